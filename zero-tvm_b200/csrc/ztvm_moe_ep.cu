// Dispatch step of the expert-parallel MoE block: every (token, slot) pair's activation row goes straight into the
// receive buffer of the rank that owns its expert, by ordinary stores to peer-mapped memory (NVLink) from one kernel.
// No collective, no host round trip: the sender picks the row's position itself, because each rank's receive buffer
// is cut into one region per SOURCE rank (seg_cap rows each) and only the source writes into its region.
//
//   region s of rank r:  rows      recv_x  [s][0 .. count)   activation rows (d f16 each) sent by rank s
//                        experts   recv_ids[s][0 .. count)   index of the row's expert inside rank r's stack
//                        sources   recv_src[s][0 .. count)   where the result row belongs in rank s's y_slots
//                                                            (token * slots_total + slot): the return address
//                        recv_cnt[s]                          count, written last by rank s
//   region `world` is local: one row per token for the replicated shared expert (when there is one).
//
// The expert matmuls then run over the whole receive buffer as ONE id list (ztvm_int4_matmul_moe_ep: regions with
// live prefixes), and the down projection's epilogue stores each result row to the source rank's y_slots through
// the return address. Ordering between ranks (all rows have landed before anyone reads; all results are back before
// the combine) is the caller's: a barrier after this kernel and one after the down projection.
#include "ztvm_kernels.h"

namespace ztvm {

__global__ void __launch_bounds__(256)
moe_ep_dispatch_kernel(const EpDispatchParams p) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t warps_per_block = blockDim.x >> 5;
  const uint32_t gwarp = blockIdx.x * warps_per_block + (threadIdx.x >> 5), nwarps = gridDim.x * warps_per_block;
  const uint32_t routed = p.tokens * p.top_k;
  const uint32_t total = routed + (p.has_shared ? p.tokens : 0u);
  const uint32_t chunks = p.d / 8u;                 // 16-byte pieces of a row
  uint32_t bad = 0;
  for (uint32_t i = gwarp; i < total; i += nwarps) {
    uint32_t t, dst_rank, local_e, src;
    if (i < routed) {
      t = i / p.top_k;
      const uint32_t s = i - t * p.top_k;
      const uint32_t e = p.ids[(size_t)t * p.ids_stride + s];
      if (e >= p.epr * p.world) { ++bad; continue; }          // warp-uniform
      dst_rank = e / p.epr;
      local_e = e - dst_rank * p.epr;
      src = t * p.slots_total + s;
    } else {                                                   // the shared expert's row of token t stays here
      t = i - routed;
      dst_rank = p.rank;
      local_e = p.epr;
      src = t * p.slots_total + p.top_k;
    }
    const uint32_t region = i < routed ? p.rank : p.world;
    uint32_t pos = 0;
    if (lane == 0) pos = atomicAdd(&p.cursors[i < routed ? dst_rank : p.world], 1u);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (pos >= p.seg_cap) { ++bad; continue; }                 // cannot happen with seg_cap >= tokens * top_k
    const size_t row = (size_t)region * p.seg_cap + pos;
    const uint4* srcp = reinterpret_cast<const uint4*>(p.x + (size_t)t * p.x_tok_stride);
    uint4* dstp = reinterpret_cast<uint4*>(p.recv_x[dst_rank] + row * p.d);
    for (uint32_t c = lane; c < chunks; c += 32u) dstp[c] = __ldg(srcp + c);
    if (lane == 0) {
      p.recv_ids[dst_rank][row] = local_e;
      p.recv_src[dst_rank][row] = src;
    }
  }
  if (bad && lane == 0) atomicAdd(p.err, bad);
  // The block that finishes last publishes the counts (every row they cover is already on its way: the fence orders
  // this block's stores, the ticket orders the blocks) and clears the cursors for the next step.
  __shared__ uint32_t is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&p.cursors[p.world + 1], 1u) == gridDim.x - 1 ? 1u : 0u;
  __syncthreads();
  if (is_last) {
    __threadfence_system();
    for (uint32_t r = threadIdx.x; r <= p.world; r += blockDim.x) {
      const uint32_t cnt = atomicExch(&p.cursors[r], 0u);
      if (r < p.world) p.recv_cnt[r][p.rank] = cnt;            // region `rank` of rank r
      else p.recv_cnt[p.rank][p.world] = cnt;                  // the local shared-expert region
    }
    if (threadIdx.x == 0) p.cursors[p.world + 1] = 0u;
    __threadfence_system();
  }
}

cudaError_t launch_moe_ep_dispatch(const EpDispatchParams& p, int sm_count, cudaStream_t st) {
  const uint32_t total = p.tokens * p.top_k + (p.has_shared ? p.tokens : 0u);
  if (total == 0) return cudaSuccess;
  const unsigned blocks = (total + 7) / 8 < (unsigned)(2 * sm_count) ? (total + 7) / 8 : (unsigned)(2 * sm_count);
  moe_ep_dispatch_kernel<<<blocks, 256, 0, st>>>(p);
  return cudaGetLastError();
}

// ---- barrier between ranks ------------------------------------------------------------------------------------------
// One warp. Lane r deals with rank r: it stores this rank's new epoch into word `rank` of rank r's flag array (release
// at system scope, after a system fence: whatever this GPU wrote before, peer stores included, is visible to whoever
// sees the flag) and then waits until word r of its own array has reached the epoch (acquire at system scope). The
// epoch lives in word `world` of the rank's own array, so replays of a captured graph keep counting. The wait is
// bounded: when it runs out, the status word is raised and the kernel returns.
__global__ void __launch_bounds__(32) peer_barrier_kernel(const PeerBarrierParams p) {
  const uint32_t lane = threadIdx.x;
  uint32_t epoch = 0;
  if (lane == 0) {
    epoch = p.flags[p.rank][p.world] + 1u;
    p.flags[p.rank][p.world] = epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  __threadfence_system();
  if (lane < p.world) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[lane] + p.rank), "r"(epoch) : "memory");
    const uint32_t* mine = p.flags[p.rank] + lane;
    const long long t0 = clock64();
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int32_t)(v - epoch) >= 0) break;
      if ((unsigned long long)(clock64() - t0) > p.wait_cycles) { atomicExch(p.status, 20u); break; }
      __nanosleep(200);
    }
  }
}

cudaError_t launch_peer_barrier(const PeerBarrierParams& p, cudaStream_t st) {
  peer_barrier_kernel<<<1, 32, 0, st>>>(p);
  return cudaGetLastError();
}

}  // namespace ztvm
