// Grouped MoE expert matmul for many (token, slot) pairs: the same contract as the ids-indirect GEMV
//   y[token, slot, :] = x[token, slot, :] * W16[ids[token, slot]]^T        (int4_matmul.gen.ts:229-254)
// but driven by an index list sorted by expert, so each expert's weights are dequantised once per 128 pairs
// and multiplied on the tensor cores instead of once per pair on CUDA cores.
//
// Planning (three small kernels over scratch memory): histogram of the expert ids, prefix sums + tile table
// (one tile = up to 128 pairs of one expert), scatter of the pair indices into expert order.
// GEMM (one CTA per tile x 128 weight rows): warp 0 TMA-loads the expert's packed weights, warp 1 issues
// tcgen05.mma, warps 2..9 gather the activation rows of the tile's pairs with 16-byte cp.async straight into
// the swizzled A slot, dequantise the B slot, and at the end scatter the rows of D to where each pair lives.
#include <mutex>

#include "ztvm_kernels.h"
#include "ztvm_moe_plan.cuh"
#include "ztvm_tc.cuh"

namespace ztvm {

constexpr int kMoeStages = 5;
constexpr int kMoeWStages = 3;
constexpr int kMoeWChunk = 4;
constexpr int kMoeWorkWarps = 8;
constexpr int kMoeThreads = 64 + kMoeWorkWarps * 32;
constexpr int kMoeBM = 128, kMoeBN = 128;

// Entry i of a segmented id list is live when it lies in the filled prefix of its region (expert-parallel form).
struct MoeSegs {
  const uint32_t* counts;
  uint32_t cap;
  __device__ __forceinline__ bool live(uint32_t i) const { return !counts || (i % cap) < counts[i / cap]; }
};

__global__ void moe_count_kernel(const uint32_t* __restrict__ ids, uint32_t tokens, uint32_t slots, uint32_t ids_stride,
                                 uint32_t E, MoeScratch sc, uint32_t* err, MoeSegs segs) {
  const uint32_t P = tokens * slots;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < P; i += gridDim.x * blockDim.x) {
    if (!segs.live(i)) continue;
    const uint32_t t = i / slots, s = i - t * slots;
    const uint32_t e = ids[(size_t)t * ids_stride + s];
    if (e < E) atomicAdd(&sc.counts[e], 1u);
    else atomicAdd(err, 1u);
  }
}

// Exclusive scan over the 1024 threads of a block (values in registers, one per thread).
__device__ __forceinline__ uint32_t moe_block_excl_scan(uint32_t v, uint32_t* warp_sums, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += t;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = warp_sums[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += t;
    }
    warp_sums[lane] = w;   // inclusive over warps
  }
  __syncthreads();
  const uint32_t base = warp ? warp_sums[warp - 1] : 0u;
  *total = warp_sums[31];
  __syncthreads();         // warp_sums may be reused by the next scan
  return base + inc - v;
}

// One block of 1024 threads, thread e = expert e (E <= 1024): offsets and tile table from the counts.
__global__ void __launch_bounds__(1024) moe_plan_kernel(uint32_t E, uint32_t tile_rows, MoeScratch sc) {
  __shared__ uint32_t warp_sums[32];
  const uint32_t e = threadIdx.x;
  const uint32_t cnt = e < E ? sc.counts[e] : 0u;
  const uint32_t nt = (cnt + tile_rows - 1) / tile_rows;
  uint32_t total_pairs, total_tiles;
  const uint32_t off = moe_block_excl_scan(cnt, warp_sums, &total_pairs);
  const uint32_t tb = moe_block_excl_scan(nt, warp_sums, &total_tiles);
  if (e < E) sc.offsets[e] = off;
  if (e == 0) { sc.offsets[E] = total_pairs; *sc.ntiles = total_tiles; }
  for (uint32_t j = 0; j < nt; ++j) {
    uint32_t* tt = sc.tiles + (size_t)(tb + j) * 3;
    tt[0] = e;
    tt[1] = off + j * tile_rows;
    tt[2] = min(tile_rows, cnt - j * tile_rows);
  }
}

// Increment of cnt[key] by every active lane, returning the lane's slot. When all active lanes of the warp hold the
// same key (the slot of a shared expert: thousands of pairs with one id), one lane adds for the warp; one atomic per
// pair on that single address would serialise the whole plan. Mixed keys take one atomic per lane (little contention).
__device__ __forceinline__ uint32_t moe_agg_add(uint32_t* cnt, uint32_t key, bool active) {
  const uint32_t amask = __ballot_sync(0xffffffffu, active);
  if (amask == 0u) return 0u;
  const int lane = threadIdx.x & 31, leader = __ffs(amask) - 1;
  const uint32_t key0 = __shfl_sync(0xffffffffu, key, leader);
  const bool uniform = __all_sync(0xffffffffu, !active || key == key0);
  if (uniform) {
    uint32_t base = 0u;
    if (lane == leader) base = atomicAdd(&cnt[key0], (uint32_t)__popc(amask));
    base = __shfl_sync(0xffffffffu, base, leader);
    return base + (uint32_t)__popc(amask & ((1u << lane) - 1u));
  }
  return active ? atomicAdd(&cnt[key], 1u) : 0u;
}

// The whole plan in ONE block for pair lists up to a few tens of thousands: histogram and cursors in shared memory,
// same scans, same tables. Pairs are walked slot-major (a warp sees 32 tokens of one slot), so the pairs of a slot
// that always carries the same expert (the shared expert) aggregate into one atomic per warp.
constexpr uint32_t kPlanSmallMax = 32768;   // pairs the one-block plan takes: 32 per thread, kept in registers
__global__ void __launch_bounds__(1024) moe_plan_small_kernel(const uint32_t* __restrict__ ids, uint32_t tokens, uint32_t slots,
                                                              uint32_t ids_stride, uint32_t E, uint32_t tile_rows,
                                                              MoeScratch sc, uint32_t* err, MoeSegs segs) {
  __shared__ uint32_t cnt_sm[1024], cur_sm[1024], warp_sums[32];
  const uint32_t e = threadIdx.x, P = tokens * slots;
  cnt_sm[e] = 0u;
  // every id of this thread is loaded up front (independent loads in flight together), then counted, then scattered
  uint32_t xs[kPlanSmallMax / 1024];
#pragma unroll
  for (int k = 0; k < (int)(kPlanSmallMax / 1024); ++k) {
    const uint32_t j = threadIdx.x + 1024u * k;                     // j = slot * tokens + token
    xs[k] = 0xFFFFFFFFu;
    if (j < P) {
      const uint32_t s = j / tokens, t = j - s * tokens;
      if (segs.live(t * slots + s)) xs[k] = ids[(size_t)t * ids_stride + s];
      else xs[k] = 0xFFFFFFFEu;                                    // not a pair at all (past a region's live rows)
    }
  }
  __syncthreads();
  uint32_t bad = 0;
#pragma unroll
  for (int k = 0; k < (int)(kPlanSmallMax / 1024); ++k) {
    if (1024u * k >= P) break;                                      // block-uniform
    if (xs[k] >= E && xs[k] < 0xFFFFFFFEu) ++bad;
    moe_agg_add(cnt_sm, xs[k], xs[k] < E);
  }
  if (bad) atomicAdd(err, bad);
  __syncthreads();
  const uint32_t cnt = e < E ? cnt_sm[e] : 0u;
  const uint32_t nt = (cnt + tile_rows - 1) / tile_rows;
  uint32_t total_pairs, total_tiles;
  const uint32_t off = moe_block_excl_scan(cnt, warp_sums, &total_pairs);
  const uint32_t tb = moe_block_excl_scan(nt, warp_sums, &total_tiles);
  cur_sm[e] = off;
  if (e < E) { sc.counts[e] = cnt; sc.offsets[e] = off; }
  if (e == 0) { sc.offsets[E] = total_pairs; *sc.ntiles = total_tiles; }
  for (uint32_t j = 0; j < nt; ++j) {
    uint32_t* tt = sc.tiles + (size_t)(tb + j) * 3;
    tt[0] = e;
    tt[1] = off + j * tile_rows;
    tt[2] = min(tile_rows, cnt - j * tile_rows);
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < (int)(kPlanSmallMax / 1024); ++k) {
    if (1024u * k >= P) break;
    const uint32_t j = threadIdx.x + 1024u * k;
    const bool ok = xs[k] < E;
    const uint32_t pos = moe_agg_add(cur_sm, xs[k], ok);
    if (ok) {
      const uint32_t s = j / tokens, t = j - s * tokens;
      sc.sorted[pos] = t * slots + s;
    }
  }
}

__global__ void moe_scatter_kernel(const uint32_t* __restrict__ ids, uint32_t tokens, uint32_t slots,
                                   uint32_t ids_stride, uint32_t E, MoeScratch sc, MoeSegs segs) {
  const uint32_t P = tokens * slots;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < P; i += gridDim.x * blockDim.x) {
    if (!segs.live(i)) continue;
    const uint32_t t = i / slots, s = i - t * slots;
    const uint32_t e = ids[(size_t)t * ids_stride + s];
    if (e < E) sc.sorted[sc.offsets[e] + atomicAdd(&sc.cursor[e], 1u)] = i;
  }
}

struct MoeGemmParams {
  const __half* S;
  const __half* B;
  const __half* X;
  __half* Y;
  uint32_t N, K, KP, SPR, slots;
  uint32_t in_slot_stride, out_slot_stride, in_tok_stride, out_tok_stride;
  MoeScratch sc;
  uint32_t* status;
};

struct MoeSmem {
  static constexpr int kABytes = kMoeBM * kGemmBK * 2;
  static constexpr int kBBytes = kMoeBN * kGemmBK * 2;
  static constexpr int kWBytes = kMoeBN * 128;
  static constexpr int kOffB = kMoeStages * kABytes;
  static constexpr int kOffW = kOffB + kMoeStages * kBBytes;
  static constexpr int kOffBar = kOffW + kMoeWStages * kWBytes;
  static constexpr int kTotal = kOffBar + 256;
};

__device__ __forceinline__ void cp_async16_sw(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

__global__ void __launch_bounds__(kMoeThreads, 1)
moe_gemm_w4_kernel(const __grid_constant__ CUtensorMap tmap_w, const MoeGemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using L = MoeSmem;
  const uint32_t tile = blockIdx.y;
  if (tile >= *p.sc.ntiles) return;   // uniform per CTA, before any barrier / TMEM use
  const uint32_t expert = p.sc.tiles[(size_t)tile * 3], r0 = p.sc.tiles[(size_t)tile * 3 + 1],
                 rows = p.sc.tiles[(size_t)tile * 3 + 2];

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t a_ring = base, b_ring = base + L::kOffB, w_ring = base + L::kOffW, bars = base + L::kOffBar;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_empty = [&](int s) { return bars + 8u * (kMoeStages + s); };
  auto bar_w_full = [&](int s) { return bars + 8u * (2 * kMoeStages + s); };
  auto bar_w_empty = [&](int s) { return bars + 8u * (2 * kMoeStages + kMoeWStages + s); };
  constexpr int kNumBars = 2 * kMoeStages + 2 * kMoeWStages + 1;
  const uint32_t bar_accum = bars + 8u * (kNumBars - 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + L::kOffBar + 8 * kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t n0 = blockIdx.x * kMoeBN;
  const uint32_t num_kb = p.K / kGemmBK;
  constexpr uint32_t kTmemCols = kMoeBN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMoeStages; ++s) {
      mbar_init(bar_full(s), kMoeWorkWarps * 32);   // every worker thread arrives itself, right after its own proxy fence
      mbar_init(bar_empty(s), 1);
    }
    for (int s = 0; s < kMoeWStages; ++s) {
      mbar_init(bar_w_full(s), 1);
      mbar_init(bar_w_empty(s), kMoeWorkWarps);
    }
    mbar_init(bar_accum, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- TMA producer: packed weights of this expert, rows [expert*N + n0, +128) of the flattened stack ----
    if (lane == 0) {
      const uint32_t num_chunks = (num_kb + kMoeWChunk - 1) / kMoeWChunk;
      uint32_t issued = 0;
      for (uint32_t c = 0; c < num_chunks; ++c) {
        const int s = c % kMoeWStages;
        const uint32_t ph = (c / kMoeWStages) & 1u;
        if (c >= kMoeWStages && !mbar_wait(bar_w_empty(s), ph ^ 1u, p.status, 6u, abort_flag)) break;
        mbar_arrive_expect_tx(bar_w_full(s), (uint32_t)L::kWBytes);
        tma_load_2d(w_ring + s * L::kWBytes, &tmap_w, bar_w_full(s), (int)(c * 32), (int)(expert * p.N + n0));
        issued = c + 1;
      }
      if (*abort_flag) {
        const uint32_t first = issued > (uint32_t)kMoeWStages ? issued - kMoeWStages : 0u;
        for (uint32_t c = first; c < issued; ++c) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar_w_full(c % kMoeWStages), (c / kMoeWStages) & 1u) &&
                 (unsigned long long)(clock64() - t0) < kWaitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_f16(kMoeBN);
      const uint64_t a0 = smem_desc_sw128(a_ring), b0 = smem_desc_sw128(b_ring);
      uint32_t s = 0, ph = 0;
      bool ok = true;
      for (uint32_t kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait(bar_full(s), ph, p.status, 2u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint64_t adesc = a0 + (uint64_t)(s * (L::kABytes >> 4)), bdesc = b0 + (uint64_t)(s * (L::kBBytes >> 4));
#pragma unroll
        for (int k = 0; k < kGemmBK / 16; ++k)
          umma_f16(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb | (uint32_t)k) ? 1u : 0u);
        umma_commit(bar_empty(s));
        if (++s == (uint32_t)kMoeStages) { s = 0; ph ^= 1u; }
      }
      if (ok) umma_commit(bar_accum);
    }
  } else {
    // ---- workers: gather A rows, dequantise B rows, then scatter the result rows ----
    const int t = threadIdx.x - 64;                 // 0..255
    const uint32_t r_tile = (uint32_t)(t >> 1), part = (uint32_t)(t & 1);
    const uint32_t row_off = (r_tile >> 3) * 1024 + (r_tile & 7) * 128;
    // source row of this thread's activation row (rows past the tile's count re-read row 0: harmless, never stored)
    const uint32_t pair = p.sc.sorted[r0 + (r_tile < rows ? r_tile : 0u)];
    const uint32_t tok = pair / p.slots, slot = pair - tok * p.slots;
    const __half* xrow = p.X + (size_t)tok * p.in_tok_stride + (size_t)slot * p.in_slot_stride;
    // weight row of this thread inside the expert
    const uint32_t wrow_idx = expert * p.N + min(n0 + r_tile, p.N - 1);
    const unsigned short* srow = reinterpret_cast<const unsigned short*>(p.S) + (size_t)wrow_idx * p.SPR;
    const unsigned short* brow = reinterpret_cast<const unsigned short*>(p.B) + (size_t)wrow_idx * p.SPR;

    auto issue_a = [&](uint32_t kb) {
      if (kb < num_kb) {
        const uint32_t dst = a_ring + (kb % kMoeStages) * L::kABytes + row_off;
        const __half* src = xrow + (size_t)kb * kGemmBK + part * 32;
#pragma unroll
        for (int c = 0; c < 4; ++c) cp_async16_sw(dst + (((part * 4 + c) ^ (r_tile & 7)) << 4), src + c * 8);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    constexpr int kLead = kMoeStages - 2;   // activation rows are fetched this many k blocks ahead
#pragma unroll
    for (int i = 0; i < kLead; ++i) issue_a((uint32_t)i);

    bool ok = true;
    for (uint32_t kb = 0; kb < num_kb && ok; ++kb) {
      const int s = (int)(kb % kMoeStages);
      const uint32_t c = kb / kMoeWChunk, j = kb % kMoeWChunk;
      const int ws = (int)(c % kMoeWStages);
      if (j == 0) ok = mbar_wait(bar_w_full(ws), (c / kMoeWStages) & 1u, p.status, 7u, abort_flag);
      uint4 wv = make_uint4(0, 0, 0, 0);
      if (ok) {
        const uint32_t chunk16 = j * 2 + part;
        wv = *reinterpret_cast<const uint4*>(gen_base + L::kOffW + ws * L::kWBytes + row_off + ((chunk16 ^ (r_tile & 7)) << 4));
      }
      // the slot that the look-ahead gather will fill was last read by the MMAs of k block kb + kLead - kMoeStages
      const uint32_t kn = kb + kLead;
      if (ok && kn < num_kb && kn >= (uint32_t)kMoeStages)
        ok = mbar_wait(bar_empty((int)(kn % kMoeStages)), ((kn / kMoeStages) & 1u) ^ 1u, p.status, 4u, abort_flag);
      if (ok) issue_a(kn); else asm volatile("cp.async.commit_group;" ::: "memory");
      if (ok) {
        const unsigned short s16 = __ldg(srow + kb), b16 = __ldg(brow + kb);   // group 64: one group per k block
        const DqGroup dq = dq_group<true>(s16, b16);
        uint8_t* rowp = gen_base + L::kOffB + s * L::kBBytes + row_off;
        const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const uint4 v = dequant_word_w16<true>(words[wi], dq);
          *reinterpret_cast<uint4*>(rowp + (((part * 4 + wi) ^ (r_tile & 7)) << 4)) = v;
        }
      }
      // The packed-weight slot is handed back only after the stores that consume its words: a release placed right
      // after the load let the refill land before the load had been performed.
      if (j == kMoeWChunk - 1 || kb + 1 == num_kb) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_w_empty(ws));
      }
      asm volatile("cp.async.wait_group %0;" ::"n"(kLead) : "memory");   // this thread's part of A(kb) has landed
      fence_proxy_async();
      mbar_arrive(bar_full(s));
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    const bool acc_ok = ok && mbar_wait(bar_accum, 0u, p.status, 5u, abort_flag);
    tc_fence_after();
    if (acc_ok) {
      const int quarter = warp & 3, half = (warp - 2) >> 2;
      const uint32_t r = (uint32_t)(quarter * 32 + lane);
      __half* dst_row = nullptr;
      if (r < rows) {
        const uint32_t pr = p.sc.sorted[r0 + r];
        const uint32_t tk = pr / p.slots, sl = pr - tk * p.slots;
        dst_row = p.Y + (size_t)tk * p.out_tok_stride + (size_t)sl * p.out_slot_stride;
      }
      const bool vec_ok = ((p.out_tok_stride | p.out_slot_stride) % 8u) == 0 && (reinterpret_cast<uintptr_t>(p.Y) & 15u) == 0;
#pragma unroll 1
      for (int cb = half; cb < kMoeBN / 32; cb += 2) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(cb * 32), v);
        tmem_ld_wait();
        const uint32_t n = n0 + cb * 32;
        if (dst_row && n < p.N) {
          if (vec_ok && n + 32 <= p.N) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 o;
              __half2 h;
              h = __floats2half2_rn(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1])); o.x = *reinterpret_cast<uint32_t*>(&h);
              h = __floats2half2_rn(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3])); o.y = *reinterpret_cast<uint32_t*>(&h);
              h = __floats2half2_rn(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5])); o.z = *reinterpret_cast<uint32_t*>(&h);
              h = __floats2half2_rn(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7])); o.w = *reinterpret_cast<uint32_t*>(&h);
              reinterpret_cast<uint4*>(dst_row + n)[i] = o;
            }
          } else {
            for (int i = 0; i < 32 && n + i < p.N; ++i) dst_row[n + i] = __float2half_rn(__uint_as_float(v[i]));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// Plan of one grouped launch: histogram of the expert ids, prefix sums + table of tiles of at most `tile_rows` pairs of
// one expert, scatter of the pair indices into expert order. The words that must start at zero are cleared here.
cudaError_t launch_moe_plan(const GemvParams& g, uint32_t tokens, uint32_t slots, const MoeScratch& sc, uint32_t tile_rows,
                            cudaStream_t st) {
  const uint32_t P = tokens * slots, E = g.experts;
  const MoeSegs segs{g.seg_counts, g.seg_cap ? g.seg_cap : 1u};
  if (P <= kPlanSmallMax) {   // short lists: one block does it all, nothing to clear beforehand
    moe_plan_small_kernel<<<1, 1024, 0, st>>>(g.ids, tokens, slots, g.ids_stride, E, tile_rows, sc, g.err_counter, segs);
    return cudaGetLastError();
  }
  cudaError_t e = cudaMemsetAsync(sc.counts, 0, ((size_t)E * 3 + 4) * 4, st);   // counts, offsets, cursor, ntiles
  if (e != cudaSuccess) return e;
  const unsigned blocks = (P + 255) / 256 > 1184 ? 1184 : (P + 255) / 256;
  moe_count_kernel<<<blocks, 256, 0, st>>>(g.ids, tokens, slots, g.ids_stride, E, sc, g.err_counter, segs);
  moe_plan_kernel<<<1, 1024, 0, st>>>(E, tile_rows, sc);
  moe_scatter_kernel<<<blocks, 256, 0, st>>>(g.ids, tokens, slots, g.ids_stride, E, sc, segs);
  return cudaGetLastError();
}

// ---- dispatch plan of the expert-parallel form ---------------------------------------------------------------------
// After the plan: pairs sorted by expert are also sorted by the rank that owns the expert (experts are dealt to ranks in
// contiguous runs of `epr`). order[i] = pair index, local_expert[i] = its expert's index inside the owner's stack,
// send_counts[r] = pairs that travel to rank r.
__global__ void moe_dispatch_finish_kernel(uint32_t E, uint32_t epr, uint32_t world, MoeScratch sc, long long* order,
                                           int* local_expert, long long* send_counts) {
  const uint32_t P = sc.offsets[E];
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < P; i += gridDim.x * blockDim.x) {
    uint32_t lo = 0, hi = E;                       // the expert e with offsets[e] <= i < offsets[e + 1]
    while (hi - lo > 1) {
      const uint32_t mid = (lo + hi) >> 1;
      if (sc.offsets[mid] <= i) lo = mid; else hi = mid;
    }
    order[i] = (long long)sc.sorted[i];
    local_expert[i] = (int)(lo % epr);
  }
  if (blockIdx.x == 0)
    for (uint32_t r = threadIdx.x; r < world; r += blockDim.x) {
      const uint32_t a = min(r * epr, E), b = min((r + 1) * epr, E);
      send_counts[r] = (long long)(sc.offsets[b] - sc.offsets[a]);
    }
}

cudaError_t launch_moe_dispatch_plan(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t epr, uint32_t world,
                                     uint32_t* scratch, long long* order, int* local_expert, long long* send_counts,
                                     cudaStream_t st) {
  const uint32_t P = tokens * slots;
  MoeScratch sc = moe_scratch_carve(scratch, g.experts, P);
  cudaError_t e = launch_moe_plan(g, tokens, slots, sc, (uint32_t)kMoeBM, st);
  if (e != cudaSuccess) return e;
  const unsigned blocks = (P + 255) / 256 > 592 ? 592 : (P + 255) / 256;
  moe_dispatch_finish_kernel<<<blocks ? blocks : 1, 256, 0, st>>>(g.experts, epr, world, sc, order, local_expert, send_counts);
  return cudaGetLastError();
}

// ---- host side -----------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn moe_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

size_t moe_grouped_scratch_bytes(uint32_t experts, uint32_t pairs) { return moe_scratch_words(experts, pairs) * 4; }

bool moe_grouped_supported(int bits, uint32_t group, uint32_t K, uint32_t N, uint32_t experts) {
  return bits == 4 && group == 64 && K % kGemmBK == 0 && N % kMoeBN == 0 && experts <= 1024;
}

cudaError_t launch_moe_grouped(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t* scratch, uint32_t* status,
                               cudaStream_t st) {
  EncodeTiledFn enc = moe_encode_fn();
  if (!enc) return cudaErrorNotSupported;
  const uint32_t P = tokens * slots, E = g.experts;
  MoeScratch sc = moe_scratch_carve(scratch, E, P);
  cudaError_t e = launch_moe_plan(g, tokens, slots, sc, (uint32_t)kMoeBM, st);
  if (e != cudaSuccess) return e;

  CUtensorMap tmap_w;
  const cuuint64_t wdims[2] = {g.KP, (cuuint64_t)E * g.N};
  const cuuint64_t wstrides[1] = {(cuuint64_t)g.KP * 4};
  const cuuint32_t wbox[2] = {32, (cuuint32_t)kMoeBN};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(g.W), wdims, wstrides, wbox, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  MoeGemmParams p;
  p.S = g.S; p.B = g.B; p.X = g.X; p.Y = reinterpret_cast<__half*>(g.Y);
  p.N = g.N; p.K = g.K; p.KP = g.KP; p.SPR = g.SPR; p.slots = slots;
  p.in_slot_stride = g.in_slot_stride; p.out_slot_stride = g.out_slot_stride;
  p.in_tok_stride = g.in_tok_stride; p.out_tok_stride = g.out_tok_stride;
  p.sc = sc; p.status = status;
  constexpr int smem = MoeSmem::kTotal + 1024;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    e = cudaFuncSetAttribute(moe_gemm_w4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const uint32_t max_tiles = (P + kMoeBM - 1) / kMoeBM + E;
  if (max_tiles > 65535u) return cudaErrorInvalidConfiguration;   // grid.y; 65536 pairs and 1024 experts stay far below
  dim3 grid(g.N / kMoeBN, max_tiles);
  moe_gemm_w4_kernel<<<grid, kMoeThreads, smem, st>>>(tmap_w, p);
  return cudaGetLastError();
}

// ---- the same matmul with its planning scratch in a fixed device array: nothing is allocated ------------------
// For callers that cannot let a matmul allocate: a serving loop whose device memory is all handed to its own pool,
// or one that cannot afford the device-wide synchronisation that growing a buffer implies. The scratch lives in the
// module's own image, so it exists (once per device) as soon as the module is loaded there.
constexpr uint32_t kMoeStaticMaxExperts = 1024, kMoeStaticMaxPairs = 65536;
constexpr size_t kMoeStaticWords = moe_scratch_words(kMoeStaticMaxExperts, kMoeStaticMaxPairs);   // 385 KB
static __device__ __align__(256) uint32_t g_moe_static_scratch[kMoeStaticWords];

bool moe_static_scratch_fits(uint32_t experts, uint64_t pairs) {
  return experts <= kMoeStaticMaxExperts && pairs <= kMoeStaticMaxPairs &&
         moe_scratch_words(experts, (uint32_t)pairs) <= kMoeStaticWords;
}

// Device address of the array on the CURRENT device. The host-side name of a __device__ array is not a device
// address: the runtime has to be asked for it, once per device (each device holds its own copy of the array).
static cudaError_t moe_static_scratch_ptr(uint32_t** out) {
  constexpr int kMaxDevices = 64;
  static uint32_t* ptrs[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (!ptrs[dev]) {
    void* addr = nullptr;
    e = cudaGetSymbolAddress(&addr, g_moe_static_scratch);
    if (e != cudaSuccess) return e;
    if (!addr) return cudaErrorInvalidSymbol;
    ptrs[dev] = static_cast<uint32_t*>(addr);
  }
  *out = ptrs[dev];
  return cudaSuccess;
}

cudaError_t launch_moe_grouped_static(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t* status,
                                      cudaStream_t st) {
  if (!moe_static_scratch_fits(g.experts, (uint64_t)tokens * slots)) return cudaErrorInvalidValue;
  uint32_t* scratch = nullptr;
  const cudaError_t e = moe_static_scratch_ptr(&scratch);
  if (e != cudaSuccess) return e;
  // launch_moe_grouped zeroes the words that must start at zero (counts, offsets, cursors, tile count) on `st`
  // before the planning kernels; the rest of the scratch is fully written before it is read.
  return launch_moe_grouped(g, tokens, slots, scratch, status, st);
}

cudaError_t launch_moe_ta_static(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t* status, int sm_count,
                                 cudaStream_t st) {
  if (!moe_static_scratch_fits(g.experts, (uint64_t)tokens * slots)) return cudaErrorInvalidValue;
  uint32_t* scratch = nullptr;
  const cudaError_t e = moe_static_scratch_ptr(&scratch);
  if (e != cudaSuccess) return e;
  return launch_moe_ta(g, tokens, slots, scratch, status, sm_count, st);   // its plan launch clears what must start at zero
}

cudaError_t launch_moe_tc_static(const GemvParams& g, uint32_t tokens, uint32_t slots, int sm_count, cudaStream_t st) {
  if (!moe_static_scratch_fits(g.experts, (uint64_t)tokens * slots)) return cudaErrorInvalidValue;
  uint32_t* scratch = nullptr;
  const cudaError_t e = moe_static_scratch_ptr(&scratch);
  if (e != cudaSuccess) return e;
  return launch_moe_tc(g, tokens, slots, scratch, sm_count, st);   // its plan launch clears what must start at zero
}

}  // namespace ztvm
