// Prefill GEMM, M > 8, 4-bit weights: y[M, N] = x[M, K] * W16[N, K]^T on tcgen05 with the DEQUANTISED WEIGHTS AS THE
// A OPERAND IN TENSOR MEMORY (replaces the matrix-unit GEMMs of int4_matmul.gen.ts:1058-1456; contract of
// ztvm_int4_matmul for M > 8).
//
// Why this orientation. With both operands in shared memory a 128 x 128 x 16 tcgen05.mma reads 8 KB per ~68 cycles,
// close to the shared-memory port's whole rate, next to the dequantisers' stores and the TMA writes (ztvm_gemm.cu).
// Here the weights take the M side of the MMA (128 weight rows = 128 TMEM
// lanes) and go from the dequantisers' registers straight into tensor memory with tcgen05.st; the activations take
// the N side (256 tokens per instruction) and are the only operand read from shared memory: 32 KB per k block
// instead of 64 + 16. D is [weight row][token] in tensor memory; the epilogue writes it transposed (a warp's 32 lanes
// are 32 consecutive output columns of one token: 64-byte stores).
//
// Roles (352 threads): warp 0 TMA-loads activation tiles (NT tokens x 64 k, 128-byte swizzle); warp 2 TMA-loads
// packed weight tiles (128 rows x 32 words = four k blocks); warps 3..10 dequantise: warp w may touch TMEM lanes
// 32 (w % 4) .. +31, so it owns those 32 weight rows, and the two warps that share a lane quarter split the k block
// in halves (16 TMEM columns each); warp 1 allocates tensor memory and issues the MMAs. Every wait is bounded
// (status word, as in ztvm_gemm.cu).
#include <type_traits>
#include "ztvm_kernels.h"
#include "ztvm_tc.cuh"

namespace ztvm {

constexpr int kTaStages = 4;        // activation tiles in shared memory and weight slices in tensor memory
constexpr int kTaWStages = 3;       // packed-weight ring (each slot holds four k blocks)
constexpr int kTaWChunk = 4;
constexpr int kTaDqWarps = 16;      // two teams of eight: a team takes every other k block
constexpr int kTaThreads = 96 + kTaDqWarps * 32;
constexpr int kTaRows = 128;        // weight rows per CTA = TMEM lanes

struct GemmTaParams {
  const __half* S;
  const __half* B;   // nullptr: symmetric
  void* Y;
  uint32_t M, N, K, SPR, group_shift, out_f32;
  uint32_t* status;
};

template <int NT>
struct GemmTaSmem {
  static constexpr int kXBytes = NT * kGemmBK * 2;            // per stage
  static constexpr int kWBytes = kTaRows * 128;               // per packed-weight slot
  static constexpr int kOffW = kTaStages * kXBytes;
  static constexpr int kOffBar = kOffW + kTaWStages * kWBytes;
  static constexpr int kTotal = kOffBar + 256;
};

template <int NT, bool AFFINE>
__global__ void __launch_bounds__(kTaThreads, 1)
gemm_w4_ta_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                  const GemmTaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using L = GemmTaSmem<NT>;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t x_ring = base, w_ring = base + L::kOffW, bars = base + L::kOffBar;
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_empty = [&](int s) { return bars + 8u * (kTaStages + s); };
  auto bar_w_full = [&](int s) { return bars + 8u * (2 * kTaStages + s); };
  auto bar_w_empty = [&](int s) { return bars + 8u * (2 * kTaStages + kTaWStages + s); };
  constexpr int kNumBars = 2 * kTaStages + 2 * kTaWStages + 1;
  const uint32_t bar_accum = bars + 8u * (kNumBars - 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + L::kOffBar + 8 * kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t n0 = blockIdx.x * kTaRows;
  const uint32_t m0 = blockIdx.y * NT;
  const uint32_t num_kb = p.K / kGemmBK;
  constexpr uint32_t kColA = NT;                                 // weight slices start after the accumulator columns
  constexpr uint32_t kTmemCols = NT + kTaStages * 32 <= 256 ? 256 : 512;

  if (threadIdx.x == 32) { tma_prefetch_desc(&tmap_x); tma_prefetch_desc(&tmap_w); }
  // Each TMA producer initialises the barriers its own copies signal and starts its first loads before the block
  // barrier: they fly while tensor memory is allocated.
  if (threadIdx.x == 0) {
    for (int s = 0; s < kTaStages; ++s) {
      mbar_init(bar_full(s), 1 + (kTaDqWarps / 2) * 32);   // the activation tile (with its byte count) + every thread of the team that writes the slice
      mbar_init(bar_empty(s), 1);
    }
    mbar_init(bar_accum, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // Programmatic dependent launch: everything before this point (and the weight / scale loads of the other warps)
    // touches nothing the previous kernel in the stream may write; the activations may be its output.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t kb = 0; kb < (uint32_t)kTaStages && kb < num_kb; ++kb) {
      mbar_arrive_expect_tx(bar_full((int)kb), (uint32_t)L::kXBytes);
#pragma unroll
      for (int b = 0; b < NT / 128; ++b)
        tma_load_2d(x_ring + kb * L::kXBytes + b * (128 * kGemmBK * 2), &tmap_x, bar_full((int)kb), (int)(kb * kGemmBK), (int)(m0 + b * 128));
    }
  }
  if (threadIdx.x == 64) {
    for (int s = 0; s < kTaWStages; ++s) {
      mbar_init(bar_w_full(s), 1);
      mbar_init(bar_w_empty(s), kTaDqWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const uint32_t nc = (num_kb + kTaWChunk - 1) / kTaWChunk;
    for (uint32_t c = 0; c < (uint32_t)kTaWStages && c < nc; ++c) {
      mbar_arrive_expect_tx(bar_w_full((int)c), (uint32_t)L::kWBytes);
      tma_load_2d(w_ring + c * L::kWBytes, &tmap_w, bar_w_full((int)c), (int)(c * 32), (int)n0);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  // The dequantisers' first scales and biases (16 groups of this thread's row) are requested before the block barrier:
  // weights are not written by the previous kernel in the stream, and the DRAM latency of these loads would otherwise
  // sit between the barrier and the first dequantised stage.
  uint4 sv_pre0 = make_uint4(0, 0, 0, 0), bv_pre0 = sv_pre0, sv_pre1 = sv_pre0, bv_pre1 = sv_pre0;
  const bool vec_sb_all = p.group_shift == 6 && (p.SPR % 8u) == 0 &&
                          ((reinterpret_cast<uintptr_t>(p.S) | reinterpret_cast<uintptr_t>(p.B)) & 15u) == 0;
  if (warp >= 3 && vec_sb_all) {
    const uint32_t row_pre = min(n0 + (uint32_t)((warp & 3) * 32 + lane), p.N - 1);
    const unsigned short* sp = reinterpret_cast<const unsigned short*>(p.S) + (size_t)row_pre * p.SPR;
    const unsigned short* bp = reinterpret_cast<const unsigned short*>(p.B) + (size_t)row_pre * p.SPR;
    sv_pre0 = __ldg(reinterpret_cast<const uint4*>(sp));
    if (AFFINE) bv_pre0 = __ldg(reinterpret_cast<const uint4*>(bp));
    if (num_kb > 8u) {
      sv_pre1 = __ldg(reinterpret_cast<const uint4*>(sp + 8));
      if (AFFINE) bv_pre1 = __ldg(reinterpret_cast<const uint4*>(bp + 8));
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ================= TMA producer: activations =================
    if (lane == 0) {
      uint32_t issued = num_kb < (uint32_t)kTaStages ? num_kb : (uint32_t)kTaStages;
      for (uint32_t kb = issued; kb < num_kb; ++kb) {
        const int s = kb % kTaStages;
        const uint32_t ph = (kb / kTaStages) & 1u;
        if (!mbar_wait(bar_empty(s), ph ^ 1u, p.status, 1u, abort_flag)) break;
        mbar_arrive_expect_tx(bar_full(s), (uint32_t)L::kXBytes);
#pragma unroll
        for (int b = 0; b < NT / 128; ++b)
          tma_load_2d(x_ring + s * L::kXBytes + b * (128 * kGemmBK * 2), &tmap_x, bar_full(s), (int)(kb * kGemmBK), (int)(m0 + b * 128));
        issued = kb + 1;
      }
      if (*abort_flag) {   // the consumer stopped: wait (bounded) until the copies already issued have landed
        const uint32_t first = issued > (uint32_t)kTaStages ? issued - kTaStages : 0u;
        for (uint32_t kb = first; kb < issued; ++kb) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar_full(kb % kTaStages), (kb / kTaStages) & 1u) &&
                 (unsigned long long)(clock64() - t0) < kWaitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_f16(NT);
      const uint64_t b0 = smem_desc_sw128(x_ring);
      uint32_t s = 0, ph = 0;
      // The thread is held at each tcgen05.mma until the pipe takes it, so a barrier poll between two k blocks would
      // be a bubble in the pipe: the next block's barrier is polled once before the last MMA of the current block is
      // issued, in the shadow of the MMAs already queued, and waited for afterwards only if that poll failed.
      bool ok = mbar_wait(bar_full(0), 0u, p.status, 2u, abort_flag);
      for (uint32_t kb = 0; kb < num_kb && ok; ++kb) {
        tc_fence_after();
        const uint64_t bdesc = b0 + (uint64_t)(s * (L::kXBytes >> 4));
        const uint32_t a_tmem = tmem_base + kColA + s * 32u;
        uint32_t s1 = s + 1u, ph1 = ph;
        if (s1 == (uint32_t)kTaStages) { s1 = 0; ph1 ^= 1u; }
        bool next_ready = true;
#pragma unroll
        for (int k = 0; k < kGemmBK / 16; ++k) {   // 16 k elements: 8 TMEM columns of A, 32 bytes along the swizzled B row
          if (k == kGemmBK / 16 - 1 && kb + 1 < num_kb) next_ready = mbar_try_wait(bar_full((int)s1), ph1);
          umma_f16_ta(tmem_base, a_tmem + (uint32_t)(8 * k), bdesc + (uint64_t)(2 * k), idesc, (kb | (uint32_t)k) ? 1u : 0u);
        }
        umma_commit(bar_empty((int)s));   // the activation tile and the weight slice are free once these MMAs have read them
        if (!next_ready) ok = mbar_wait(bar_full((int)s1), ph1, p.status, 2u, abort_flag);
        s = s1; ph = ph1;
      }
      if (ok) umma_commit(bar_accum);
    }
  } else if (warp == 2) {
    // ================= TMA producer: packed weights =================
    if (lane == 0) {
      const uint32_t num_chunks = (num_kb + kTaWChunk - 1) / kTaWChunk;
      uint32_t issued = num_chunks < (uint32_t)kTaWStages ? num_chunks : (uint32_t)kTaWStages;
      for (uint32_t c = issued; c < num_chunks; ++c) {
        const int s = c % kTaWStages;
        const uint32_t ph = (c / kTaWStages) & 1u;
        if (!mbar_wait(bar_w_empty(s), ph ^ 1u, p.status, 6u, abort_flag)) break;
        mbar_arrive_expect_tx(bar_w_full(s), (uint32_t)L::kWBytes);
        tma_load_2d(w_ring + s * L::kWBytes, &tmap_w, bar_w_full(s), (int)(c * 32), (int)n0);
        issued = c + 1;
      }
      if (*abort_flag) {
        const uint32_t first = issued > (uint32_t)kTaWStages ? issued - kTaWStages : 0u;
        for (uint32_t c = first; c < issued; ++c) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar_w_full(c % kTaWStages), (c / kTaWStages) & 1u) &&
                 (unsigned long long)(clock64() - t0) < kWaitCycles) {}
        }
      }
    }
  } else {
    // ================= dequantisers (warps 3..18), then epilogue =================
    // Two teams of eight warps take the k blocks in turn (team = k block mod 2). Inside a team, thread
    // (quarter, lane) of half h owns weight row 32 quarter + lane and the 32-code half h of the block. A warp runs its
    // block as one dependent chain (wait, load, dequantise, store to tensor memory, wait for the store, arrive), about
    // twice as long as the tensor pipe needs for the block's MMAs: with one team the pipe idles half of the time, with
    // two the chains of consecutive blocks overlap.
    const int quarter = warp & 3;                       // TMEM lanes this warp may touch: [32 * quarter, +32)
    const uint32_t wpart = (uint32_t)(warp - 3) >> 2;   // 0..3
    const uint32_t part = wpart & 1u;                   // which half of the k block
    const uint32_t team = wpart >> 1;
    const uint32_t r_tile = (uint32_t)(quarter * 32 + lane);
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int gshift = (int)p.group_shift;
    const uint32_t row = min(n0 + r_tile, p.N - 1);
    const unsigned short* srow = reinterpret_cast<const unsigned short*>(p.S) + (size_t)row * p.SPR;
    const unsigned short* brow = reinterpret_cast<const unsigned short*>(p.B) + (size_t)row * p.SPR;
    bool ok = true;
    // group 64: eight groups per 16-byte load, fetched eight k blocks ahead; scalar loads otherwise
    const bool vec_sb = vec_sb_all;
    uint4 sv_cur = sv_pre0, bv_cur = bv_pre0, sv_nxt = sv_pre1, bv_nxt = bv_pre1;
    auto load_sb8 = [&](uint4& sv, uint4& bv, uint32_t kb8) {
      if (kb8 >= num_kb) return;
      sv = __ldg(reinterpret_cast<const uint4*>(srow + kb8));
      if (AFFINE) bv = __ldg(reinterpret_cast<const uint4*>(brow + kb8));
    };
    auto pick16 = [](const uint4& v, int i) -> unsigned short {
      const uint32_t wsel = (i >> 1) == 0 ? v.x : (i >> 1) == 1 ? v.y : (i >> 1) == 2 ? v.z : v.w;
      return (unsigned short)((i & 1) ? (wsel >> 16) : (wsel & 0xFFFFu));
    };

    const uint8_t* const wrow_sm = gen_base + L::kOffW + (r_tile >> 3) * 1024 + (r_tile & 7) * 128;
    constexpr int kUnroll = 8;
    auto run = [&](auto team_c) {
      constexpr int TEAM = decltype(team_c)::value;
      for (uint32_t kb0 = 0; kb0 < num_kb && ok; kb0 += kUnroll) {
#pragma unroll
        for (int i = TEAM; i < kUnroll; i += 2) {
          const uint32_t kb = kb0 + i;
          if (kb >= num_kb || !ok) break;
          const int s = (int)(kb % kTaStages);
          const uint32_t ph = (kb / kTaStages) & 1u;
          const uint32_t c = kb / kTaWChunk;
          const int ws = (int)(c % kTaWStages);
          const int j = i % kTaWChunk;
          if (j == TEAM) ok = mbar_wait(bar_w_full(ws), (c / kTaWStages) & 1u, p.status, 7u, abort_flag);
          uint4 wv = make_uint4(0, 0, 0, 0);
          if (ok) wv = *reinterpret_cast<const uint4*>(wrow_sm + ws * L::kWBytes + ((((uint32_t)j * 2 + part) ^ (r_tile & 7)) << 4));
          // the TMEM slice of stage s was last read by the MMAs of k block kb - kTaStages
          if (ok && kb >= (uint32_t)kTaStages) {
            ok = mbar_wait(bar_empty(s), ph ^ 1u, p.status, 4u, abort_flag);
            tc_fence_after();
          }
          if (ok) {
            unsigned short s16, b16 = 0;
            if (vec_sb) {
              s16 = pick16(sv_cur, i);
              if (AFFINE) b16 = pick16(bv_cur, i);
            } else {
              const uint32_t g = (kb * kGemmBK + part * 32) >> gshift;
              s16 = __ldg(srow + g);
              if (AFFINE) b16 = __ldg(brow + g);
            }
            const DqGroup dq = dq_group<AFFINE>(s16, b16);
            const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
            uint32_t a[16];
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
              const uint4 v = dequant_word_w16<AFFINE>(words[wi], dq);
              a[4 * wi] = v.x; a[4 * wi + 1] = v.y; a[4 * wi + 2] = v.z; a[4 * wi + 3] = v.w;
            }
            // 32 weights of this row = 16 TMEM columns (two k-adjacent f16 per column) of this thread's lane
            tmem_st16(tmem_base + lane_base + kColA + (uint32_t)s * 32u + part * 16u, a);
            tmem_st_wait();
          }
          // the packed slot goes back to the producer only after the stores that consumed its words; a warp signals
          // after its team's last k block of the slot
          if (j + 2 >= kTaWChunk || kb + 2 >= num_kb) {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_w_empty(ws));
          }
          tc_fence_before();
          mbar_arrive(bar_full(s));   // every thread arrives itself (also on abort)
        }
        if (vec_sb) {
          sv_cur = sv_nxt; bv_cur = bv_nxt;
          load_sb8(sv_nxt, bv_nxt, kb0 + 2 * kUnroll);
        }
      }
      // a last slot that holds one k block only has nothing for the second team: it still hands the slot back
      if (TEAM == 1 && (num_kb % kTaWChunk) == 1u) {
        const uint32_t c = (num_kb - 1u) / kTaWChunk;
        const int ws = (int)(c % kTaWStages);
        if (ok) ok = mbar_wait(bar_w_full(ws), (c / kTaWStages) & 1u, p.status, 7u, abort_flag);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_w_empty(ws));
      }
    };
    if (team == 0) run(std::integral_constant<int, 0>{}); else run(std::integral_constant<int, 1>{});
    // ---- epilogue: D[weight row][token] in TMEM -> y[token][weight row] ------------------------------------------
    const bool acc_ok = ok && mbar_wait(bar_accum, 0u, p.status, 5u, abort_flag);
    tc_fence_after();
    asm volatile("griddepcontrol.wait;" ::: "memory");   // y may still be read by the previous kernel in the stream
    // f16 rows of whole 16-byte pieces: the tile is turned round in the (now idle) activation ring. Phase 1: a thread
    // stores its weight row's 32 tokens of a block as f16 into stage[token][row] (a warp fills 64 consecutive bytes
    // per instruction). Phase 2: half a warp reads one token's 256 bytes and stores them to y in 16-byte pieces.
    // All sixteen warps reach the named barrier (also when a wait ran out: they then skip the memory work).
    static_assert(NT * kTaRows * 2 <= kTaStages * L::kXBytes, "the output stage lives in the activation ring");
    const bool staged = !p.out_f32 && (p.N % 8u) == 0;
    if (staged) {
      const uint32_t stage = x_ring;
      if (acc_ok) {
#pragma unroll 1
        for (int cb = (int)wpart; cb < NT / 32; cb += 4) {
          uint32_t v[32];
          tmem_ld32(tmem_base + lane_base + (uint32_t)(cb * 32), v);
          tmem_ld_wait();
          const uint32_t col = stage + (uint32_t)(cb * 32) * (kTaRows * 2u) + r_tile * 2u;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const unsigned short hv = __half_as_ushort(__float2half_rn(__uint_as_float(v[i])));
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(col + (uint32_t)i * (kTaRows * 2u)), "h"(hv) : "memory");
          }
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kTaDqWarps * 32) : "memory");
      if (acc_ok) {
        const uint32_t w16 = (uint32_t)(warp - 3);                 // 0..15
        const uint32_t sub = (uint32_t)lane >> 4, piece = (uint32_t)lane & 15u;
        const uint32_t n = n0 + piece * 8u;
        const uint4* const stage_g = reinterpret_cast<const uint4*>(gen_base);
#pragma unroll 4
        for (uint32_t t = w16 * 2u + sub; t < (uint32_t)NT; t += 2u * kTaDqWarps) {
          const uint32_t m = m0 + t;
          if (m < p.M && n < p.N)
            *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.Y) + (size_t)m * p.N + n) = stage_g[t * (kTaRows * 2u / 16u) + piece];
        }
      }
    } else if (acc_ok) {
      const uint32_t n = n0 + r_tile;
      // the four warps of a quarter take the 32-token blocks in turn
#pragma unroll 1
      for (int cb = (int)wpart; cb < NT / 32; cb += 4) {
        uint32_t v[32];
        tmem_ld32(tmem_base + lane_base + (uint32_t)(cb * 32), v);
        tmem_ld_wait();
        const uint32_t m_first = m0 + cb * 32;
        if (n < p.N) {
          if (p.out_f32) {
            float* dst = reinterpret_cast<float*>(p.Y) + (size_t)m_first * p.N + n;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (m_first + i < p.M) dst[(size_t)i * p.N] = __uint_as_float(v[i]);
          } else {
            __half* dst = reinterpret_cast<__half*>(p.Y) + (size_t)m_first * p.N + n;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (m_first + i < p.M) dst[(size_t)i * p.N] = __float2half_rn(__uint_as_float(v[i]));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ---- host side ---------------------------------------------------------------------------------------------
typedef CUresult (*TaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TaEncodeFn ta_encode_fn() {
  static TaEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TaEncodeFn>(ptr);
  }
  return fn;
}

template <int NT, bool AFFINE>
static cudaError_t launch_ta_one(const CUtensorMap& tx, const CUtensorMap& tw, const GemmTaParams& p, cudaStream_t st) {
  auto kern = gemm_w4_ta_kernel<NT, AFFINE>;
  constexpr int smem = GemmTaSmem<NT>::kTotal + 1024;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + kTaRows - 1) / kTaRows, (p.M + NT - 1) / NT);
  cfg.blockDim = dim3(kTaThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, tx, tw, p);
}

cudaError_t launch_gemm_w4_ta(const uint32_t* W, const __half* S, const __half* B, const __half* X, void* Y, uint32_t M,
                              uint32_t N, uint32_t K, uint32_t group_shift, bool out_f32, uint32_t* status, cudaStream_t st) {
  TaEncodeFn enc = ta_encode_fn();
  if (!enc) return cudaErrorNotSupported;
  const cuuint32_t estr[2] = {1, 1};
  CUtensorMap tx, tw;
  const cuuint64_t xdims[2] = {K, M};
  const cuuint64_t xstrides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t xbox[2] = {(cuuint32_t)kGemmBK, 128};
  CUresult r = enc(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(X), xdims, xstrides, xbox, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  const cuuint64_t wdims[2] = {K / 8, N};
  const cuuint64_t wstrides[1] = {(cuuint64_t)(K / 8) * 4};
  const cuuint32_t wbox[2] = {32, (cuuint32_t)kTaRows};
  r = enc(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(W), wdims, wstrides, wbox, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  GemmTaParams p;
  p.S = S; p.B = B; p.Y = Y;
  p.M = M; p.N = N; p.K = K; p.SPR = K >> group_shift; p.group_shift = group_shift;
  p.out_f32 = out_f32 ? 1u : 0u;
  p.status = status;
  const bool affine = B != nullptr;
  // 256 tokens per instruction unless that leaves most SMs without a tile (M = 256 on 8192 rows: 64 CTAs of 256 tokens
  // or 128 CTAs of 128)
  const uint64_t ctas256 = (uint64_t)((N + kTaRows - 1) / kTaRows) * ((M + 255) / 256);
  if (M > 128 && (M > 256 || ctas256 >= 111)) return affine ? launch_ta_one<256, true>(tx, tw, p, st) : launch_ta_one<256, false>(tx, tw, p, st);
  return affine ? launch_ta_one<128, true>(tx, tw, p, st) : launch_ta_one<128, false>(tx, tw, p, st);
}

}  // namespace ztvm
