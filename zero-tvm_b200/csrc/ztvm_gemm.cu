// Prefill GEMM for 4-bit group-quantised weights on the 5th-generation tensor cores, both operands in shared memory.
// Serves 8 < M <= 128 (64-row weight tiles give twice as many CTAs as ztvm_gemm_ta.cu's 128-row tiles) and, with
// ZTVM_GEMM=sm, every M for comparison.
//
//   y[m, n] = sum_k x[m, k] * W16[n, k],   W16 = f16_rne(fl32(s * q + b))   (or s * (q - 7))
//
// W16 is the value the reference's numpy dequantiser produces (scripts/make-dsv2-layer-ref.py:108-116)
// and what its matrix-unit GEMMs feed their f16 fragments (int4_matmul.gen.ts:1173-1178); accumulation is
// f32 in tensor memory. kind::f16 takes the f16 activations unchanged, so x is never rounded.
//
// One CTA computes a (MB x 128 tokens) x (BN weight rows) tile:
//   warp 0      TMA producer for activations: tiles x[128 x 64] (128-byte swizzle) into a ring of STAGES slots
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) per 16-wide k step and
//               per 128-token block, accumulators live in TMEM; tcgen05.commit releases the ring slot
//   warp 2      TMA producer for packed weights: tiles W[BN rows x 32 words] (= 256 codes, four k blocks, whole
//               128-byte lines per row) into a ring of its own, so the code stream runs far ahead of its use
//   warps 3..10 dequantisers, as two groups of four warps on alternate k blocks: per 64-wide k block a thread reads
//               its row's codes from shared memory and the group's scale/bias, builds the f16 weights with the SAME
//               device function the parity hook uses, and writes them in the tensor core's K-major 128B-swizzled layout.
//               After the main loop the same eight warps drain TMEM (tcgen05.ld) and store y.
// Every mbarrier wait is bounded (about a second); a wait that runs out raises a status word, the roles
// stop, in-flight copies are waited for (bounded), TMEM is freed and the kernel returns.
#include "ztvm_kernels.h"
#include "ztvm_tc.cuh"

namespace ztvm {

constexpr int kGemmStages = 4;       // activation / dequantised-weight ring
constexpr int kGemmWStages = 2;      // packed-weight ring (each slot holds four k blocks)
constexpr int kGemmWChunk = 4;       // k blocks per packed-weight slot: 32 words = 128 bytes per row
constexpr int kGemmDqWarps = 8;      // dequantiser warps (two per SM sub-partition)
constexpr int kGemmThreads = 96 + kGemmDqWarps * 32;   // two TMA warps + MMA warp + dequantisers
struct GemmParams {
  const uint32_t* W;
  const __half* S;
  const __half* B;   // nullptr: symmetric
  void* Y;
  uint32_t M, N, K, KP, SPR, group_shift, out_f32;
  uint32_t* status;  // [1]: timeout code
  uint32_t tma_store;  // 1: f16 output through shared memory + TMA store (needs N % 8 == 0)
  uint32_t x_tx_bytes; // bytes one activation stage receives: the TMA box holds min(128, M rounded up to 8) rows per 128-token block
};

// Dynamic shared memory carve-up (1024-byte aligned): A ring | B ring | barriers | tmem slot | abort flag
template <int MB, int BN>
struct GemmSmem {
  static constexpr int kABytes = MB * 128 * kGemmBK * 2;  // per stage
  static constexpr int kBBytes = BN * kGemmBK * 2;
  static constexpr int kOffB = kGemmStages * kABytes;
  static constexpr int kWBytes = BN * 128;                 // per packed-weight slot
  static constexpr int kOffW = kOffB + kGemmStages * kBBytes;
  static constexpr int kOffBar = kOffW + kGemmWStages * kWBytes;
  static constexpr int kTotal = kOffBar + 256;
};

template <int MB, int BN, bool AFFINE>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_w4_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
               const __grid_constant__ CUtensorMap tmap_y, const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using L = GemmSmem<MB, BN>;
  // align the dynamic region to 1024 bytes (swizzle atoms and UMMA descriptors assume it)
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t a_ring = base, b_ring = base + L::kOffB, w_ring = base + L::kOffW, bars = base + L::kOffBar;
  // barrier layout: full[S] (activation bytes + one arrival per dequantiser warp), empty[S], w_full[WS],
  // w_empty[WS], accum, then tmem slot and abort flag
  auto bar_full = [&](int s) { return bars + 8u * s; };
  auto bar_empty = [&](int s) { return bars + 8u * (kGemmStages + s); };
  auto bar_w_full = [&](int s) { return bars + 8u * (2 * kGemmStages + s); };
  auto bar_w_empty = [&](int s) { return bars + 8u * (2 * kGemmStages + kGemmWStages + s); };
  constexpr int kNumBars = 2 * kGemmStages + 2 * kGemmWStages + 1;
  const uint32_t bar_accum = bars + 8u * (kNumBars - 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + L::kOffBar + 8 * kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t n0 = blockIdx.x * BN;
  const uint32_t m0 = blockIdx.y * (MB * 128);
  const uint32_t num_kb = p.K / kGemmBK;
  constexpr uint32_t kTmemCols = (MB * BN) <= 32 ? 32 : (MB * BN) <= 64 ? 64 : (MB * BN) <= 128 ? 128 : (MB * BN) <= 256 ? 256 : 512;

  if (threadIdx.x == 32) { tma_prefetch_desc(&tmap_x); tma_prefetch_desc(&tmap_w); tma_prefetch_desc(&tmap_y); }
  // Each TMA producer initialises the barriers its own copies signal and starts its first loads right away: they
  // fly while the other warps allocate tensor memory and meet at the block barrier below. Everyone else touches
  // those barriers only after that barrier.
  if (threadIdx.x == 0) {
    for (int s = 0; s < kGemmStages; ++s) {
      mbar_init(bar_full(s), 1 + kGemmDqWarps * 32 / 2);   // the TMA producer's arrival (with the byte count) + every thread of one dequantiser group
      mbar_init(bar_empty(s), 1);
    }
    mbar_init(bar_accum, 1);
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // Programmatic dependent launch: nothing before this point (nor the weight / scale loads of the other warps)
    // touches what the previous kernel in the stream may write; the activations may be its output.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (uint32_t kb = 0; kb < (uint32_t)kGemmStages && kb < num_kb; ++kb) {
      mbar_arrive_expect_tx(bar_full((int)kb), p.x_tx_bytes);
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
        tma_load_2d(a_ring + kb * L::kABytes + mb * (128 * kGemmBK * 2), &tmap_x, bar_full((int)kb), (int)(kb * kGemmBK),
                    (int)(m0 + mb * 128));
    }
  }
  if (threadIdx.x == 64) {
    for (int s = 0; s < kGemmWStages; ++s) {
      mbar_init(bar_w_full(s), 1);
      mbar_init(bar_w_empty(s), kGemmDqWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const uint32_t num_chunks0 = (num_kb + kGemmWChunk - 1) / kGemmWChunk;
    for (uint32_t c = 0; c < (uint32_t)kGemmWStages && c < num_chunks0; ++c) {
      mbar_arrive_expect_tx(bar_w_full((int)c), (uint32_t)L::kWBytes);
      tma_load_2d(w_ring + c * L::kWBytes, &tmap_w, bar_w_full((int)c), (int)(c * 32), (int)n0);
    }
  }
  if (warp == 1) {  // the MMA warp owns the TMEM allocation
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      uint32_t issued = num_kb < (uint32_t)kGemmStages ? num_kb : (uint32_t)kGemmStages;   // the first stages went out before the block barrier
      for (uint32_t kb = issued; kb < num_kb; ++kb) {
        const int s = kb % kGemmStages;
        const uint32_t ph = (kb / kGemmStages) & 1u;
        if (kb >= kGemmStages && !mbar_wait(bar_empty(s), ph ^ 1u, p.status, 1u, abort_flag)) break;
        mbar_arrive_expect_tx(bar_full(s), p.x_tx_bytes);
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
          tma_load_2d(a_ring + s * L::kABytes + mb * (128 * kGemmBK * 2), &tmap_x, bar_full(s), (int)(kb * kGemmBK),
                      (int)(m0 + mb * 128));
        issued = kb + 1;
      }
      // if the consumer stopped, wait (bounded) until the copies already issued have landed
      if (*abort_flag) {
        const uint32_t first = issued > (uint32_t)kGemmStages ? issued - kGemmStages : 0u;
        for (uint32_t kb = first; kb < issued; ++kb) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar_full(kb % kGemmStages), (kb / kGemmStages) & 1u) &&
                 (unsigned long long)(clock64() - t0) < kWaitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_f16(BN);
      const uint64_t a0 = smem_desc_sw128(a_ring), b0 = smem_desc_sw128(b_ring);
      uint32_t s = 0, ph = 0;
      bool ok = true, ready = false;   // ready: the current stage's barrier was already seen complete by an early poll
      for (uint32_t kb = 0; kb < num_kb; ++kb) {
        if (!ready) ok = mbar_wait(bar_full(s), ph, p.status, 2u, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint64_t bdesc = b0 + (uint64_t)(s * (L::kBBytes >> 4));
        const uint32_t ns = s + 1 == (uint32_t)kGemmStages ? 0u : s + 1;
        const uint32_t nph = ns == 0 ? ph ^ 1u : ph;
        bool ready_next = false;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const uint64_t adesc = a0 + (uint64_t)(s * (L::kABytes >> 4) + mb * ((128 * kGemmBK * 2) >> 4));
#pragma unroll
          for (int k = 0; k < kGemmBK / 16; ++k) {
            // advance both descriptors by 16 elements = 32 bytes inside the swizzle row: +2 in the (>>4) address field
            umma_f16(tmem_base + (uint32_t)(mb * BN), adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc,
                     (kb | (uint32_t)k) ? 1u : 0u);
            // the tensor pipe is busy with what was just queued: poll the next stage's barrier in its shadow
            if (mb == MB - 1 && k == kGemmBK / 16 - 2 && kb + 1 < num_kb) ready_next = mbar_try_wait(bar_full(ns), nph);
          }
        }
        umma_commit(bar_empty(s));   // the slot is free once these MMAs have read it
        s = ns; ph = nph; ready = ready_next;
      }
      if (ok) umma_commit(bar_accum);  // all accumulators final
    }
  } else if (warp == 2) {
    // ================= TMA producer: packed weights =================
    if (lane == 0) {
      const uint32_t num_chunks = (num_kb + kGemmWChunk - 1) / kGemmWChunk;
      uint32_t issued = num_chunks < (uint32_t)kGemmWStages ? num_chunks : (uint32_t)kGemmWStages;   // sent before the block barrier
      for (uint32_t c = issued; c < num_chunks; ++c) {
        const int s = c % kGemmWStages;
        const uint32_t ph = (c / kGemmWStages) & 1u;
        if (c >= kGemmWStages && !mbar_wait(bar_w_empty(s), ph ^ 1u, p.status, 6u, abort_flag)) break;
        mbar_arrive_expect_tx(bar_w_full(s), (uint32_t)L::kWBytes);
        tma_load_2d(w_ring + s * L::kWBytes, &tmap_w, bar_w_full(s), (int)(c * 32), (int)n0);
        issued = c + 1;
      }
      if (*abort_flag) {
        const uint32_t first = issued > (uint32_t)kGemmWStages ? issued - kGemmWStages : 0u;
        for (uint32_t c = first; c < issued; ++c) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar_w_full(c % kGemmWStages), (c / kGemmWStages) & 1u) &&
                 (unsigned long long)(clock64() - t0) < kWaitCycles) {}
        }
      }
    }
  } else {
    // ================= dequantisers (warps 3..10), then epilogue =================
    // The dequantisers work as two groups of four warps that take alternate k blocks. One k block is a chain of waits,
    // shared loads, conversions and stores whose latency, not its instruction count, set the pace when every thread
    // worked on every k block; two groups keep two k blocks in flight.
    const int t = threadIdx.x - 96;                  // 0..255
    constexpr int kDqGroups = 2;
    constexpr int GT = kGemmDqWarps * 32 / kDqGroups;   // threads per group
    constexpr int TPR = GT / BN;                     // threads per weight row (BN = 128 -> 1, 64 -> 2)
    constexpr int WPT = (kGemmBK / 8) / TPR;         // 8-code words per thread per k block (8, 4)
    static_assert(TPR >= 1 && WPT >= 2 && TPR * WPT == 8, "unsupported BN");
    const int grp = t / GT, tg = t % GT;
    const int gshift = (int)p.group_shift;
    const uint32_t r_tile = (uint32_t)(tg / TPR);    // weight row within the tile
    const uint32_t part = (uint32_t)(tg % TPR);      // which run of WPT words of the 8-word k block
    const uint32_t row = min(n0 + r_tile, p.N - 1);
    const unsigned short* srow = reinterpret_cast<const unsigned short*>(p.S) + (size_t)row * p.SPR;
    const unsigned short* brow = reinterpret_cast<const unsigned short*>(p.B) + (size_t)row * p.SPR;
    bool ok = true;
    // Scales and biases: eight groups per 16-byte load (group 64 = one group per k block) when the row's group
    // count keeps the loads aligned, fetched eight k blocks ahead; scalar loads otherwise.
    const bool vec_sb = gshift == 6 && (p.SPR % 8u) == 0 && ((reinterpret_cast<uintptr_t>(p.S) | reinterpret_cast<uintptr_t>(p.B)) & 15u) == 0;
    uint4 sv_cur = make_uint4(0, 0, 0, 0), bv_cur = sv_cur, sv_nxt = sv_cur, bv_nxt = sv_cur;
    auto load_sb8 = [&](uint4& sv, uint4& bv, uint32_t kb8) {   // groups kb8 .. kb8+7
      if (kb8 >= num_kb) return;
      sv = __ldg(reinterpret_cast<const uint4*>(srow + kb8));
      if (AFFINE) bv = __ldg(reinterpret_cast<const uint4*>(brow + kb8));
    };
    auto pick16 = [](const uint4& v, int i) -> unsigned short {   // i is a compile-time constant after unrolling
      const uint32_t wsel = (i >> 1) == 0 ? v.x : (i >> 1) == 1 ? v.y : (i >> 1) == 2 ? v.z : v.w;
      return (unsigned short)((i & 1) ? (wsel >> 16) : (wsel & 0xFFFFu));
    };
    if (vec_sb) { load_sb8(sv_cur, bv_cur, 0); load_sb8(sv_nxt, bv_nxt, 8); }

    // this thread's row inside a swizzled tile (dequantised ring and packed ring share the row geometry)
    const uint32_t row_off = (r_tile >> 3) * 1024 + (r_tile & 7) * 128;
    uint8_t* const brow_sm = gen_base + L::kOffB + row_off;
    const uint8_t* const wrow_sm = gen_base + L::kOffW + row_off;
    constexpr int kUnroll = 8;   // = groups per scale vector; a multiple of kGemmWChunk
    for (uint32_t kb0 = 0; kb0 < num_kb && ok; kb0 += kUnroll) {
#pragma unroll
      for (int i = 0; i < kUnroll; ++i) {
        const uint32_t kb = kb0 + i;
        if (kb >= num_kb || !ok) break;
        if ((i & 1) != grp) continue;                     // the other group's k block
        const int s = (int)(kb % kGemmStages);
        const uint32_t ph = (kb / kGemmStages) & 1u;
        const uint32_t c = kb / kGemmWChunk;              // packed-weight chunk and slot
        const int ws = (int)(c % kGemmWStages);
        constexpr int kJ = kGemmWChunk;
        const int j = i % kJ;                             // k block inside the chunk (kb0 is a multiple of 8)
        if (j == grp) ok = mbar_wait(bar_w_full(ws), (c / kGemmWStages) & 1u, p.status, 7u, abort_flag);   // this group's first k block of the chunk
        // codes of this k block: words [j*8 + part*WPT, +WPT) of the row's 32-word line
        uint32_t wv[WPT];
        if (ok) {
          const uint8_t* wl = wrow_sm + ws * L::kWBytes;
#pragma unroll
          for (int q4 = 0; q4 < (WPT + 3) / 4; ++q4) {
            const uint32_t word0 = (uint32_t)j * 8 + part * WPT + q4 * 4;
            const uint32_t chunk16 = word0 >> 2;
            const uint8_t* src = wl + ((chunk16 ^ (r_tile & 7)) << 4) + (word0 & 3) * 4;
            if constexpr (WPT == 2) {
              const uint2 v = *reinterpret_cast<const uint2*>(src);
              wv[0] = v.x; wv[1] = v.y;
            } else {
              const uint4 v = *reinterpret_cast<const uint4*>(src);
              wv[4 * q4] = v.x; wv[4 * q4 + 1] = v.y; wv[4 * q4 + 2] = v.z; wv[4 * q4 + 3] = v.w;
            }
          }
        }
        if (ok && kb >= (uint32_t)kGemmStages) ok = mbar_wait(bar_empty(s), ph ^ 1u, p.status, 4u, abort_flag);
        if (ok) {
          uint8_t* rowp = brow_sm + s * L::kBBytes;
          unsigned short s16, b16 = 0;
          if (vec_sb) {
            s16 = pick16(sv_cur, i);
            if (AFFINE) b16 = pick16(bv_cur, i);
          } else {
            const uint32_t g = (kb * kGemmBK + part * WPT * 8) >> gshift;
            s16 = __ldg(srow + g);
            if (AFFINE) b16 = __ldg(brow + g);
          }
          DqGroup dq = dq_group<AFFINE>(s16, b16);
#pragma unroll
          for (int wi = 0; wi < WPT; ++wi) {
            if (WPT == 8 && wi == 4 && gshift == 5) {   // group 32: the second half of the block is the next group
              const uint32_t g = (kb * kGemmBK + 32) >> gshift;
              dq = dq_group<AFFINE>(__ldg(srow + g), AFFINE ? __ldg(brow + g) : (unsigned short)0);
            }
            const uint4 v = dequant_word_w16<AFFINE>(wv[wi], dq);
            const uint32_t chunk = part * WPT + wi;                      // 16-byte chunk of the 128-byte row
            *reinterpret_cast<uint4*>(rowp + ((chunk ^ (r_tile & 7)) << 4)) = v;
          }
          fence_proxy_async();   // make the generic-proxy stores visible to the tensor core's async proxy
        }
        // Last read of the packed slot: it goes back to the producer only after the stores that consume its words.
        // (A release straight after the loads let the refill land before the loads had been performed.)
        if (j + kDqGroups >= kJ || kb + kDqGroups >= num_kb) {   // this group's last k block of the chunk
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_w_empty(ws));
        }
        mbar_arrive(bar_full(s));   // every thread arrives itself, right after its own proxy fence (also on abort)
      }
      if (vec_sb) {
        sv_cur = sv_nxt; bv_cur = bv_nxt;
        load_sb8(sv_nxt, bv_nxt, kb0 + 2 * kUnroll);
      }
    }
    // ---- epilogue: TMEM -> registers -> y ---------------------------------------------------------
    const bool acc_ok = ok && mbar_wait(bar_accum, 0u, p.status, 5u, abort_flag);
    tc_fence_after();
    asm volatile("griddepcontrol.wait;" ::: "memory");   // y may still be read by the previous kernel in the stream
    if (acc_ok && p.tma_store) {
      // f16 output: registers -> shared memory in the 128-byte swizzle (two 64-column halves per 128-token block,
      // in the activation ring, which is idle once the accumulators are final) -> one TMA store per half.
      // The store clips rows past M and columns past N by itself.
      const int quarter = warp & 3;                      // TMEM lanes this warp may read: [32*quarter, +32)
      const int half = (warp - 3) >> 2;                  // two warps share a quarter: even / odd column blocks
      const uint32_t r = (uint32_t)(quarter * 32 + lane);   // row (token) inside the 128-token block
#pragma unroll 1
      for (int mb = 0; mb < MB; ++mb) {
#pragma unroll 1
        for (int cb = half; cb < BN / 32; cb += 2) {
          uint32_t v[32];
          tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mb * BN + cb * 32), v);
          tmem_ld_wait();
          uint8_t* tile = gen_base + (mb * (BN / 64) + (cb >> 1)) * (128 * 128) + (r >> 3) * 1024 + (r & 7) * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o;
            __half2 h;
            h = __floats2half2_rn(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1])); o.x = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3])); o.y = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5])); o.z = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7])); o.w = *reinterpret_cast<uint32_t*>(&h);
            const uint32_t chunk = (uint32_t)((cb & 1) * 4 + i);
            *reinterpret_cast<uint4*>(tile + ((chunk ^ (r & 7)) << 4)) = o;
          }
        }
      }
      fence_proxy_async();
      asm volatile("bar.sync 1, %0;" ::"n"(kGemmDqWarps * 32) : "memory");   // the eight epilogue warps only
      if (threadIdx.x == 96) {
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
          for (int hh = 0; hh < BN / 64; ++hh)
            tma_store_2d(&tmap_y, base + (uint32_t)((mb * (BN / 64) + hh) * (128 * 128)), (int)(n0 + hh * 64), (int)(m0 + mb * 128));
        tma_store_commit_and_wait();
      }
    } else if (acc_ok) {
      const int quarter = warp & 3;                      // TMEM lanes this warp may read: [32*quarter, +32)
      const int half = (warp - 3) >> 2;                  // two warps share a quarter: even / odd column blocks
#pragma unroll 1
      for (int mb = 0; mb < MB; ++mb) {
        const uint32_t m = m0 + mb * 128 + quarter * 32 + lane;
#pragma unroll 1
        for (int cb = half; cb < BN / 32; cb += 2) {
          uint32_t v[32];
          tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mb * BN + cb * 32), v);
          tmem_ld_wait();
          const uint32_t n = n0 + cb * 32;
          if (m < p.M && n < p.N) {
            if (p.out_f32) {
              float* dst = reinterpret_cast<float*>(p.Y) + (size_t)m * p.N + n;
              if (n + 32 <= p.N && (p.N & 3u) == 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  reinterpret_cast<float4*>(dst)[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                                  __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
              } else {
                for (int i = 0; i < 32 && n + i < p.N; ++i) dst[i] = __uint_as_float(v[i]);
              }
            } else {
              __half* dst = reinterpret_cast<__half*>(p.Y) + (size_t)m * p.N + n;
              if (n + 32 <= p.N && (p.N & 7u) == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  uint4 o;
                  __half2 h;
                  h = __floats2half2_rn(__uint_as_float(v[8 * i]), __uint_as_float(v[8 * i + 1])); o.x = *reinterpret_cast<uint32_t*>(&h);
                  h = __floats2half2_rn(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3])); o.y = *reinterpret_cast<uint32_t*>(&h);
                  h = __floats2half2_rn(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5])); o.z = *reinterpret_cast<uint32_t*>(&h);
                  h = __floats2half2_rn(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7])); o.w = *reinterpret_cast<uint32_t*>(&h);
                  reinterpret_cast<uint4*>(dst)[i] = o;
                }
              } else {
                for (int i = 0; i < 32 && n + i < p.N; ++i) dst[i] = __float2half_rn(__uint_as_float(v[i]));
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ---- host side --------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
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

template <int MB, int BN, bool AFFINE>
static cudaError_t launch_gemm_one(const CUtensorMap& tmap, const CUtensorMap& tmap_w, const CUtensorMap& tmap_y, const GemmParams& p, cudaStream_t st) {
  auto kern = gemm_w4_kernel<MB, BN, AFFINE>;
  constexpr int smem = GemmSmem<MB, BN>::kTotal + 1024;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((p.N + BN - 1) / BN, (p.M + MB * 128 - 1) / (MB * 128));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, tmap, tmap_w, tmap_y, p);
}

bool gemm_w4_supported(int bits, uint32_t group, uint32_t K) {
  return bits == 4 && (group == 32 || group == 64 || group == 128) && K % kGemmBK == 0;
}

cudaError_t launch_gemm_w4(const uint32_t* W, const __half* S, const __half* B, const __half* X, void* Y, uint32_t M,
                           uint32_t N, uint32_t K, uint32_t group_shift, bool out_f32, uint32_t* status, cudaStream_t st) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return cudaErrorNotSupported;
  CUtensorMap tmap;
  const cuuint64_t dims[2] = {K, M};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  // A box much taller than the tensor (M < 32 under a 128-row box) made every activation load and output store slow
  // (22 us against 13 us per launch on 8192 x 2048): the boxes hold only the rows there are. Rows of the stage that no
  // copy fills feed accumulator rows that are never stored.
  const uint32_t box_rows = M >= 128 ? 128u : (M + 7u) & ~7u;
  const cuuint32_t box[2] = {(cuuint32_t)kGemmBK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(X), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  // packed weights: u32 [N][K/8], box = 32 words (four k blocks, one 128-byte line) x BN rows
  const uint32_t bn = M > 128 ? 128u : 64u;
  CUtensorMap tmap_w;
  const cuuint64_t wdims[2] = {K / 8, N};
  const cuuint64_t wstrides[1] = {(cuuint64_t)(K / 8) * 4};
  const cuuint32_t wbox[2] = {32, bn};
  r = enc(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(W), wdims, wstrides, wbox, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  // f16 output [M][N]: box = 64 columns (one 128-byte swizzle row) x 128 rows
  CUtensorMap tmap_y = tmap_w;
  const bool tma_store = !out_f32 && (N % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15u) == 0);
  if (tma_store) {
    const cuuint64_t ydims[2] = {N, M};
    const cuuint64_t ystrides[1] = {(cuuint64_t)N * 2};
    const cuuint32_t ybox[2] = {64, box_rows};
    r = enc(&tmap_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, Y, ydims, ystrides, ybox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  }
  GemmParams p;
  p.tma_store = tma_store ? 1u : 0u;
  p.x_tx_bytes = (M > 128 ? 2u : 1u) * box_rows * (uint32_t)(kGemmBK * 2);
  p.W = W; p.S = S; p.B = B; p.Y = Y;
  p.M = M; p.N = N; p.K = K; p.KP = K / 8; p.SPR = K >> group_shift; p.group_shift = group_shift;
  p.out_f32 = out_f32 ? 1u : 0u;
  p.status = status;
  const bool affine = B != nullptr;
  if (M > 128) {
    return affine ? launch_gemm_one<2, 128, true>(tmap, tmap_w, tmap_y, p, st) : launch_gemm_one<2, 128, false>(tmap, tmap_w, tmap_y, p, st);
  }
  return affine ? launch_gemm_one<1, 64, true>(tmap, tmap_w, tmap_y, p, st) : launch_gemm_one<1, 64, false>(tmap, tmap_w, tmap_y, p, st);
}

}  // namespace ztvm
