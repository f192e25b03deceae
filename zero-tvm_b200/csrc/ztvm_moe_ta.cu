// Grouped MoE expert matmul on tcgen05 with the DEQUANTISED EXPERT WEIGHTS AS THE A OPERAND IN TENSOR MEMORY:
//   y[token, slot, :] = x[token, slot, :] * W16[ids[token, slot]]^T        (int4_matmul.gen.ts:229-254)
// for launches where an expert sees many pairs. The pairs of one expert (sorted by the plan, ztvm_moe_plan.cuh) take
// the N side of the MMA, up to 128 per tile, so an expert's weights are dequantised ONCE per 128 pairs and per 128
// output rows, and go from the dequantisers' registers straight into tensor memory (tcgen05.st) instead of through
// shared memory. The activation rows of the tile's pairs are the only shared-memory operand: gathered with 16-byte
// cp.async into the 128-byte-swizzled K-major layout.
//
// Persistent: one CTA per SM walks the units (tile of pairs, 128 weight rows) u = blockIdx.x, + gridDim.x, ...; two
// accumulator sets in tensor memory let the epilogue of unit i run under the main loop of unit i + 1, and every
// pipeline (packed weights, activations, weight slices) keeps running across unit boundaries.
//
// Roles (576 threads): warp 0 TMA-loads packed weights (128 rows x 32 words = four k blocks per slot); warp 1 owns
// tensor memory and issues the MMAs; warps 2..9 dequantise (warp w touches TMEM lanes 32 (w % 4) .. +31 = its 32
// weight rows; the two warps of a lane quarter split a k block in halves); warps 10..13 gather activations (one pair
// row per thread); warps 14..17 read finished accumulators and scatter them to where each pair lives. Every wait is
// bounded: on expiry a status word is raised, the roles stop, copies in flight are waited for, TMEM is freed.
#include <mutex>

#include "ztvm_kernels.h"
#include "ztvm_moe_plan.cuh"
#include "ztvm_tc.cuh"

namespace ztvm {

#ifdef ZTVM_MTA_PROF
__device__ unsigned long long g_mta_prof[64];
#define PROF_DECL(n) long long prof_acc[n] = {}; long long prof_t = 0; (void)prof_t
#define PROF_T0() prof_t = clock64()
#define PROF_ADD(i) do { const long long t_ = clock64(); prof_acc[i] += t_ - prof_t; prof_t = t_; } while (0)
#define PROF_OUT(base, n, cond) do { if (blockIdx.x == 0 && (cond)) for (int i_ = 0; i_ < n; ++i_) g_mta_prof[base + i_] = (unsigned long long)prof_acc[i_]; } while (0)
#else
#define PROF_DECL(n)
#define PROF_T0()
#define PROF_ADD(i)
#define PROF_OUT(base, n, cond)
#endif

constexpr int kMtaBK = 128;          // k elements per pipeline stage = two 64-element swizzle atoms = two scale groups
constexpr int kMtaStages = 4;        // stages: activation tiles in shared memory, weight slices in tensor memory
constexpr int kMtaWStages = 4;       // packed-weight ring; a slot holds 256 codes per row = two stages
constexpr int kMtaWPerSlot = 2;      // stages per packed-weight slot
constexpr int kMtaNP = 128;          // pairs per tile = widest MMA N used
constexpr int kMtaRows = 128;        // weight rows per unit = TMEM lanes
#ifndef ZTVM_MTA_DQWARPS
#define ZTVM_MTA_DQWARPS 16
#endif
constexpr int kMtaDqWarps = ZTVM_MTA_DQWARPS, kMtaGaWarps = 4, kMtaEpWarps = 4;
constexpr int kMtaParts = kMtaDqWarps / 4;          // dequantiser warps per lane quarter: each takes 128 / parts codes of a stage
constexpr int kMtaWpt = 16 / kMtaParts;             // packed words per thread and stage
static_assert(kMtaParts == 2 || kMtaParts == 4, "two or four dequantiser warps per lane quarter");
constexpr int kMtaThreads = 64 + (kMtaDqWarps + kMtaGaWarps + kMtaEpWarps) * 32;
constexpr int kMtaLead = kMtaStages - 2;   // activation rows are fetched this many stages ahead
constexpr uint32_t kMtaColA = 2 * kMtaNP;  // TMEM: two accumulator sets, then the weight slices (64 columns each)
constexpr uint32_t kMtaSliceCols = kMtaBK / 2;
constexpr uint32_t kMtaTmemCols = 512;
constexpr int kMtaUnitTable = 256;   // units of a CTA kept in shared memory (further ones are read from the plan directly)
static_assert(kMtaColA + kMtaStages * kMtaSliceCols <= kMtaTmemCols, "tensor memory columns");

struct MoeTaParams {
  const __half* S;
  const __half* B;
  const __half* X;
  __half* Y;
  uint32_t N, K, SPR, slots, NB;
  uint32_t in_slot_stride, out_slot_stride, in_tok_stride, out_tok_stride;
  MoeScratch sc;
  uint32_t* status;
  // expert-parallel form: the output row of pair i lives at y_seg[i / seg_cap] + dst_index[i] * out_tok_stride
  const uint32_t* dst_index;
  uint32_t seg_cap;
  __half* y_seg[9];
};

struct MtaSmem {
  static constexpr int kXHalf = kMtaNP * 128;                    // one swizzle atom column: 128 rows x 64 k
  static constexpr int kXBytes = 2 * kXHalf;                     // per stage
  static constexpr int kWBytes = kMtaRows * 128;                 // per packed-weight slot
  static constexpr int kOffW = kMtaStages * kXBytes;
  static constexpr int kOffBar = kOffW + kMtaWStages * kWBytes;
  static constexpr int kOffUnits = kOffBar + 256;                // this CTA's first kMtaUnitTable units: expert, r0, rows, n0
  static constexpr int kTotal = kOffUnits + kMtaUnitTable * 16;
};

// N consecutive 32-bit columns of this thread's TMEM lane from registers (N = 16 or 32).
template <int N>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t* v) {
  static_assert(N == 32 || N == 16, "16 or 32 columns");
  if constexpr (N == 32) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[N - 16]), "r"(v[N - 15]),
          "r"(v[N - 14]), "r"(v[N - 13]), "r"(v[N - 12]), "r"(v[N - 11]), "r"(v[N - 10]), "r"(v[N - 9]), "r"(v[N - 8]),
          "r"(v[N - 7]), "r"(v[N - 6]), "r"(v[N - 5]), "r"(v[N - 4]), "r"(v[N - 3]), "r"(v[N - 2]), "r"(v[N - 1])
        : "memory");
  } else {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
  }
}

__global__ void __launch_bounds__(kMtaThreads, 1)
moe_ta_kernel(const __grid_constant__ CUtensorMap tmap_w, const MoeTaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using L = MtaSmem;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t x_ring = base, w_ring = base + L::kOffW, bars = base + L::kOffBar;
  // full: dequantiser warps (weight slice in tensor memory) + gather warps (activation tile) -> MMA; empty: MMA -> both
  auto bar_full = [&](uint32_t s) { return bars + 8u * s; };
  auto bar_empty = [&](uint32_t s) { return bars + 8u * (kMtaStages + s); };
  auto bar_w_full = [&](uint32_t s) { return bars + 8u * (2 * kMtaStages + s); };
  auto bar_w_empty = [&](uint32_t s) { return bars + 8u * (2 * kMtaStages + kMtaWStages + s); };
  auto bar_acc_full = [&](uint32_t s) { return bars + 8u * (2 * kMtaStages + 2 * kMtaWStages + s); };
  auto bar_acc_empty = [&](uint32_t s) { return bars + 8u * (2 * kMtaStages + 2 * kMtaWStages + 2 + s); };
  constexpr int kNumBars = 2 * kMtaStages + 2 * kMtaWStages + 4;
  static_assert(8 * kNumBars + 8 <= 256, "barrier block");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + L::kOffBar + 8 * kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t num_kb = p.K / kGemmBK;                       // 64-element k blocks (= scale groups)
  const uint32_t num_st = (num_kb + 1) / 2;                    // stages of 128 (the last may hold one k block only)
  const uint32_t num_chunks = (num_st + kMtaWPerSlot - 1) / kMtaWPerSlot;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMtaStages; ++s) {
      mbar_init(bar_full(s), kMtaDqWarps + kMtaGaWarps);   // one arrival per producing warp
      mbar_init(bar_empty(s), 1);
    }
    for (int s = 0; s < kMtaWStages; ++s) {
      mbar_init(bar_w_full(s), 1);
      mbar_init(bar_w_empty(s), kMtaDqWarps);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_acc_full(s), 1);
      mbar_init(bar_acc_empty(s), kMtaEpWarps);
    }
    *abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x == 32) tma_prefetch_desc(&tmap_w);
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kMtaTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // The plan (tile table, sorted pair list) and the activations are written by kernels earlier in the stream.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // Units of this CTA: blockIdx.x, + gridDim.x, ... Their descriptors are copied from the plan into shared memory once
  // (a role that had to chase tile table -> pair list in global memory at every unit start stalled the whole pipeline
  // for microseconds per unit).
  const uint32_t total_units = *p.sc.ntiles * p.NB;
  const uint32_t my_units = total_units > blockIdx.x ? (total_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
  uint4* unit_tab = reinterpret_cast<uint4*>(gen_base + L::kOffUnits);
  auto unit_global = [&](uint32_t ui) {
    const uint32_t u = blockIdx.x + ui * gridDim.x;
    const uint32_t tile = u / p.NB;
    return make_uint4(p.sc.tiles[(size_t)tile * 3], p.sc.tiles[(size_t)tile * 3 + 1], p.sc.tiles[(size_t)tile * 3 + 2],
                      (u - tile * p.NB) * kMtaRows);
  };
  for (uint32_t ui = threadIdx.x; ui < my_units && ui < (uint32_t)kMtaUnitTable; ui += blockDim.x) unit_tab[ui] = unit_global(ui);
  __syncthreads();
  auto unit_of = [&](uint32_t ui, uint32_t& expert, uint32_t& r0, uint32_t& rows, uint32_t& n0) {
    const uint4 v = ui < (uint32_t)kMtaUnitTable ? unit_tab[ui] : unit_global(ui);
    expert = v.x; r0 = v.y; rows = v.z; n0 = v.w;
  };

  if (warp == 0) {
    // ================= TMA producer: packed weights of the unit's expert, rows [expert * N + n0, +128) ============
    if (lane == 0) {
      uint32_t gc = 0, issued = 0;
      bool ok = true;
      PROF_DECL(3);
      PROF_T0();
      for (uint32_t ui = 0; ui < my_units && ok; ++ui) {
        uint32_t expert, r0, rows, n0;
        unit_of(ui, expert, r0, rows, n0);
        PROF_ADD(0);
        for (uint32_t c = 0; c < num_chunks; ++c, ++gc) {
          const uint32_t s = gc % kMtaWStages, ph = (gc / kMtaWStages) & 1u;
          if (gc >= (uint32_t)kMtaWStages && !mbar_wait(bar_w_empty(s), ph ^ 1u, p.status, 6u, abort_flag)) { ok = false; break; }
          PROF_ADD(1);
          mbar_arrive_expect_tx(bar_w_full(s), (uint32_t)L::kWBytes);
          tma_load_2d(w_ring + s * L::kWBytes, &tmap_w, bar_w_full(s), (int)(c * 32), (int)(expert * p.N + n0));
          issued = gc + 1;
          PROF_ADD(2);
        }
      }
      PROF_OUT(0, 3, true);
      if (*abort_flag) {   // the consumers stopped: wait (bounded) until the copies already issued have landed
        const uint32_t first = issued > (uint32_t)kMtaWStages ? issued - kMtaWStages : 0u;
        for (uint32_t c = first; c < issued; ++c) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar_w_full(c % kMtaWStages), (c / kMtaWStages) & 1u) &&
                 (unsigned long long)(clock64() - t0) < kWaitCycles) {}
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    // One tcgen05.commit per 128-element stage: a commit keeps the issuing thread for a couple of hundred cycles, about
    // as long as the MMAs of a 64-element k block of a 64-pair tile take on the tensor pipe.
    if (lane == 0) {
      const uint64_t b0 = smem_desc_sw128(x_ring);
      uint32_t gst = 0;
      bool ok = true;
      PROF_DECL(5);
      PROF_T0();
      for (uint32_t ui = 0; ui < my_units && ok; ++ui) {
        uint32_t expert, r0, rows, n0;
        unit_of(ui, expert, r0, rows, n0);
        PROF_ADD(0);
        const uint32_t n_mma = rows <= 16u ? 16u : ((rows + 15u) & ~15u);
        const uint32_t idesc = idesc_f16((int)n_mma);
        const uint32_t ab = ui & 1u;
        // this accumulator set was last read by the epilogue of unit ui - 2
        if (ui >= 2u && !mbar_wait(bar_acc_empty(ab), ((ui >> 1) & 1u) ^ 1u, p.status, 8u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        PROF_ADD(1);
        const uint32_t d_tmem = tmem_base + ab * (uint32_t)kMtaNP;
        for (uint32_t st = 0; st < num_st; ++st, ++gst) {
          const uint32_t s = gst % kMtaStages, ph = (gst / kMtaStages) & 1u;
          if (!mbar_wait(bar_full(s), ph, p.status, 2u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          PROF_ADD(2);
          const uint64_t bdesc = b0 + (uint64_t)(s * (L::kXBytes >> 4));
          const uint32_t a_tmem = tmem_base + kMtaColA + s * kMtaSliceCols;
          const int nk = (2 * st + 1 < num_kb) ? 8 : 4;            // 16-element steps in this stage
#ifdef ZTVM_MTA_NOMMA
          if (nk == 99)
#endif
#pragma unroll
          for (int k = 0; k < 8; ++k)   // 16 k elements: 8 TMEM columns of A, 32 bytes along the swizzled row of atom k / 4
            if (k < nk)
              umma_f16_ta(d_tmem, a_tmem + (uint32_t)(8 * k), bdesc + (uint64_t)((k >> 2) * (L::kXHalf >> 4) + 2 * (k & 3)), idesc,
                          (st | (uint32_t)k) ? 1u : 0u);
          PROF_ADD(3);
          umma_commit(bar_empty(s));   // the activation tile and the weight slice are free once these MMAs have read them
          PROF_ADD(4);
        }
        if (ok) umma_commit(bar_acc_full(ab));
      }
      PROF_OUT(8, 5, true);
    }
  } else if (warp < 2 + kMtaDqWarps) {
    // ================= dequantisers (warps 2..9) =================
    // Thread (quarter, lane) owns weight row 32 quarter + lane of the unit; the two warps of a quarter take one scale
    // group (64 codes) of the stage each: 8 words in, 32 columns of tensor memory out.
    const int quarter = warp & 3;                       // TMEM lanes this warp may touch: [32 * quarter, +32)
    const uint32_t part = (uint32_t)(warp - 2) >> 2;    // which 128 / kMtaParts codes of the stage
    const uint32_t r_tile = (uint32_t)(quarter * 32 + lane);
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint8_t* const wrow_sm = gen_base + L::kOffW + (r_tile >> 3) * 1024 + (r_tile & 7) * 128;
    uint32_t gst = 0, gc = 0;
    bool ok = true;
    PROF_DECL(7);
    PROF_T0();
    // Scales and biases of this thread's row, eight groups (= four stages) per 16-byte load. The loads run as one stream
    // over (unit, block of four stages), two items ahead of their use, so a unit's first scales are already in
    // registers when the unit starts. This thread's group of stage st is k block 2 st + gsel. Rows whose group count is
    // no multiple of eight (or unaligned tables) load the two f16 values per stage instead.
    const bool vec_sb = (p.SPR % 8u) == 0 && ((reinterpret_cast<uintptr_t>(p.S) | reinterpret_cast<uintptr_t>(p.B)) & 15u) == 0;
    const uint32_t nblk = (num_st + 3u) / 4u;
    auto row_of = [&](uint32_t ui) -> size_t {
      uint32_t expert, r0, rows, n0;
      unit_of(ui, expert, r0, rows, n0);
      return (size_t)expert * p.N + min(n0 + r_tile, p.N - 1);
    };
    auto load_sb8 = [&](uint4& sv, uint4& bv, uint32_t item) {     // item = ui * nblk + block
      if (!vec_sb || item >= my_units * nblk) return;
      const uint32_t ui = item / nblk, blk = item - ui * nblk;
      const size_t off = row_of(ui) * p.SPR + 8u * blk;
      sv = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.S) + off));
      bv = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.B) + off));
    };
    auto pick16 = [](const uint4& v, uint32_t i) -> unsigned short {
      const uint32_t wsel = (i >> 1) == 0 ? v.x : (i >> 1) == 1 ? v.y : (i >> 1) == 2 ? v.z : v.w;
      return (unsigned short)((i & 1) ? (wsel >> 16) : (wsel & 0xFFFFu));
    };
    uint4 sv_cur = make_uint4(0, 0, 0, 0), bv_cur = sv_cur, sv_nxt = sv_cur, bv_nxt = sv_cur;
    load_sb8(sv_cur, bv_cur, 0);
    load_sb8(sv_nxt, bv_nxt, 1);
    uint32_t item = 0;
    for (uint32_t ui = 0; ui < my_units && ok; ++ui) {
      const size_t row = row_of(ui);
      const unsigned short* srow = reinterpret_cast<const unsigned short*>(p.S) + row * p.SPR;
      const unsigned short* brow = reinterpret_cast<const unsigned short*>(p.B) + row * p.SPR;
      for (uint32_t st0 = 0; st0 < num_st && ok; st0 += 4) {
#pragma unroll
        for (int si = 0; si < 4; ++si) {
          const uint32_t st = st0 + si;
          if (st >= num_st || !ok) break;
          const uint32_t g = gst + st;
          const uint32_t s = g % kMtaStages, ph = (g / kMtaStages) & 1u;
          const uint32_t c = gc + st / kMtaWPerSlot, ws = c % kMtaWStages;
          const uint32_t j = (uint32_t)si % kMtaWPerSlot;          // st0 is a multiple of 4
          const uint32_t gsel = part * 2u / kMtaParts;          // which of the stage's two scale groups
          const uint32_t kb = 2u * st + gsel;
          PROF_ADD(0);
          if (j == 0) ok = mbar_wait(bar_w_full(ws), (c / kMtaWStages) & 1u, p.status, 7u, abort_flag);
          PROF_ADD(1);
          uint4 wq[kMtaWpt / 4];
#pragma unroll
          for (int q = 0; q < kMtaWpt / 4; ++q) {   // 16-byte chunks of this row's 128 bytes of the slot, swizzled by the row
            const uint32_t ch = 4u * j + part * (kMtaWpt / 4) + q;
            wq[q] = ok ? *reinterpret_cast<const uint4*>(wrow_sm + ws * L::kWBytes + ((ch ^ (r_tile & 7)) << 4)) : make_uint4(0, 0, 0, 0);
          }
          PROF_ADD(2);
          // the TMEM slice of stage s was last read by the MMAs of stage g - kMtaStages
          if (ok && g >= (uint32_t)kMtaStages) {
            ok = mbar_wait(bar_empty(s), ph ^ 1u, p.status, 4u, abort_flag);
            tc_fence_after();
          }
          PROF_ADD(3);
          if (ok && kb < num_kb) {
            unsigned short s16, b16;
            if (vec_sb) {
              s16 = pick16(sv_cur, 2u * (uint32_t)si + gsel);
              b16 = pick16(bv_cur, 2u * (uint32_t)si + gsel);
            } else {
              s16 = __ldg(srow + kb);
              b16 = __ldg(brow + kb);
            }
            const DqGroup dq = dq_group<true>(s16, b16);
            uint32_t a[4 * kMtaWpt];
#pragma unroll
            for (int wi = 0; wi < kMtaWpt; ++wi) {
              const uint4& src = wq[wi >> 2];
              const uint32_t word = (wi & 3) == 0 ? src.x : (wi & 3) == 1 ? src.y : (wi & 3) == 2 ? src.z : src.w;
#ifndef ZTVM_MTA_NOMATH
              const uint4 v = dequant_word_w16<true>(word, dq);
#else
              const uint4 v = make_uint4(word, word + dq.s16, word ^ 3u, word + 1u);
#endif
              a[4 * wi] = v.x; a[4 * wi + 1] = v.y; a[4 * wi + 2] = v.z; a[4 * wi + 3] = v.w;
            }
            // 8 weights per word = 4 TMEM columns (two k-adjacent f16 per column) of this thread's lane
            const uint32_t taddr = tmem_base + lane_base + kMtaColA + s * kMtaSliceCols + part * (4u * kMtaWpt);
#ifndef ZTVM_MTA_NOST
            tmem_st_cols<4 * kMtaWpt>(taddr, a);
#else
            if (a[0] == 0x12345678u && a[7] == 0x9abcdef0u) tmem_st_cols<4 * kMtaWpt>(taddr, a);
#endif
            PROF_ADD(4);
            tmem_st_wait();
            PROF_ADD(5);
          }
          // the packed slot goes back to the producer only after the stores that consumed its words
          if (j == kMtaWPerSlot - 1 || st + 1 == num_st) {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_w_empty(ws));
          }
          // every lane's stores to tensor memory are complete (wait::st above); one lane signals for the warp
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_full(s));   // (also on abort)
          PROF_ADD(6);
        }
        sv_cur = sv_nxt; bv_cur = bv_nxt;
        load_sb8(sv_nxt, bv_nxt, item + 2u);
        ++item;
      }
      gst += num_st;
      gc += num_chunks;
    }
    PROF_OUT(16, 7, threadIdx.x == 64);
  } else if (warp < 2 + kMtaDqWarps + kMtaGaWarps) {
    // ================= gather: activation rows of the tile's pairs into the swizzled B stages =================
    // Lane mapping for coalescing: the eight lanes t % 8 = 0..7 copy the eight 16-byte chunks of one 128-byte row
    // segment, so a warp-wide cp.async touches 4 rows (4 lines), not 32. Thread t serves rows t / 8 + 16 i, i = 0..7.
    const uint32_t t = threadIdx.x - (2 + kMtaDqWarps) * 32;      // 0..127
    const uint32_t chunk = t & 7u, rbase = t >> 3;
    uint32_t gst = 0;
    bool ok = true;
    PROF_DECL(4);
    PROF_T0();
    // the pair indices of unit ui + 1 are fetched while unit ui streams
    uint32_t pr_nxt[8];
    auto load_pairs = [&](uint32_t ui) {
#pragma unroll
      for (int i = 0; i < 8; ++i) pr_nxt[i] = 0xFFFFFFFFu;
      if (ui >= my_units) return;
      uint32_t expert, r0, rows, n0;
      unit_of(ui, expert, r0, rows, n0);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t r = rbase + 16u * i;
        if (r < rows) pr_nxt[i] = p.sc.sorted[r0 + r];
      }
    };
    load_pairs(0);
    for (uint32_t ui = 0; ui < my_units && ok; ++ui) {
      const __half* xrow[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        xrow[i] = nullptr;
        if (pr_nxt[i] != 0xFFFFFFFFu) {
          const uint32_t pair = pr_nxt[i];
          const uint32_t tok = pair / p.slots, slot = pair - tok * p.slots;
          xrow[i] = p.X + (size_t)tok * p.in_tok_stride + (size_t)slot * p.in_slot_stride + chunk * 8u;
        }
      }
      load_pairs(ui + 1);
      auto issue = [&](uint32_t st) -> bool {      // false: a wait ran out
        bool good = true;
        if (st < num_st) {
          const uint32_t g = gst + st, s = g % kMtaStages;
          if (g >= (uint32_t)kMtaStages) good = mbar_wait(bar_empty(s), ((g / kMtaStages) & 1u) ^ 1u, p.status, 3u, abort_flag);
          if (good) {
            const uint32_t dst0 = x_ring + s * L::kXBytes;
            const bool two = 2 * st + 1 < num_kb;              // the stage holds both 64-element atoms
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (!xrow[i]) continue;
              const uint32_t r = rbase + 16u * i;
              const uint32_t dst = dst0 + (r >> 3) * 1024u + (r & 7u) * 128u + ((chunk ^ (r & 7u)) << 4);
              const __half* src = xrow[i] + (size_t)st * kMtaBK;
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
              if (two) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)L::kXHalf), "l"(src + 64) : "memory");
            }
          }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        return good;
      };
#pragma unroll
      for (int i = 0; i < kMtaLead; ++i) ok = ok && issue((uint32_t)i);
      PROF_ADD(0);
      for (uint32_t st = 0; st < num_st; ++st) {
        if (ok) ok = issue(st + kMtaLead); else asm volatile("cp.async.commit_group;" ::: "memory");
        PROF_ADD(1);
        asm volatile("cp.async.wait_group %0;" ::"n"(kMtaLead) : "memory");   // this thread's row of stage st has landed
        PROF_ADD(2);
        fence_proxy_async();              // each thread publishes its own row to the async proxy, then one lane signals
        __syncwarp();
        if ((t & 31u) == 0) mbar_arrive(bar_full((gst + st) % kMtaStages));   // (also on abort)
        PROF_ADD(3);
      }
      gst += num_st;
    }
    PROF_OUT(24, 4, t == 0);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else {
    // ================= epilogue: D[weight row][pair] in TMEM -> y rows of the pairs =================
    const int quarter = warp & 3;
    const uint32_t r_tile = (uint32_t)(quarter * 32 + lane);
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    bool ok = true;
    PROF_DECL(2);
    PROF_T0();
    for (uint32_t ui = 0; ui < my_units && ok; ++ui) {
      uint32_t expert, r0, rows, n0;
      unit_of(ui, expert, r0, rows, n0);
      const uint32_t ab = ui & 1u;
      if (!mbar_wait(bar_acc_full(ab), (ui >> 1) & 1u, p.status, 5u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      PROF_ADD(0);
      const uint32_t n = n0 + r_tile;
      for (uint32_t cb = 0; cb * 32u < rows; ++cb) {
        // lane i looks up where pair cb * 32 + i lives; the addresses are then passed round the warp
        unsigned long long my_dst = 0ull;
        if (cb * 32u + lane < rows) {
          const uint32_t pr = p.sc.sorted[r0 + cb * 32u + lane];
          if (p.dst_index) {
            my_dst = reinterpret_cast<unsigned long long>(p.y_seg[pr / p.seg_cap] + (size_t)p.dst_index[pr] * p.out_tok_stride);
          } else {
            const uint32_t tk = pr / p.slots, sl = pr - tk * p.slots;
            my_dst = reinterpret_cast<unsigned long long>(p.Y + (size_t)tk * p.out_tok_stride + (size_t)sl * p.out_slot_stride);
          }
        }
        uint32_t v[32];
        tmem_ld32(tmem_base + lane_base + ab * (uint32_t)kMtaNP + cb * 32u, v);
        tmem_ld_wait();
        const uint32_t lim = rows - cb * 32u;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const unsigned long long d = __shfl_sync(0xffffffffu, my_dst, i);
          if ((uint32_t)i < lim && n < p.N) reinterpret_cast<__half*>(d)[n] = __float2half_rn(__uint_as_float(v[i]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty(ab));
      PROF_ADD(1);
    }
    PROF_OUT(32, 2, threadIdx.x == (2 + kMtaDqWarps + kMtaGaWarps) * 32);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kMtaTmemCols);
}

// ---- host side -----------------------------------------------------------------------------------------
typedef CUresult (*MtaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static MtaEncodeFn mta_encode_fn() {
  static MtaEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<MtaEncodeFn>(ptr);
  }
  return fn;
}

// Encoded tensor maps of expert stacks, kept per (address, shape): an engine calls with the same few stacks for ever.
static cudaError_t mta_weight_map(const uint32_t* W, uint32_t KP, uint64_t rows, CUtensorMap* out) {
  struct Entry { const uint32_t* W; uint32_t KP; uint64_t rows; CUtensorMap map; };
  constexpr int kSlots = 32;
  static Entry cache[kSlots];
  static int used = 0, next = 0;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < used; ++i)
    if (cache[i].W == W && cache[i].KP == KP && cache[i].rows == rows) { *out = cache[i].map; return cudaSuccess; }
  MtaEncodeFn enc = mta_encode_fn();
  if (!enc) return cudaErrorNotSupported;
  const cuuint64_t wdims[2] = {KP, rows};
  const cuuint64_t wstrides[1] = {(cuuint64_t)KP * 4};
  const cuuint32_t wbox[2] = {32, (cuuint32_t)kMtaRows};
  const cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(W), wdims, wstrides, wbox, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
  const int slot = used < kSlots ? used++ : (next = (next + 1) % kSlots);
  cache[slot] = Entry{W, KP, rows, m};
  *out = m;
  return cudaSuccess;
}

#ifdef ZTVM_MTA_PROF
extern "C" __attribute__((visibility("default"))) int ztvm_mta_prof_read(unsigned long long* out) {
  return (int)cudaMemcpyFromSymbol(out, g_mta_prof, sizeof(unsigned long long) * 64);
}
#endif

bool moe_ta_supported(int bits, uint32_t group, uint32_t K, uint32_t N, uint32_t experts) {
  return bits == 4 && group == 64 && K % kGemmBK == 0 && K >= (uint32_t)kGemmBK && N % 8 == 0 && experts <= 1024;
}

cudaError_t launch_moe_ta(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t* scratch, uint32_t* status,
                          int sm_count, cudaStream_t st, bool reuse_plan) {
  static_assert(kMtaNP == (int)kMoeTaTileRows, "tile rows");
  const uint32_t P = tokens * slots, E = g.experts;
  MoeScratch sc = moe_scratch_carve(scratch, E, P);
  cudaError_t e = reuse_plan ? cudaSuccess : launch_moe_plan(g, tokens, slots, sc, (uint32_t)kMtaNP, st);
  if (e != cudaSuccess) return e;
  CUtensorMap tmap_w;
  e = mta_weight_map(g.W, g.KP, (uint64_t)E * g.N, &tmap_w);
  if (e != cudaSuccess) return e;
  MoeTaParams p;
  p.S = g.S; p.B = g.B; p.X = g.X; p.Y = reinterpret_cast<__half*>(g.Y);
  p.N = g.N; p.K = g.K; p.SPR = g.SPR; p.slots = slots; p.NB = (g.N + kMtaRows - 1) / kMtaRows;
  p.in_slot_stride = g.in_slot_stride; p.out_slot_stride = g.out_slot_stride;
  p.in_tok_stride = g.in_tok_stride; p.out_tok_stride = g.out_tok_stride;
  p.sc = sc; p.status = status;
  p.dst_index = g.dst_index; p.seg_cap = g.seg_cap ? g.seg_cap : 1u;
  for (int i = 0; i < 9; ++i) p.y_seg[i] = reinterpret_cast<__half*>(g.y_seg[i]);
  constexpr int smem = MtaSmem::kTotal + 1024;
  static bool attr_set[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 64 && !attr_set[dev]) {
      e = cudaFuncSetAttribute(moe_ta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return e;
      attr_set[dev] = true;
    }
  }
  // upper bound of the units (the kernel reads the real count): no more CTAs than that, one per SM
  const uint64_t max_units = ((uint64_t)(P + kMtaNP - 1) / kMtaNP + E) * p.NB;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(max_units < (uint64_t)sm_count ? max_units : (uint64_t)sm_count));
  cfg.blockDim = dim3(kMtaThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, moe_ta_kernel, tmap_w, p);
}

}  // namespace ztvm
