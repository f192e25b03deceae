// Grouped MoE expert matmul on tcgen05 with the DEQUANTISED EXPERT WEIGHTS AS THE A OPERAND IN TENSOR MEMORY:
//   y[token, slot, :] = x[token, slot, :] * W16[ids[token, slot]]^T        (int4_matmul.gen.ts:229-254)
// for launches where an expert sees many pairs. The pairs of one expert (sorted by the plan, ztvm_moe_plan.cuh) take
// the N side of the MMA, up to 128 per tile, so an expert's weights are dequantised ONCE per 128 pairs, and go from the
// dequantisers' registers straight into tensor memory (tcgen05.st) instead of through shared memory. The activation
// rows of the tile's pairs are the only shared-memory operand: gathered with 16-byte cp.async into the
// 128-byte-swizzled K-major layout, eight lanes per 128-byte row segment (coalesced).
//
// Unit of work = (tile of pairs, 256 weight rows): two 128-row halves share every gathered activation stage, which
// halves the activation traffic per weight byte (with 128-row units the re-gathering of x for every row block, not
// the arithmetic, set the pace). Persistent: one CTA per SM walks its units blockIdx.x, + gridDim.x, ...; the unit
// descriptors are copied from the plan into shared memory once, and pair lists and scales of the next unit are
// fetched while the current one streams, so nothing chases pointers through global memory at a unit boundary. Every
// pipeline (packed weights, activations, weight slices) keeps running across unit boundaries.
//
// Roles (832 threads): warp 0 TMA-loads packed weights (two boxes of 128 rows x 32 words = four k blocks per slot);
// warp 1 owns tensor memory and issues the MMAs (eight per 64-element stage, one commit); warps 2..17 dequantise
// (warp w touches TMEM lanes 32 (w % 4) .. +31; the four warps of a lane quarter take the two row halves x the two
// 32-code halves of a stage); warps 18..21 gather activations; warps 22..25 read finished accumulators and scatter
// them to where each pair lives (or, in the expert-parallel form, to the rank it came from). One arrival per warp on
// the shared-memory barriers. Every wait is bounded: on expiry a status word is raised, the roles stop, copies in
// flight are waited for, TMEM is freed.
#include <mutex>

#include "ztvm_kernels.h"
#include "ztvm_moe_plan.cuh"
#include "ztvm_tc.cuh"

namespace ztvm {

constexpr int kMtaStages = 4;        // weight slices in tensor memory (64 k elements x two row halves each)
constexpr int kMtaXStages = 4;       // activation tiles in shared memory (64 k elements each), a ring of their own
constexpr int kMtaWStages = 4;       // packed-weight ring; a slot holds four k blocks of both row halves
constexpr int kMtaWChunk = 4;        // k blocks per packed-weight slot
constexpr int kMtaNP = 128;          // pairs per tile = widest MMA N used
constexpr int kMtaRows = 128;        // weight rows per half = TMEM lanes
constexpr int kMtaUnitRows = 2 * kMtaRows;
constexpr int kMtaDqWarps = 16, kMtaGaWarps = 4, kMtaEpWarps = 4;
constexpr int kMtaThreads = 64 + (kMtaDqWarps + kMtaGaWarps + kMtaEpWarps) * 32;
constexpr int kMtaLead = kMtaXStages - 2;  // activation rows are fetched this many stages ahead
constexpr uint32_t kMtaColA = 2 * kMtaNP;  // TMEM: one accumulator per row half, then the weight slices (32 columns each)
constexpr uint32_t kMtaTmemCols = 512;
constexpr int kMtaUnitTable = 256;   // units of a CTA kept in shared memory (further ones are read from the plan directly)
static_assert(kMtaColA + kMtaStages * 2 * 32 <= kMtaTmemCols, "tensor memory columns");

struct MoeTaParams {
  const __half* S;
  const __half* B;
  const __half* X;
  __half* Y;
  uint32_t N, K, SPR, slots, NB;      // NB: 256-row blocks of N
  uint32_t in_slot_stride, out_slot_stride, in_tok_stride, out_tok_stride;
  MoeScratch sc;
  uint32_t* status;
  // expert-parallel form: the output row of pair i lives at y_seg[i / seg_cap] + dst_index[i] * out_tok_stride
  const uint32_t* dst_index;
  uint32_t seg_cap;
  __half* y_seg[9];
  uint32_t vec_out;                   // every output row starts on a 16-byte boundary: rows leave in 16-byte stores
};

struct MtaSmem {
  static constexpr int kXBytes = kMtaNP * 128;                   // per stage: 128 pair rows x 64 k
  static constexpr int kWHalf = kMtaRows * 128;                  // one row half of a packed-weight slot
  static constexpr int kWBytes = 2 * kWHalf;
  static constexpr int kOffW = kMtaXStages * kXBytes;
  static constexpr int kOffBar = kOffW + kMtaWStages * kWBytes;
  static constexpr int kOffUnits = kOffBar + 256;                // this CTA's first kMtaUnitTable units: expert, r0, rows, n0
  static constexpr int kStagePitch = kMtaUnitRows * 2;           // epilogue stage: 32 pairs x 256 weight rows, f16
  static constexpr int kOffStage = kOffUnits + kMtaUnitTable * 16;
  static constexpr int kOffDst = kOffStage + 32 * kStagePitch;   // output row address of each pair of a unit, two units
  static constexpr int kTotal = kOffDst + 2 * kMtaNP * 8;
};

// Named barrier 1: the epilogue warps among themselves (barrier 0 is __syncthreads).
__device__ __forceinline__ void ep_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kMtaEpWarps * 32) : "memory"); }
__device__ __forceinline__ bool ep_bar_and(bool pred) {
  uint32_t r;
  asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, 1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
               : "=r"(r) : "r"((uint32_t)pred), "n"(kMtaEpWarps * 32) : "memory");
  return r != 0u;
}

__global__ void __launch_bounds__(kMtaThreads, 1)
moe_ta_kernel(const __grid_constant__ CUtensorMap tmap_w, const MoeTaParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  using L = MtaSmem;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t x_ring = base, w_ring = base + L::kOffW, bars = base + L::kOffBar;
  // a_*: weight slices in tensor memory (dequantisers <-> MMA); x_*: activation tiles in shared memory (gather <-> MMA)
  auto bar_full = [&](uint32_t s) { return bars + 8u * s; };
  auto bar_empty = [&](uint32_t s) { return bars + 8u * (kMtaStages + s); };
  auto bar_x_full = [&](uint32_t s) { return bars + 8u * (2 * kMtaStages + s); };
  auto bar_x_empty = [&](uint32_t s) { return bars + 8u * (2 * kMtaStages + kMtaXStages + s); };
  constexpr int kBarW = 2 * kMtaStages + 2 * kMtaXStages;
  auto bar_w_full = [&](uint32_t s) { return bars + 8u * (kBarW + s); };
  auto bar_w_empty = [&](uint32_t s) { return bars + 8u * (kBarW + kMtaWStages + s); };
  const uint32_t bar_acc_full = bars + 8u * (kBarW + 2 * kMtaWStages);
  const uint32_t bar_acc_empty = bar_acc_full + 8u;
  constexpr int kNumBars = kBarW + 2 * kMtaWStages + 2;
  static_assert(8 * kNumBars + 8 <= 256, "barrier block");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + L::kOffBar + 8 * kNumBars);
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t num_kb = p.K / kGemmBK;                       // 64-element stages (= scale groups)
  const uint32_t num_chunks = (num_kb + kMtaWChunk - 1) / kMtaWChunk;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMtaStages; ++s) {
      mbar_init(bar_full(s), kMtaDqWarps);   // one arrival per dequantiser warp
      mbar_init(bar_empty(s), 1);
    }
    for (int s = 0; s < kMtaXStages; ++s) {
      mbar_init(bar_x_full(s), kMtaGaWarps);  // one arrival per gather warp
      mbar_init(bar_x_empty(s), 1);
    }
    for (int s = 0; s < kMtaWStages; ++s) {
      mbar_init(bar_w_full(s), 1);
      mbar_init(bar_w_empty(s), kMtaDqWarps);
    }
    mbar_init(bar_acc_full, 1);
    mbar_init(bar_acc_empty, kMtaEpWarps);
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

  const uint32_t total_units = *p.sc.ntiles * p.NB;
  const uint32_t my_units = total_units > blockIdx.x ? (total_units - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
  uint4* unit_tab = reinterpret_cast<uint4*>(gen_base + L::kOffUnits);
  auto unit_global = [&](uint32_t ui) {
    const uint32_t u = blockIdx.x + ui * gridDim.x;
    const uint32_t tile = u / p.NB;
    return make_uint4(p.sc.tiles[(size_t)tile * 3], p.sc.tiles[(size_t)tile * 3 + 1], p.sc.tiles[(size_t)tile * 3 + 2],
                      (u - tile * p.NB) * kMtaUnitRows);
  };
  for (uint32_t ui = threadIdx.x; ui < my_units && ui < (uint32_t)kMtaUnitTable; ui += blockDim.x) unit_tab[ui] = unit_global(ui);
  __syncthreads();
  auto unit_of = [&](uint32_t ui, uint32_t& expert, uint32_t& r0, uint32_t& rows, uint32_t& n0) {
    const uint4 v = ui < (uint32_t)kMtaUnitTable ? unit_tab[ui] : unit_global(ui);
    expert = v.x; r0 = v.y; rows = v.z; n0 = v.w;
  };

  if (warp == 0) {
    // ================= TMA producer: packed weights, rows [expert * N + n0, +256) as two boxes of 128 ============
    if (lane == 0) {
      uint32_t gc = 0, issued = 0;
      bool ok = true;
      for (uint32_t ui = 0; ui < my_units && ok; ++ui) {
        uint32_t expert, r0, rows, n0;
        unit_of(ui, expert, r0, rows, n0);
        for (uint32_t c = 0; c < num_chunks; ++c, ++gc) {
          const uint32_t s = gc % kMtaWStages, ph = (gc / kMtaWStages) & 1u;
          if (gc >= (uint32_t)kMtaWStages && !mbar_wait(bar_w_empty(s), ph ^ 1u, p.status, 6u, abort_flag, 400u)) { ok = false; break; }
          mbar_arrive_expect_tx(bar_w_full(s), (uint32_t)L::kWBytes);
          tma_load_2d(w_ring + s * L::kWBytes, &tmap_w, bar_w_full(s), (int)(c * 32), (int)(expert * p.N + n0));
          tma_load_2d(w_ring + s * L::kWBytes + L::kWHalf, &tmap_w, bar_w_full(s), (int)(c * 32), (int)(expert * p.N + n0 + kMtaRows));
          issued = gc + 1;
        }
      }
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
    if (lane == 0) {
      const uint64_t b0 = smem_desc_sw128(x_ring);
      uint32_t gst = 0;
      bool ok = true;
      for (uint32_t ui = 0; ui < my_units && ok; ++ui) {
        uint32_t expert, r0, rows, n0;
        unit_of(ui, expert, r0, rows, n0);
        const uint32_t n_mma = rows <= 16u ? 16u : ((rows + 15u) & ~15u);
        const uint32_t idesc = idesc_f16((int)n_mma);
        const bool two = n0 + kMtaRows < p.N;                       // the second row half holds rows of this expert
        // the accumulators were last read by the epilogue of the previous unit
        if (ui >= 1u && !mbar_wait(bar_acc_empty, (ui & 1u) ^ 1u, p.status, 8u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (uint32_t kb = 0; kb < num_kb; ++kb, ++gst) {
          const uint32_t s = gst % kMtaStages, ph = (gst / kMtaStages) & 1u;
          const uint32_t xs = gst % kMtaXStages, xph = (gst / kMtaXStages) & 1u;
          if (!mbar_wait(bar_x_full(xs), xph, p.status, 9u, abort_flag)) { ok = false; break; }
          if (!mbar_wait(bar_full(s), ph, p.status, 2u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t bdesc = b0 + (uint64_t)(xs * (L::kXBytes >> 4));
          const uint32_t a_tmem = tmem_base + kMtaColA + s * 64u;
#pragma unroll
          for (int k = 0; k < kGemmBK / 16; ++k)   // 16 k elements: 8 TMEM columns of A, 32 bytes along the swizzled B row
            umma_f16_ta(tmem_base, a_tmem + (uint32_t)(8 * k), bdesc + (uint64_t)(2 * k), idesc, (kb | (uint32_t)k) ? 1u : 0u);
          if (two) {
#pragma unroll
            for (int k = 0; k < kGemmBK / 16; ++k)
              umma_f16_ta(tmem_base + (uint32_t)kMtaNP, a_tmem + 32u + (uint32_t)(8 * k), bdesc + (uint64_t)(2 * k), idesc,
                          (kb | (uint32_t)k) ? 1u : 0u);
          }
          umma_commit(bar_empty(s));   // the weight slices and the activation tile are free once these MMAs have read them
          umma_commit(bar_x_empty(xs));
        }
        if (ok) umma_commit(bar_acc_full);
      }
    }
  } else if (warp < 2 + kMtaDqWarps) {
    // ================= dequantisers (warps 2..17) =================
    // Thread (quarter, lane) of part p owns weight row 128 (p / 2) + 32 quarter + lane of the unit and the 32-code half
    // p % 2 of every stage: 4 words in, 16 columns of tensor memory out.
    const int quarter = warp & 3;                       // TMEM lanes this warp may touch: [32 * quarter, +32)
    const uint32_t part = (uint32_t)(warp - 2) >> 2;    // 0..3
    const uint32_t half = part >> 1, khalf = part & 1u;
    const uint32_t r_half = (uint32_t)(quarter * 32 + lane);            // row inside the half
    const uint32_t r_unit = half * kMtaRows + r_half;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint8_t* const wrow_sm = gen_base + L::kOffW + half * L::kWHalf + (r_half >> 3) * 1024 + (r_half & 7) * 128;
    // Scales and biases of this thread's row, eight groups (= eight stages) per 16-byte load. The loads run as one stream
    // over (unit, block of eight stages), two items ahead of their use, so a unit's first scales are already in
    // registers when the unit starts. Rows whose group count is no multiple of eight (or unaligned tables) load the
    // two f16 values per stage instead.
    const bool vec_sb = (p.SPR % 8u) == 0 && ((reinterpret_cast<uintptr_t>(p.S) | reinterpret_cast<uintptr_t>(p.B)) & 15u) == 0;
    const uint32_t nblk = (num_kb + 7u) / 8u;
    auto row_of = [&](uint32_t ui) -> size_t {
      uint32_t expert, r0, rows, n0;
      unit_of(ui, expert, r0, rows, n0);
      return (size_t)expert * p.N + min(n0 + r_unit, p.N - 1);
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
    uint32_t gst = 0, gc = 0, item = 0;
    bool ok = true;
    for (uint32_t ui = 0; ui < my_units && ok; ++ui) {
      const size_t row = row_of(ui);
      const unsigned short* srow = reinterpret_cast<const unsigned short*>(p.S) + row * p.SPR;
      const unsigned short* brow = reinterpret_cast<const unsigned short*>(p.B) + row * p.SPR;
      for (uint32_t kb0 = 0; kb0 < num_kb && ok; kb0 += 8) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t kb = kb0 + i;
          if (kb >= num_kb || !ok) break;
          const uint32_t g = gst + kb;
          const uint32_t s = g % kMtaStages, ph = (g / kMtaStages) & 1u;
          const uint32_t c = gc + kb / kMtaWChunk, ws = c % kMtaWStages;
          const uint32_t j = (uint32_t)i % kMtaWChunk;              // kb0 is a multiple of 8
          if (j == 0) ok = mbar_wait(bar_w_full(ws), (c / kMtaWStages) & 1u, p.status, 7u, abort_flag);
          uint4 wv = make_uint4(0, 0, 0, 0);   // 16-byte chunk 2 j + khalf of this row's 128 bytes of the slot, swizzled by the row
          if (ok) wv = *reinterpret_cast<const uint4*>(wrow_sm + ws * L::kWBytes + (((2u * j + khalf) ^ (r_half & 7)) << 4));
          // the TMEM slices of stage s were last read by the MMAs of stage g - kMtaStages
          if (ok && g >= (uint32_t)kMtaStages) {
            ok = mbar_wait(bar_empty(s), ph ^ 1u, p.status, 4u, abort_flag);
            tc_fence_after();
          }
          if (ok) {
            unsigned short s16, b16;
            if (vec_sb) {
              s16 = pick16(sv_cur, (uint32_t)i);
              b16 = pick16(bv_cur, (uint32_t)i);
            } else {
              s16 = __ldg(srow + kb);
              b16 = __ldg(brow + kb);
            }
            const DqGroup dq = dq_group<true>(s16, b16);
            const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
            uint32_t a[16];
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
              const uint4 v = dequant_word_w16<true>(words[wi], dq);
              a[4 * wi] = v.x; a[4 * wi + 1] = v.y; a[4 * wi + 2] = v.z; a[4 * wi + 3] = v.w;
            }
            // 32 weights of this row = 16 TMEM columns (two k-adjacent f16 per column) of this thread's lane
            tmem_st16(tmem_base + lane_base + kMtaColA + s * 64u + half * 32u + khalf * 16u, a);
            tmem_st_wait();
          }
          // the packed slot goes back to the producer only after the stores that consumed its words
          if (j == kMtaWChunk - 1 || kb + 1 == num_kb) {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_w_empty(ws));
          }
          // every lane's stores to tensor memory are complete (wait::st above); one lane signals for the warp. (A few
          // hundred arrivals per stage on one shared-memory barrier would cost more than the dequantisation.)
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_full(s));   // (also on abort)
        }
        sv_cur = sv_nxt; bv_cur = bv_nxt;
        load_sb8(sv_nxt, bv_nxt, item + 2u);
        ++item;
      }
      gst += num_kb;
      gc += num_chunks;
    }
  } else if (warp < 2 + kMtaDqWarps + kMtaGaWarps) {
    // ================= gather: activation rows of the tile's pairs into the swizzled B stages =================
    // Lane mapping for coalescing: the eight lanes t % 8 = 0..7 copy the eight 16-byte chunks of one 128-byte row
    // segment, so a warp-wide cp.async touches 4 rows (4 lines), not 32. Thread t serves rows t / 8 + 16 i, i = 0..7.
    const uint32_t t = threadIdx.x - (2 + kMtaDqWarps) * 32;      // 0..127
    const uint32_t chunk = t & 7u, rbase = t >> 3;
    uint32_t gst = 0;
    bool ok = true;
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
      auto issue = [&](uint32_t kb) -> bool {      // false: a wait ran out
        bool good = true;
        if (kb < num_kb) {
          const uint32_t g = gst + kb, s = g % kMtaXStages;
          if (g >= (uint32_t)kMtaXStages) good = mbar_wait(bar_x_empty(s), ((g / kMtaXStages) & 1u) ^ 1u, p.status, 3u, abort_flag);
          if (good) {
            const uint32_t dst0 = x_ring + s * L::kXBytes;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (!xrow[i]) continue;
              const uint32_t r = rbase + 16u * i;
              const uint32_t dst = dst0 + (r >> 3) * 1024u + (r & 7u) * 128u + ((chunk ^ (r & 7u)) << 4);
              asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(xrow[i] + (size_t)kb * kGemmBK) : "memory");
            }
          }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        return good;
      };
#pragma unroll
      for (int i = 0; i < kMtaLead; ++i) ok = ok && issue((uint32_t)i);
      for (uint32_t kb = 0; kb < num_kb; ++kb) {
        if (ok) ok = issue(kb + kMtaLead); else asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(kMtaLead) : "memory");   // this thread's pieces of stage kb have landed
        fence_proxy_async();              // each thread publishes its own pieces to the async proxy, then one lane signals
        __syncwarp();
        if ((t & 31u) == 0) mbar_arrive(bar_x_full((gst + kb) % kMtaXStages));   // (also on abort)
      }
      gst += num_kb;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else {
    // ================= epilogue: D[weight row][pair] in TMEM -> y rows of the pairs =================
    // A thread holds one weight row of 32 pairs, an output row wants 256 weight rows of one pair side by side: the tile
    // turns round in shared memory, 32 pairs at a time. Phase 1: every thread stores its 32 values as f16 into
    // stage[pair][weight row] (a warp's 32 lanes fill 64 consecutive bytes). Phase 2: a warp reads one pair's 512 bytes
    // (16 per lane) and stores them to the pair's output row in one instruction. The accumulators are free again as
    // soon as the last 32 pairs have been read, before their rows have left.
    const int quarter = warp & 3;
    const uint32_t r_half = (uint32_t)(quarter * 32 + lane);
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t stage = base + L::kOffStage;
    unsigned long long* const dst_tabs = reinterpret_cast<unsigned long long*>(gen_base + L::kOffDst);
    const uint4* const stage_g = reinterpret_cast<const uint4*>(gen_base + L::kOffStage);
    const bool vec_out = p.vec_out != 0u;
    for (uint32_t ui = 0; ui < my_units; ++ui) {
      uint32_t expert, r0, rows, n0;
      unit_of(ui, expert, r0, rows, n0);
      // where the output rows of this unit's pairs start: warp q looks up pairs 32 q .. 32 q + 31 while the unit's
      // MMAs are still running (two dependent global loads per pair); two tables, so a slow warp may still be reading
      // the previous unit's
      unsigned long long* const dst_tab = dst_tabs + (ui & 1u) * (uint32_t)kMtaNP;
      {
        const uint32_t col = (uint32_t)quarter * 32u + (uint32_t)lane;
        unsigned long long my_dst = 0ull;
        if (col < rows) {
          const uint32_t pr = p.sc.sorted[r0 + col];
          if (p.dst_index) {
            my_dst = reinterpret_cast<unsigned long long>(p.y_seg[pr / p.seg_cap] + (size_t)p.dst_index[pr] * p.out_tok_stride);
          } else {
            const uint32_t tk = pr / p.slots, sl = pr - tk * p.slots;
            my_dst = reinterpret_cast<unsigned long long>(p.Y + (size_t)tk * p.out_tok_stride + (size_t)sl * p.out_slot_stride);
          }
        }
        dst_tab[col] = my_dst;
      }
      const bool got = mbar_wait(bar_acc_full, ui & 1u, p.status, 5u, abort_flag, 400u);
      // the four warps leave together or not at all: none may be left alone at a barrier below
      if (!ep_bar_and(got)) break;
      tc_fence_after();
      const bool two = n0 + kMtaRows < p.N;
      const uint32_t ncb = (rows + 31u) / 32u;
      for (uint32_t cb = 0; cb < ncb; ++cb) {
        const uint32_t lim = min(32u, rows - cb * 32u);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (h == 1 && !two) break;                                   // warp-uniform
          uint32_t v[32];
          tmem_ld32(tmem_base + lane_base + (uint32_t)h * kMtaNP + cb * 32u, v);
          tmem_ld_wait();
          const uint32_t col = stage + ((uint32_t)h * kMtaRows + r_half) * 2u;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const unsigned short hv = __half_as_ushort(__float2half_rn(__uint_as_float(v[i])));
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(col + (uint32_t)i * (uint32_t)L::kStagePitch), "h"(hv) : "memory");
          }
        }
        if (cb + 1 == ncb) {       // the accumulators have been read: the next unit's MMAs may start
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_acc_empty);
        }
        ep_bar();
        // rows out: warp q takes pairs q, q + 4, ...; lane l the eight weight rows n0 + 8 l .. of the pair
        const uint32_t n = n0 + 8u * (uint32_t)lane;
        const bool mine = n < p.N && (two || lane < 16);               // N % 8 == 0: eight rows are in or out together
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t i = (uint32_t)quarter + 4u * (uint32_t)j;
          if (i >= lim) break;
          __half* const d = reinterpret_cast<__half*>(dst_tab[cb * 32u + i]) + n;
          if (mine) {
            const uint4 q = stage_g[i * (L::kStagePitch / 16) + lane];
            if (vec_out) {
              *reinterpret_cast<uint4*>(d) = q;
            } else {
              const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                d[2 * e] = __ushort_as_half((unsigned short)(w4[e] & 0xFFFFu));
                d[2 * e + 1] = __ushort_as_half((unsigned short)(w4[e] >> 16));
              }
            }
          }
        }
        ep_bar();                  // the stage is free for the next 32 pairs
      }
    }
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
  p.N = g.N; p.K = g.K; p.SPR = g.SPR; p.slots = slots; p.NB = (g.N + kMtaUnitRows - 1) / kMtaUnitRows;
  p.in_slot_stride = g.in_slot_stride; p.out_slot_stride = g.out_slot_stride;
  p.in_tok_stride = g.in_tok_stride; p.out_tok_stride = g.out_tok_stride;
  p.sc = sc; p.status = status;
  p.dst_index = g.dst_index; p.seg_cap = g.seg_cap ? g.seg_cap : 1u;
  for (int i = 0; i < 9; ++i) p.y_seg[i] = reinterpret_cast<__half*>(g.y_seg[i]);
  uintptr_t lowbits = ((uintptr_t)g.out_tok_stride | (uintptr_t)g.out_slot_stride) * 2u;
  if (g.dst_index) { for (int i = 0; i < 9; ++i) lowbits |= reinterpret_cast<uintptr_t>(g.y_seg[i]); }
  else lowbits |= reinterpret_cast<uintptr_t>(g.Y);
  p.vec_out = (lowbits & 15u) == 0 ? 1u : 0u;
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
