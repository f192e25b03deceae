// Persistent decode GEMV for 4-bit / group-64 weights, M = 1..8, with the warp-level matrix unit as the multiplier
// array (int4_matmul.gen.ts:170-571 for M = 1, :580-695 for the runtime-M matvec).
//
// Why this shape. At HBM rate one SM has to consume ~45 codes per clock. The CUDA-core paths top out near 54
// (M = 1) and pay M times the FMAs for M > 1; mma.sync.m16n8k16 multiplies 16 weight rows x 16 codes x 8 tokens per
// instruction (measured 73 codes/clk/SM with the unpack below), the same for every M <= 8. So the kernel is built
// around keeping the memory pipe full and the per-tile fixed work small:
//   * grid = one CTA per SM; CTA b owns the contiguous rows [b*N/G, (b+1)*N/G): perfectly balanced in bytes.
//   * K is cut in slices of 256 codes. Warp (ks, rg) owns slice ks of the current K tile (16 slices = 4096 codes)
//     and walks the CTA's 16-row tiles rg, rg+RG, ...; with K < 4096 the spare warps take other row tiles (RG > 1).
//     The activations of a slice live in registers as ready-made B fragments (32 registers), loaded once per K
//     tile: no shared-memory traffic for x at all.
//   * weights, scales and biases of a (tile, slice) -- 16 x 128 B + 16 x 16 B -- travel global -> shared with
//     per-lane cp.async into a ring of kTcDepth stages per warp (147 KB in flight per SM); no block-level barrier
//     is involved in the streaming itself.
//   * a nibble masked where it sits is an f16 subnormal (q * 2^-24 or q * 2^-20): the A fragments are 2 shifts and
//     8 ANDs per 16 codes, the products are exact, each 64-code group is summed inside the matrix unit and folded
//     into the f32 accumulators with round-to-nearest FMAs:  acc += s*2^24*lo + s*2^20*hi + b*sum(x).
//   * every kTcRounds rounds the K-slice partials of the warps meet in shared memory (double-buffered, one
//     __syncthreads per meeting, fixed summation order: results are deterministic).
#include <cstdlib>

#include "ztvm_device.cuh"
#include "ztvm_kernels.h"
#include "ztvm_stream_mma.cuh"

namespace ztvm {

constexpr uint32_t kTcMaxAccBytes = 32 * 1024;       // cross-K-tile accumulators (only when K > 4096)
// rounds between two meetings: the partial buffers hold 2 x warps x rounds x 16 rows x NT floats
__host__ __device__ constexpr int tc_rounds(int nt) { return nt <= 4 ? 4 : 2; }


// NT = tokens padded to a power of two. The eight columns of an MMA are (group, token) pairs: with NT tokens one
// accumulator collects GPA = 8 / NT scale groups side by side (the B fragment of a column is zero in the MMAs of the
// other groups), so the per-group fold after the MMAs is spread over the lanes of a quad instead of being repeated
// by each of them: lane (g, c) owns columns 2c and 2c + 1.
// W = warps per CTA: 16 (one CTA per SM, the whole shared memory as its ring) for projections that keep an SM busy for
// tens of microseconds; 8 (two CTAs fit an SM: registers and shared memory halve) for small ones, so that the CTAs of
// the NEXT launch in the stream -- already started under programmatic dependent launch -- sit beside this launch's and
// stream their first weights while it finishes, instead of waiting for the SM to empty.
template <int NT, bool AFFINE, int W>
__global__ void __launch_bounds__(W * 32, 16 / W)
gemv_tc_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t tc_smem[];
  constexpr int GPA = 8 / NT;                               // groups per accumulator (only 4 exist per tile)
  constexpr int NA = GPA >= 4 ? 1 : 4 / GPA;                // accumulators per tile
  constexpr int kTcRounds = tc_rounds(NT);                  // rounds between two meetings of the K-slice partials
  constexpr int kBlkRows = kTcRounds * 16;                  // rows a warp covers between two meetings
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;

  const uint32_t slices = p.K / kTcSlice;
  const uint32_t KS = slices < (uint32_t)W ? slices : (uint32_t)W;
  const uint32_t RG = (uint32_t)W / KS;
  const uint32_t ks = (uint32_t)warp % KS, rg = (uint32_t)warp / KS;
  const bool warp_active = rg < RG;
  const uint32_t num_kt = (slices + KS - 1) / KS;

  // Rows of this CTA. Plain form: the contiguous rows [r0, r0 + nrows). Paired form (gate rows, then up rows, in one
  // weight): the CTA owns output rows [r0, r0 + prows) and walks their gate and up tiles alternately -- tile 2j holds
  // gate rows r0 + 16 j .., tile 2j + 1 the up rows pair_rows further down -- so that both halves of an output meet in
  // the same block of rounds. `nrows` counts tile slots x 16 there.
  const bool paired = p.pair_rows != 0u;
  const uint32_t out_rows = paired ? p.pair_rows : p.N;
  const uint32_t r0 = (uint32_t)((uint64_t)blockIdx.x * out_rows / gridDim.x);
  const uint32_t r1 = (uint32_t)((uint64_t)(blockIdx.x + 1) * out_rows / gridDim.x);
  const uint32_t prows = r1 - r0;
  const uint32_t ntiles = paired ? 2u * ((prows + 15) / 16) : (prows + 15) / 16;
  const uint32_t nrows = paired ? ntiles * 16u : prows;
  // first weight row of the tile that starts at CTA-relative row `trow`, and how many of its 16 rows exist
  auto tile_row = [&](uint32_t trow) -> uint32_t {
    if (!paired) return r0 + trow;
    const uint32_t t = trow >> 4;
    return (t & 1u) * p.pair_rows + r0 + (t >> 1) * 16u;
  };
  auto tile_live = [&](uint32_t trow) -> uint32_t {
    const uint32_t first = paired ? (trow >> 5) * 16u : trow;
    return prows - first < 16u ? prows - first : 16u;
  };
  uint32_t rounds = (ntiles + RG - 1) / RG;
  rounds = (rounds + kTcRounds - 1) / kTcRounds * kTcRounds;
  const uint32_t total = num_kt * rounds;                   // (K tile, round) steps of every warp

  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(tc_smem) + (uint32_t)warp * (kTcDepth * kTcTileBytes);
  float* partial = reinterpret_cast<float*>(tc_smem + (W * kTcDepth * kTcTileBytes));            // [2][warps][kBlkRows][NT]
  float* acc_sm = partial + 2 * W * kBlkRows * NT;                       // [nrows][M], only if num_kt > 1

  // ---- producer side: one (tile, slice) per step, issued kTcDepth - 1 steps ahead ----------------------------
  const uint32_t cp_row = (uint32_t)lane >> 3, cp_chunk = (uint32_t)lane & 7;   // codes: 4 rows x 8 chunks per pass
  const uint32_t sb_row = (uint32_t)lane >> 1, sb_which = (uint32_t)lane & 1;   // scales / biases: 16 rows x 2
  const uint32_t cp_dst = cp_row * 128 + (((cp_chunk >> 1) ^ (cp_row & 3)) << 5) + ((cp_chunk & 1) << 4);
  const uint32_t sb_dst = kTcTileW + sb_row * 16 + sb_which * 8;
  const size_t row4 = (size_t)4 * p.KP;
  uint32_t i_step = 0, i_kt = 0, i_rd = 0;                  // the next step to issue, as (K tile, round)
  // Running addresses of this lane's pieces of the next tile (plain form: rows advance by RG tiles per round, slices
  // by KS per K tile), so a step costs a few adds instead of 64-bit multiplies; the paired form computes its rows.
  const uint32_t* const src_base = p.W + (size_t)(r0 + rg * 16 + cp_row) * p.KP + ks * 32 + cp_chunk * 4;
  const __half* const sb_base = (sb_which ? p.B : p.S) + (size_t)(r0 + rg * 16 + sb_row) * p.SPR + ks * 4;
  const size_t src_round = (size_t)RG * 16 * p.KP, sb_round = (size_t)RG * 16 * p.SPR;
  const uint32_t* src_run = src_base;
  const __half* sb_run = sb_base;
  uint32_t i_trow = rg * 16, i_slot = 0;
  auto issue = [&]() {
    if (warp_active && i_step < total) {
      const uint32_t sl = i_kt * KS + ks;
      const uint32_t trow = i_trow;                         // first row of the tile, CTA-relative
      if (sl < slices && trow < nrows) {
        const uint32_t st = ring + i_slot * kTcTileBytes;
        const uint32_t* src = src_run;
        const __half* sbp = sb_run;
        uint32_t live = nrows - trow < 16u ? nrows - trow : 16u;
        if (paired) {
          const uint32_t wrow = tile_row(trow);
          live = tile_live(trow);
          src = p.W + (size_t)(wrow + cp_row) * p.KP + sl * 32 + cp_chunk * 4;
          sbp = (sb_which ? p.B : p.S) + (size_t)(wrow + sb_row) * p.SPR + sl * 4;
        }
        if (live == 16u) {
#pragma unroll
          for (int i = 0; i < 4; ++i) tc_cp16(st + cp_dst + i * 512, src + i * row4);   // (row + 4i) & 3 == row & 3
          if (AFFINE || sb_which == 0) tc_cp8(st + sb_dst, sbp);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (cp_row + 4 * i < live) tc_cp16(st + cp_dst + i * 512, src + i * row4);
          if (sb_row < live && (AFFINE || sb_which == 0)) tc_cp8(st + sb_dst, sbp);
        }
      }
    }
    tc_commit();
    ++i_step;
    if (++i_slot == (uint32_t)kTcDepth) i_slot = 0;
    src_run += src_round; sb_run += sb_round; i_trow += RG * 16;
    if (++i_rd == rounds) {
      i_rd = 0; ++i_kt;
      i_trow = rg * 16;
      src_run = src_base + (size_t)i_kt * KS * 32;
      sb_run = sb_base + (size_t)i_kt * KS * 4;
    }
  };
#pragma unroll
  for (int i = 0; i < kTcDepth - 1; ++i) issue();

  // everything above reads only weights; activations and outputs belong to the stream order
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // B fragments of this warp's slice: column g of the MMA = (group jn within an accumulator, token tn)
  uint32_t xf[4][2][4];          // [group][word step][lo k0-7, lo k8-15, hi k0-7, hi k8-15]
  unsigned long long xs2[NA];    // sums of x over the groups that columns 2c, 2c + 1 of accumulator a stand for
  const int jn = g / NT, tn = g % NT;
  auto load_x = [&](uint32_t kt) {
    const uint32_t sl = kt * KS + ks;
    const bool tok_ok = warp_active && sl < slices && (uint32_t)tn < p.M;
    const __half* xr = p.X + (size_t)tn * p.x_row_stride + (size_t)sl * kTcSlice;
    float part[4];
#pragma unroll
    for (int tq = 0; tq < 4; ++tq) {
      const bool on = tok_ok && (tq % GPA) == jn;
      float sum = 0.f;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (on) raw = *reinterpret_cast<const uint4*>(xr + (8 * tq + 2 * c + u) * 8);
        // raw = (x0x1, x2x3, x4x5, x6x7) -> (x0x4, x2x6 | x1x5, x3x7): the pair order of the masked code words
        xf[tq][u][0] = __byte_perm(raw.x, raw.z, 0x5410);
        xf[tq][u][1] = __byte_perm(raw.y, raw.w, 0x5410);
        xf[tq][u][2] = __byte_perm(raw.x, raw.z, 0x7632);
        xf[tq][u][3] = __byte_perm(raw.y, raw.w, 0x7632);
        const float2 a = __half22float2(u32_as_h2(raw.x)), b = __half22float2(u32_as_h2(raw.y)),
                     d = __half22float2(u32_as_h2(raw.z)), e = __half22float2(u32_as_h2(raw.w));
        sum += ((a.x + a.y) + (b.x + b.y)) + ((d.x + d.y) + (e.x + e.y));
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);          // every lane of quad g: sum over group tq of token tn
      part[tq] = sum;
    }
#pragma unroll
    for (int a = 0; a < NA; ++a) {
      float r2[2];
#pragma unroll
      for (int v = 0; v < 2; ++v) {
        const int col = 2 * c + v, want = a * GPA + col / NT;   // the group this lane folds for that column
        float r = 0.f;
#pragma unroll
        for (int tq = 0; tq < 4; ++tq) {
          const float t = __shfl_sync(0xffffffffu, part[tq], col * 4);
          if (tq == want) r = t;
        }
        r2[v] = r;
      }
      xs2[a] = tc_pk(r2[0], r2[1]);
    }
  };
  load_x(0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  unsigned long long acc[kTcRounds][2];   // per round and row half: the two columns of this lane, packed
#pragma unroll
  for (int q = 0; q < kTcRounds; ++q) acc[q][0] = acc[q][1] = 0ull;
  const unsigned long long k16 = tc_pk(16.f, 16.f);
  const float kZero[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t swz = ((uint32_t)g & 3u);
  // where this lane finds the scale (and, 8 bytes on, the bias) of the group it folds, inside a row's 16 bytes
  const uint32_t sc_off = NT == 1 ? 4u * ((uint32_t)c & 1u) : NT == 2 ? 2u * (uint32_t)c : NT == 4 ? 2u * ((uint32_t)c >> 1) : 0u;

  uint32_t step = 0, meet = 0;   // meet: running count of meetings, its parity picks the partial buffer
  for (uint32_t kt = 0; kt < num_kt; ++kt) {
    if (kt) load_x(kt);
    const bool slice_ok = warp_active && kt * KS + ks < slices;
    for (uint32_t blk = 0; blk < rounds / kTcRounds; ++blk, ++meet) {
#pragma unroll
      for (int q = 0; q < kTcRounds; ++q, ++step) {
        issue();
        asm volatile("cp.async.wait_group %0;" ::"n"(kTcDepth - 1) : "memory");
        __syncwarp();
        const uint32_t trow = ((blk * kTcRounds + q) * RG + rg) * 16;
        if (slice_ok && trow < nrows) {
          const uint32_t st = ring + (step % kTcDepth) * kTcTileBytes;
          float clo[NA][4], chi[NA][4];
#pragma unroll
          for (int tq = 0; tq < 4; ++tq) {
            const int a = NA == 1 ? 0 : tq / GPA;
            const bool first = NA == 1 ? tq == 0 : (tq % GPA) == 0;
            const uint32_t off = (((uint32_t)tq ^ swz) << 5) + ((uint32_t)c << 3);
            const uint2 wg = tc_lds64(st + (uint32_t)g * 128 + off), wh = tc_lds64(st + (uint32_t)(g + 8) * 128 + off);
            {
              const Inplace4 cg = codes4_inplace(wg.x), ch = codes4_inplace(wh.x);   // rows g and g + 8
              if (first) {
                tc_mma(clo[a], cg.lo04, ch.lo04, cg.lo26, ch.lo26, xf[tq][0][0], xf[tq][0][1], kZero);
                tc_mma(chi[a], cg.hi15, ch.hi15, cg.hi37, ch.hi37, xf[tq][0][2], xf[tq][0][3], kZero);
              } else {
                tc_mma(clo[a], cg.lo04, ch.lo04, cg.lo26, ch.lo26, xf[tq][0][0], xf[tq][0][1], clo[a]);
                tc_mma(chi[a], cg.hi15, ch.hi15, cg.hi37, ch.hi37, xf[tq][0][2], xf[tq][0][3], chi[a]);
              }
            }
            {
              const Inplace4 cg = codes4_inplace(wg.y), ch = codes4_inplace(wh.y);
              tc_mma(clo[a], cg.lo04, ch.lo04, cg.lo26, ch.lo26, xf[tq][1][0], xf[tq][1][1], clo[a]);
              tc_mma(chi[a], cg.hi15, ch.hi15, cg.hi37, ch.hi37, xf[tq][1][2], xf[tq][1][3], chi[a]);
            }
          }
          // fold: column 2c + v of accumulator a is one (group, token); its scale and bias sit at sc_off (+ 8)
#pragma unroll
          for (int a = 0; a < NA; ++a)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t rowp = st + kTcTileW + (uint32_t)(g + 8 * h) * 16 + sc_off + (NT == 4 ? 4u * a : NT == 8 ? 2u * a : 0u);
              float s[2], b[2];
              if constexpr (NT == 1) {      // columns 2c, 2c + 1 are two groups
                const float2 s2 = __half22float2(u32_as_h2(tc_lds32(rowp)));
                s[0] = s2.x; s[1] = s2.y;
                if (AFFINE) {
                  const float2 b2 = __half22float2(u32_as_h2(tc_lds32(rowp + 8)));
                  b[0] = b2.x; b[1] = b2.y;
                }
              } else {                      // both columns belong to one group
                s[0] = s[1] = __half2float(__ushort_as_half((unsigned short)tc_lds16(rowp)));
                if (AFFINE) b[0] = b[1] = __half2float(__ushort_as_half((unsigned short)tc_lds16(rowp + 8)));
              }
              if (!AFFINE) { b[0] = -7.f * s[0]; b[1] = -7.f * s[1]; }
              // (2^24 lo + 2^20 hi) / 2^20, then the scale and the bias term, two columns per instruction
              const unsigned long long t2 = tc_ffma2(tc_pk(clo[a][2 * h], clo[a][2 * h + 1]), k16, tc_pk(chi[a][2 * h], chi[a][2 * h + 1]));
              unsigned long long r = acc[q][h];
              r = tc_ffma2(tc_pk(s[0] * 1048576.f, s[1] * 1048576.f), t2, r);
              r = tc_ffma2(tc_pk(b[0], b[1]), xs2[a], r);
              acc[q][h] = r;
            }
        }
        __syncwarp();   // every lane is done with the stage before the next issue refills it
      }
      // ---- meeting: K-slice partials of the block's rows -> shared, then one fixed-order sum per output --------
      float* mine = partial + ((size_t)((meet & 1u) * W + (uint32_t)warp) * kBlkRows) * NT;
#pragma unroll
      for (int q = 0; q < kTcRounds; ++q)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float2 av = tc_unpk(acc[q][h]);
          float v0 = slice_ok ? av.x : 0.f, v1 = slice_ok ? av.y : 0.f;
          acc[q][h] = 0ull;
          float* dst = mine + (q * 16 + g + 8 * h) * NT;
          if constexpr (NT == 1) {          // the quad's columns are groups of token 0
            v0 += v1;
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            if (c == 0) dst[0] = v0;
          } else if constexpr (NT == 2) {   // lane c holds group c of tokens 0, 1
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1); v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2); v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            if (c == 0) *reinterpret_cast<float2*>(dst) = make_float2(v0, v1);
          } else if constexpr (NT == 4) {   // lanes c and c ^ 2 hold the two groups of tokens 2(c & 1) + v
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2); v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            if (c < 2) *reinterpret_cast<float2*>(dst + 2 * c) = make_float2(v0, v1);
          } else {
            *reinterpret_cast<float2*>(dst + 2 * c) = make_float2(v0, v1);
          }
        }
      __syncthreads();
      const float* buf = partial + (size_t)(meet & 1u) * W * kBlkRows * NT;
      const uint32_t outs = (uint32_t)kTcRounds * RG * 16u * p.M;
      // the meeting's sums are taken by a different warp each time, so no warp falls behind the others for good
      for (uint32_t i = (threadIdx.x + (uint32_t)(W * 32) - 32u * (meet & (uint32_t)(W - 1))) & (uint32_t)(W * 32 - 1); i < outs; i += blockDim.x) {
        const uint32_t tok = i % p.M, br = i / p.M;           // br: row inside the block's R*RG tiles
        const uint32_t r16 = br & 15u, tb = br >> 4;
        const uint32_t q = tb / RG, rgi = tb - q * RG;
        const uint32_t row = ((blk * kTcRounds + q) * RG + rgi) * 16 + r16;
        if (row >= nrows || r16 >= tile_live(row & ~15u)) continue;
        float v = 0.f;
        for (uint32_t k2 = 0; k2 < KS; ++k2) v += buf[((size_t)(rgi * KS + k2) * kBlkRows + q * 16 + r16) * NT + tok];
        if (num_kt > 1) {
          float* a = acc_sm + (size_t)row * p.M + tok;
          if (kt) v += *a;
          if (kt + 1 < num_kt) { *a = v; continue; }
        }
        if (paired) {
          // The thread that holds an up row (odd tile) finishes the output: the gate row's sum is one tile back, in the
          // same block (tiles per block are even and blocks start on even tiles). Its own thread wrote nothing.
          const uint32_t tile = row >> 4;
          if ((tile & 1u) == 0u) continue;
          const uint32_t tg = tb - 1u, qg = tg / RG, rgg = tg - qg * RG;
          float gsum = 0.f;
          for (uint32_t k2 = 0; k2 < KS; ++k2) gsum += buf[((size_t)(rgg * KS + k2) * kBlkRows + qg * 16 + r16) * NT + tok];
          if (num_kt > 1 && kt) gsum += acc_sm[(size_t)(row - 16u) * p.M + tok];
          const float silu = gsum * (1.0f / (1.0f + expf(-gsum)));
          reinterpret_cast<__half*>(p.Y)[(size_t)tok * p.y_row_stride + r0 + (tile >> 1) * 16u + r16] = __float2half_rn(v * silu);
          continue;
        }
        const size_t o = (size_t)tok * p.y_row_stride + r0 + row;
        if (p.out_f32) {
          reinterpret_cast<float*>(p.Y)[o] = v;
          for (uint32_t k2 = 0; k2 < p.n_more; ++k2) reinterpret_cast<float*>(p.y_more[k2])[o] = v;   // peers (NVLink stores)
        } else {
          const __half hv = __float2half_rn(v);
          reinterpret_cast<__half*>(p.Y)[o] = hv;
          for (uint32_t k2 = 0; k2 < p.n_more; ++k2) reinterpret_cast<__half*>(p.y_more[k2])[o] = hv;
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---- host side --------------------------------------------------------------------------------------------
// Shared-memory accumulators (only when K spans several K tiles of W slices) must fit beside the ring.
static unsigned tc_grid_for(const GemvParams& p, int sm_count) {
  const uint32_t out_rows = p.pair_rows ? p.pair_rows : p.N;
  return out_rows < (uint32_t)sm_count ? out_rows : (unsigned)sm_count;
}
// rows of the cross-K-tile accumulators of one CTA (paired form: gate and up tile slots, 16 rows each)
static uint64_t tc_acc_rows(const GemvParams& p, unsigned grid) {
  const uint32_t out_rows = p.pair_rows ? p.pair_rows : p.N;
  const uint64_t rows = ((uint64_t)out_rows + grid - 1) / grid + 1;
  return p.pair_rows ? 2 * ((rows + 15) / 16) * 16 : rows;
}
static bool tc_acc_fits(const GemvParams& p, int sm_count, int warps) {
  const uint32_t slices = p.K / kTcSlice;
  if (slices <= (uint32_t)warps) return true;
  return tc_acc_rows(p, tc_grid_for(p, sm_count)) * p.M * 4 <= (warps == 8 ? kTcMaxAccBytes / 2 : kTcMaxAccBytes);
}
// warps per CTA for a problem: 8 (two CTAs per SM) while an SM's share of the weights is small, else 16
static int tc_warps_for(const GemvParams& p, int sm_count) {
  static const int forced = [] { const char* e = getenv("ZTVM_GEMV_WARPS"); return e ? atoi(e) : 0; }();   // measurement knob
  int w = 16;
  if (forced == 8 || forced == 16) w = forced;
  else if (p.K / kTcSlice <= 8u && (uint64_t)p.N * p.KP * 4 / (uint64_t)sm_count <= 384u * 1024u) w = 8;   // one K tile only
  if (w == 8 && !tc_acc_fits(p, sm_count, 8)) w = 16;
  return w;
}
bool gemv_tc_supported(const GemvParams& p, int bits, int sm_count) {
  if (bits != 4 || p.group_shift != 6 || p.M < 1 || p.M > 8) return false;
  if (p.pair_rows && (p.N != 2 * p.pair_rows || p.out_f32 || p.n_more)) return false;
  if (p.K % kTcSlice || p.K == 0 || p.N == 0) return false;
  if (p.x_row_stride % 8 || (reinterpret_cast<uintptr_t>(p.X) & 15u)) return false;
  if ((reinterpret_cast<uintptr_t>(p.W) & 15u) || (reinterpret_cast<uintptr_t>(p.S) & 7u) ||
      (p.B && (reinterpret_cast<uintptr_t>(p.B) & 7u)))
    return false;
  return tc_acc_fits(p, sm_count, tc_warps_for(p, sm_count));
}

template <int NT, bool AFFINE, int W>
static cudaError_t launch_tc_one(const GemvParams& p, unsigned grid, size_t smem, cudaStream_t st) {
  auto kern = gemv_tc_kernel<NT, AFFINE, W>;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, W == 16 ? 227 * 1024 : 112 * 1024);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(W * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  static const bool no_pdl = [] { const char* e = getenv("ZTVM_NO_PDL"); return e && e[0] == '1'; }();   // measurement knob
  cfg.numAttrs = no_pdl ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int W>
static cudaError_t launch_tc_w(const GemvParams& p, int sm_count, cudaStream_t st) {
  const unsigned grid = tc_grid_for(p, sm_count);
  const int nt = p.M == 1 ? 1 : p.M == 2 ? 2 : p.M <= 4 ? 4 : 8;
  size_t smem = (size_t)W * kTcDepth * kTcTileBytes + (size_t)2 * W * tc_rounds(nt) * 16 * nt * 4;
  if (p.K / kTcSlice > (uint32_t)W) smem += (size_t)tc_acc_rows(p, grid) * p.M * 4;
  const bool affine = p.B != nullptr;
  switch (nt) {
    case 1: return affine ? launch_tc_one<1, true, W>(p, grid, smem, st) : launch_tc_one<1, false, W>(p, grid, smem, st);
    case 2: return affine ? launch_tc_one<2, true, W>(p, grid, smem, st) : launch_tc_one<2, false, W>(p, grid, smem, st);
    case 4: return affine ? launch_tc_one<4, true, W>(p, grid, smem, st) : launch_tc_one<4, false, W>(p, grid, smem, st);
    default: return affine ? launch_tc_one<8, true, W>(p, grid, smem, st) : launch_tc_one<8, false, W>(p, grid, smem, st);
  }
}

cudaError_t launch_gemv_tc(const GemvParams& p, int sm_count, cudaStream_t st) {
  return tc_warps_for(p, sm_count) == 8 ? launch_tc_w<8>(p, sm_count, st) : launch_tc_w<16>(p, sm_count, st);
}

}  // namespace ztvm
