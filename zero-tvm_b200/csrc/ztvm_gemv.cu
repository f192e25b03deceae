// Decode GEMV (M = 1..8) for packed 4-bit / 3-bit group-quantised weights, and its
// ids-indirect MoE form. HBM-bound by design: every weight word is read once with 128-bit
// streaming loads, dequantised in registers, accumulated in f32 and reduced with warp
// shuffles. No tensor cores.
//
// Arithmetic (src/compiler/shaders/int4_matmul.gen.ts:78-96, :388-464): for a run of codes that
// shares one (scale, bias) pair,  sum x_i*(s*q_i + b) = s * sum x_i*q_i + b * sum x_i.  The
// products x_i*q_i are formed in f32 from exact integer codes, so the only roundings are the
// f32 accumulations. The symmetric flavour w = s*(q-7) is the same expression with b = -7*s.
//
// Work split: a "unit" is 32 consecutive codes of one row (4 words at 4 bits, 3 words at 3
// bits); lane l of a warp owns units l, l+32, ... of each of the ROWS rows the warp is
// responsible for, and keeps the matching 32 activations (per batch row) in registers across
// those rows. Activations are staged once per CTA in shared memory as f32 in a lane-interleaved
// order, so the 128-bit shared loads are conflict-free.
#include "ztvm_device.cuh"
#include "ztvm_kernels.h"

namespace ztvm {

constexpr int kGemvWarps = 4;          // warps per CTA
constexpr int kGemvTileElems = 16384;  // f32 activation elements staged per K tile (64 KB)

// shared layout of one staged activation row of `units` units: float4 (j, u) -> [(u/32)*256 + j*32 + u%32]
__device__ __forceinline__ int xs_f4_index(int u, int j) { return ((u >> 5) << 8) + (j << 5) + (u & 31); }

template <int BITS, int MT, int ROWS, bool MOE>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_kernel(const GemvParams p) {
  extern __shared__ float4 smem_f4[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  constexpr int WPU = BITS;  // words per 32-code unit: 8 bits -> 8, 4 bits -> 4, 3 bits -> 3

  const uint32_t* __restrict__ W = p.W;
  const __half* __restrict__ S = p.S;
  const __half* __restrict__ Bv = p.B;
  const __half* __restrict__ X = p.X;
  size_t out_base = 0;
  if (MOE) {
    const uint32_t token = blockIdx.y, slot = blockIdx.z;
    const uint32_t expert = p.ids[(size_t)token * p.ids_stride + slot];
    if (expert >= p.experts) {
      if (threadIdx.x == 0 && blockIdx.x == 0) atomicAdd(p.err_counter, 1u);
      return;
    }
    W += (size_t)expert * p.N * p.KP;
    S += (size_t)expert * p.N * p.SPR;
    if (Bv) Bv += (size_t)expert * p.N * p.SPR;
    X += (size_t)token * p.in_tok_stride + (size_t)slot * p.in_slot_stride;
    out_base = (size_t)token * p.out_tok_stride + (size_t)slot * p.out_slot_stride;
  }

  const uint32_t row0 = (blockIdx.x * kGemvWarps + warp) * ROWS;
  const uint32_t units = p.K >> 5;
  const uint32_t tile_units = p.tile_units;  // multiple of 32
  const int gshift = p.group_shift - 5;      // unit index -> group index (group >= 32)

  // per-row bases (rows past N are clamped for the loads and masked at the store)
  const uint32_t* wrow[ROWS];
  const __half* srow[ROWS];
  const __half* brow[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    uint32_t row = min(row0 + r, p.N - 1);
    wrow[r] = W + (size_t)row * p.KP;
    srow[r] = S + (size_t)row * p.SPR;
    brow[r] = Bv ? Bv + (size_t)row * p.SPR : nullptr;
  }

  float acc[ROWS][MT];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[r][m] = 0.f;

  float* xsum_sm = reinterpret_cast<float*>(smem_f4 + (size_t)MT * tile_units * 8);  // [MT][tile_units]

  for (uint32_t tu0 = 0; tu0 < units; tu0 += tile_units) {
    const uint32_t tu = min(tile_units, units - tu0);
    if (tu0) __syncthreads();  // previous tile fully consumed
    // ---- stage activations: f16 global -> f32 shared, 8 elements per thread-step --------
    for (uint32_t i = threadIdx.x; i < MT * tu * 4; i += blockDim.x) {
      const uint32_t m = i / (tu * 4), rem = i - m * tu * 4;
      const uint32_t u = rem >> 2, j2 = rem & 3;  // unit, pair of float4 within the unit
      float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
      if (m < p.M) {
        const uint4 raw = *reinterpret_cast<const uint4*>(X + (size_t)m * p.x_row_stride + ((size_t)(tu0 + u) << 5) + (j2 << 3));
        const float2 a = __half22float2(u32_as_h2(raw.x)), b = __half22float2(u32_as_h2(raw.y)),
                     c = __half22float2(u32_as_h2(raw.z)), d = __half22float2(u32_as_h2(raw.w));
        lo = make_float4(a.x, a.y, b.x, b.y);
        hi = make_float4(c.x, c.y, d.x, d.y);
      }
      float4* dst = smem_f4 + (size_t)m * tile_units * 8;
      dst[xs_f4_index(u, 2 * j2)] = lo;
      dst[xs_f4_index(u, 2 * j2 + 1)] = hi;
    }
    __syncthreads();
    // ---- per-unit activation sums (the bias term's multiplier) ----------------------------
    for (uint32_t i = threadIdx.x; i < MT * tu; i += blockDim.x) {
      const uint32_t m = i / tu, u = i - m * tu;
      const float4* src = smem_f4 + (size_t)m * tile_units * 8;
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 v = src[xs_f4_index(u, j)];
        s += (v.x + v.y) + (v.z + v.w);
      }
      xsum_sm[m * tile_units + u] = s;
    }
    __syncthreads();

    // ---- stream the weights ---------------------------------------------------------------
    for (uint32_t it = lane; it < tu; it += 32) {
      const uint32_t u = tu0 + it;
      uint32_t w[ROWS][WPU];
      float sc[ROWS], bi[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        if constexpr (BITS == 4) {
          const uint4 v = ld_stream_u4(wrow[r] + (size_t)u * 4);
          w[r][0] = v.x; w[r][1] = v.y; w[r][2] = v.z; w[r][3] = v.w;
        } else if constexpr (BITS == 8) {
          const uint4 v0 = ld_stream_u4(wrow[r] + (size_t)u * 8), v1 = ld_stream_u4(wrow[r] + (size_t)u * 8 + 4);
          w[r][0] = v0.x; w[r][1] = v0.y; w[r][2] = v0.z; w[r][3] = v0.w;
          w[r][4] = v1.x; w[r][5] = v1.y; w[r][6] = v1.z; w[r][7] = v1.w;
        } else {
#pragma unroll
          for (int k = 0; k < WPU; ++k) w[r][k] = ld_stream_u32(wrow[r] + (size_t)u * 3 + k);
        }
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const uint32_t g = u >> gshift;
        sc[r] = ld_f16_as_f32(srow[r] + g);
        bi[r] = brow[r] ? ld_f16_as_f32(brow[r] + g) : -7.0f * sc[r];
      }
      float d[ROWS][MT];
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int m = 0; m < MT; ++m) d[r][m] = 0.f;

#pragma unroll
      for (int j = 0; j < 4; ++j) {  // four 8-code blocks of the unit
        float xv[MT][8];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const float4* src = smem_f4 + (size_t)m * tile_units * 8;
          const float4 a = src[xs_f4_index(it, 2 * j)], b = src[xs_f4_index(it, 2 * j + 1)];
          xv[m][0] = a.x; xv[m][1] = a.y; xv[m][2] = a.z; xv[m][3] = a.w;
          xv[m][4] = b.x; xv[m][5] = b.y; xv[m][6] = b.z; xv[m][7] = b.w;
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          float q[8];
          if constexpr (BITS == 4) codes4_f32(w[r][j], q);
          else if constexpr (BITS == 8) codes8_f32(w[r][2 * j], w[r][2 * j + 1], q);
          else codes3_f32(window3(w[r][0], w[r][1], w[r][2], j), q);
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            float t = d[r][m];
#pragma unroll
            for (int i = 0; i < 8; ++i) t = fmaf(xv[m][i], q[i], t);
            d[r][m] = t;
          }
        }
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float xs = xsum_sm[m * tile_units + it];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r][m] = fmaf(bi[r], xs, fmaf(sc[r], d[r][m], acc[r][m]));
      }
    }
  }

  // ---- reduce across the warp and store ------------------------------------------------------
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const float v = warp_sum(acc[r][m]);
      const uint32_t row = row0 + r;
      if (lane == 0 && row < p.N && (uint32_t)m < p.M) {
        const size_t o = MOE ? out_base + row : (size_t)m * p.y_row_stride + row;
        if (p.out_f32) reinterpret_cast<float*>(p.Y)[o] = v;
        else reinterpret_cast<__half*>(p.Y)[o] = __float2half_rn(v);
      }
    }
}

// ---- M = 1, 4-bit: f16 x f16 -> f32 FMAs on codes masked in place ---------------------------------
// A nibble masked where it sits, (w & 0x000F000F) / (w & 0x00F000F0), is a pair of f16 subnormals
// q * 2^-24 / q * 2^-20. fma.rn.f32.f16 multiplies two f16 operands exactly and accumulates in f32 with
// round-to-nearest, so no conversion instruction is needed at all: per 8 codes one shift, four ANDs and
// eight FMAs. The two power-of-two classes accumulate separately and are folded into the scale.
// Activations stay f16 in shared memory, each 8-block permuted to (x0,x4)(x1,x5)(x2,x6)(x3,x7) so that
// register halves line up with the masked code pairs.
__device__ __forceinline__ float fma_f16_lo(uint32_t xp, uint32_t qp, float acc) {
  unsigned short xl, xh, ql, qh;
  asm("mov.b32 {%0,%1}, %2;" : "=h"(xl), "=h"(xh) : "r"(xp));
  asm("mov.b32 {%0,%1}, %2;" : "=h"(ql), "=h"(qh) : "r"(qp));
  asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(xl), "h"(ql));
  return acc;
}
__device__ __forceinline__ float fma_f16_hi(uint32_t xp, uint32_t qp, float acc) {
  unsigned short xl, xh, ql, qh;
  asm("mov.b32 {%0,%1}, %2;" : "=h"(xl), "=h"(xh) : "r"(xp));
  asm("mov.b32 {%0,%1}, %2;" : "=h"(ql), "=h"(qh) : "r"(qp));
  asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(xh), "h"(qh));
  return acc;
}

// shared layout: 16-byte item (unit u, word j) at [(u/32)*128 + j*32 + u%32]
__device__ __forceinline__ int xh_index(int u, int j) { return ((u >> 5) << 7) + (j << 5) + (u & 31); }

template <int ROWS, bool MOE>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_fma_m1_kernel(const GemvParams p) {
  extern __shared__ float4 smem_f4[];
  uint4* xsm = reinterpret_cast<uint4*>(smem_f4);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  const uint32_t* __restrict__ W = p.W;
  const __half* __restrict__ S = p.S;
  const __half* __restrict__ Bv = p.B;
  const __half* __restrict__ X = p.X;
  size_t out_base = 0;
  if (MOE) {
    const uint32_t token = blockIdx.y, slot = blockIdx.z;
    const uint32_t expert = p.ids[(size_t)token * p.ids_stride + slot];
    if (expert >= p.experts) {
      if (threadIdx.x == 0 && blockIdx.x == 0) atomicAdd(p.err_counter, 1u);
      return;
    }
    W += (size_t)expert * p.N * p.KP;
    S += (size_t)expert * p.N * p.SPR;
    if (Bv) Bv += (size_t)expert * p.N * p.SPR;
    X += (size_t)token * p.in_tok_stride + (size_t)slot * p.in_slot_stride;
    out_base = (size_t)token * p.out_tok_stride + (size_t)slot * p.out_slot_stride;
  }
  const uint32_t row0 = (blockIdx.x * kGemvWarps + warp) * ROWS;
  const uint32_t units = p.K >> 5;
  const uint32_t units_up = (units + 31) & ~31u;
  const int gshift = p.group_shift - 5;
  const uint32_t* wrow[ROWS];
  const __half* srow[ROWS];
  const __half* brow[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const uint32_t row = min(row0 + r, p.N - 1);
    wrow[r] = W + (size_t)row * p.KP;
    srow[r] = S + (size_t)row * p.SPR;
    brow[r] = Bv ? Bv + (size_t)row * p.SPR : nullptr;
  }
  // first round of weights goes out before the activations are staged
  uint4 wcur[ROWS];
  {
    const uint32_t u = min((uint32_t)lane, units - 1);
#pragma unroll
    for (int r = 0; r < ROWS; ++r) wcur[r] = ld_stream_u4(wrow[r] + (size_t)u * 4);
  }
  float* xsum_sm = reinterpret_cast<float*>(xsm + (size_t)units_up * 4);
  for (uint32_t i = threadIdx.x; i < units * 4; i += blockDim.x) {
    const uint32_t u = i >> 2, j = i & 3;
    const uint4 raw = *reinterpret_cast<const uint4*>(X + ((size_t)u << 5) + (j << 3));
    uint4 o;  // (x0x1,x2x3,x4x5,x6x7) -> (x0x4, x1x5, x2x6, x3x7)
    o.x = __byte_perm(raw.x, raw.z, 0x5410);
    o.y = __byte_perm(raw.x, raw.z, 0x7632);
    o.z = __byte_perm(raw.y, raw.w, 0x5410);
    o.w = __byte_perm(raw.y, raw.w, 0x7632);
    xsm[xh_index(u, j)] = o;
  }
  __syncthreads();
  for (uint32_t u = threadIdx.x; u < units; u += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 v = xsm[xh_index(u, j)];
      const float2 a = __half22float2(u32_as_h2(v.x)), b = __half22float2(u32_as_h2(v.y)),
                   c = __half22float2(u32_as_h2(v.z)), d = __half22float2(u32_as_h2(v.w));
      s += ((a.x + a.y) + (b.x + b.y)) + ((c.x + c.y) + (d.x + d.y));
    }
    xsum_sm[u] = s;
  }
  __syncthreads();

  float acc[ROWS];
#pragma unroll
  for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;

  for (uint32_t u = lane; u < units; u += 32) {
    uint4 wnext[ROWS];
    {
      const uint32_t un = min(u + 32, units - 1);
#pragma unroll
      for (int r = 0; r < ROWS; ++r) wnext[r] = ld_stream_u4(wrow[r] + (size_t)un * 4);
    }
    float sc[ROWS], bi[ROWS];
    const uint32_t grp = u >> gshift;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      sc[r] = ld_f16_as_f32(srow[r] + grp);
      bi[r] = brow[r] ? ld_f16_as_f32(brow[r] + grp) : -7.0f * sc[r];
    }
    float dlo[ROWS], dhi[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) dlo[r] = dhi[r] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 xp = xsm[xh_index(u, j)];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const uint32_t w = j == 0 ? wcur[r].x : j == 1 ? wcur[r].y : j == 2 ? wcur[r].z : wcur[r].w;
        const Inplace4 ip = codes4_inplace(w);
        const uint32_t a0 = ip.lo04, a1 = ip.hi15, a2 = ip.lo26, a3 = ip.hi37;
        float lo = dlo[r], hi = dhi[r];
        lo = fma_f16_lo(xp.x, a0, lo); lo = fma_f16_hi(xp.x, a0, lo);   // x0*q0, x4*q4
        hi = fma_f16_lo(xp.y, a1, hi); hi = fma_f16_hi(xp.y, a1, hi);   // x1*q1, x5*q5
        lo = fma_f16_lo(xp.z, a2, lo); lo = fma_f16_hi(xp.z, a2, lo);   // x2*q2, x6*q6
        hi = fma_f16_lo(xp.w, a3, hi); hi = fma_f16_hi(xp.w, a3, hi);   // x3*q3, x7*q7
        dlo[r] = lo; dhi[r] = hi;
      }
    }
    const float xs = xsum_sm[u];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      float a = acc[r];
      a = fmaf(sc[r] * 16777216.f, dlo[r], a);
      a = fmaf(sc[r] * 1048576.f, dhi[r], a);
      acc[r] = fmaf(bi[r], xs, a);
      wcur[r] = wnext[r];
    }
  }
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const float v = warp_sum(acc[r]);
    const uint32_t row = row0 + r;
    if (lane == 0 && row < p.N) {
      const size_t o = MOE ? out_base + row : (size_t)row;
      if (p.out_f32) reinterpret_cast<float*>(p.Y)[o] = v;
      else reinterpret_cast<__half*>(p.Y)[o] = __float2half_rn(v);
    }
  }
}

// ---- M = 1, 4-bit, dense: persistent form ----------------------------------------------------------
// One CTA per SM slot (grid = 2 x SM count): the CTA owns a contiguous slice of the output rows, stages
// the activation vector ONCE, and its eight warps walk their sub-slices in steps of ROWS rows. Loads of
// step i+1 (weights, scale, bias) are in flight while step i is multiplied. The kernel is written for
// programmatic dependent launch: everything that does not depend on the previous kernel in the stream
// (the first weight loads) is issued before griddepcontrol.wait; activations are read and outputs are
// written only after it, and dependents are released as soon as the activations are staged.
constexpr int kPersistWarps = 8;

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Weights travel global -> shared with per-lane 16-byte cp.async copies into a ring of DEPTH stages per
// warp: the bytes in flight are bounded by shared memory (DEPTH x ROWS x 512 B per warp), not by
// registers, and a lane only ever reads back the slots it filled itself, so no barrier is involved.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int ROWS, int DEPTH>
__global__ void __launch_bounds__(kPersistWarps * 32, 2)
gemv_fma_m1_persist_kernel(const GemvParams p) {
  extern __shared__ float4 smem_f4[];
  uint4* xsm = reinterpret_cast<uint4*>(smem_f4);
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const uint32_t units = p.K >> 5;
  const uint32_t units_up = (units + 31) & ~31u;
  const uint32_t ipr = units_up >> 5;  // lane iterations per row
  const int gshift = p.group_shift - 5;
  float* xsum_sm = reinterpret_cast<float*>(xsm + (size_t)units_up * 4);
  // ring[warp][stage][row][lane]
  uint4* ring = reinterpret_cast<uint4*>(xsum_sm + units_up) + (size_t)warp * DEPTH * ROWS * 32 + lane;

  // rows of this CTA, then of this warp
  const uint32_t cta_lo = (uint32_t)(((uint64_t)p.N * blockIdx.x) / gridDim.x);
  const uint32_t cta_hi = (uint32_t)(((uint64_t)p.N * (blockIdx.x + 1)) / gridDim.x);
  const uint32_t cnt = cta_hi - cta_lo;
  const uint32_t r_lo = cta_lo + (cnt * warp) / kPersistWarps;
  const uint32_t r_hi = cta_lo + (cnt * (warp + 1)) / kPersistWarps;
  const uint32_t nsteps = (r_hi - r_lo + ROWS - 1) / ROWS;
  const uint32_t total = nsteps * ipr;

  const uint16_t* S16 = reinterpret_cast<const uint16_t*>(p.S);
  const uint16_t* B16 = reinterpret_cast<const uint16_t*>(p.B);
  // Three cursors walk the same flattened (row step, lane iteration) sequence: weights DEPTH-1 ahead,
  // scale/bias two ahead, and the multiply. Each keeps its own counters, advanced without divisions.
  struct Cursor {
    uint32_t it, ui, row[ROWS];
  };
  auto cursor_rows = [&](Cursor& c, uint32_t step) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) c.row[r] = min(r_lo + step * ROWS + r, r_hi - 1);
  };
  auto cursor_next = [&](Cursor& c) {
    ++c.it;
    if (++c.ui == ipr) {
      c.ui = 0;
      if (c.it < total) {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) c.row[r] = min(c.row[r] + ROWS, r_hi - 1);
      }
    }
  };
  Cursor cw, cs;
  cw.it = cw.ui = cs.it = cs.ui = 0;
  if (total) { cursor_rows(cw, 0); cursor_rows(cs, 0); }
  uint32_t wslot = 0;  // ring slot the weight cursor fills next
  // one commit group per flattened iteration (empty past the end, so the group count stays uniform)
  auto issue_w = [&]() {
    if (cw.it < total) {
      const uint32_t u = min(cw.ui * 32 + lane, units - 1);
      uint4* slot = ring + (size_t)wslot * ROWS * 32;
#pragma unroll
      for (int r = 0; r < ROWS; ++r) cp_async16(slot + r * 32, p.W + (size_t)cw.row[r] * p.KP + (size_t)u * 4);
      cursor_next(cw);
    }
    wslot = wslot + 1 == DEPTH ? 0 : wslot + 1;
    cp_async_commit();
  };
  struct SB { uint32_t s[ROWS], b[ROWS]; };  // raw f16 bits
  auto issue_sb = [&](SB& f) {
    if (cs.it >= total) return;
    const uint32_t grp = min(cs.ui * 32 + lane, units - 1) >> gshift;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      f.s[r] = __ldg(S16 + (size_t)cs.row[r] * p.SPR + grp);
      f.b[r] = B16 ? (uint32_t)__ldg(B16 + (size_t)cs.row[r] * p.SPR + grp) : 0u;
    }
    cursor_next(cs);
  };

  // weights, scales and biases do not depend on the previous kernel: fill the ring before waiting on it
#pragma unroll
  for (int d = 0; d < DEPTH - 1; ++d) issue_w();
  SB sb0, sb1;
  issue_sb(sb0);
  issue_sb(sb1);

  pdl_wait();  // the previous kernel in the stream may have produced the activations
  // ---- stage activations (f16, pair-permuted) and their per-unit sums ---------------------------------
  {
    const uint32_t one2 = 0x3C003C00u;  // (1.0, 1.0) in f16
    for (uint32_t i = threadIdx.x; i < units_up * 4; i += blockDim.x) {
      const uint32_t u = i >> 2, j = i & 3;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (u < units) raw = *reinterpret_cast<const uint4*>(p.X + ((size_t)u << 5) + (j << 3));
      uint4 o;  // (x0x1,x2x3,x4x5,x6x7) -> (x0x4, x1x5, x2x6, x3x7)
      o.x = __byte_perm(raw.x, raw.z, 0x5410);
      o.y = __byte_perm(raw.x, raw.z, 0x7632);
      o.z = __byte_perm(raw.y, raw.w, 0x5410);
      o.w = __byte_perm(raw.y, raw.w, 0x7632);
      xsm[xh_index(u, j)] = o;
      // sum of the 8 values in f32 (x * 1.0 accumulated), then over the 4 blocks of the unit
      float sx = 0.f;
      sx = fma_f16_lo(o.x, one2, sx); sx = fma_f16_hi(o.x, one2, sx);
      sx = fma_f16_lo(o.y, one2, sx); sx = fma_f16_hi(o.y, one2, sx);
      sx = fma_f16_lo(o.z, one2, sx); sx = fma_f16_hi(o.z, one2, sx);
      sx = fma_f16_lo(o.w, one2, sx); sx = fma_f16_hi(o.w, one2, sx);
      sx += __shfl_xor_sync(0xffffffffu, sx, 1);
      sx += __shfl_xor_sync(0xffffffffu, sx, 2);
      if (j == 0) xsum_sm[u] = sx;
    }
  }
  __syncthreads();
  pdl_launch_dependents();

  float acc[ROWS];
  uint32_t cslot = 0, row_out = r_lo;
  for (uint32_t step = 0; step < nsteps; ++step, row_out += ROWS) {
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
    for (uint32_t ui = 0; ui < ipr; ++ui) {
      issue_w();
      SB sb2;
      issue_sb(sb2);
      cp_async_wait<DEPTH - 1>();  // the group of this iteration has landed
      const uint32_t u = ui * 32 + lane;
      if (u < units) {
        const uint4* slot = ring + (size_t)cslot * ROWS * 32;
        uint4 wv[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) wv[r] = slot[r * 32];
        float dlo[ROWS], dhi[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) dlo[r] = dhi[r] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 xp = xsm[xh_index(u, j)];
#pragma unroll
          for (int r = 0; r < ROWS; ++r) {
            const uint32_t w = j == 0 ? wv[r].x : j == 1 ? wv[r].y : j == 2 ? wv[r].z : wv[r].w;
            const Inplace4 ip = codes4_inplace(w);
            const uint32_t a0 = ip.lo04, a1 = ip.hi15, a2 = ip.lo26, a3 = ip.hi37;
            float lo = dlo[r], hi = dhi[r];
            lo = fma_f16_lo(xp.x, a0, lo); lo = fma_f16_hi(xp.x, a0, lo);
            hi = fma_f16_lo(xp.y, a1, hi); hi = fma_f16_hi(xp.y, a1, hi);
            lo = fma_f16_lo(xp.z, a2, lo); lo = fma_f16_hi(xp.z, a2, lo);
            hi = fma_f16_lo(xp.w, a3, hi); hi = fma_f16_hi(xp.w, a3, hi);
            dlo[r] = lo; dhi[r] = hi;
          }
        }
        const float xs = xsum_sm[u];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          const float sc = __half2float(__ushort_as_half((unsigned short)sb0.s[r]));
          const float bias = B16 ? __half2float(__ushort_as_half((unsigned short)sb0.b[r])) : -7.0f * sc;
          const float d = fmaf(dlo[r], 16.f, dhi[r]);           // in units of 2^-20
          acc[r] = fmaf(bias, xs, fmaf(sc * 1048576.f, d, acc[r]));
        }
      }
      cslot = cslot + 1 == DEPTH ? 0 : cslot + 1;
      sb0 = sb1; sb1 = sb2;
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float v = warp_sum(acc[r]);
      const uint32_t row = row_out + r;
      if (lane == 0 && row < r_hi) {
        if (p.out_f32) reinterpret_cast<float*>(p.Y)[row] = v;
        else reinterpret_cast<__half*>(p.Y)[row] = __float2half_rn(v);
      }
    }
  }
  cp_async_wait<0>();
}

// ---- host-side launch ------------------------------------------------------------------------
template <int BITS, int MT, int ROWS, bool MOE>
static cudaError_t launch_one(const GemvParams& p, dim3 grid, size_t smem, cudaStream_t st) {
  auto kern = gemv_kernel<BITS, MT, ROWS, MOE>;
  static bool attr_set[16] = {};  // per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  kern<<<grid, kGemvWarps * 32, smem, st>>>(p);
  return cudaGetLastError();
}

template <int ROWS, bool MOE>
static cudaError_t launch_fma_m1(const GemvParams& p, dim3 grid, cudaStream_t st) {
  auto kern = gemv_fma_m1_kernel<ROWS, MOE>;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const uint32_t units = p.K >> 5, units_up = (units + 31) & ~31u;
  const size_t smem = (size_t)units_up * 64 + (size_t)units_up * 4;
  kern<<<grid, kGemvWarps * 32, smem, st>>>(p);
  return cudaGetLastError();
}

template <int ROWS, int DEPTH>
static cudaError_t launch_fma_m1_persist(const GemvParams& p, int sm_count, cudaStream_t st) {
  auto kern = gemv_fma_m1_persist_kernel<ROWS, DEPTH>;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  const uint32_t units = p.K >> 5, units_up = (units + 31) & ~31u;
  const size_t smem = (size_t)units_up * 64 + (size_t)units_up * 4 + (size_t)kPersistWarps * DEPTH * ROWS * 512;
  // One or two CTAs per SM, whichever wastes fewer of the ROWS-row steps on the warps' last, partial step.
  auto efficiency = [&](uint32_t ctas) {
    const double rpw = (double)p.N / ((double)ctas * kPersistWarps);
    const double steps = (double)((uint32_t)((rpw + ROWS - 1e-9) / ROWS) + 0);
    return rpw / ((steps < 1 ? 1 : steps) * ROWS);
  };
  uint32_t grid = efficiency((uint32_t)sm_count * 2) + 0.15 >= efficiency((uint32_t)sm_count) ? (uint32_t)sm_count * 2
                                                                                              : (uint32_t)sm_count;
  const uint32_t max_ctas = (p.N + kPersistWarps - 1) / kPersistWarps;  // at least one row per warp
  if (grid > max_ctas) grid = max_ctas;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kPersistWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int BITS, int MT, bool MOE>
static cudaError_t launch_rows(const GemvParams& p, int rows, dim3 grid, size_t smem, cudaStream_t st) {
  if (rows == 4) return launch_one<BITS, MT, 4, MOE>(p, grid, smem, st);
  if (rows == 2) return launch_one<BITS, MT, 2, MOE>(p, grid, smem, st);
  return launch_one<BITS, MT, 1, MOE>(p, grid, smem, st);
}

cudaError_t launch_gemv(GemvParams p, int bits, bool moe, uint32_t tokens, uint32_t slots, int sm_count,
                        cudaStream_t st) {
  const int mt = p.M <= 1 ? 1 : p.M <= 2 ? 2 : p.M <= 4 ? 4 : 8;
  // rows per warp: 4 when that still leaves every SM several CTAs, else fewer
  const uint64_t pairs = moe ? (uint64_t)tokens * slots : 1;
  int rows = 4;
  while (rows > 1 && ((uint64_t)(p.N + kGemvWarps * rows - 1) / (kGemvWarps * rows)) * pairs < (uint64_t)sm_count * 4)
    rows >>= 1;
  if ((mt == 8 || bits == 8) && rows > 2) rows = 2;  // register pressure
  const uint32_t units = p.K >> 5;
  uint32_t tile_units = (uint32_t)(kGemvTileElems / mt) >> 5;
  const uint32_t units_up = (units + 31) & ~31u;
  if (tile_units > units_up) tile_units = units_up;
  p.tile_units = tile_units;
  const size_t smem = (size_t)mt * tile_units * (128 + 4);
  dim3 grid((p.N + kGemvWarps * rows - 1) / (kGemvWarps * rows), moe ? tokens : 1, moe ? slots : 1);
  if (bits == 4 && mt == 1 && !moe && p.K <= 20480) {  // dense 4-bit decode row: persistent FMA kernel
    const uint32_t rows_per_warp = p.N / ((uint32_t)sm_count * 2 * kPersistWarps);
    (void)rows_per_warp;
    return launch_fma_m1_persist<4, 4>(p, sm_count, st);
  }
  if (bits == 4 && mt == 1 && p.K <= 40960) {  // 4-bit decode row: the conversion-free FMA kernel
    if (moe) return rows == 4 ? launch_fma_m1<4, true>(p, grid, st) : rows == 2 ? launch_fma_m1<2, true>(p, grid, st) : launch_fma_m1<1, true>(p, grid, st);
    return rows == 4 ? launch_fma_m1<4, false>(p, grid, st) : rows == 2 ? launch_fma_m1<2, false>(p, grid, st) : launch_fma_m1<1, false>(p, grid, st);
  }
#define ZTVM_MT(BITS_, MOE_)                                                            \
  switch (mt) {                                                                          \
    case 1: return launch_rows<BITS_, 1, MOE_>(p, rows, grid, smem, st);                 \
    case 2: return launch_rows<BITS_, 2, MOE_>(p, rows, grid, smem, st);                 \
    case 4: return launch_rows<BITS_, 4, MOE_>(p, rows, grid, smem, st);                 \
    default: return launch_rows<BITS_, 8, MOE_>(p, rows, grid, smem, st);                \
  }
  if (moe) {
    if (bits == 4) return launch_rows<4, 1, true>(p, rows, grid, smem, st);
    return launch_rows<3, 1, true>(p, rows, grid, smem, st);
  }
  if (bits == 4) { ZTVM_MT(4, false) }
  if (bits == 8) { ZTVM_MT(8, false) }
  ZTVM_MT(3, false)
#undef ZTVM_MT
}

}  // namespace ztvm
