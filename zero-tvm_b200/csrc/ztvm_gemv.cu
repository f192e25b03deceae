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
  constexpr int WPU = BITS;  // words per 32-code unit: 4 bits -> 4, 3 bits -> 3

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
  if (mt == 8 && rows > 2) rows = 2;  // register budget
  const uint32_t units = p.K >> 5;
  uint32_t tile_units = (uint32_t)(kGemvTileElems / mt) >> 5;
  const uint32_t units_up = (units + 31) & ~31u;
  if (tile_units > units_up) tile_units = units_up;
  p.tile_units = tile_units;
  const size_t smem = (size_t)mt * tile_units * (128 + 4);
  dim3 grid((p.N + kGemvWarps * rows - 1) / (kGemvWarps * rows), moe ? tokens : 1, moe ? slots : 1);
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
  ZTVM_MT(3, false)
#undef ZTVM_MT
}

}  // namespace ztvm
