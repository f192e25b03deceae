// Decode GEMV for 4-bit weights, M = 1..8, on the warp-level matrix unit.
//
// Why not plain FMAs: at 6.5 TB/s a B200 streams 13 T codes/s, i.e. 45 codes per clock per SM.
// Unpack + convert + FMA on the CUDA cores measured 28 codes/clk/SM (issue-bound); the same
// products on mma.sync.m16n8k16 measured 73, for up to eight activation rows at once. The kernel
// stays bandwidth-bound by design: the matrix unit is only the multiplier array.
//
// Exactness: a nibble masked in place, (w & 0x000F000F) or (w & 0x00F000F0), IS a pair of f16
// subnormals with values q * 2^-24 resp. q * 2^-20 (no magic constant, no subtraction). The MMA forms
// x*q exactly and accumulates in f32; the two power-of-two classes keep separate accumulators and are
// folded into the group scale afterwards (s * 2^24, s * 2^20 are exact). Per scale group:
//   acc += s * sum x_i q_i + b * sum x_i          (int4_matmul.gen.ts:78-96, :388-464)
// so the arithmetic is the reference GEMV's, with a different (pairwise) summation order.
//
// Mapping: a CTA owns 16 weight rows; its warps split K in chunks of whole scale groups. In a warp,
// lane (g = lane/4, c = lane%4) holds rows g and g+8 and, per group, WPL = group/32 consecutive words
// starting at word c*WPL of the group: the four lanes of a quad together hold exactly one group, which
// is what one MMA sums over. Word t of the lane feeds two MMAs (the 2^-24 and the 2^-20 class):
//   A = {wg & m, wh & m, (wg >> 8) & m, (wh >> 8) & m}       rows g | g+8, codes (q0,q4 | q2,q6) resp. (q1,q5 | q3,q7)
//   B = activations of token g for the same 8-code block, stored in shared memory already permuted to
//       [x0,x4,x2,x6, x1,x5,x3,x7] and laid out so that a quarter-warp reads 128 contiguous bytes.
#include "ztvm_device.cuh"
#include "ztvm_kernels.h"

namespace ztvm {

constexpr int kMmaRows = 16;       // weight rows per CTA
constexpr int kMmaMaxWarps = 8;
constexpr int kMmaBatch = 4;       // scale groups per load batch

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1, const float (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

template <int WPL>
struct WordVec;
template <> struct WordVec<1> { uint32_t w[1]; };
template <> struct WordVec<2> { uint32_t w[2]; };
template <> struct WordVec<4> { uint32_t w[4]; };

template <int WPL>
__device__ __forceinline__ WordVec<WPL> load_words(const uint32_t* p, bool valid) {
  WordVec<WPL> v;
#pragma unroll
  for (int i = 0; i < WPL; ++i) v.w[i] = 0u;
  if (valid) {
    if constexpr (WPL == 4) {
      const uint4 t = ld_stream_u4(p);
      v.w[0] = t.x; v.w[1] = t.y; v.w[2] = t.z; v.w[3] = t.w;
    } else if constexpr (WPL == 2) {
      asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.w[0]), "=r"(v.w[1]) : "l"(p));
    } else {
      v.w[0] = ld_stream_u32(p);
    }
  }
  return v;
}

// Shared-memory item (16 bytes = one permuted 8-code activation block) of group `grp` (tile-relative),
// word t, token tok, quad lane c.
template <int WPL, int NTOK>
__device__ __forceinline__ int xitem(int grp, int t, int tok, int c) {
  return ((grp * WPL + t) * NTOK + tok) * 4 + c;
}

template <int WPL, int NTOK, bool MOE>
__global__ void __launch_bounds__(kMmaMaxWarps * 32)
gemv_mma_kernel(const GemvParams p) {
  extern __shared__ uint4 smem_u4[];
  constexpr int GROUP = WPL * 32;
  constexpr int NV = NTOK <= 1 ? 1 : 2;  // tokens per lane that can be live: (2c) and (2c+1)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, c = lane & 3;

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

  const uint32_t row0 = blockIdx.x * kMmaRows;
  const uint32_t ra = min(row0 + g, p.N - 1), rb = min(row0 + g + 8, p.N - 1);
  const uint32_t* wa = W + (size_t)ra * p.KP + c * WPL;
  const uint32_t* wb = W + (size_t)rb * p.KP + c * WPL;
  const __half* sa = S + (size_t)ra * p.SPR;
  const __half* sb = S + (size_t)rb * p.SPR;
  const __half* ba = Bv ? Bv + (size_t)ra * p.SPR : nullptr;
  const __half* bb = Bv ? Bv + (size_t)rb * p.SPR : nullptr;

  const uint32_t groups = p.SPR;
  const uint32_t tile_groups = p.tile_units;  // groups staged per K tile (multiple of kMmaBatch)
  float* xsum_sm = reinterpret_cast<float*>(smem_u4 + (size_t)tile_groups * WPL * NTOK * 4);  // [tile_groups][NTOK]
  float* red_sm = xsum_sm + (size_t)tile_groups * NTOK;                                        // [nwarps][16][8]

  // live accumulators: [row half][token 2c | 2c+1]
  float acc[2][NV];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int v = 0; v < NV; ++v) acc[h][v] = 0.f;

  const bool vec_sb = (p.SPR % 4 == 0);  // 8-byte loads of 4 consecutive scales are aligned
  const float kZero[4] = {0.f, 0.f, 0.f, 0.f};

  for (uint32_t tg0 = 0; tg0 < groups; tg0 += tile_groups) {
    const uint32_t tg = min(tile_groups, groups - tg0);
    // this warp's chunk of the tile, a multiple of the batch size
    uint32_t gpw = (tg + nwarps - 1) / nwarps;
    gpw = (gpw + kMmaBatch - 1) / kMmaBatch * kMmaBatch;
    const uint32_t gbeg = min((uint32_t)warp * gpw, tg), gend = min(gbeg + gpw, tg);

    // ---- first batch of weights goes out before anything else ---------------------------------
    WordVec<WPL> qa[kMmaBatch], qb[kMmaBatch];
#pragma unroll
    for (int i = 0; i < kMmaBatch; ++i) {
      const uint32_t gi = gbeg + i;
      const bool ok = gi < gend;
      qa[i] = load_words<WPL>(wa + (size_t)(tg0 + gi) * (GROUP / 8), ok);
      qb[i] = load_words<WPL>(wb + (size_t)(tg0 + gi) * (GROUP / 8), ok);
    }

    if (tg0) __syncthreads();  // previous tile fully consumed
    // ---- stage activations: 8-element blocks, permuted to the MMA pair order ---------------------
    {
      const uint32_t nblk = tg * (GROUP / 8);
      for (uint32_t i = threadIdx.x; i < nblk * NTOK; i += blockDim.x) {
        const uint32_t tok = i / nblk, blk = i - tok * nblk;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (tok < p.M) raw = *reinterpret_cast<const uint4*>(X + (size_t)tok * p.x_row_stride + (size_t)(tg0 * (GROUP / 8) + blk) * 8);
        // raw = (x0x1, x2x3, x4x5, x6x7) -> (x0x4, x2x6, x1x5, x3x7)
        uint4 o;
        o.x = __byte_perm(raw.x, raw.z, 0x5410);
        o.y = __byte_perm(raw.y, raw.w, 0x5410);
        o.z = __byte_perm(raw.x, raw.z, 0x7632);
        o.w = __byte_perm(raw.y, raw.w, 0x7632);
        const uint32_t grp = blk / (GROUP / 8), wi = blk % (GROUP / 8);
        smem_u4[xitem<WPL, NTOK>(grp, wi % WPL, tok, wi / WPL)] = o;
      }
    }
    __syncthreads();
    // ---- per-(group, token) activation sums: the bias term's multiplier ---------------------------
    for (uint32_t i = threadIdx.x; i < tg * NTOK; i += blockDim.x) {
      const uint32_t grp = i / NTOK, tok = i - grp * NTOK;
      float s = 0.f;
#pragma unroll
      for (int t = 0; t < WPL; ++t)
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const uint4 v = smem_u4[xitem<WPL, NTOK>(grp, t, tok, cc)];
          const float2 a = __half22float2(u32_as_h2(v.x)), b = __half22float2(u32_as_h2(v.y)),
                       d = __half22float2(u32_as_h2(v.z)), e = __half22float2(u32_as_h2(v.w));
          s += ((a.x + a.y) + (b.x + b.y)) + ((d.x + d.y) + (e.x + e.y));
        }
      xsum_sm[grp * NTOK + tok] = s;
    }
    __syncthreads();

    // ---- stream this warp's groups ---------------------------------------------------------------
    for (uint32_t gb = gbeg; gb < gend; gb += kMmaBatch) {
      // scales / biases of the batch
      float sc[2][kMmaBatch], bi[2][kMmaBatch];
      if (vec_sb && gb + kMmaBatch <= gend) {
        const uint2 s0 = __ldg(reinterpret_cast<const uint2*>(sa + tg0 + gb)), s1 = __ldg(reinterpret_cast<const uint2*>(sb + tg0 + gb));
        float2 t;
        t = __half22float2(u32_as_h2(s0.x)); sc[0][0] = t.x; sc[0][1] = t.y;
        t = __half22float2(u32_as_h2(s0.y)); sc[0][2] = t.x; sc[0][3] = t.y;
        t = __half22float2(u32_as_h2(s1.x)); sc[1][0] = t.x; sc[1][1] = t.y;
        t = __half22float2(u32_as_h2(s1.y)); sc[1][2] = t.x; sc[1][3] = t.y;
        if (ba) {
          const uint2 b0 = __ldg(reinterpret_cast<const uint2*>(ba + tg0 + gb)), b1 = __ldg(reinterpret_cast<const uint2*>(bb + tg0 + gb));
          t = __half22float2(u32_as_h2(b0.x)); bi[0][0] = t.x; bi[0][1] = t.y;
          t = __half22float2(u32_as_h2(b0.y)); bi[0][2] = t.x; bi[0][3] = t.y;
          t = __half22float2(u32_as_h2(b1.x)); bi[1][0] = t.x; bi[1][1] = t.y;
          t = __half22float2(u32_as_h2(b1.y)); bi[1][2] = t.x; bi[1][3] = t.y;
        } else {
#pragma unroll
          for (int i = 0; i < kMmaBatch; ++i) { bi[0][i] = -7.f * sc[0][i]; bi[1][i] = -7.f * sc[1][i]; }
        }
      } else {
#pragma unroll
        for (int i = 0; i < kMmaBatch; ++i) {
          const bool ok = gb + i < gend;
          sc[0][i] = ok ? ld_f16_as_f32(sa + tg0 + gb + i) : 0.f;
          sc[1][i] = ok ? ld_f16_as_f32(sb + tg0 + gb + i) : 0.f;
          bi[0][i] = !ok ? 0.f : ba ? ld_f16_as_f32(ba + tg0 + gb + i) : -7.f * sc[0][i];
          bi[1][i] = !ok ? 0.f : bb ? ld_f16_as_f32(bb + tg0 + gb + i) : -7.f * sc[1][i];
        }
      }
      // prefetch the next batch of weights
      WordVec<WPL> na[kMmaBatch], nb[kMmaBatch];
#pragma unroll
      for (int i = 0; i < kMmaBatch; ++i) {
        const uint32_t gi = gb + kMmaBatch + i;
        const bool ok = gi < gend;
        na[i] = load_words<WPL>(wa + (size_t)(tg0 + gi) * (GROUP / 8), ok);
        nb[i] = load_words<WPL>(wb + (size_t)(tg0 + gi) * (GROUP / 8), ok);
      }

#pragma unroll
      for (int i = 0; i < kMmaBatch; ++i) {
        if (gb + i >= gend) break;
        float clo[4], chi[4];
#pragma unroll
        for (int t = 0; t < WPL; ++t) {
          uint4 xb = make_uint4(0u, 0u, 0u, 0u);
          if (g < NTOK) xb = smem_u4[xitem<WPL, NTOK>(gb + i, t, g, c)];
          const uint32_t wg = qa[i].w[t], wh = qb[i].w[t];
          const Inplace4 cg = codes4_inplace(wg), ch = codes4_inplace(wh);
          if (t == 0) {
            mma_16816(clo, cg.lo04, ch.lo04, cg.lo26, ch.lo26, xb.x, xb.y, kZero);
            mma_16816(chi, cg.hi15, ch.hi15, cg.hi37, ch.hi37, xb.z, xb.w, kZero);
          } else {
            mma_16816(clo, cg.lo04, ch.lo04, cg.lo26, ch.lo26, xb.x, xb.y, clo);
            mma_16816(chi, cg.hi15, ch.hi15, cg.hi37, ch.hi37, xb.z, xb.w, chi);
          }
        }
        // fold the group: acc += s*(2^24*lo + 2^20*hi) + b*xsum
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float s24 = sc[h][i] * 16777216.f, s20 = sc[h][i] * 1048576.f;
#pragma unroll
          for (int v = 0; v < NV; ++v) {
            const int tok = 2 * c + v;
            const float xs = tok < NTOK ? xsum_sm[(gb + i) * NTOK + tok] : 0.f;
            float a = acc[h][v];
            a = fmaf(s24, clo[2 * h + v], a);
            a = fmaf(s20, chi[2 * h + v], a);
            a = fmaf(bi[h][i], xs, a);
            acc[h][v] = a;
          }
        }
      }
#pragma unroll
      for (int i = 0; i < kMmaBatch; ++i) { qa[i] = na[i]; qb[i] = nb[i]; }
    }
  }

  // ---- reduce across the warps of the CTA (each covered a different K chunk) and store ------------
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int tok = 2 * c + v;
      if (tok < NTOK) red_sm[(warp * kMmaRows + g + 8 * h) * 8 + tok] = acc[h][v];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < kMmaRows * NTOK; i += blockDim.x) {
    const int r = i / NTOK, tok = i - r * NTOK;
    float v = 0.f;
    for (int w = 0; w < nwarps; ++w) v += red_sm[(w * kMmaRows + r) * 8 + tok];
    const uint32_t row = row0 + r;
    if (row < p.N && (uint32_t)tok < p.M) {
      const size_t o = MOE ? out_base + row : (size_t)tok * p.y_row_stride + row;
      if (p.out_f32) reinterpret_cast<float*>(p.Y)[o] = v;
      else reinterpret_cast<__half*>(p.Y)[o] = __float2half_rn(v);
    }
  }
}

// ---- host-side launch ------------------------------------------------------------------------------
template <int WPL, int NTOK, bool MOE>
static cudaError_t launch_mma_one(const GemvParams& p, dim3 grid, int threads, size_t smem, cudaStream_t st) {
  auto kern = gemv_mma_kernel<WPL, NTOK, MOE>;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  kern<<<grid, threads, smem, st>>>(p);
  return cudaGetLastError();
}

template <int WPL, bool MOE>
static cudaError_t launch_mma_tok(const GemvParams& p, int ntok, dim3 grid, int threads, size_t smem, cudaStream_t st) {
  if (MOE || ntok == 1) return launch_mma_one<WPL, 1, MOE>(p, grid, threads, smem, st);
  if constexpr (!MOE) {
    if (ntok == 2) return launch_mma_one<WPL, 2, false>(p, grid, threads, smem, st);
    if (ntok == 4) return launch_mma_one<WPL, 4, false>(p, grid, threads, smem, st);
    return launch_mma_one<WPL, 8, false>(p, grid, threads, smem, st);
  }
  return cudaErrorInvalidValue;
}

bool gemv_mma_supported(int bits, uint32_t group) { return bits == 4 && (group == 32 || group == 64 || group == 128); }

cudaError_t launch_gemv_mma(GemvParams p, bool moe, uint32_t tokens, uint32_t slots, cudaStream_t st) {
  const uint32_t group = 1u << p.group_shift;
  const int wpl = (int)group / 32;
  const int ntok = p.M <= 1 ? 1 : p.M <= 2 ? 2 : p.M <= 4 ? 4 : 8;
  const uint32_t groups = p.SPR;
  // warps per CTA: one batch of groups per warp when K is short, up to eight warps
  int nwarps = (int)((groups + kMmaBatch - 1) / kMmaBatch);
  nwarps = nwarps < 1 ? 1 : nwarps > kMmaMaxWarps ? kMmaMaxWarps : nwarps;
  // groups staged per K tile: activations (f16) + sums within ~64 KB
  const uint32_t per_group = group * 2u * ntok + 4u * ntok;
  uint32_t tile_groups = (64u * 1024u / per_group) / kMmaBatch * kMmaBatch;
  const uint32_t groups_up = (groups + kMmaBatch - 1) / kMmaBatch * kMmaBatch;
  if (tile_groups > groups_up) tile_groups = groups_up;
  p.tile_units = tile_groups;
  const size_t smem = (size_t)tile_groups * per_group + (size_t)nwarps * kMmaRows * 8 * 4;
  dim3 grid((p.N + kMmaRows - 1) / kMmaRows, moe ? tokens : 1, moe ? slots : 1);
  const int threads = nwarps * 32;
  if (moe) {
    if (wpl == 2) return launch_mma_tok<2, true>(p, 1, grid, threads, smem, st);
    if (wpl == 4) return launch_mma_tok<4, true>(p, 1, grid, threads, smem, st);
    return launch_mma_tok<1, true>(p, 1, grid, threads, smem, st);
  }
  if (wpl == 2) return launch_mma_tok<2, false>(p, ntok, grid, threads, smem, st);
  if (wpl == 4) return launch_mma_tok<4, false>(p, ntok, grid, threads, smem, st);
  return launch_mma_tok<1, false>(p, ntok, grid, threads, smem, st);
}

}  // namespace ztvm
