// Grouped MoE expert matmul, streaming form: the contract of the ids-indirect GEMV
//   y[token, slot, :] = x[token, slot, :] * W[ids[token, slot]]^T        (int4_matmul.gen.ts:229-254)
// for token counts where an expert sees a handful of pairs (a few hundred tokens over 256 experts). There the job
// is bound by reading every active expert's weights once, not by the multiplies, so it is built like the
// persistent decode GEMV (ztvm_gemv_tc.cu) rather than like the tensor-core tiles of ztvm_moe_gemm.cu:
//   * the plan (ztvm_moe_plan.cuh) sorts the pairs by expert and cuts each expert's list into chunks of <= 8 pairs:
//     a chunk is the 8 columns of an mma.sync.m16n8k16;
//   * work unit = (chunk, 16 weight rows). The units, in chunk-major order, are split evenly over one CTA per SM;
//     inside a CTA warp (ks, rg) owns K slice ks (256 codes) and walks units rg, rg + RG, ...;
//   * a warp keeps the chunk's activations as B fragments in registers and reloads them when its unit sequence
//     crosses into the next chunk; weights / scales / biases stream through the per-warp cp.async ring;
//   * codes enter the MMA as f16 subnormals masked in place (exact products), each 64-code group is folded with its
//     scale and bias by round-to-nearest f32 FMAs, K-slice partials meet in shared memory in a fixed order.
// An expert with more than 8 pairs is streamed once per chunk (the repeats hit L2): the host side sends launches
// with many pairs per expert to the tensor-core tiles instead.
#include "ztvm_moe_plan.cuh"
#include "ztvm_stream_mma.cuh"

namespace ztvm {

constexpr int kMtRounds = 2;                       // rounds between two meetings of the K-slice partials
constexpr int kMtBlkRows = kMtRounds * 16;
constexpr int kMtPartialBytes = 2 * kTcWarps * kMtBlkRows * 8 * 4;

struct MoeTcParams {
  const uint32_t* W;
  const __half* S;
  const __half* B;
  const __half* X;
  __half* Y;
  uint32_t N, K, KP, SPR, slots;
  uint32_t in_slot_stride, out_slot_stride, in_tok_stride, out_tok_stride;
  MoeScratch sc;
};

__global__ void __launch_bounds__(kTcWarps * 32, 1)
moe_tc_kernel(const MoeTcParams p) {
  extern __shared__ __align__(128) uint8_t mt_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;

  const uint32_t KS = p.K / kTcSlice;                        // <= 16, checked by the launcher
  const uint32_t RG = (uint32_t)kTcWarps / KS;
  const uint32_t ks = (uint32_t)warp % KS, rg = (uint32_t)warp / KS;
  const bool warp_active = rg < RG;
  const uint32_t TPE = p.N / 16;                             // units per chunk
  const uint32_t nchunks = *p.sc.ntiles;
  const uint64_t U = (uint64_t)nchunks * TPE;
  const uint32_t u0 = (uint32_t)(U * blockIdx.x / gridDim.x), u1 = (uint32_t)(U * (blockIdx.x + 1) / gridDim.x);
  uint32_t rounds = (u1 - u0 + RG - 1) / RG;
  rounds = (rounds + kMtRounds - 1) / kMtRounds * kMtRounds;

  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(mt_smem) + (uint32_t)warp * (kTcDepth * kTcTileBytes);
  float* partial = reinterpret_cast<float*>(mt_smem + kTcRingBytes);            // [2][warps][kMtBlkRows][8]

  // ---- producer side -----------------------------------------------------------------------------------------
  const uint32_t cp_row = (uint32_t)lane >> 3, cp_chunk = (uint32_t)lane & 7;
  const uint32_t sb_row = (uint32_t)lane >> 1, sb_which = (uint32_t)lane & 1;
  const uint32_t cp_dst = cp_row * 128 + (((cp_chunk >> 1) ^ (cp_row & 3)) << 5) + ((cp_chunk & 1) << 4);
  const uint32_t sb_dst = kTcTileW + sb_row * 16 + sb_which * 8;
  const size_t row4 = (size_t)4 * p.KP;
  const bool affine = p.B != nullptr;
  // the unit the next issue will fetch, as (chunk, tile inside the chunk), and that chunk's expert
  uint32_t i_rd = 0, i_ec = (u0 + rg) / TPE, i_tile = (u0 + rg) - i_ec * TPE, i_expert = 0xFFFFFFFFu, i_ec_loaded = 0xFFFFFFFFu;
  auto issue = [&]() {
    const uint32_t u = u0 + i_rd * RG + rg;
    if (warp_active && i_rd < rounds && u < u1) {
      if (i_ec != i_ec_loaded) { i_expert = p.sc.tiles[(size_t)i_ec * 3]; i_ec_loaded = i_ec; }
      const uint32_t st = ring + (i_rd % kTcDepth) * kTcTileBytes;
      const size_t row = (size_t)i_expert * p.N + (size_t)i_tile * 16;
      const uint32_t* src = p.W + (row + cp_row) * p.KP + ks * 32 + cp_chunk * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) tc_cp16(st + cp_dst + i * 512, src + i * row4);
      if (affine || sb_which == 0) tc_cp8(st + sb_dst, (sb_which ? p.B : p.S) + (row + sb_row) * p.SPR + ks * 4);
    }
    tc_commit();
    ++i_rd;
    i_tile += RG;
    while (i_tile >= TPE) { i_tile -= TPE; ++i_ec; }
  };
#pragma unroll
  for (int i = 0; i < kTcDepth - 1; ++i) issue();

  // ---- consumer side -----------------------------------------------------------------------------------------
  uint32_t xf[4][2][4];           // B fragments of the current chunk: column g = its g-th pair
  unsigned long long xs2[4];      // per group: sums of x for the pairs of columns 2c, 2c + 1
  auto load_chunk = [&](uint32_t ec) {
    const uint32_t first = p.sc.tiles[(size_t)ec * 3 + 1], ntok = p.sc.tiles[(size_t)ec * 3 + 2];
    const bool on = (uint32_t)g < ntok;
    const __half* xr = p.X;
    if (on) {
      const uint32_t pair = p.sc.sorted[first + g];
      const uint32_t tok = pair / p.slots, slot = pair - tok * p.slots;
      xr = p.X + (size_t)tok * p.in_tok_stride + (size_t)slot * p.in_slot_stride + (size_t)ks * kTcSlice;
    }
#pragma unroll
    for (int tq = 0; tq < 4; ++tq) {
      float sum = 0.f;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (on) raw = *reinterpret_cast<const uint4*>(xr + (8 * tq + 2 * c + u) * 8);
        xf[tq][u][0] = __byte_perm(raw.x, raw.z, 0x5410);
        xf[tq][u][1] = __byte_perm(raw.y, raw.w, 0x5410);
        xf[tq][u][2] = __byte_perm(raw.x, raw.z, 0x7632);
        xf[tq][u][3] = __byte_perm(raw.y, raw.w, 0x7632);
        const float2 a = __half22float2(u32_as_h2(raw.x)), b = __half22float2(u32_as_h2(raw.y)),
                     d = __half22float2(u32_as_h2(raw.z)), e = __half22float2(u32_as_h2(raw.w));
        sum += ((a.x + a.y) + (b.x + b.y)) + ((d.x + d.y) + (e.x + e.y));
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      xs2[tq] = tc_pk(__shfl_sync(0xffffffffu, sum, (2 * c) * 4), __shfl_sync(0xffffffffu, sum, (2 * c + 1) * 4));
    }
  };

  unsigned long long acc[kMtRounds][2];
#pragma unroll
  for (int q = 0; q < kMtRounds; ++q) acc[q][0] = acc[q][1] = 0ull;
  const float kZero[4] = {0.f, 0.f, 0.f, 0.f};
  const unsigned long long k16 = tc_pk(16.f, 16.f);
  const uint32_t swz = ((uint32_t)g & 3u);
  uint32_t c_ec = (u0 + rg) / TPE, c_tile = (u0 + rg) - c_ec * TPE, c_loaded = 0xFFFFFFFFu;

  uint32_t step = 0;
  for (uint32_t blk = 0; blk < rounds / kMtRounds; ++blk) {
#pragma unroll
    for (int q = 0; q < kMtRounds; ++q, ++step) {
      issue();
      const uint32_t u = u0 + step * RG + rg;
      const bool live = warp_active && u < u1;
      if (live && c_ec != c_loaded) { load_chunk(c_ec); c_loaded = c_ec; }   // warp-uniform
      asm volatile("cp.async.wait_group %0;" ::"n"(kTcDepth - 1) : "memory");
      __syncwarp();
      if (live) {
        const uint32_t st = ring + (step % kTcDepth) * kTcTileBytes;
        const uint4 sg = tc_lds128(st + kTcTileW + (uint32_t)g * 16), sh = tc_lds128(st + kTcTileW + (uint32_t)(g + 8) * 16);
        const uint32_t sw[2][2] = {{sg.x, sg.y}, {sh.x, sh.y}}, bw[2][2] = {{sg.z, sg.w}, {sh.z, sh.w}};
#pragma unroll
        for (int tq = 0; tq < 4; ++tq) {
          const uint32_t off = (((uint32_t)tq ^ swz) << 5) + ((uint32_t)c << 3);
          const uint2 wg = tc_lds64(st + (uint32_t)g * 128 + off), wh = tc_lds64(st + (uint32_t)(g + 8) * 128 + off);
          float clo[4], chi[4];
          {
            const Inplace4 cg = codes4_inplace(wg.x), ch = codes4_inplace(wh.x);   // rows g and g + 8
            tc_mma(clo, cg.lo04, ch.lo04, cg.lo26, ch.lo26, xf[tq][0][0], xf[tq][0][1], kZero);
            tc_mma(chi, cg.hi15, ch.hi15, cg.hi37, ch.hi37, xf[tq][0][2], xf[tq][0][3], kZero);
          }
          {
            const Inplace4 cg = codes4_inplace(wg.y), ch = codes4_inplace(wh.y);
            tc_mma(clo, cg.lo04, ch.lo04, cg.lo26, ch.lo26, xf[tq][1][0], xf[tq][1][1], clo);
            tc_mma(chi, cg.hi15, ch.hi15, cg.hi37, ch.hi37, xf[tq][1][2], xf[tq][1][3], chi);
          }
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float2 s2 = __half22float2(u32_as_h2(sw[h][tq >> 1]));
            const float s = ((tq & 1) ? s2.y : s2.x) * 1048576.f;
            float b;
            if (affine) {
              const float2 b2 = __half22float2(u32_as_h2(bw[h][tq >> 1]));
              b = (tq & 1) ? b2.y : b2.x;
            } else {
              b = -7.f * ((tq & 1) ? s2.y : s2.x);
            }
            const unsigned long long t2 = tc_ffma2(tc_pk(clo[2 * h], clo[2 * h + 1]), k16, tc_pk(chi[2 * h], chi[2 * h + 1]));
            unsigned long long r = acc[q][h];
            r = tc_ffma2(tc_pk(s, s), t2, r);
            r = tc_ffma2(tc_pk(b, b), xs2[tq], r);
            acc[q][h] = r;
          }
        }
      }
      __syncwarp();
      c_tile += RG;
      while (c_tile >= TPE) { c_tile -= TPE; ++c_ec; }
    }
    // ---- meeting ------------------------------------------------------------------------------------------------
    float* mine = partial + ((size_t)((blk & 1u) * kTcWarps + (uint32_t)warp) * kMtBlkRows) * 8;
#pragma unroll
    for (int q = 0; q < kMtRounds; ++q)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        *reinterpret_cast<float2*>(mine + (q * 16 + g + 8 * h) * 8 + 2 * c) = tc_unpk(acc[q][h]);
        acc[q][h] = 0ull;
      }
    __syncthreads();
    const float* buf = partial + (size_t)(blk & 1u) * kTcWarps * kMtBlkRows * 8;
    const uint32_t outs = (uint32_t)kMtRounds * RG * 128u;
    for (uint32_t i = (threadIdx.x + 512u - 32u * (blk & 15u)) & 511u; i < outs; i += blockDim.x) {
      const uint32_t r16 = i & 15u, col = (i >> 4) & 7u, tb = i >> 7;
      const uint32_t q = tb / RG, rgi = tb - q * RG;
      const uint32_t u = u0 + (blk * kMtRounds + q) * RG + rgi;
      if (u >= u1) continue;
      const uint32_t ec = u / TPE, tile = u - ec * TPE;
      if (col >= p.sc.tiles[(size_t)ec * 3 + 2]) continue;
      float v = 0.f;
      for (uint32_t k2 = 0; k2 < KS; ++k2) v += buf[((size_t)(rgi * KS + k2) * kMtBlkRows + q * 16 + r16) * 8 + col];
      const uint32_t pair = p.sc.sorted[p.sc.tiles[(size_t)ec * 3 + 1] + col];
      const uint32_t tok = pair / p.slots, slot = pair - tok * p.slots;
      p.Y[(size_t)tok * p.out_tok_stride + (size_t)slot * p.out_slot_stride + tile * 16 + r16] = __float2half_rn(v);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---- host side ---------------------------------------------------------------------------------------------
bool moe_tc_supported(const GemvParams& g, int bits) {
  if (bits != 4 || g.group_shift != 6) return false;
  if (g.K == 0 || g.K % kTcSlice || g.K / kTcSlice > (uint32_t)kTcWarps || g.N == 0 || g.N % 16) return false;
  if ((g.in_slot_stride | g.in_tok_stride) % 8 || (reinterpret_cast<uintptr_t>(g.X) & 15u)) return false;
  if ((reinterpret_cast<uintptr_t>(g.W) & 15u) || (reinterpret_cast<uintptr_t>(g.S) & 7u) ||
      (g.B && (reinterpret_cast<uintptr_t>(g.B) & 7u)))
    return false;
  return g.experts <= 1024;
}

cudaError_t launch_moe_tc(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t* scratch, int sm_count,
                          cudaStream_t st, bool reuse_plan) {
  const uint32_t P = tokens * slots;
  MoeScratch sc = moe_scratch_carve(scratch, g.experts, P);
  cudaError_t e = reuse_plan ? cudaSuccess : launch_moe_plan(g, tokens, slots, sc, kMoeTcTileRows, st);
  if (e != cudaSuccess) return e;
  MoeTcParams p;
  p.W = g.W; p.S = g.S; p.B = g.B; p.X = g.X; p.Y = reinterpret_cast<__half*>(g.Y);
  p.N = g.N; p.K = g.K; p.KP = g.KP; p.SPR = g.SPR; p.slots = slots;
  p.in_slot_stride = g.in_slot_stride; p.out_slot_stride = g.out_slot_stride;
  p.in_tok_stride = g.in_tok_stride; p.out_tok_stride = g.out_tok_stride;
  p.sc = sc;
  constexpr int smem = kTcRingBytes + kMtPartialBytes;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    e = cudaFuncSetAttribute(moe_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  moe_tc_kernel<<<sm_count, kTcWarps * 32, smem, st>>>(p);
  return cudaGetLastError();
}

}  // namespace ztvm
