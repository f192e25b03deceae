// Persistent decode GEMV for 3-bit / group-64 weights, M = 1 (the q3 GEMV body, int4_matmul.gen.ts:409-448): the design
// of ztvm_gemv_tc.cu — one CTA per SM, K cut in 256-code slices owned by warps, per-warp cp.async ring, activations as
// MMA B fragments in registers, fixed-order meeting of the K-slice partials — with an unpack made for a bit stream
// whose codes do not sit on nibble boundaries.
//
// A 3-bit code anywhere in bits 0..9 of a 16-bit half is still an f16 subnormal: (7 << o) & half = q * 2^(o-24), and
// the power of two is moved onto the activation of that slot (x * 2^-o is exact unless |x| < 2^(o-14), where it
// rounds at 2^-25: far below the output tolerance), so every product is q * x * 2^-24 and one accumulator serves.
// A 32-bit window of the row's bit stream that starts on code i holds codes i, i+1, i+2 in its low half (offsets 0, 3,
// 6) and i+6, i+7 in its high half (offsets 2, 5): two ANDs give the register pairs (i | i+6) and (i+1 | i+7), i.e.
// one funnel shift + two ANDs per four codes. Windows at i = 0, 2, 4 (mod 12) tile the stream in pairs.
//
// Lane (g, c) of a warp owns scale group c of the slice (64 codes = 6 words of rows g and g + 8): all window
// positions are compile-time constants, and because the lane's k slots all belong to group c, the B fragment puts
// their activations in MMA column c only — the accumulator's columns are the groups, as in the 4-bit kernel for M = 1.
// 64 = 5 * 12 + 4: fifteen full windows and two that use their low half only, 17 MMAs per (16 rows x 256 codes).
#include <cstdlib>

#include "ztvm_device.cuh"
#include "ztvm_kernels.h"
#include "ztvm_stream_mma.cuh"

namespace ztvm {

constexpr int kT3RowBytes = 96;                          // 256 codes of one row
constexpr int kT3TileW = 16 * kT3RowBytes;               // 1536
constexpr int kT3TileBytes = kT3TileW + 16 * 16;         // + per row 4 scales, 4 biases (f16)
constexpr int kT3RingBytes = kTcWarps * kTcDepth * kT3TileBytes;
constexpr int kT3Rounds = 4;
constexpr int kT3Views = kCodes3Views;
constexpr uint32_t kT3MaxAccBytes = 32 * 1024;

// first code of window k inside the lane's group (the unpack itself is codes3_inplace, shared with the parity hook)
__host__ __device__ constexpr int t3_code(int k) { return codes3_view_first(k); }

__global__ void __launch_bounds__(kTcWarps * 32, 1)
gemv_tc3_kernel(const GemvParams p) {   // 3-bit weights exist only in the affine layout
  extern __shared__ __align__(128) uint8_t t3_smem[];
  constexpr int kBlkRows = kT3Rounds * 16;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;

  const uint32_t slices = p.K / kTcSlice;
  const uint32_t KS = slices < (uint32_t)kTcWarps ? slices : (uint32_t)kTcWarps;
  const uint32_t RG = (uint32_t)kTcWarps / KS;
  const uint32_t ks = (uint32_t)warp % KS, rg = (uint32_t)warp / KS;
  const bool warp_active = rg < RG;
  const uint32_t num_kt = (slices + KS - 1) / KS;

  const uint32_t r0 = (uint32_t)((uint64_t)blockIdx.x * p.N / gridDim.x);
  const uint32_t r1 = (uint32_t)((uint64_t)(blockIdx.x + 1) * p.N / gridDim.x);
  const uint32_t nrows = r1 - r0;
  const uint32_t ntiles = (nrows + 15) / 16;
  uint32_t rounds = (ntiles + RG - 1) / RG;
  rounds = (rounds + kT3Rounds - 1) / kT3Rounds * kT3Rounds;
  const uint32_t total = num_kt * rounds;

  const uint32_t ring = (uint32_t)__cvta_generic_to_shared(t3_smem) + (uint32_t)warp * (kTcDepth * kT3TileBytes);
  float* partial = reinterpret_cast<float*>(t3_smem + kT3RingBytes);            // [2][warps][kBlkRows]
  float* acc_sm = partial + 2 * kTcWarps * kBlkRows;                            // [nrows], only if num_kt > 1

  // ---- producer side: 16 rows x 6 chunks of 16 bytes = three copies per lane, plus scales / biases -------------
  const uint32_t sb_row = (uint32_t)lane >> 1, sb_which = (uint32_t)lane & 1;
  const uint32_t sb_dst = kT3TileW + sb_row * 16 + sb_which * 8;
  uint32_t i_step = 0, i_kt = 0, i_rd = 0;
  // this lane's three 16-byte pieces of a tile (row, chunk) and their running source addresses: rows advance by RG tiles
  // per round, slices by KS per K tile
  uint32_t cp_row3[3], cp_dst3[3];
  const uint32_t* src_base[3];
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const uint32_t q = (uint32_t)lane + 32u * i, row = q / 6, j = q - row * 6;
    cp_row3[i] = row;
    cp_dst3[i] = row * kT3RowBytes + j * 16;
    src_base[i] = p.W + (size_t)(r0 + rg * 16 + row) * p.KP + ks * 24 + j * 4;
  }
  const __half* const sb_base = (sb_which ? p.B : p.S) + (size_t)(r0 + rg * 16 + sb_row) * p.SPR + ks * 4;
  const size_t src_round = (size_t)RG * 16 * p.KP, sb_round = (size_t)RG * 16 * p.SPR;
  size_t src_off = 0, sb_off = 0;
  uint32_t i_trow = rg * 16, i_slot = 0;
  auto issue = [&]() {
    if (warp_active && i_step < total) {
      const uint32_t sl = i_kt * KS + ks;
      const uint32_t trow = i_trow;
      if (sl < slices && trow < nrows) {
        const uint32_t st = ring + i_slot * kT3TileBytes;
#pragma unroll
        for (int i = 0; i < 3; ++i)
          if (trow + cp_row3[i] < nrows) tc_cp16(st + cp_dst3[i], src_base[i] + src_off);
        if (trow + sb_row < nrows) tc_cp8(st + sb_dst, sb_base + sb_off);
      }
    }
    tc_commit();
    ++i_step;
    if (++i_slot == (uint32_t)kTcDepth) i_slot = 0;
    src_off += src_round; sb_off += sb_round; i_trow += RG * 16;
    if (++i_rd == rounds) {
      i_rd = 0; ++i_kt;
      i_trow = rg * 16;
      src_off = (size_t)i_kt * KS * 24;
      sb_off = (size_t)i_kt * KS * 4;
    }
  };
#pragma unroll
  for (int i = 0; i < kTcDepth - 1; ++i) issue();

  asm volatile("griddepcontrol.wait;" ::: "memory");   // everything above reads only weights

  // B fragments: the lane's k slots are the codes of group c, their activations sit in MMA column c, i.e. in the lanes
  // with g == c; slot offsets 0 / 2 / 3 / 5 inside a half become factors 1, 1/4, 1/8, 1/32 on the activation.
  uint32_t xb[kT3Views][2];
  float xs[2];                   // sum of x over the groups of columns 2c, 2c + 1 (the bias term's multiplier)
  auto load_x = [&](uint32_t kt) {
    const uint32_t sl = kt * KS + ks;
    const bool on = warp_active && sl < slices && g == c;
    const __half* xr = p.X + (size_t)sl * kTcSlice + 64 * c;
    __align__(16) __half h[64];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if (on) raw = *reinterpret_cast<const uint4*>(xr + 8 * i);
      *reinterpret_cast<uint4*>(&h[8 * i]) = raw;
    }
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 64; ++i) sum += __half2float(h[i]);
    const __half q4 = __float2half(0.25f), q8 = __float2half(0.125f), q32 = __float2half(0.03125f);
#pragma unroll
    for (int k = 0; k < kT3Views; ++k) {
      const int i = t3_code(k);
      const __half z = __float2half(0.f);
      const __half a0 = h[i], a1 = k < 15 ? __hmul(h[i + 6], q4) : z;          // register 0: code i | code i + 6
      const __half b0 = __hmul(h[i + 1], q8), b1 = k < 15 ? __hmul(h[i + 7], q32) : z;   // register 1: i + 1 | i + 7
      const __half2 r0v = __halves2half2(a0, a1), r1v = __halves2half2(b0, b1);
      xb[k][0] = *reinterpret_cast<const uint32_t*>(&r0v);
      xb[k][1] = *reinterpret_cast<const uint32_t*>(&r1v);
    }
    // lane (G, G) holds the sum of group G: lanes folding columns 2c, 2c + 1 fetch it from lane 5 G
#pragma unroll
    for (int v = 0; v < 2; ++v) {
      const int G = 2 * c + v;
      const float t = __shfl_sync(0xffffffffu, sum, (5 * G) & 31);
      xs[v] = G < 4 ? t : 0.f;
    }
  };
  load_x(0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  float acc[kT3Rounds][2][2];
#pragma unroll
  for (int q = 0; q < kT3Rounds; ++q)
#pragma unroll
    for (int h = 0; h < 2; ++h) acc[q][h][0] = acc[q][h][1] = 0.f;
  const float kZero[4] = {0.f, 0.f, 0.f, 0.f};

  uint32_t step = 0, meet = 0;
  for (uint32_t kt = 0; kt < num_kt; ++kt) {
    if (kt) load_x(kt);
    const bool slice_ok = warp_active && kt * KS + ks < slices;
    for (uint32_t blk = 0; blk < rounds / kT3Rounds; ++blk, ++meet) {
#pragma unroll
      for (int q = 0; q < kT3Rounds; ++q, ++step) {
        issue();
        asm volatile("cp.async.wait_group %0;" ::"n"(kTcDepth - 1) : "memory");
        __syncwarp();
        const uint32_t trow = ((blk * kT3Rounds + q) * RG + rg) * 16;
        if (slice_ok && trow < nrows) {
          const uint32_t st = ring + (step % kTcDepth) * kT3TileBytes;
          uint32_t w[6], u[6];   // group c of rows g and g + 8
#pragma unroll
          for (int i = 0; i < 3; ++i) {
            const uint2 a = tc_lds64(st + (uint32_t)g * kT3RowBytes + 24u * c + 8u * i);
            const uint2 b = tc_lds64(st + (uint32_t)(g + 8) * kT3RowBytes + 24u * c + 8u * i);
            w[2 * i] = a.x; w[2 * i + 1] = a.y; u[2 * i] = b.x; u[2 * i + 1] = b.y;
          }
          float d0[4], d1[4];   // two accumulation chains
#pragma unroll
          for (int k = 0; k < kT3Views; ++k) {
            uint32_t w0, w1, u0, u1;
            codes3_inplace(w, k, w0, w1);
            codes3_inplace(u, k, u0, u1);
            if (k == 0) tc_mma(d0, w0, u0, w1, u1, xb[k][0], xb[k][1], kZero);
            else if (k == 1) tc_mma(d1, w0, u0, w1, u1, xb[k][0], xb[k][1], kZero);
            else if (k & 1) tc_mma(d1, w0, u0, w1, u1, xb[k][0], xb[k][1], d1);
            else tc_mma(d0, w0, u0, w1, u1, xb[k][0], xb[k][1], d0);
          }
          // fold: columns 2c, 2c + 1 of the accumulator are groups 2c, 2c + 1 (lanes with c >= 2 hold empty columns)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t rowp = st + kT3TileW + (uint32_t)(g + 8 * h) * 16 + 4u * ((uint32_t)c & 1u);
            const float2 s2 = __half22float2(u32_as_h2(tc_lds32(rowp)));
            const float2 b2 = __half22float2(u32_as_h2(tc_lds32(rowp + 8)));
            const float t0 = d0[2 * h] + d1[2 * h], t1 = d0[2 * h + 1] + d1[2 * h + 1];
            acc[q][h][0] = fmaf(b2.x, xs[0], fmaf(s2.x * 16777216.f, t0, acc[q][h][0]));
            acc[q][h][1] = fmaf(b2.y, xs[1], fmaf(s2.y * 16777216.f, t1, acc[q][h][1]));
          }
        }
        __syncwarp();
      }
      // ---- meeting ----------------------------------------------------------------------------------------------
      float* mine = partial + (size_t)((meet & 1u) * kTcWarps + (uint32_t)warp) * kBlkRows;
#pragma unroll
      for (int q = 0; q < kT3Rounds; ++q)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float v0 = slice_ok ? acc[q][h][0] + acc[q][h][1] : 0.f;
          acc[q][h][0] = acc[q][h][1] = 0.f;
          v0 += __shfl_xor_sync(0xffffffffu, v0, 1);        // groups 0, 1 (c = 0) + groups 2, 3 (c = 1)
          if (c == 0) mine[q * 16 + g + 8 * h] = v0;
        }
      __syncthreads();
      const float* buf = partial + (size_t)(meet & 1u) * kTcWarps * kBlkRows;
      const uint32_t outs = (uint32_t)kT3Rounds * RG * 16u;
      for (uint32_t i = (threadIdx.x + 512u - 32u * (meet & 15u)) & 511u; i < outs; i += blockDim.x) {
        const uint32_t r16 = i & 15u, tb = i >> 4;
        const uint32_t q = tb / RG, rgi = tb - q * RG;
        const uint32_t row = ((blk * kT3Rounds + q) * RG + rgi) * 16 + r16;
        if (row >= nrows) continue;
        float v = 0.f;
        for (uint32_t k2 = 0; k2 < KS; ++k2) v += buf[(size_t)(rgi * KS + k2) * kBlkRows + q * 16 + r16];
        if (num_kt > 1) {
          float* a = acc_sm + row;
          if (kt) v += *a;
          if (kt + 1 < num_kt) { *a = v; continue; }
        }
        const size_t o = (size_t)r0 + row;
        if (p.out_f32) reinterpret_cast<float*>(p.Y)[o] = v;
        else reinterpret_cast<__half*>(p.Y)[o] = __float2half_rn(v);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---- host side ---------------------------------------------------------------------------------------------
bool gemv_tc3_supported(const GemvParams& p, int bits, int sm_count) {
  if (bits != 3 || p.group_shift != 6 || p.M != 1 || !p.B) return false;
  if (p.K % kTcSlice || p.K == 0 || p.N == 0) return false;
  if ((reinterpret_cast<uintptr_t>(p.X) & 15u) || (reinterpret_cast<uintptr_t>(p.W) & 15u) ||
      (reinterpret_cast<uintptr_t>(p.S) & 7u) || (p.B && (reinterpret_cast<uintptr_t>(p.B) & 7u)))
    return false;
  if (p.K / kTcSlice > (uint32_t)kTcWarps) {
    const uint32_t grid = p.N < (uint32_t)sm_count ? p.N : (uint32_t)sm_count;
    if ((((uint64_t)p.N + grid - 1) / grid + 1) * 4 > kT3MaxAccBytes) return false;
  }
  return true;
}

static cudaError_t launch_tc3_one(const GemvParams& p, unsigned grid, size_t smem, cudaStream_t st) {
  auto kern = gemv_tc3_kernel;
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kTcWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

cudaError_t launch_gemv_tc3(const GemvParams& p, int sm_count, cudaStream_t st) {
  const unsigned grid = p.N < (uint32_t)sm_count ? p.N : (unsigned)sm_count;
  size_t smem = kT3RingBytes + (size_t)2 * kTcWarps * kT3Rounds * 16 * 4;
  if (p.K / kTcSlice > (uint32_t)kTcWarps) smem += (((size_t)p.N + grid - 1) / grid + 1) * 4;
  return launch_tc3_one(p, grid, smem, st);
}

}  // namespace ztvm
