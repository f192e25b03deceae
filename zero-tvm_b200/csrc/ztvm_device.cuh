// Device-side building blocks shared by every kernel of the library: code unpacking, the two
// canonical dequantisers, small load/reduce helpers. The parity hooks (ztvm_unpack_codes,
// ztvm_dequant) call exactly these functions, so what they materialise is what the fused
// kernels consume.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ztvm {

// ---- loads ---------------------------------------------------------------------------------
// Streaming 128-bit load: weights are read exactly once, so they bypass L1 allocation.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float ld_f16_as_f32(const __half* p) { return __half2float(__ldg(p)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- 4-bit codes ---------------------------------------------------------------------------
// Code i of a word sits at bits [4i, 4i+4). The eight codes come out as four half2 holding the
// exact integers, in the pair order (q0,q4) (q1,q5) (q2,q6) (q3,q7):
//   (w & 0x000F000F) | 0x64006400 is the half pair (1024+q0, 1024+q4): the nibble lands in the
//   low mantissa bits of 1024.0; (w & 0x00F000F0) | 0x54005400 is (64+q1, 64+q5): the nibble
//   lands four bits up in the mantissa of 64.0, whose ulp is 1/16. One shift by 8 gives the
//   other four. Subtracting the offsets in half precision is exact.
struct Codes8 {
  __half2 p04, p15, p26, p37;
};
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & b) | c
  return r;
}
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

__device__ __forceinline__ Codes8 unpack4(uint32_t w) {
  const __half2 k1024 = u32_as_h2(0x64006400u), k64 = u32_as_h2(0x54005400u);
  const uint32_t w8 = w >> 8;
  Codes8 c;
  c.p04 = __hsub2(u32_as_h2(lop3_and_or(w, 0x000F000Fu, 0x64006400u)), k1024);
  c.p15 = __hsub2(u32_as_h2(lop3_and_or(w, 0x00F000F0u, 0x54005400u)), k64);
  c.p26 = __hsub2(u32_as_h2(lop3_and_or(w8, 0x000F000Fu, 0x64006400u)), k1024);
  c.p37 = __hsub2(u32_as_h2(lop3_and_or(w8, 0x00F000F0u, 0x54005400u)), k64);
  return c;
}
// The same eight codes WITHOUT any arithmetic: a nibble masked where it sits is already an f16 subnormal,
// (w & 0x000F) = q * 2^-24 and (w & 0x00F0) = q * 2^-20 in each 16-bit half. The four registers hold the pairs
// (q0,q4) * 2^-24, (q1,q5) * 2^-20, (q2,q6) * 2^-24, (q3,q7) * 2^-20. Every streaming kernel (the persistent GEMV, the
// tiled GEMVs, the streaming grouped MoE kernel) feeds its multiplier array with exactly these registers, and the
// parity hook ztvm_unpack_codes_streamed turns them back into integers.
struct Inplace4 {
  uint32_t lo04, hi15, lo26, hi37;
};
__device__ __forceinline__ Inplace4 codes4_inplace(uint32_t w) {
  const uint32_t w8 = w >> 8;
  Inplace4 c;
  c.lo04 = w & 0x000F000Fu;
  c.hi15 = w & 0x00F000F0u;
  c.lo26 = w8 & 0x000F000Fu;
  c.hi37 = w8 & 0x00F000F0u;
  return c;
}
constexpr float kInplaceLoScale = 16777216.f;   // 2^24: subnormal of the low-nibble mask -> integer code
constexpr float kInplaceHiScale = 1048576.f;    // 2^20: subnormal of the high-nibble mask -> integer code

// The eight codes as f32, in natural order q[0..7].
__device__ __forceinline__ void codes4_f32(uint32_t w, float q[8]) {
  Codes8 c = unpack4(w);
  float2 a = __half22float2(c.p04), b = __half22float2(c.p15), d = __half22float2(c.p26),
         e = __half22float2(c.p37);
  q[0] = a.x; q[4] = a.y; q[1] = b.x; q[5] = b.y; q[2] = d.x; q[6] = d.y; q[3] = e.x; q[7] = e.y;
}

// ---- 8-bit codes ---------------------------------------------------------------------------
// Four codes per word, code i at bits [8i, 8i+8) (src/compiler/shaders/int8_affine_matvec.wgsl,
// moe_router_logits.wgsl: `(word >> (8u * n)) & 255u`). A block of eight codes is two words.
__device__ __forceinline__ void codes8_f32(uint32_t w0, uint32_t w1, float q[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    q[i] = (float)((w0 >> (8 * i)) & 255u);
    q[4 + i] = (float)((w1 >> (8 * i)) & 255u);
  }
}

// ---- 3-bit codes ---------------------------------------------------------------------------
// A row is one LSB-first bitstream; 32 codes occupy exactly three words. Codes 8b..8b+7 of such a
// triple are the 24-bit window starting at bit 24b.
__device__ __forceinline__ uint32_t window3(uint32_t w0, uint32_t w1, uint32_t w2, int b) {
  // b: 0..3 (compile-time after unrolling)
  switch (b) {
    case 0: return w0 & 0xFFFFFFu;
    case 1: return ((w0 >> 24) | (w1 << 8)) & 0xFFFFFFu;
    case 2: return ((w1 >> 16) | (w2 << 16)) & 0xFFFFFFu;
    default: return w2 >> 8;
  }
}
__device__ __forceinline__ void codes3_f32(uint32_t win, float q[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] = (float)((win >> (3 * i)) & 7u);
}

// In-place 3-bit codes for the matrix unit. `w` holds one scale group of a row: 64 codes = 192 bits = six words.
// A 3-bit code anywhere in bits 0..9 of a 16-bit half is an f16 subnormal q * 2^(o-24) (o = its bit offset in the half).
// View k (0..16) is the 32-bit window of the stream that starts on code c = codes3_view_first(k): its low half holds
// codes c, c+1 at offsets 0, 3 and its high half codes c+6, c+7 at offsets 2, 5, so two ANDs give
//   r0 = (code c | code c+6)   with values q * 2^-24 | q * 2^-22
//   r1 = (code c+1 | code c+7) with values q * 2^-21 | q * 2^-19
// Views 0..14 tile codes 0..59 in pairs (c = 12 (k/3) + 2 (k%3)); views 15, 16 cover codes 60..63 with their low half
// only. The powers of two are moved onto the activations by the kernel that multiplies.
__host__ __device__ constexpr int codes3_view_first(int k) { return k < 15 ? 12 * (k / 3) + 2 * (k % 3) : 60 + 2 * (k - 15); }
constexpr int kCodes3Views = 17;
__device__ __forceinline__ void codes3_inplace(const uint32_t (&w)[6], int k, uint32_t& r0, uint32_t& r1) {
  constexpr uint32_t kM0 = 0x001C0007u, kM1 = 0x00E00038u;
  const int bit = 3 * codes3_view_first(k), j = bit >> 5, sh = bit & 31;
  uint32_t v;
  if (sh == 0) v = w[j];
  else if (sh <= 8 || j == 5) v = w[j] >> sh;             // the window fits in one word
  else v = __funnelshift_r(w[j], w[j + 1 < 6 ? j + 1 : 5], sh);
  r0 = v & (k < 15 ? kM0 : (kM0 & 0xFFFFu));
  r1 = v & (k < 15 ? kM1 : (kM1 & 0xFFFFu));
}

// ---- canonical dequantisers ----------------------------------------------------------------
// W32 = fl32(s*q + b) (affine) or fl32(s*(q-7)) (symmetric). s*q is exact in f32 (11-bit
// significand times a 4-bit integer), so fmaf and mul-then-add give the same bits.
template <bool AFFINE>
__device__ __forceinline__ float dequant_w32(float q, float s, float b) {
  return AFFINE ? fmaf(s, q, b) : s * (q - 7.0f);
}
// W16 = f16_rne(W32): the value a tensor-core GEMM multiplies with.
template <bool AFFINE>
__device__ __forceinline__ __half dequant_w16(float q, float s, float b) {
  return __float2half_rn(dequant_w32<AFFINE>(q, s, b));
}

}  // namespace ztvm
