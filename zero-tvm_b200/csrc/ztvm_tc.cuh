// Tensor-core plumbing shared by the GEMM kernels: mbarrier / TMA / tcgen05 wrappers (inline PTX for sm_100a),
// shared-memory and instruction descriptors, and the f16 weight builder.
#pragma once
#include <cuda.h>

#include "ztvm_device.cuh"

namespace ztvm {

constexpr int kGemmBK = 64;         // k elements per stage = one 128-byte swizzle row of f16
constexpr unsigned long long kWaitCycles = 2000000000ull;  // ~1 s at 2 GHz

// ---- PTX wrappers ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false (and a raised status word) when the phase does not complete in about a second.
// `nap_ns`: sleep between polls. A role that waits for a whole main loop (an epilogue, a producer many slots ahead)
// passes a long nap: its polls are instructions taken from the warps that have work.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t* status, uint32_t code,
                                          volatile uint32_t* abort_flag, uint32_t nap_ns = 40u) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    // A waiting warp shares its scheduler with warps that have work: between polls it sleeps, and the abort flag and
    // the clock are looked at once per 32 polls only.
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      __nanosleep(nap_ns);
    }
    if (*abort_flag) return false;
    if ((unsigned long long)(clock64() - t0) > kWaitCycles) {
      *abort_flag = 1u;
      atomicExch(status, code);
      return false;
    }
  }
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tmap, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
// Commits the bulk stores issued so far and waits until their shared-memory source has been read (the staging tile may
// then be reused or the CTA may exit; the global writes complete on their own before the grid is reported finished).
__device__ __forceinline__ void tma_store_commit_and_wait() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], f16 inputs, f32 accumulate
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
// The same MMA with the A operand in tensor memory (lane = row of A, one 32-bit column = two k-adjacent f16).
__device__ __forceinline__ void umma_f16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes (64 f16) in the 128-byte
// swizzle: 8-row groups are 1024 bytes apart (stride byte offset), the leading byte offset is unused,
// descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);          // start address >> 4, bits [0,14)
  d |= (uint64_t)1 << 16;                            // leading byte offset (ignored for swizzled K-major)
  d |= (uint64_t)(1024u >> 4) << 32;                 // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                            // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
  return d;
}
// Instruction descriptor: f32 accumulate, f16 A and B, both K-major, M = 128, N = BN.
__host__ __device__ constexpr uint32_t idesc_f16(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// ---- the f16 weight builder of the tensor-core GEMMs -----------------------------------------------------------------
// Canonical weight: W16 = f16_rne(fl32(s*q + b)) (affine) or f16_rne(s*(q-7)) (symmetric), q the exact integer code.
//
// Fast path: one half-precision FMA per PAIR of codes. hfma2 rounds the exact value s*q + b once, to f16; the canonical
// definition rounds it to f32 first. The two agree whenever s*q + b is exactly representable in f32, because the first
// rounding is then the identity. With s = Ms * 2^es and b = Mb * 2^eb (|Ms|, |Mb| < 2^11, es / eb the exponents of the
// last place: max(E, 1) - 25 for a biased exponent field E) and q <= 15, the sum is an integer below 2^24 times
// 2^min(es, eb) as soon as -12 <= es - eb <= 8 (or one of the two is zero): exact in f32. Real checkpoints sit well
// inside (b is a few times s); a group outside takes the slow path below, which builds the f32 value explicitly. So
// both paths give the canonical bits, always; the fast one needs no f16 <-> f32 conversion at all (those run on the
// quarter-rate conversion unit and used to bound every kernel that dequantises on the fly).
struct DqGroup {
  __half2 s2, b2;        // scale / bias of the group in both halves
  float sf, bf;          // the same, widened (slow path)
  unsigned short s16;
  bool fast;
};
template <bool AFFINE>
__device__ __forceinline__ DqGroup dq_group(unsigned short s16, unsigned short b16) {
  DqGroup g;
  g.s16 = s16;
  g.s2 = u32_as_h2((uint32_t)s16 * 0x10001u);
  g.b2 = u32_as_h2((uint32_t)b16 * 0x10001u);
  g.sf = __half2float(__ushort_as_half(s16));
  g.bf = AFFINE ? __half2float(__ushort_as_half(b16)) : 0.f;
  if (AFFINE) {
    const int es = max((int)((s16 >> 10) & 31u), 1), eb = max((int)((b16 >> 10) & 31u), 1);
    const int d = es - eb;
    g.fast = (s16 & 0x7FFFu) == 0u || (b16 & 0x7FFFu) == 0u || (d >= -12 && d <= 8);
  } else {
    g.fast = true;       // s * (q - 7): an 11-bit by 4-bit product is exact in f32 whatever the scale
  }
  return g;
}

__device__ __forceinline__ uint32_t h2_as_u32(const __half2& h) { return *reinterpret_cast<const uint32_t*>(&h); }

// Dequantise one 8-code word into 8 f16 weights in natural order (as one uint4).
template <bool AFFINE>
__device__ __forceinline__ uint4 dequant_word_w16(uint32_t w, const DqGroup& g) {
  const Codes8 c = unpack4(w);  // exact integer codes as f16 pairs (q0,q4)(q1,q5)(q2,q6)(q3,q7)
  uint4 o;
  if (g.fast) {
    __half2 r04, r15, r26, r37;
    if (AFFINE) {
      r04 = __hfma2(c.p04, g.s2, g.b2); r15 = __hfma2(c.p15, g.s2, g.b2);
      r26 = __hfma2(c.p26, g.s2, g.b2); r37 = __hfma2(c.p37, g.s2, g.b2);
    } else {
      const __half2 k7 = u32_as_h2(0x47004700u);   // 7.0
      r04 = __hmul2(__hsub2(c.p04, k7), g.s2); r15 = __hmul2(__hsub2(c.p15, k7), g.s2);
      r26 = __hmul2(__hsub2(c.p26, k7), g.s2); r37 = __hmul2(__hsub2(c.p37, k7), g.s2);
    }
    o.x = __byte_perm(h2_as_u32(r04), h2_as_u32(r15), 0x5410);   // (w0, w1)
    o.y = __byte_perm(h2_as_u32(r26), h2_as_u32(r37), 0x5410);   // (w2, w3)
    o.z = __byte_perm(h2_as_u32(r04), h2_as_u32(r15), 0x7632);   // (w4, w5)
    o.w = __byte_perm(h2_as_u32(r26), h2_as_u32(r37), 0x7632);   // (w6, w7)
    return o;
  }
  // slow path: fma.rn.f32.f16 multiplies the two f16 operands exactly and adds the f32 bias with one rounding (the same
  // bits as dequant_w32<true>: s*q is exact in f32 either way), then one round-to-nearest-even to f16
  float v[8];
  auto two = [&](const __half2& q2, int i_lo, int i_hi) {
    unsigned short q_lo, q_hi;
    asm("mov.b32 {%0,%1}, %2;" : "=h"(q_lo), "=h"(q_hi) : "r"(h2_as_u32(q2)));
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(v[i_lo]) : "h"(g.s16), "h"(q_lo), "f"(g.bf));
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(v[i_hi]) : "h"(g.s16), "h"(q_hi), "f"(g.bf));
  };
  two(c.p04, 0, 4);
  two(c.p15, 1, 5);
  two(c.p26, 2, 6);
  two(c.p37, 3, 7);
  o.x = h2_as_u32(__floats2half2_rn(v[0], v[1]));
  o.y = h2_as_u32(__floats2half2_rn(v[2], v[3]));
  o.z = h2_as_u32(__floats2half2_rn(v[4], v[5]));
  o.w = h2_as_u32(__floats2half2_rn(v[6], v[7]));
  return o;
}

}  // namespace ztvm
