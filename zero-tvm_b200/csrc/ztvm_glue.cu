// Parity hooks (unpack / dequant) and the MoE glue kernels around the expert matmuls:
// router top-k, SiLU*up, weighted combine.
#include "ztvm_device.cuh"
#include "ztvm_kernels.h"
#include "ztvm_tc.cuh"

namespace ztvm {

// ---- parity hooks ------------------------------------------------------------------------------
// One thread per 8-code block. 4-bit: block = one word. 3-bit: block j of a 32-code unit is the
// 24-bit window at bit 24j of the unit's three words.
template <int BITS>
__device__ __forceinline__ void load_block_codes(const uint32_t* W, uint32_t KP, uint32_t n, uint32_t blk, float q[8]) {
  const uint32_t* row = W + (size_t)n * KP;
  if constexpr (BITS == 4) {
    codes4_f32(row[blk], q);
  } else if constexpr (BITS == 8) {
    codes8_f32(row[2 * blk], row[2 * blk + 1], q);
  } else {
    const uint32_t u = blk >> 2, j = blk & 3;
    const uint32_t w0 = row[u * 3], w1 = row[u * 3 + 1], w2 = row[u * 3 + 2];
    uint32_t win;
    switch (j) {
      case 0: win = window3(w0, w1, w2, 0); break;
      case 1: win = window3(w0, w1, w2, 1); break;
      case 2: win = window3(w0, w1, w2, 2); break;
      default: win = window3(w0, w1, w2, 3); break;
    }
    codes3_f32(win, q);
  }
}

template <int BITS>
__global__ void unpack_codes_kernel(const uint32_t* W, uint8_t* codes, uint32_t N, uint32_t K) {
  const uint32_t nblk = K >> 3, KP = K * BITS / 32;
  const size_t total = (size_t)N * nblk;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t n = (uint32_t)(i / nblk), blk = (uint32_t)(i - (size_t)n * nblk);
    float q[8];
    load_block_codes<BITS>(W, KP, n, blk, q);
    uint2 o;
    o.x = (uint32_t)q[0] | ((uint32_t)q[1] << 8) | ((uint32_t)q[2] << 16) | ((uint32_t)q[3] << 24);
    o.y = (uint32_t)q[4] | ((uint32_t)q[5] << 8) | ((uint32_t)q[6] << 16) | ((uint32_t)q[7] << 24);
    *reinterpret_cast<uint2*>(codes + i * 8) = o;
  }
}

template <int BITS, bool AFFINE, bool AS_F16>
__global__ void dequant_kernel(const uint32_t* W, const __half* S, const __half* B, void* out, uint32_t N, uint32_t K,
                               uint32_t group_shift) {
  const uint32_t nblk = K >> 3, KP = K * BITS / 32, SPR = K >> group_shift;
  const size_t total = (size_t)N * nblk;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t n = (uint32_t)(i / nblk), blk = (uint32_t)(i - (size_t)n * nblk);
    const uint32_t g = (blk << 3) >> group_shift;
    if constexpr (AS_F16 && BITS == 4) {
      // the tensor-core GEMMs (dense and grouped) build their f16 operand with dequant_word_w16: so does the hook
      const unsigned short s16 = reinterpret_cast<const unsigned short*>(S)[(size_t)n * SPR + g];
      const unsigned short b16 = AFFINE ? reinterpret_cast<const unsigned short*>(B)[(size_t)n * SPR + g] : (unsigned short)0;
      const uint4 v = dequant_word_w16<AFFINE>(W[(size_t)n * KP + blk], dq_group<AFFINE>(s16, b16));
      *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(out) + i * 8) = v;
      continue;
    }
    float q[8];
    load_block_codes<BITS>(W, KP, n, blk, q);
    const float s = __half2float(S[(size_t)n * SPR + g]);
    const float b = AFFINE ? __half2float(B[(size_t)n * SPR + g]) : 0.f;
    if constexpr (AS_F16) {
      __half h[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) h[k] = dequant_w16<AFFINE>(q[k], s, b);
      *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(out) + i * 8) = *reinterpret_cast<uint4*>(h);
    } else {
      float4 lo, hi;
      lo.x = dequant_w32<AFFINE>(q[0], s, b); lo.y = dequant_w32<AFFINE>(q[1], s, b);
      lo.z = dequant_w32<AFFINE>(q[2], s, b); lo.w = dequant_w32<AFFINE>(q[3], s, b);
      hi.x = dequant_w32<AFFINE>(q[4], s, b); hi.y = dequant_w32<AFFINE>(q[5], s, b);
      hi.z = dequant_w32<AFFINE>(q[6], s, b); hi.w = dequant_w32<AFFINE>(q[7], s, b);
      float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + i * 8);
      o[0] = lo; o[1] = hi;
    }
  }
}

// The codes as the streaming kernels see them: in-place masks that are f16 subnormals (codes4_inplace / codes3_inplace,
// the functions those kernels call), scaled back to integers. 4-bit: one thread per word. 3-bit: one thread per
// (row, scale group of 64 codes = six words), the unit a lane of the 3-bit GEMV owns.
__device__ __forceinline__ uint32_t sub_to_code(uint32_t halfbits, float scale) {
  return (uint32_t)(__half2float(__ushort_as_half((unsigned short)halfbits)) * scale);
}
template <int BITS>
__global__ void unpack_codes_streamed_kernel(const uint32_t* W, uint8_t* codes, uint32_t N, uint32_t K) {
  if constexpr (BITS == 4) {
    const uint32_t KP = K >> 3;
    const size_t total = (size_t)N * KP;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
      const Inplace4 c = codes4_inplace(W[i]);
      uint32_t q[8];
      q[0] = sub_to_code(c.lo04 & 0xFFFFu, kInplaceLoScale); q[4] = sub_to_code(c.lo04 >> 16, kInplaceLoScale);
      q[1] = sub_to_code(c.hi15 & 0xFFFFu, kInplaceHiScale); q[5] = sub_to_code(c.hi15 >> 16, kInplaceHiScale);
      q[2] = sub_to_code(c.lo26 & 0xFFFFu, kInplaceLoScale); q[6] = sub_to_code(c.lo26 >> 16, kInplaceLoScale);
      q[3] = sub_to_code(c.hi37 & 0xFFFFu, kInplaceHiScale); q[7] = sub_to_code(c.hi37 >> 16, kInplaceHiScale);
      uint2 o;
      o.x = q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24);
      o.y = q[4] | (q[5] << 8) | (q[6] << 16) | (q[7] << 24);
      *reinterpret_cast<uint2*>(codes + i * 8) = o;
    }
  } else {
    const uint32_t groups = K >> 6, KP = K / 32 * 3;
    const size_t total = (size_t)N * groups;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
      const uint32_t n = (uint32_t)(i / groups), g = (uint32_t)(i - (size_t)n * groups);
      uint32_t w[6];
#pragma unroll
      for (int j = 0; j < 6; ++j) w[j] = W[(size_t)n * KP + g * 6 + j];
      uint8_t* dst = codes + (size_t)n * K + (size_t)g * 64;
#pragma unroll
      for (int k = 0; k < kCodes3Views; ++k) {
        uint32_t r0, r1;
        codes3_inplace(w, k, r0, r1);
        const int c0 = codes3_view_first(k);
        dst[c0] = (uint8_t)sub_to_code(r0 & 0xFFFFu, 16777216.f);            // offset 0: q * 2^-24
        dst[c0 + 1] = (uint8_t)sub_to_code(r1 & 0xFFFFu, 2097152.f);         // offset 3: q * 2^-21
        if (k < 15) {
          dst[c0 + 6] = (uint8_t)sub_to_code(r0 >> 16, 4194304.f);           // offset 2: q * 2^-22
          dst[c0 + 7] = (uint8_t)sub_to_code(r1 >> 16, 524288.f);            // offset 5: q * 2^-19
        }
      }
    }
  }
}

static inline unsigned grid_for(size_t total, int block) {
  size_t g = (total + block - 1) / block;
  return (unsigned)(g > 148 * 32 ? 148 * 32 : (g ? g : 1));
}

cudaError_t launch_unpack_codes(const uint32_t* W, uint8_t* codes, uint32_t N, uint32_t K, int bits, cudaStream_t st) {
  const size_t total = (size_t)N * (K >> 3);
  if (bits == 4) unpack_codes_kernel<4><<<grid_for(total, 256), 256, 0, st>>>(W, codes, N, K);
  else if (bits == 8) unpack_codes_kernel<8><<<grid_for(total, 256), 256, 0, st>>>(W, codes, N, K);
  else unpack_codes_kernel<3><<<grid_for(total, 256), 256, 0, st>>>(W, codes, N, K);
  return cudaGetLastError();
}

cudaError_t launch_unpack_codes_streamed(const uint32_t* W, uint8_t* codes, uint32_t N, uint32_t K, int bits, cudaStream_t st) {
  if (bits == 4) unpack_codes_streamed_kernel<4><<<grid_for((size_t)N * (K >> 3), 256), 256, 0, st>>>(W, codes, N, K);
  else unpack_codes_streamed_kernel<3><<<grid_for((size_t)N * (K >> 6), 256), 256, 0, st>>>(W, codes, N, K);
  return cudaGetLastError();
}

cudaError_t launch_dequant(const uint32_t* W, const __half* S, const __half* B, void* out, uint32_t N, uint32_t K,
                           int bits, uint32_t group_shift, bool affine, bool as_f16, cudaStream_t st) {
  const size_t total = (size_t)N * (K >> 3);
  const unsigned g = grid_for(total, 256);
#define ZTVM_DQ(BITS_, AFF_, F16_) dequant_kernel<BITS_, AFF_, F16_><<<g, 256, 0, st>>>(W, S, B, out, N, K, group_shift)
  if (bits == 4) {
    if (affine) { if (as_f16) ZTVM_DQ(4, true, true); else ZTVM_DQ(4, true, false); }
    else        { if (as_f16) ZTVM_DQ(4, false, true); else ZTVM_DQ(4, false, false); }
  } else if (bits == 8) {
    if (as_f16) ZTVM_DQ(8, true, true); else ZTVM_DQ(8, true, false);
  } else {
    if (as_f16) ZTVM_DQ(3, true, true); else ZTVM_DQ(3, true, false);
  }
#undef ZTVM_DQ
  return cudaGetLastError();
}

// ---- embedding rows (embedding_affine.wgsl:38-57, embedding_affine_int8.wgsl) ------------------------------
// out[t][:] = the dequantised row input_ids[t] of an affine-quantised table, f16: the canonical W16 (what the vendor
// dequantiser stores), through the same word dequantiser as the GEMMs for 4-bit codes. One thread per 8 values.
template <int BITS>
__global__ void embedding_affine_kernel(const int32_t* __restrict__ input_ids, const uint32_t* __restrict__ W,
                                        const __half* __restrict__ S, const __half* __restrict__ B, __half* __restrict__ out,
                                        uint32_t seq_len, uint32_t D, uint32_t vocab, uint32_t* err) {
  const uint32_t nblk = D >> 3, KP = D * BITS / 32, SPR = D >> 6;
  const size_t total = (size_t)seq_len * nblk;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t t = (uint32_t)(i / nblk), blk = (uint32_t)(i - (size_t)t * nblk);
    const int32_t id = input_ids[t];
    if (id < 0 || (uint32_t)id >= vocab) {          // counted, the row is left untouched
      if (blk == 0) atomicAdd(err, 1u);
      continue;
    }
    const size_t n = (size_t)id;
    const uint32_t g = blk >> 3;
    const unsigned short s16 = reinterpret_cast<const unsigned short*>(S)[n * SPR + g];
    const unsigned short b16 = reinterpret_cast<const unsigned short*>(B)[n * SPR + g];
    uint4 v;
    if constexpr (BITS == 4) {
      v = dequant_word_w16<true>(W[n * KP + blk], dq_group<true>(s16, b16));
    } else {
      float q[8];
      codes8_f32(W[n * KP + 2 * blk], W[n * KP + 2 * blk + 1], q);
      const float sf = __half2float(__ushort_as_half(s16)), bf = __half2float(__ushort_as_half(b16));
      __half h[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) h[k] = dequant_w16<true>(q[k], sf, bf);
      v = *reinterpret_cast<uint4*>(h);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * D + (size_t)blk * 8) = v;
  }
}
cudaError_t launch_embedding_affine(const int32_t* input_ids, const uint32_t* W, const __half* S, const __half* B, __half* out,
                                    uint32_t seq_len, uint32_t D, uint32_t vocab, int bits, uint32_t* err, cudaStream_t st) {
  const size_t total = (size_t)seq_len * (D >> 3);
  if (total == 0) return cudaSuccess;
  if (bits == 4) embedding_affine_kernel<4><<<grid_for(total, 256), 256, 0, st>>>(input_ids, W, S, B, out, seq_len, D, vocab, err);
  else embedding_affine_kernel<8><<<grid_for(total, 256), 256, 0, st>>>(input_ids, W, S, B, out, seq_len, D, vocab, err);
  return cudaGetLastError();
}

// ---- f16 matvec with f32 accumulation and f32 output (moe_router_logits_f16.wgsl) -------------------------------
// y[t][e] = sum_i f32(x[t][i]) * f32(w[e][i]). One warp per (row e, slab of up to 8 tokens); 16-byte loads.
__global__ void __launch_bounds__(256) f16_matvec_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                                                          float* __restrict__ y, uint32_t D, uint32_t rows, uint32_t tokens) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint32_t t0 = blockIdx.y * 8u;
  if (e >= rows) return;
  const uint32_t nt = min(8u, tokens - t0);
  float acc[8];
#pragma unroll
  for (int m = 0; m < 8; ++m) acc[m] = 0.f;
  for (uint32_t c = lane; c < D / 8u; c += 32u) {
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w + (size_t)e * D) + c);
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      if ((uint32_t)m >= nt) break;
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + (size_t)(t0 + m) * D) + c);
      const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 a = __half22float2(u32_as_h2(xw[k])), b = __half22float2(u32_as_h2(ww[k]));
        acc[m] = fmaf(a.x, b.x, acc[m]);
        acc[m] = fmaf(a.y, b.y, acc[m]);
      }
    }
  }
  for (uint32_t i = (D / 8u) * 8u + lane; i < D; i += 32u)        // tail when D % 8 != 0
    for (uint32_t m = 0; m < nt; ++m)
      acc[m] = fmaf(__half2float(x[(size_t)(t0 + m) * D + i]), __half2float(w[(size_t)e * D + i]), acc[m]);
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && (uint32_t)m < nt) y[(size_t)(t0 + m) * rows + e] = v;
  }
}
cudaError_t launch_f16_matvec(const __half* x, const __half* w, float* y, uint32_t D, uint32_t rows, uint32_t tokens, cudaStream_t st) {
  if (rows == 0 || tokens == 0) return cudaSuccess;
  for (uint32_t t0 = 0; t0 < tokens; t0 += 8u * 65535u) {       // grid.y carries the token slab
    const uint32_t nt = min(tokens - t0, 8u * 65535u);
    dim3 grid((rows + 7) / 8, (nt + 7) / 8);
    f16_matvec_kernel<<<grid, 256, 0, st>>>(x + (size_t)t0 * D, w, y + (size_t)t0 * rows, D, rows, nt);
  }
  return cudaGetLastError();
}

// ---- router top-k ------------------------------------------------------------------------------
// One warp per token. Each lane keeps experts lane, lane+32, ... (up to 32 per lane, E <= 1024) in
// registers. softmax over the E routed experts in f32, then K rounds of arg-max; ties go to the lower
// expert index; the winner is masked with -1. Scores are written in descending order, then the shared
// expert (index E) with sigmoid of its own logit when present (moe_router_topk.wgsl:83-135).
constexpr int kTopkPerLane = 32;

template <int PER>
__global__ void __launch_bounds__(128) route_topk_kernel(const float* __restrict__ logits, uint32_t* __restrict__ ids,
                                                          float* __restrict__ scores, uint32_t tokens, uint32_t E,
                                                          uint32_t K, uint32_t norm_topk, uint32_t has_shared) {
  const int lane = threadIdx.x & 31;
  const uint32_t tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= tokens) return;
  const float* l = logits + (size_t)tok * (E + has_shared);
  const size_t obase = (size_t)tok * (K + has_shared);

  float pv[PER];
  float m = -3.0e38f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const uint32_t e = (uint32_t)i * 32 + lane;
    const float v = e < E ? l[e] : -3.0e38f;
    pv[i] = v;
    m = fmaxf(m, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const uint32_t e = (uint32_t)i * 32 + lane;
    const float v = e < E ? expf(pv[i] - m) : 0.f;
    pv[i] = e < E ? v : -1.f;
    s += e < E ? v : 0.f;
  }
  const float denom = warp_sum(s);

  float total = 0.f;
  float my_top = 0.f;  // lane k keeps the k-th winner
  for (uint32_t k = 0; k < K; ++k) {
    float bv = -1.f;
    uint32_t bi = 0xffffffffu;
#pragma unroll
    for (int i = 0; i < PER; ++i) {  // ascending expert index within the lane: strict > keeps the lower one
      if (pv[i] > bv) { bv = pv[i]; bi = (uint32_t)i * 32 + lane; }
    }
    float best = bv;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
    uint32_t widx = bv == best ? bi : 0xffffffffu;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) widx = min(widx, __shfl_xor_sync(0xffffffffu, widx, o));
    total += best;
    if ((uint32_t)lane == k) my_top = best;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      if ((uint32_t)i * 32 + lane == widx) pv[i] = -1.f;
    if (lane == 0) ids[obase + k] = widx;
  }
  const float scale = norm_topk ? 1.0f / total : 1.0f / denom;
  if ((uint32_t)lane < K) scores[obase + lane] = my_top * scale;
  if (has_shared && lane == 0) {
    ids[obase + K] = E;
    scores[obase + K] = 1.0f / (1.0f + expf(-l[E]));
  }
}

cudaError_t launch_route_topk(const float* logits, uint32_t* ids, float* scores, uint32_t tokens, uint32_t E,
                              uint32_t K, bool norm_topk, bool has_shared, cudaStream_t st) {
  const unsigned grid = (tokens + 3) / 4;
  if (E <= 256) route_topk_kernel<8><<<grid, 128, 0, st>>>(logits, ids, scores, tokens, E, K, norm_topk, has_shared);
  else route_topk_kernel<kTopkPerLane><<<grid, 128, 0, st>>>(logits, ids, scores, tokens, E, K, norm_topk, has_shared);
  return cudaGetLastError();
}

// ---- SiLU * up -----------------------------------------------------------------------------------
// Rows of [gate(ffn) | up(ffn)] f16 -> f16 [ffn]; f32 arithmetic (silu_mul.wgsl:40-43).
__device__ __forceinline__ float silu_mul_one(float g, float u) {
  const float sg = g * (1.0f / (1.0f + expf(-g)));
  return u * sg;
}
// VEC = 8: eight elements per thread (16-byte loads and stores; ffn % 8 == 0, 16-byte aligned buffers), else one.
template <int VEC>
__global__ void silu_mul_kernel(const __half* __restrict__ gate_up, __half* __restrict__ h, uint32_t rows, uint32_t ffn,
                                const uint32_t* __restrict__ seg_counts, uint32_t seg_cap) {
  const uint32_t per_row = ffn / VEC;
  const size_t total = (size_t)rows * per_row;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / per_row, c = (i - r * per_row) * VEC;
    if (seg_counts && (uint32_t)(r % seg_cap) >= seg_counts[r / seg_cap]) continue;   // past the region's live rows
    if constexpr (VEC == 8) {
      const uint4 gv = *reinterpret_cast<const uint4*>(gate_up + r * 2 * ffn + c);
      const uint4 uv = *reinterpret_cast<const uint4*>(gate_up + r * 2 * ffn + ffn + c);
      const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
      uint32_t ow[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 g2 = __half22float2(u32_as_h2(gw[k])), u2 = __half22float2(u32_as_h2(uw[k]));
        const __half2 o = __floats2half2_rn(silu_mul_one(g2.x, u2.x), silu_mul_one(g2.y, u2.y));
        ow[k] = *reinterpret_cast<const uint32_t*>(&o);
      }
      *reinterpret_cast<uint4*>(h + r * ffn + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    } else {
      const float g = __half2float(gate_up[r * 2 * ffn + c]);
      const float u = __half2float(gate_up[r * 2 * ffn + ffn + c]);
      h[r * ffn + c] = __float2half_rn(silu_mul_one(g, u));
    }
  }
}
cudaError_t launch_silu_mul(const __half* gate_up, __half* h, uint32_t rows, uint32_t ffn, cudaStream_t st,
                            const uint32_t* seg_counts, uint32_t seg_cap) {
  const size_t total = (size_t)rows * ffn;
  if (total == 0) return cudaSuccess;
  const bool vec = ffn % 8 == 0 && ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(h)) & 15u) == 0;
  if (vec) silu_mul_kernel<8><<<grid_for(total / 8, 256), 256, 0, st>>>(gate_up, h, rows, ffn, seg_counts, seg_cap ? seg_cap : 1u);
  else silu_mul_kernel<1><<<grid_for(total, 256), 256, 0, st>>>(gate_up, h, rows, ffn, seg_counts, seg_cap ? seg_cap : 1u);
  return cudaGetLastError();
}

// The same over f32 [gate(ffn) | up(ffn)] rows: the second step of the fused FFN on shapes the paired GEMV does not
// take (fused_ffn.wgsl keeps both dot products in f32 up to the final store).
__global__ void silu_mul_f32_kernel(const float* __restrict__ gate_up, __half* __restrict__ h, uint32_t rows, uint32_t ffn) {
  const size_t total = (size_t)rows * ffn;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / ffn, c = i - r * ffn;
    h[i] = __float2half_rn(silu_mul_one(gate_up[r * 2 * ffn + c], gate_up[r * 2 * ffn + ffn + c]));
  }
}
cudaError_t launch_silu_mul_f32(const float* gate_up, __half* h, uint32_t rows, uint32_t ffn, cudaStream_t st) {
  const size_t total = (size_t)rows * ffn;
  if (total == 0) return cudaSuccess;
  silu_mul_f32_kernel<<<grid_for(total, 256), 256, 0, st>>>(gate_up, h, rows, ffn);
  return cudaGetLastError();
}

// ---- weighted combine -----------------------------------------------------------------------------
// out[t][i] = f16(sum_s score[t][s] * f32(y[t][s][i])), slots added in index order (moe_combine.wgsl:39-43).
template <int VEC>
__global__ void moe_combine_kernel(const __half* __restrict__ y, const float* __restrict__ scores, __half* __restrict__ out,
                                   uint32_t tokens, uint32_t slots, uint32_t d) {
  const uint32_t per_row = d / VEC;
  const size_t total = (size_t)tokens * per_row;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / per_row, c = (i - t * per_row) * VEC;
    float acc[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] = 0.f;
    for (uint32_t s = 0; s < slots; ++s) {
      const float sc = scores[t * slots + s];
      const __half* src = y + (t * slots + s) * d + c;
      if constexpr (VEC == 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(src);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __half22float2(u32_as_h2(w[k]));
          acc[2 * k] = __fadd_rn(acc[2 * k], __fmul_rn(sc, f.x));
          acc[2 * k + 1] = __fadd_rn(acc[2 * k + 1], __fmul_rn(sc, f.y));
        }
      } else {
        acc[0] = __fadd_rn(acc[0], __fmul_rn(sc, __half2float(src[0])));
      }
    }
    if constexpr (VEC == 8) {
      uint32_t ow[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __half2 o = __floats2half2_rn(acc[2 * k], acc[2 * k + 1]);
        ow[k] = *reinterpret_cast<const uint32_t*>(&o);
      }
      *reinterpret_cast<uint4*>(out + t * d + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    } else {
      out[t * d + c] = __float2half_rn(acc[0]);
    }
  }
}
cudaError_t launch_moe_combine(const __half* y_slots, const float* scores, __half* out, uint32_t tokens,
                               uint32_t slots, uint32_t d, cudaStream_t st) {
  const size_t total = (size_t)tokens * d;
  if (total == 0) return cudaSuccess;
  const bool vec = d % 8 == 0 && ((reinterpret_cast<uintptr_t>(y_slots) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
  if (vec) moe_combine_kernel<8><<<grid_for(total / 8, 256), 256, 0, st>>>(y_slots, scores, out, tokens, slots, d);
  else moe_combine_kernel<1><<<grid_for(total, 256), 256, 0, st>>>(y_slots, scores, out, tokens, slots, d);
  return cudaGetLastError();
}

}  // namespace ztvm
