/* CPU oracle, fast twin of ztvm_oracle.py (plain C + OpenMP).
 *
 * TEST INFRASTRUCTURE ONLY: linked by nothing in the shipped library. It is
 * loaded by the test-suite, the smoke check and the CPU-baseline / reference
 * arm of the benchmark, always as the checker or the timed CPU baseline.
 *
 * It restates the arithmetic of the Zero-TVM int4/int3 dequant-matmul shaders
 * (paths relative to the reference project):
 *   unpack      src/compiler/shaders/int4_matmul.gen.ts:157-167 (4-bit), :409-448 (3-bit windows)
 *   GEMV order  src/compiler/shaders/int4_matmul.gen.ts:388-408,449-464 (per word s*dot + b*xs, f32)
 *   batched     src/compiler/shaders/int4_matmul.gen.ts:580-695 (same math per batch row)
 *   f32 dequant src/compiler/shaders/int4_matmul.gen.ts:1001-1002
 *   f16 dequant scripts/make-dsv2-layer-ref.py:108-116 (f16 of the f32 value)
 *   MoE ids     src/compiler/shaders/int4_matmul.gen.ts:229-254
 *   routing     src/compiler/shaders/moe_router_topk.wgsl:83-135
 *   silu / combine  src/compiler/shaders/silu_mul.wgsl:40-43, moe_combine.wgsl:39-43
 *
 * Parity status: the 4-bit affine dequantiser is pinned through tests/golden
 * (outputs of the reference's own numpy dequant_from); the rest is pinned by
 * formula against ztvm_oracle.py ("parity unpinned" versus executed reference).
 *
 * Build: see oracle/Makefile (no -march=native: the .so travels to other hosts;
 * -ffp-contract=off keeps mul+add roundings identical to numpy's).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float h2f(uint16_t h) {
  _Float16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}
static inline uint16_t f2h(float f) {
  _Float16 v = (_Float16)f; /* round-to-nearest-even */
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}

int zo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* code k of a row ------------------------------------------------------- */
static inline uint32_t code4(const uint32_t* row, long k) { return (row[k >> 3] >> (4 * (k & 7))) & 15u; }

/* 3-bit: 8-code block blk = 24-bit window at bit 24*blk (gen.ts:436-439,412-414) */
static inline uint32_t window3(const uint32_t* row, long blk) {
  uint64_t bit = (uint64_t)blk * 24u;
  uint32_t sh = (uint32_t)(bit & 31u);
  uint32_t win = row[bit >> 5] >> sh;
  if (sh > 8u) win |= row[(bit >> 5) + 1] << (32u - sh);
  return win & 0xFFFFFFu;
}

/* 8 codes of block blk into q[8] */
static inline void block_codes(const uint32_t* row, long blk, int bits, float q[8]) {
  if (bits == 4) {
    uint32_t p = row[blk];
    for (int i = 0; i < 8; ++i) q[i] = (float)((p >> (4 * i)) & 15u);
  } else if (bits == 8) { /* four bytes per word (int8_affine_matvec.wgsl: (word >> 8n) & 255) */
    for (int i = 0; i < 8; ++i) q[i] = (float)((row[2 * blk + (i >> 2)] >> (8 * (i & 3))) & 255u);
  } else {
    uint32_t w = window3(row, blk);
    for (int i = 0; i < 8; ++i) q[i] = (float)((w >> (3 * i)) & 7u);
  }
}

void zo_unpack_codes(const uint32_t* W, uint8_t* q, long N, long K, int bits) {
  long KP = K * bits / 32;
#pragma omp parallel for schedule(static)
  for (long n = 0; n < N; ++n) {
    const uint32_t* row = W + n * KP;
    for (long blk = 0; blk < K / 8; ++blk) {
      float c[8];
      block_codes(row, blk, bits, c);
      for (int i = 0; i < 8; ++i) q[n * K + blk * 8 + i] = (uint8_t)c[i];
    }
  }
}

/* W32 = fl32(s*q + b) | fl32(s*(q-7));  out_f16 != 0 -> W16 = f16_rne(W32) */
void zo_dequant(const uint32_t* W, const uint16_t* s, const uint16_t* b, void* out, long N, long K, int bits,
                int group, int affine, int out_f16) {
  long KP = K * bits / 32, SPR = K / group;
#pragma omp parallel for schedule(static)
  for (long n = 0; n < N; ++n) {
    const uint32_t* row = W + n * KP;
    for (long blk = 0; blk < K / 8; ++blk) {
      float c[8];
      block_codes(row, blk, bits, c);
      long g = (blk * 8) / group;
      float sc = h2f(s[n * SPR + g]);
      float bi = affine ? h2f(b[n * SPR + g]) : 0.0f;
      for (int i = 0; i < 8; ++i) {
        float w = affine ? (sc * c[i] + bi) : (sc * (c[i] - 7.0f));
        long o = n * K + blk * 8 + i;
        if (out_f16) ((uint16_t*)out)[o] = f2h(w);
        else ((float*)out)[o] = w;
      }
    }
  }
}

/* y[m,n] = sum_k f64(x[m,k]) * f64(Wdq[n,k]); Wdq = W32, or W16 when w16 != 0. */
void zo_matmul_f64(const uint16_t* x, const uint32_t* W, const uint16_t* s, const uint16_t* b, double* y, long M,
                   long N, long K, int bits, int group, int affine, int w16) {
  long KP = K * bits / 32, SPR = K / group;
#pragma omp parallel
  {
    double* wrow = (double*)malloc(sizeof(double) * (size_t)K);
#pragma omp for schedule(static)
    for (long n = 0; n < N; ++n) {
      const uint32_t* row = W + n * KP;
      for (long blk = 0; blk < K / 8; ++blk) {
        float c[8];
        block_codes(row, blk, bits, c);
        long g = (blk * 8) / group;
        float sc = h2f(s[n * SPR + g]);
        float bi = affine ? h2f(b[n * SPR + g]) : 0.0f;
        for (int i = 0; i < 8; ++i) {
          float w = affine ? (sc * c[i] + bi) : (sc * (c[i] - 7.0f));
          if (w16) w = h2f(f2h(w));
          wrow[blk * 8 + i] = (double)w;
        }
      }
      for (long m = 0; m < M; ++m) {
        const uint16_t* xr = x + m * K;
        double acc = 0.0;
        for (long k = 0; k < K; ++k) acc += (double)h2f(xr[k]) * wrow[k];
        y[m * N + n] = acc;
      }
    }
    free(wrow);
  }
}

/* One output in the shader's order: lane t owns blocks t, t+lanes, ...; per block
 * acc += s*((x0q0+x1q1)+(x2q2+x3q3)+...) + b*(x0+...+x7); lanes summed pairwise. */
static inline float gemv_row_ref(const float* xf, const uint32_t* row, const uint16_t* s, const uint16_t* b,
                                 long K, int bits, int group, int affine, int lanes) {
  float acc[64];
  for (int t = 0; t < lanes; ++t) acc[t] = 0.0f;
  long nblk = K / 8;
  for (long blk = 0; blk < nblk; ++blk) {
    float c[8];
    block_codes(row, blk, bits, c);
    const float* xi = xf + blk * 8;
    long g = (blk * 8) / group;
    float sc = h2f(s[g]);
    float t0, t1, t2, t3;
    if (affine) {
      t0 = xi[0] * c[0] + xi[1] * c[1];
      t1 = xi[2] * c[2] + xi[3] * c[3];
      t2 = xi[4] * c[4] + xi[5] * c[5];
      t3 = xi[6] * c[6] + xi[7] * c[7];
    } else {
      t0 = xi[0] * (c[0] - 7.0f) + xi[1] * (c[1] - 7.0f);
      t1 = xi[2] * (c[2] - 7.0f) + xi[3] * (c[3] - 7.0f);
      t2 = xi[4] * (c[4] - 7.0f) + xi[5] * (c[5] - 7.0f);
      t3 = xi[6] * (c[6] - 7.0f) + xi[7] * (c[7] - 7.0f);
    }
    float term = sc * (((t0 + t1) + t2) + t3);
    if (affine) {
      float xs = xi[0];
      for (int i = 1; i < 8; ++i) xs += xi[i];
      term = term + h2f(b[g]) * xs;
    }
    int t = (int)(blk % lanes);
    acc[t] = acc[t] + term;
  }
  for (int w = lanes / 2; w >= 1; w /= 2)
    for (int t = 0; t < w; ++t) acc[t] = acc[t] + acc[t + w];
  return acc[0];
}

/* y[m,n] (f16 or f32) in reference GEMV order; this is the timed CPU baseline. */
void zo_gemv_ref(const uint16_t* x, const uint32_t* W, const uint16_t* s, const uint16_t* b, void* y, long M,
                 long N, long K, int bits, int group, int affine, int out_f32, int lanes) {
  long KP = K * bits / 32, SPR = K / group;
  float* xf = (float*)malloc(sizeof(float) * (size_t)(M * K));
  for (long i = 0; i < M * K; ++i) xf[i] = h2f(x[i]);
#pragma omp parallel for schedule(static)
  for (long n = 0; n < N; ++n) {
    for (long m = 0; m < M; ++m) {
      float v = gemv_row_ref(xf + m * K, W + n * KP, s + n * SPR, affine ? b + n * SPR : NULL, K, bits, group,
                             affine, lanes);
      if (out_f32) ((float*)y)[m * N + n] = v;
      else ((uint16_t*)y)[m * N + n] = f2h(v);
    }
  }
  free(xf);
}

/* ids-indirect expert GEMV (gen.ts:229-254): for (token, slot): expert = ids[token*ids_stride + slot];
 * in  = x + token*in_tok_stride + slot*in_slot_stride;  out = y + token*out_tok_stride + slot*out_slot_stride. */
void zo_moe_gemv_ref(const uint16_t* x, const uint32_t* W, const uint16_t* s, const uint16_t* b, uint16_t* y,
                     const uint32_t* ids, long tokens, long slots, long N, long K, int bits, int group,
                     long in_slot_stride, long out_slot_stride, long in_tok_stride, long out_tok_stride,
                     long ids_stride) {
  long KP = K * bits / 32, SPR = K / group;
#pragma omp parallel
  {
    float* xf = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(dynamic, 1) collapse(2)
    for (long t = 0; t < tokens; ++t) {
      for (long sl = 0; sl < slots; ++sl) {
        long e = ids[t * ids_stride + sl];
        const uint16_t* xin = x + t * in_tok_stride + sl * in_slot_stride;
        for (long k = 0; k < K; ++k) xf[k] = h2f(xin[k]);
        uint16_t* out = y + t * out_tok_stride + sl * out_slot_stride;
        for (long n = 0; n < N; ++n) {
          float v = gemv_row_ref(xf, W + (e * N + n) * KP, s + (e * N + n) * SPR, b + (e * N + n) * SPR, K, bits,
                                 group, 1, 32);
          out[n] = f2h(v);
        }
      }
    }
    free(xf);
  }
}

/* f64 version of the same indirection, over W32 (w16 = 0) or W16 (w16 = 1) */
void zo_moe_matmul_f64(const uint16_t* x, const uint32_t* W, const uint16_t* s, const uint16_t* b, double* y,
                       const uint32_t* ids, long tokens, long slots, long N, long K, int bits, int group,
                       long in_slot_stride, long in_tok_stride, long ids_stride, int w16) {
  long KP = K * bits / 32, SPR = K / group;
#pragma omp parallel
  {
    double* xd = (double*)malloc(sizeof(double) * (size_t)K);
#pragma omp for schedule(dynamic, 1) collapse(2)
    for (long t = 0; t < tokens; ++t) {
      for (long sl = 0; sl < slots; ++sl) {
        long e = ids[t * ids_stride + sl];
        const uint16_t* xin = x + t * in_tok_stride + sl * in_slot_stride;
        for (long k = 0; k < K; ++k) xd[k] = (double)h2f(xin[k]);
        double* out = y + (t * slots + sl) * N;
        for (long n = 0; n < N; ++n) {
          const uint32_t* row = W + (e * N + n) * KP;
          double acc = 0.0;
          for (long blk = 0; blk < K / 8; ++blk) {
            float c[8];
            block_codes(row, blk, bits, c);
            long g = (blk * 8) / group;
            float sc = h2f(s[(e * N + n) * SPR + g]), bi = h2f(b[(e * N + n) * SPR + g]);
            for (int i = 0; i < 8; ++i) {
              float w = sc * c[i] + bi;
              if (w16) w = h2f(f2h(w));
              acc += xd[blk * 8 + i] * (double)w;
            }
          }
          out[n] = acc;
        }
      }
    }
    free(xd);
  }
}

/* softmax over E -> K arg-max rounds (ties to the lower index) -> renormalise;
 * slot K = expert E with sigmoid(logit[E]) when has_shared (moe_router_topk.wgsl:83-135). */
void zo_router_topk(const float* logits, uint32_t* ids, float* scores, long tokens, int E, int K, int norm_topk,
                    int has_shared) {
  int rows = E + (has_shared ? 1 : 0), S = K + (has_shared ? 1 : 0);
#pragma omp parallel
  {
    float* p = (float*)malloc(sizeof(float) * (size_t)E);
#pragma omp for schedule(static)
    for (long t = 0; t < tokens; ++t) {
      const float* l = logits + t * rows;
      float peak = -3.0e38f;
      for (int e = 0; e < E; ++e) peak = l[e] > peak ? l[e] : peak;
      float denom = 0.0f;
      for (int e = 0; e < E; ++e) {
        p[e] = expf(l[e] - peak);
        denom += p[e];
      }
      float total = 0.0f;
      for (int k = 0; k < K; ++k) {
        float bv = -1.0f;
        int bi = 0;
        for (int e = 0; e < E; ++e)
          if (p[e] > bv) { bv = p[e]; bi = e; }
        ids[t * S + k] = (uint32_t)bi;
        scores[t * S + k] = bv;
        total += bv;
        p[bi] = -1.0f;
      }
      float scale = norm_topk ? 1.0f / total : 1.0f / denom;
      for (int k = 0; k < K; ++k) scores[t * S + k] *= scale;
      if (has_shared) {
        ids[t * S + K] = (uint32_t)E;
        scores[t * S + K] = 1.0f / (1.0f + expf(-l[E]));
      }
    }
    free(p);
  }
}

/* h = f16(up * gate * 1/(1+exp(-gate))), rows of [gate(ffn) | up(ffn)] (silu_mul.wgsl:40-43) */
void zo_silu_mul(const uint16_t* gate_up, uint16_t* h, long rows, long ffn) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < rows; ++r)
    for (long i = 0; i < ffn; ++i) {
      float g = h2f(gate_up[r * 2 * ffn + i]), u = h2f(gate_up[r * 2 * ffn + ffn + i]);
      float sg = g * (1.0f / (1.0f + expf(-g)));
      h[r * ffn + i] = f2h(u * sg);
    }
}

/* out[t] = f16(sum_s score[t,s]*f32(y[t,s])) (moe_combine.wgsl:39-43) */
void zo_moe_combine(const uint16_t* y_slots, const float* scores, uint16_t* out, long tokens, long slots, long d) {
#pragma omp parallel for schedule(static)
  for (long t = 0; t < tokens; ++t)
    for (long i = 0; i < d; ++i) {
      float acc = 0.0f;
      for (long s = 0; s < slots; ++s) acc = acc + scores[t * slots + s] * h2f(y_slots[(t * slots + s) * d + i]);
      out[t * d + i] = f2h(acc);
    }
}
