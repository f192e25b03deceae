// C ABI of libztvm_b200.so: context, argument validation, kernel selection. Every entry point
// validates before it launches and reports through a status code plus a thread-local message.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "../../include/ztvm_b200.h"
#include "ztvm_kernels.h"

struct ztvm_ctx {
  uint32_t magic;
  int no_gemm;    // env ZTVM_NO_GEMM=1: keep M > 8 on GEMV slabs (a measurement knob)
  // 0 auto: the persistent matrix-unit GEMV where its shape rules allow, else M = 1 on the CUDA-core FMA GEMV and
  // M = 2..8 on the tiled matrix-unit GEMV; 1: FMA always; 2: tiled matrix unit always; 3: like 0 but M = 1 stays on
  // the FMA GEMV (env ZTVM_GEMV_PATH=fma|mma|tc|tc_m2, a measurement knob)
  int gemv_path;
  int device;
  int sm_count;
  cudaStream_t stream;
  uint32_t* err_counter;  // device word: out-of-range expert ids seen by the MoE kernels
  // staging for the host-buffer entry point (grown on demand, freed at destroy)
  void* h_pinned; size_t h_pinned_bytes;
  void* d_x; size_t d_x_bytes;
  // lanes of ztvm_int4_matmul_host_async: a stream and device buffers each, used round robin
  struct HostLane { cudaStream_t stream; void* d_x; size_t d_x_bytes; void* d_y; size_t d_y_bytes; } lanes[3];
  uint32_t next_lane;
  void* d_y; size_t d_y_bytes;
  // plan scratch of the grouped MoE matmul (grown on demand: a call that needs more synchronises the device,
  // reallocates and goes on; make one call at the largest size before capturing a graph)
  void* d_ws; size_t d_ws_bytes;
  void* d_ffn; size_t d_ffn_bytes;      // f32 gate/up rows of ztvm_fused_ffn's two-launch form
  // env ZTVM_MOE_GROUPED (a measurement knob): 0 forces the per-pair GEMV, 1 the tensor-core tiles, 2 the streaming
  // grouped kernel; unset = by size (below 128 pairs per-pair; then streaming while an expert sees few pairs)
  int moe_grouped;
  int gemm_sm;      // env ZTVM_GEMM=sm: the GEMM with both operands in shared memory (a measurement knob)
  // what the plan in d_ws was built from (ztvm_int4_matmul_moe_ep reuse_plan)
  const void* plan_ids; const void* plan_segs; uint32_t plan_tokens, plan_tile_rows, plan_experts, plan_slots, plan_stride;
  int plan_reuse;   // ztvm_moe_plan_reuse: consecutive ztvm_int4_matmul_moe calls over one id list share its plan
  int moe_tiles_sm; // env ZTVM_MOE_TILES=sm: the grouped MoE tiles with both operands in shared memory (a measurement knob)
};

namespace {

constexpr uint32_t kMagic = 0x5a54564du;  // "ZTVM"
thread_local char g_err[512] = "";

ztvm_status fail(ztvm_status s, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return s;
}
ztvm_status cuda_fail(cudaError_t e, const char* what) {
  return fail(ZTVM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}
#define ZTVM_CUDA(call)                                      \
  do {                                                       \
    cudaError_t e_ = (call);                                 \
    if (e_ != cudaSuccess) return cuda_fail(e_, #call);      \
  } while (0)

ztvm_status check_ctx(ztvm_ctx* ctx) {
  if (!ctx) return fail(ZTVM_ERR_BAD_CONTEXT, "context is NULL");
  if (ctx->magic != kMagic) return fail(ZTVM_ERR_BAD_CONTEXT, "context is not live (destroyed or corrupt)");
  int dev = -1;
  ZTVM_CUDA(cudaGetDevice(&dev));
  if (dev != ctx->device) ZTVM_CUDA(cudaSetDevice(ctx->device));
  return ZTVM_OK;
}

// True when `p` is page-locked host memory known to the runtime (cudaHostAlloc / cudaHostRegister).
bool host_is_pinned(const void* p) {
  cudaPointerAttributes a;
  if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
    cudaGetLastError();   // older runtimes report plain malloc memory as an error: clear it
    return false;
  }
  return a.type == cudaMemoryTypeHost;
}

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

int log2_exact(uint32_t v) {
  if (v == 0 || (v & (v - 1))) return -1;
  int s = 0;
  while ((1u << s) != v) ++s;
  return s;
}

// Layout rules shared by every matmul entry point.
ztvm_status check_desc(const ztvm_mm_desc* d, bool need_m) {
  if (!d) return fail(ZTVM_ERR_NULL_POINTER, "desc is NULL");
  if (d->bits != 4 && d->bits != 3 && d->bits != 8)
    return fail(ZTVM_ERR_UNSUPPORTED, "bits=%u: 8, 4 and 3 are implemented", d->bits);
  if (d->bits != 4 && !d->affine)
    return fail(ZTVM_ERR_UNSUPPORTED, "%u-bit weights exist only in the affine layout", d->bits);
  const int gs = log2_exact(d->group);
  if (gs < 5 || gs > 8) return fail(ZTVM_ERR_BAD_DIMS, "group=%u: must be a power of two in [32, 256]", d->group);
  if (d->K == 0 || d->N == 0) return fail(ZTVM_ERR_BAD_DIMS, "K=%u N=%u: must be non-zero", d->K, d->N);
  if (d->K % d->group) return fail(ZTVM_ERR_BAD_DIMS, "K=%u is not a multiple of group=%u", d->K, d->group);
  if (need_m && d->M == 0) return fail(ZTVM_ERR_BAD_DIMS, "M=0");
  if ((uint64_t)d->N * (d->K / 32 * d->bits) > 0xFFFFFFFFull * 4ull)
    return fail(ZTVM_ERR_TOO_LARGE, "N*K too large");
  return ZTVM_OK;
}

bool use_mma(const ztvm_ctx* ctx, const ztvm_mm_desc* d, uint32_t m) {
  if (!ztvm::gemv_mma_supported((int)d->bits, d->group)) return false;
  return ctx->gemv_path == 2 || ((ctx->gemv_path == 0 || ctx->gemv_path == 3) && m > 1);
}

ztvm::GemvParams gemv_params(const ztvm_mm_desc* d, void* y, const void* x, const void* s, const void* w,
                             const void* b) {
  ztvm::GemvParams p;
  memset(&p, 0, sizeof(p));
  p.W = static_cast<const uint32_t*>(w);
  p.S = static_cast<const __half*>(s);
  p.B = d->affine ? static_cast<const __half*>(b) : nullptr;
  p.X = static_cast<const __half*>(x);
  p.Y = y;
  p.K = d->K; p.N = d->N; p.M = d->M;
  p.KP = d->K / 32 * d->bits;
  p.SPR = d->K / d->group;
  p.group_shift = (uint32_t)log2_exact(d->group);
  p.out_f32 = d->out_f32 ? 1u : 0u;
  p.x_row_stride = d->K;
  p.y_row_stride = d->N;
  return p;
}

ztvm_status check_buffers(const ztvm_mm_desc* d, const void* y, const void* x, const void* s, const void* w,
                          const void* b) {
  if (!y || !x || !s || !w) return fail(ZTVM_ERR_NULL_POINTER, "y/x/scales/packed_w must be non-NULL");
  if (d->affine && !b) return fail(ZTVM_ERR_NULL_POINTER, "affine weights need biases");
  if (!aligned(w, 16) || !aligned(x, 16)) return fail(ZTVM_ERR_ALIGNMENT, "packed_w and x must be 16-byte aligned");
  if (!aligned(s, 8) || (b && !aligned(b, 8)) || !aligned(y, d->out_f32 ? 4 : 2))
    return fail(ZTVM_ERR_ALIGNMENT, "scales/biases must be 8-byte aligned, y aligned to its element type");
  return ZTVM_OK;
}

ztvm_status grow(void** p, size_t* have, size_t need, bool pinned) {
  if (*have >= need) return ZTVM_OK;
  if (*p) {
    if (pinned) ZTVM_CUDA(cudaFreeHost(*p)); else ZTVM_CUDA(cudaFree(*p));
    *p = nullptr; *have = 0;
  }
  size_t cap = need + need / 2;
  if (pinned) ZTVM_CUDA(cudaMallocHost(p, cap)); else ZTVM_CUDA(cudaMalloc(p, cap));
  *have = cap;
  return ZTVM_OK;
}

}  // namespace

extern "C" {

int32_t ztvm_version(void) { return 100; }

const char* ztvm_status_string(ztvm_status s) {
  switch (s) {
    case ZTVM_OK: return "ok";
    case ZTVM_ERR_NULL_POINTER: return "null pointer";
    case ZTVM_ERR_BAD_DIMS: return "bad dimensions";
    case ZTVM_ERR_UNSUPPORTED: return "unsupported combination";
    case ZTVM_ERR_ALIGNMENT: return "misaligned buffer";
    case ZTVM_ERR_CUDA: return "CUDA error";
    case ZTVM_ERR_BAD_CONTEXT: return "bad context";
    case ZTVM_ERR_TOO_LARGE: return "size beyond limit";
    default: return "unknown status";
  }
}

const char* ztvm_last_error(ztvm_ctx*) { return g_err; }

ztvm_status ztvm_init(int32_t device_ordinal, ztvm_ctx** out_ctx) {
  if (!out_ctx) return fail(ZTVM_ERR_NULL_POINTER, "out_ctx is NULL");
  *out_ctx = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceCount (no usable CUDA device: this library has no CPU path)");
  if (device_ordinal < 0 || device_ordinal >= count)
    return fail(ZTVM_ERR_BAD_CONTEXT, "device %d out of range (%d devices)", device_ordinal, count);
  ZTVM_CUDA(cudaSetDevice(device_ordinal));
  cudaDeviceProp prop;
  ZTVM_CUDA(cudaGetDeviceProperties(&prop, device_ordinal));
  if (prop.major != 10)
    return fail(ZTVM_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", device_ordinal,
                prop.major, prop.minor);
  ztvm_ctx* c = new (std::nothrow) ztvm_ctx();
  if (!c) return fail(ZTVM_ERR_CUDA, "out of host memory");
  memset(c, 0, sizeof(*c));
  c->device = device_ordinal;
  c->sm_count = prop.multiProcessorCount;
  e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&c->err_counter), 256);
  if (e == cudaSuccess) e = cudaMemset(c->err_counter, 0, 256);
  if (e != cudaSuccess) {
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
    return cuda_fail(e, "context set-up");
  }
  const char* ng = getenv("ZTVM_NO_GEMM");
  c->no_gemm = (ng && ng[0] == '1') ? 1 : 0;
  const char* gk = getenv("ZTVM_GEMM");
  c->gemm_sm = (gk && !strcmp(gk, "sm")) ? 1 : 0;
  const char* mt = getenv("ZTVM_MOE_TILES");
  c->moe_tiles_sm = (mt && !strcmp(mt, "sm")) ? 1 : 0;
  const char* mg = getenv("ZTVM_MOE_GROUPED");
  c->moe_grouped = !mg ? -1 : (mg[0] == '1' ? 1 : mg[0] == '2' ? 2 : 0);
  const char* gp = getenv("ZTVM_GEMV_PATH");
  c->gemv_path = !gp ? 0 : !strcmp(gp, "fma") ? 1 : !strcmp(gp, "mma") ? 2 : !strcmp(gp, "tc_m2") ? 3 : 0;
  c->magic = kMagic;
  *out_ctx = c;
  return ZTVM_OK;
}

ztvm_status ztvm_destroy(ztvm_ctx* ctx) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  cudaStreamSynchronize(ctx->stream);
  if (ctx->h_pinned) cudaFreeHost(ctx->h_pinned);
  if (ctx->d_x) cudaFree(ctx->d_x);
  if (ctx->d_y) cudaFree(ctx->d_y);
  if (ctx->d_ws) cudaFree(ctx->d_ws);
  if (ctx->d_ffn) cudaFree(ctx->d_ffn);
  for (auto& l : ctx->lanes) {
    if (l.stream) { cudaStreamSynchronize(l.stream); cudaStreamDestroy(l.stream); }
    if (l.d_x) cudaFree(l.d_x);
    if (l.d_y) cudaFree(l.d_y);
  }
  cudaFree(ctx->err_counter);
  cudaStreamDestroy(ctx->stream);
  ctx->magic = 0;
  delete ctx;
  return ZTVM_OK;
}

ztvm_status ztvm_sync(ztvm_ctx* ctx) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  ZTVM_CUDA(cudaStreamSynchronize(ctx->stream));
  return ZTVM_OK;
}

ztvm_status ztvm_int4_matmul(ztvm_ctx* ctx, const ztvm_mm_desc* d, void* y, const void* x, const void* scales,
                             const void* packed_w, const void* biases, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if ((s = check_desc(d, true))) return s;
  if ((s = check_buffers(d, y, x, scales, packed_w, biases))) return s;
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  // Up to 16 rows the GEMV in slabs of eight wins: it re-streams the weights once per slab at HBM speed, while the
  // tensor-core kernels dequantise every code once at ~12 codes per clock and SM whatever M is (measured on
  // 8192 x 2048: 9.4 us against 21 us at M = 16, 14 against 13 us at M = 24). It is also the reference's choice for
  // short chunks (runtime-M matvec, exact codes and f32 weights; its GEMMs start at 64 rows).
  if (d->M > 16 && ztvm::gemm_w4_supported((int)d->bits, d->group, d->K) && !ctx->no_gemm) {
    if (!aligned(y, 16)) return fail(ZTVM_ERR_ALIGNMENT, "y must be 16-byte aligned for the GEMM path");
    // M > 128: weights as the A operand in tensor memory (256 tokens per instruction); up to 128 rows the tiles with
    // both operands in shared memory, whose 64-row weight tiles give twice as many CTAs
    auto launch = (ctx->gemm_sm || d->M <= 128) ? ztvm::launch_gemm_w4 : ztvm::launch_gemm_w4_ta;
    ZTVM_CUDA(launch(static_cast<const uint32_t*>(packed_w), static_cast<const __half*>(scales),
                     d->affine ? static_cast<const __half*>(biases) : nullptr, static_cast<const __half*>(x), y, d->M, d->N,
                     d->K, (uint32_t)log2_exact(d->group), d->out_f32 != 0, ctx->err_counter + 1, st));
    return ZTVM_OK;
  }
  // Otherwise rows are processed in slabs of at most 8 by the GEMV.
  for (uint32_t m0 = 0; m0 < d->M; m0 += 8) {
    ztvm_mm_desc dd = *d;
    dd.M = d->M - m0 < 8 ? d->M - m0 : 8;
    ztvm::GemvParams p = gemv_params(&dd, y, x, scales, packed_w, biases);
    p.X = static_cast<const __half*>(x) + (size_t)m0 * d->K;
    p.Y = d->out_f32 ? static_cast<void*>(static_cast<float*>(y) + (size_t)m0 * d->N)
                     : static_cast<void*>(static_cast<__half*>(y) + (size_t)m0 * d->N);
    const bool want_tc = ctx->gemv_path == 0 || (ctx->gemv_path == 3 && dd.M > 1);
    if (want_tc && ztvm::gemv_tc_supported(p, (int)d->bits, ctx->sm_count)) ZTVM_CUDA(ztvm::launch_gemv_tc(p, ctx->sm_count, st));
    else if (want_tc && ztvm::gemv_tc3_supported(p, (int)d->bits, ctx->sm_count)) ZTVM_CUDA(ztvm::launch_gemv_tc3(p, ctx->sm_count, st));
    else if (use_mma(ctx, d, dd.M)) ZTVM_CUDA(ztvm::launch_gemv_mma(p, false, 1, 1, st));
    else ZTVM_CUDA(ztvm::launch_gemv(p, (int)d->bits, false, 1, 1, ctx->sm_count, st));
  }
  return ZTVM_OK;
}

ztvm_status ztvm_peer_barrier(ztvm_ctx* ctx, uint32_t* const* flags, uint32_t world, uint32_t rank, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!flags) return fail(ZTVM_ERR_NULL_POINTER, "flags is NULL");
  if (world == 0 || world > 8 || rank >= world) return fail(ZTVM_ERR_BAD_DIMS, "world=%u rank=%u: 1..8 ranks", world, rank);
  ztvm::PeerBarrierParams p;
  memset(&p, 0, sizeof(p));
  for (uint32_t r = 0; r < world; ++r) {
    if (!flags[r] || !aligned(flags[r], 4)) return fail(ZTVM_ERR_NULL_POINTER, "flags[%u] missing or misaligned", r);
    p.flags[r] = flags[r];
  }
  p.world = world; p.rank = rank;
  p.wait_cycles = 2000000000ull;      // about a second
  p.status = ctx->err_counter + 1;
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ZTVM_CUDA(ztvm::launch_peer_barrier(p, st));
  return ZTVM_OK;
}

ztvm_status ztvm_int4_matmul_nshard(ztvm_ctx* ctx, const ztvm_mm_desc* d, void* const* y_dsts, uint32_t world, uint32_t rank,
                                    uint32_t y_row_stride, const void* x, const void* scales, const void* packed_w,
                                    const void* biases, uint32_t* const* flags, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (world == 0 || world > 8 || rank >= world) return fail(ZTVM_ERR_BAD_DIMS, "world=%u rank=%u: 1..8 ranks", world, rank);
  // a rank whose shard is empty (N_total smaller than the rank count allows) still takes part in the barrier
  if (d && d->N > 0 && (s = ztvm_int4_matmul_multi(ctx, d, y_dsts, world, y_row_stride, x, scales, packed_w, biases, stream))) return s;
  return ztvm_peer_barrier(ctx, flags, world, rank, stream);
}

ztvm_status ztvm_moe_ffn_ep(ztvm_ctx* ctx, const ztvm_moe_ffn_ep_args* a, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!a) return fail(ZTVM_ERR_NULL_POINTER, "args is NULL");
  const ztvm_moe_ep_layout* L = &a->layout;
  if (L->world == 0 || L->world > 8 || L->rank >= L->world) return fail(ZTVM_ERR_BAD_DIMS, "world=%u rank=%u: 1..8 ranks", L->world, L->rank);
  if (!a->gate_up || !a->h) return fail(ZTVM_ERR_NULL_POINTER, "gate_up/h scratch is NULL");
  if (a->ffn == 0 || a->d == 0) return fail(ZTVM_ERR_BAD_DIMS, "d=%u ffn=%u", a->d, a->ffn);
  for (uint32_t r = 0; r < L->world; ++r)
    if (!a->y_slots[r] || !a->flags[r]) return fail(ZTVM_ERR_NULL_POINTER, "y_slots / flags of rank %u missing", r);
  const uint32_t slots = a->top_k + (a->has_shared ? 1u : 0u);
  const uint32_t regions = L->world + 1u;
  const uint64_t rows_total = (uint64_t)regions * L->seg_cap;
  if (rows_total >= (1ull << 31)) return fail(ZTVM_ERR_TOO_LARGE, "(world + 1) * seg_cap = %llu rows", (unsigned long long)rows_total);
  if ((s = ztvm_moe_ep_dispatch(ctx, L, a->ids, a->tokens, a->top_k, a->has_shared, a->ids_stride, a->x, a->d, a->x_tok_stride, stream))) return s;
  if ((s = ztvm_peer_barrier(ctx, a->flags, L->world, L->rank, stream))) return s;
  ztvm_moe_ep_rows rows;
  memset(&rows, 0, sizeof(rows));
  rows.seg_counts = L->recv_cnt[L->rank];
  rows.seg_cap = L->seg_cap;
  rows.segments = regions;
  const uint32_t E1 = L->experts_per_rank + (a->has_shared ? 1u : 0u);
  ztvm_moe_desc gu = {{a->d, a->ffn, 1, 64, 4, 1, 0}, E1, 1, (uint32_t)rows_total, 0, 2 * a->ffn, a->d, 2 * a->ffn, 1};
  // a result row goes to y_seg[region] + recv_src[i] * d: recv_src = token * slots + slot indexes rows of d elements
  ztvm_moe_desc dn = {{a->ffn, a->d, 1, 64, 4, 1, 0}, E1, 1, (uint32_t)rows_total, 0, a->d, a->ffn, a->d, 1};
  (void)slots;
  const uint32_t* rids = L->recv_ids[L->rank];
  if ((s = ztvm_int4_matmul_moe_ep(ctx, &gu, &rows, a->gate_up, L->recv_x[L->rank], a->gate_scales, a->gate_w, a->gate_biases, rids, stream))) return s;
  rows.reuse_plan = 1;
  if ((s = ztvm_int4_matmul_moe_ep(ctx, &gu, &rows, static_cast<__half*>(a->gate_up) + a->ffn, L->recv_x[L->rank], a->up_scales, a->up_w,
                                   a->up_biases, rids, stream))) return s;
  if ((s = ztvm_silu_mul_rows(ctx, &rows, a->ffn, a->h, a->gate_up, stream))) return s;
  rows.dst_index = L->recv_src[L->rank];
  for (uint32_t r = 0; r < L->world; ++r) rows.y_seg[r] = a->y_slots[r];
  rows.y_seg[L->world] = a->y_slots[L->rank];        // the local region's rows belong to this rank's own tokens
  if ((s = ztvm_int4_matmul_moe_ep(ctx, &dn, &rows, a->y_slots[L->rank], a->h, a->down_scales, a->down_w, a->down_biases, rids, stream))) return s;
  return ztvm_peer_barrier(ctx, a->flags, L->world, L->rank, stream);
}

ztvm_status ztvm_fused_ffn(ztvm_ctx* ctx, const ztvm_mm_desc* d, void* h, const void* x, const void* scales,
                           const void* packed_w, const void* biases, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if ((s = check_desc(d, true))) return s;
  if (d->out_f32) return fail(ZTVM_ERR_UNSUPPORTED, "the fused FFN stores f16");
  if (d->N > 0x7FFFFFFFu) return fail(ZTVM_ERR_TOO_LARGE, "ffn=%u: 2 * ffn rows must fit 32 bits", d->N);
  ztvm_mm_desc gu = *d;
  gu.N = 2 * d->N;
  if ((s = check_buffers(&gu, h, x, scales, packed_w, biases))) return s;
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  if (d->M <= 8 && ctx->gemv_path == 0) {
    ztvm::GemvParams p = gemv_params(&gu, h, x, scales, packed_w, biases);
    p.pair_rows = d->N;
    p.y_row_stride = d->N;
    if (ztvm::gemv_tc_supported(p, (int)d->bits, ctx->sm_count)) {
      ZTVM_CUDA(ztvm::launch_gemv_tc(p, ctx->sm_count, st));
      return ZTVM_OK;
    }
  }
  const size_t need = (size_t)d->M * gu.N * sizeof(float);
  if (ctx->d_ffn_bytes < need) {
    ZTVM_CUDA(cudaDeviceSynchronize());
    if ((s = grow(&ctx->d_ffn, &ctx->d_ffn_bytes, need, false))) return s;
  }
  gu.out_f32 = 1;
  if ((s = ztvm_int4_matmul(ctx, &gu, ctx->d_ffn, x, scales, packed_w, biases, st))) return s;
  ZTVM_CUDA(ztvm::launch_silu_mul_f32(static_cast<const float*>(ctx->d_ffn), static_cast<__half*>(h), d->M, d->N, st));
  return ZTVM_OK;
}

// One router logit per (token, row): the exact-code GEMV in slabs of eight tokens for quantised routers (never the f16
// tensor-core GEMM: logits feed a softmax and a top-k, so they keep the f32-accumulated exact-code arithmetic of the
// reference's matvec whatever the token count), a plain f16 matvec for routers stored in f16.
ztvm_status ztvm_moe_router_logits(ztvm_ctx* ctx, uint32_t D, uint32_t rows, uint32_t tokens, uint32_t bits, float* logits,
                                   const void* x, const void* w, const void* scales, const void* biases, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!logits || !x || !w) return fail(ZTVM_ERR_NULL_POINTER, "logits/x/w must be non-NULL");
  if (D == 0 || rows == 0) return fail(ZTVM_ERR_BAD_DIMS, "D=%u rows=%u: must be non-zero", D, rows);
  if (tokens == 0) return ZTVM_OK;
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  if (bits == 16) {
    if (!aligned(x, 16) || !aligned(w, 16) || D % 8) return fail(ZTVM_ERR_ALIGNMENT, "f16 router: x and w 16-byte aligned, D %% 8 == 0");
    ZTVM_CUDA(ztvm::launch_f16_matvec(static_cast<const __half*>(x), static_cast<const __half*>(w), logits, D, rows, tokens, st));
    return ZTVM_OK;
  }
  if (bits != 8 && bits != 4) return fail(ZTVM_ERR_UNSUPPORTED, "router bits=%u: 16, 8 and 4 are implemented", bits);
  ztvm_mm_desc d = {D, rows, tokens, 64, bits, 1, 1};
  if ((s = check_desc(&d, true))) return s;
  if ((s = check_buffers(&d, logits, x, scales, w, biases))) return s;
  const int keep = ctx->no_gemm;
  ctx->no_gemm = 1;
  s = ztvm_int4_matmul(ctx, &d, logits, x, scales, w, biases, st);
  ctx->no_gemm = keep;
  return s;
}

ztvm_status ztvm_embedding_affine(ztvm_ctx* ctx, uint32_t D, uint32_t bits, uint32_t vocab, uint32_t seq_len, void* out,
                                  const int32_t* input_ids, const void* scales, const void* weights, const void* biases,
                                  void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!out || !input_ids || !scales || !weights || !biases) return fail(ZTVM_ERR_NULL_POINTER, "out/input_ids/scales/weights/biases must be non-NULL");
  if (bits != 4 && bits != 8) return fail(ZTVM_ERR_UNSUPPORTED, "embedding bits=%u: 4 and 8 are implemented", bits);
  if (D == 0 || D % 64 || vocab == 0) return fail(ZTVM_ERR_BAD_DIMS, "D=%u must be a non-zero multiple of the group size 64, vocab=%u non-zero", D, vocab);
  if (!aligned(out, 16) || !aligned(weights, 4)) return fail(ZTVM_ERR_ALIGNMENT, "out must be 16-byte aligned");
  if (seq_len == 0) return ZTVM_OK;
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ZTVM_CUDA(ztvm::launch_embedding_affine(input_ids, static_cast<const uint32_t*>(weights), static_cast<const __half*>(scales),
                                          static_cast<const __half*>(biases), static_cast<__half*>(out), seq_len, D, vocab,
                                          (int)bits, ctx->err_counter, st));
  return ZTVM_OK;
}

ztvm_status ztvm_int4_matmul_multi(ztvm_ctx* ctx, const ztvm_mm_desc* d, void* const* y_dsts, uint32_t n_dst,
                                   uint32_t y_row_stride, const void* x, const void* scales, const void* packed_w,
                                   const void* biases, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if ((s = check_desc(d, true))) return s;
  if (!y_dsts) return fail(ZTVM_ERR_NULL_POINTER, "y_dsts is NULL");
  if (n_dst < 1 || n_dst > 8) return fail(ZTVM_ERR_BAD_DIMS, "n_dst=%u must be 1..8", n_dst);
  for (uint32_t i = 0; i < n_dst; ++i)
    if (!y_dsts[i]) return fail(ZTVM_ERR_NULL_POINTER, "y_dsts[%u] is NULL", i);
  if ((s = check_buffers(d, y_dsts[0], x, scales, packed_w, biases))) return s;
  if (d->M > 8) return fail(ZTVM_ERR_UNSUPPORTED, "the multi-destination form is the decode GEMV: M=%u exceeds 8", d->M);
  if (y_row_stride < d->N) return fail(ZTVM_ERR_BAD_DIMS, "y_row_stride=%u < N=%u", y_row_stride, d->N);
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ztvm::GemvParams p = gemv_params(d, y_dsts[0], x, scales, packed_w, biases);
  p.y_row_stride = y_row_stride;
  p.n_more = n_dst - 1;
  for (uint32_t i = 1; i < n_dst; ++i) p.y_more[i - 1] = y_dsts[i];
  if (!ztvm::gemv_tc_supported(p, (int)d->bits, ctx->sm_count))
    return fail(ZTVM_ERR_UNSUPPORTED,
                "the multi-destination form runs the persistent GEMV only: bits=4, group=64, K %% 256 == 0, 16-byte aligned "
                "x and weights (got bits=%u group=%u K=%u)", d->bits, d->group, d->K);
  ZTVM_CUDA(ztvm::launch_gemv_tc(p, ctx->sm_count, st));
  return ZTVM_OK;
}

ztvm_status ztvm_int4_matmul_host(ztvm_ctx* ctx, const ztvm_mm_desc* d, void* y_host, const void* x_host,
                                  const void* scales, const void* packed_w, const void* biases) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if ((s = check_desc(d, true))) return s;
  if (!y_host || !x_host) return fail(ZTVM_ERR_NULL_POINTER, "y_host/x_host must be non-NULL");
  const size_t xb = (size_t)d->M * d->K * 2, yb = (size_t)d->M * d->N * (d->out_f32 ? 4 : 2);
  // Page-locked caller buffers are copied by the DMA engines directly; pageable ones go through the context's
  // pinned staging buffer (an extra host memcpy each way).
  const bool x_pinned = host_is_pinned(x_host), y_pinned = host_is_pinned(y_host);
  const size_t stage = (x_pinned ? 0 : xb) + (y_pinned ? 0 : yb);
  if (stage && (s = grow(&ctx->h_pinned, &ctx->h_pinned_bytes, stage, true))) return s;
  if ((s = grow(&ctx->d_x, &ctx->d_x_bytes, xb, false))) return s;
  if ((s = grow(&ctx->d_y, &ctx->d_y_bytes, yb, false))) return s;
  char* hp = static_cast<char*>(ctx->h_pinned);
  const void* x_src = x_host;
  if (!x_pinned) { memcpy(hp, x_host, xb); x_src = hp; }
  void* y_dst = y_pinned ? y_host : static_cast<void*>(hp + (x_pinned ? 0 : xb));
  ZTVM_CUDA(cudaMemcpyAsync(ctx->d_x, x_src, xb, cudaMemcpyHostToDevice, ctx->stream));
  if ((s = ztvm_int4_matmul(ctx, d, ctx->d_y, ctx->d_x, scales, packed_w, biases, ctx->stream))) return s;
  ZTVM_CUDA(cudaMemcpyAsync(y_dst, ctx->d_y, yb, cudaMemcpyDeviceToHost, ctx->stream));
  ZTVM_CUDA(cudaStreamSynchronize(ctx->stream));
  if (!y_pinned) memcpy(y_host, y_dst, yb);
  return ZTVM_OK;
}

// The host-buffer call without the wait: copy-in, matmul and copy-out are queued on one of three lanes (a stream and a
// pair of device buffers each), taken round robin, so that while one call's kernel runs the next call's activations
// arrive and the previous call's results leave (the two copy directions and the SMs work at the same time).
ztvm_status ztvm_int4_matmul_host_async(ztvm_ctx* ctx, const ztvm_mm_desc* d, void* y_host, const void* x_host,
                                        const void* scales, const void* packed_w, const void* biases) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if ((s = check_desc(d, true))) return s;
  if (!y_host || !x_host) return fail(ZTVM_ERR_NULL_POINTER, "y_host/x_host must be non-NULL");
  if (!host_is_pinned(x_host) || !host_is_pinned(y_host))
    return fail(ZTVM_ERR_UNSUPPORTED, "the asynchronous host form copies straight from / to the caller's buffers: they must be page-locked");
  const size_t xb = (size_t)d->M * d->K * 2, yb = (size_t)d->M * d->N * (d->out_f32 ? 4 : 2);
  ztvm_ctx::HostLane& l = ctx->lanes[ctx->next_lane];
  ctx->next_lane = (ctx->next_lane + 1u) % 3u;
  if (!l.stream) ZTVM_CUDA(cudaStreamCreateWithFlags(&l.stream, cudaStreamNonBlocking));
  if (l.d_x_bytes < xb || l.d_y_bytes < yb) {
    ZTVM_CUDA(cudaStreamSynchronize(l.stream));      // the lane's earlier calls still use its buffers
    if ((s = grow(&l.d_x, &l.d_x_bytes, xb, false))) return s;
    if ((s = grow(&l.d_y, &l.d_y_bytes, yb, false))) return s;
  }
  ZTVM_CUDA(cudaMemcpyAsync(l.d_x, x_host, xb, cudaMemcpyHostToDevice, l.stream));
  if ((s = ztvm_int4_matmul(ctx, d, l.d_y, l.d_x, scales, packed_w, biases, l.stream))) return s;
  ZTVM_CUDA(cudaMemcpyAsync(y_host, l.d_y, yb, cudaMemcpyDeviceToHost, l.stream));
  return ZTVM_OK;
}

ztvm_status ztvm_host_wait(ztvm_ctx* ctx) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  for (auto& l : ctx->lanes)
    if (l.stream) ZTVM_CUDA(cudaStreamSynchronize(l.stream));
  return ZTVM_OK;
}

// Which grouped kernel serves a MoE launch: 0 none (per-pair GEMV), 1 tensor-core tiles with the weights in tensor
// memory, 2 streaming kernel, 3 tensor-core tiles with both operands in shared memory (ZTVM_MOE_TILES=sm, or shapes
// only it takes). `forced` is the context's ZTVM_MOE_GROUPED knob (-1 = by size).
static int moe_pick(const ztvm_ctx* ctx, const ztvm_moe_desc* md, const ztvm::GemvParams& p, const void* y) {
  const int forced = ctx->moe_grouped;
  const ztvm_mm_desc* d = &md->mm;
  const uint64_t pairs = (uint64_t)md->tokens * md->slots;
  const bool ta_ok = ztvm::moe_ta_supported((int)d->bits, d->group, d->K, d->N, md->experts);
  const bool sm_ok = (md->out_slot_stride | md->out_tok_stride) % 8 == 0 && aligned(y, 16) && !p.dst_index &&
                     ztvm::moe_grouped_supported((int)d->bits, d->group, d->K, d->N, md->experts);
  const int tiles = ctx->moe_tiles_sm ? (sm_ok ? 3 : ta_ok ? 1 : 0) : (ta_ok ? 1 : sm_ok ? 3 : 0);
  const bool stream_ok = ztvm::moe_tc_supported(p, (int)d->bits) && !p.dst_index;
  // Where the two grouped kernels cross (measured on the 257-expert block, hidden 2048, ffn 512): the tiles cost the same
  // whatever the pair count (every expert's weights are dequantised once: ~100 us per projection), the streaming kernel
  // grows with the 8-pair chunks it walks (gate: 35 us + 0.020 us per pair; down, with its short K: 48 us + 0.028 us per
  // pair). They meet near 12.6 pairs per expert for the long-K projections and 6.6 for the short-K one; one threshold
  // for both keeps the three projections of a block on one kernel, whose plan they can then share.
  const bool few_per_expert = pairs < 10ull * md->experts;
  if (forced == 1) return tiles ? tiles : stream_ok ? 2 : 0;
  if (forced == 2) return stream_ok ? 2 : tiles;
  return (stream_ok && (few_per_expert || !tiles)) ? 2 : tiles;
}

static ztvm::GemvParams moe_params(ztvm_ctx* ctx, const ztvm_moe_desc* md, void* y, const void* x, const void* scales,
                                   const void* packed_w, const void* biases, const uint32_t* ids) {
  ztvm_mm_desc dd = md->mm;
  dd.M = 1;
  ztvm::GemvParams p = gemv_params(&dd, y, x, scales, packed_w, biases);
  p.ids = ids;
  p.experts = md->experts;
  p.in_slot_stride = md->in_slot_stride; p.out_slot_stride = md->out_slot_stride;
  p.in_tok_stride = md->in_tok_stride; p.out_tok_stride = md->out_tok_stride;
  p.ids_stride = md->ids_stride;
  p.err_counter = ctx->err_counter;
  return p;
}

ztvm_status ztvm_int4_matmul_moe(ztvm_ctx* ctx, const ztvm_moe_desc* md, void* y, const void* x, const void* scales,
                                 const void* packed_w, const void* biases, const uint32_t* ids, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!md) return fail(ZTVM_ERR_NULL_POINTER, "desc is NULL");
  const ztvm_mm_desc* d = &md->mm;
  if ((s = check_desc(d, false))) return s;
  if (!d->affine) return fail(ZTVM_ERR_UNSUPPORTED, "MoE expert weights are affine-quantised only");
  if (d->bits == 8) return fail(ZTVM_ERR_UNSUPPORTED, "MoE expert weights are 4-bit or 3-bit");
  if (d->out_f32) return fail(ZTVM_ERR_UNSUPPORTED, "MoE expert matmuls write f16");
  if (d->M > 1) return fail(ZTVM_ERR_BAD_DIMS, "MoE matmul is per (token, slot): mm.M must be 1 (or 0)");
  if ((s = check_buffers(d, y, x, scales, packed_w, biases))) return s;
  if (!ids) return fail(ZTVM_ERR_NULL_POINTER, "ids is NULL");
  if (md->tokens == 0) return ZTVM_OK;
  if (md->slots == 0 || md->experts == 0) return fail(ZTVM_ERR_BAD_DIMS, "slots and experts must be non-zero");
  if (md->slots > 65535) return fail(ZTVM_ERR_TOO_LARGE, "slots=%u exceeds 65535", md->slots);
  if (md->ids_stride < md->slots) return fail(ZTVM_ERR_BAD_DIMS, "ids_stride=%u < slots=%u", md->ids_stride, md->slots);
  if ((md->in_slot_stride | md->in_tok_stride) % 8)
    return fail(ZTVM_ERR_ALIGNMENT, "input strides must be multiples of 8 elements (16-byte activation loads)");
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ztvm_mm_desc dd = *d;
  dd.M = 1;
  // Many pairs: sort them by expert. While an expert sees only a few pairs the job is bound by streaming each active
  // expert's weights once (streaming kernel); with many pairs per expert it is a real contraction (tensor-core tiles,
  // each expert's weights dequantised once per 128 pairs).
  const uint64_t pairs = (uint64_t)md->tokens * md->slots;
  const bool want_grouped = ctx->moe_grouped < 0 ? pairs >= 128 : ctx->moe_grouped >= 1;
  if (want_grouped && pairs < (1ull << 31)) {
    const ztvm::GemvParams p = moe_params(ctx, md, y, x, scales, packed_w, biases, ids);
    const int pick = moe_pick(ctx, md, p, y);
    if (pick) {
      const size_t need = ztvm::moe_grouped_scratch_bytes(md->experts, (uint32_t)pairs);
      if (ctx->d_ws_bytes < need) {
        ZTVM_CUDA(cudaDeviceSynchronize());
        if ((s = grow(&ctx->d_ws, &ctx->d_ws_bytes, need, false))) return s;
        ctx->plan_ids = nullptr;
      }
      uint32_t* ws = static_cast<uint32_t*>(ctx->d_ws);
      const uint32_t tile_rows = pick == 2 ? ztvm::kMoeTcTileRows : ztvm::kMoeTaTileRows;
      // gate, up and down of one step walk the same id list: with ztvm_moe_plan_reuse on, its plan is built once
      const bool reuse = ctx->plan_reuse && pick != 3 && ctx->plan_ids == ids && ctx->plan_segs == nullptr &&
                         ctx->plan_tokens == md->tokens && ctx->plan_slots == md->slots && ctx->plan_stride == md->ids_stride &&
                         ctx->plan_tile_rows == tile_rows && ctx->plan_experts == md->experts;
      if (pick == 2) ZTVM_CUDA(ztvm::launch_moe_tc(p, md->tokens, md->slots, ws, ctx->sm_count, st, reuse));
      else if (pick == 1) ZTVM_CUDA(ztvm::launch_moe_ta(p, md->tokens, md->slots, ws, ctx->err_counter + 1, ctx->sm_count, st, reuse));
      else ZTVM_CUDA(ztvm::launch_moe_grouped(p, md->tokens, md->slots, ws, ctx->err_counter + 1, st));
      ctx->plan_ids = pick != 3 ? ids : nullptr; ctx->plan_segs = nullptr; ctx->plan_tokens = md->tokens; ctx->plan_slots = md->slots;
      ctx->plan_stride = md->ids_stride; ctx->plan_tile_rows = tile_rows; ctx->plan_experts = md->experts;
      return ZTVM_OK;
    }
  }
  // grid.y carries the token: split very long token lists into slabs of 65535
  for (uint32_t t0 = 0; t0 < md->tokens; t0 += 65535) {
    const uint32_t nt = md->tokens - t0 < 65535 ? md->tokens - t0 : 65535;
    ztvm::GemvParams p = gemv_params(&dd, y, x, scales, packed_w, biases);
    p.X = static_cast<const __half*>(x) + (size_t)t0 * md->in_tok_stride;
    p.Y = static_cast<__half*>(y) + (size_t)t0 * md->out_tok_stride;
    p.ids = ids + (size_t)t0 * md->ids_stride;
    p.experts = md->experts;
    p.in_slot_stride = md->in_slot_stride; p.out_slot_stride = md->out_slot_stride;
    p.in_tok_stride = md->in_tok_stride; p.out_tok_stride = md->out_tok_stride;
    p.ids_stride = md->ids_stride;
    p.err_counter = ctx->err_counter;
    if (use_mma(ctx, d, 1)) ZTVM_CUDA(ztvm::launch_gemv_mma(p, true, nt, md->slots, st));
    else ZTVM_CUDA(ztvm::launch_gemv(p, (int)d->bits, true, nt, md->slots, ctx->sm_count, st));
  }
  return ZTVM_OK;
}

ztvm_status ztvm_int4_matmul_moe_noalloc(ztvm_ctx* ctx, const ztvm_moe_desc* md, void* y, const void* x,
                                         const void* scales, const void* packed_w, const void* biases,
                                         const uint32_t* ids, void* stream) {
  ztvm_status s = check_ctx(ctx);   // also makes the context's device current: the scratch array is per device
  if (s) return s;
  if (!md) return fail(ZTVM_ERR_NULL_POINTER, "desc is NULL");
  const ztvm_mm_desc* d = &md->mm;
  if ((s = check_desc(d, false))) return s;
  if (!d->affine) return fail(ZTVM_ERR_UNSUPPORTED, "MoE expert weights are affine-quantised only");
  if (d->out_f32) return fail(ZTVM_ERR_UNSUPPORTED, "MoE expert matmuls write f16");
  if (d->M > 1) return fail(ZTVM_ERR_BAD_DIMS, "MoE matmul is per (token, slot): mm.M must be 1 (or 0)");
  if ((s = check_buffers(d, y, x, scales, packed_w, biases))) return s;
  if (!ids) return fail(ZTVM_ERR_NULL_POINTER, "ids is NULL");
  if (md->tokens == 0) return ZTVM_OK;
  if (md->slots == 0 || md->experts == 0) return fail(ZTVM_ERR_BAD_DIMS, "slots and experts must be non-zero");
  if (md->ids_stride < md->slots) return fail(ZTVM_ERR_BAD_DIMS, "ids_stride=%u < slots=%u", md->ids_stride, md->slots);
  const uint64_t pairs = (uint64_t)md->tokens * md->slots;
  if (!ztvm::moe_static_scratch_fits(md->experts, pairs))
    return fail(ZTVM_ERR_TOO_LARGE,
                "tokens*slots=%llu, experts=%u exceed the fixed scratch of this entry point (at most %u pairs, %u experts): "
                "split the token list or call ztvm_int4_matmul_moe",
                (unsigned long long)pairs, md->experts, (unsigned)ZTVM_MOE_NOALLOC_MAX_PAIRS,
                (unsigned)ZTVM_MOE_NOALLOC_MAX_EXPERTS);
  if ((md->in_slot_stride | md->in_tok_stride) % 8)
    return fail(ZTVM_ERR_ALIGNMENT, "input strides must be multiples of 8 elements (16-byte activation loads)");
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  const ztvm::GemvParams p = moe_params(ctx, md, y, x, scales, packed_w, biases, ids);
  const int pick = moe_pick(ctx, md, p, y);   // the same choice ztvm_int4_matmul_moe makes
  if (!pick)
    return fail(ZTVM_ERR_UNSUPPORTED,
                "this entry point runs the grouped kernels only: bits=4, group=64, K %% 64 == 0, N %% 8 == 0 "
                "(got bits=%u group=%u K=%u N=%u)", d->bits, d->group, d->K, d->N);
  if (pick == 2) ZTVM_CUDA(ztvm::launch_moe_tc_static(p, md->tokens, md->slots, ctx->sm_count, st));
  else if (pick == 1) ZTVM_CUDA(ztvm::launch_moe_ta_static(p, md->tokens, md->slots, ctx->err_counter + 1, ctx->sm_count, st));
  else ZTVM_CUDA(ztvm::launch_moe_grouped_static(p, md->tokens, md->slots, ctx->err_counter + 1, st));
  return ZTVM_OK;
}

ztvm_status ztvm_moe_plan_reuse(ztvm_ctx* ctx, int32_t enable) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  ctx->plan_reuse = enable ? 1 : 0;
  ctx->plan_ids = nullptr;
  return ZTVM_OK;
}

ztvm_status ztvm_moe_route_topk(ztvm_ctx* ctx, uint32_t E, uint32_t K, uint32_t norm_topk, uint32_t has_shared,
                                uint32_t tokens, uint32_t* ids, float* scores, const float* logits, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!ids || !scores || !logits) return fail(ZTVM_ERR_NULL_POINTER, "ids/scores/logits must be non-NULL");
  if (E == 0 || E > 1024) return fail(ZTVM_ERR_TOO_LARGE, "E=%u: 1..1024 routed experts supported", E);
  if (K == 0 || K > 32 || K > E) return fail(ZTVM_ERR_BAD_DIMS, "K=%u: need 1 <= K <= min(32, E)", K);
  if (tokens == 0) return ZTVM_OK;
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ctx->plan_ids = nullptr;   // a new id list: whatever plan the context holds describes the old one
  ZTVM_CUDA(ztvm::launch_route_topk(logits, ids, scores, tokens, E, K, norm_topk != 0, has_shared != 0, st));
  return ZTVM_OK;
}

ztvm_status ztvm_moe_dispatch_plan(ztvm_ctx* ctx, const uint32_t* ids, uint32_t tokens, uint32_t slots, uint32_t ids_stride,
                                   uint32_t experts, uint32_t experts_per_rank, uint32_t world, int64_t* order,
                                   int32_t* local_expert, int64_t* send_counts, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!ids || !order || !local_expert || !send_counts) return fail(ZTVM_ERR_NULL_POINTER, "ids/order/local_expert/send_counts must be non-NULL");
  if (experts == 0 || experts > 1024) return fail(ZTVM_ERR_TOO_LARGE, "experts=%u: 1..1024 supported", experts);
  if (experts_per_rank == 0 || world == 0 || (uint64_t)experts_per_rank * world < experts)
    return fail(ZTVM_ERR_BAD_DIMS, "experts_per_rank=%u x world=%u does not cover experts=%u", experts_per_rank, world, experts);
  if (slots == 0 || ids_stride < slots) return fail(ZTVM_ERR_BAD_DIMS, "need 1 <= slots <= ids_stride (slots=%u, ids_stride=%u)", slots, ids_stride);
  const uint64_t pairs = (uint64_t)tokens * slots;
  if (pairs >= (1ull << 31)) return fail(ZTVM_ERR_TOO_LARGE, "tokens*slots=%llu", (unsigned long long)pairs);
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  if (tokens == 0) {
    ZTVM_CUDA(cudaMemsetAsync(send_counts, 0, (size_t)world * 8, st));
    return ZTVM_OK;
  }
  const size_t need = ztvm::moe_grouped_scratch_bytes(experts, (uint32_t)pairs);
  if (ctx->d_ws_bytes < need) {
    ZTVM_CUDA(cudaDeviceSynchronize());
    if ((s = grow(&ctx->d_ws, &ctx->d_ws_bytes, need, false))) return s;
  }
  ctx->plan_ids = nullptr;
  ztvm::GemvParams p;
  memset(&p, 0, sizeof(p));
  p.ids = ids;
  p.experts = experts;
  p.ids_stride = ids_stride;
  p.err_counter = ctx->err_counter;
  ZTVM_CUDA(ztvm::launch_moe_dispatch_plan(p, tokens, slots, experts_per_rank, world, static_cast<uint32_t*>(ctx->d_ws),
                                           reinterpret_cast<long long*>(order), local_expert,
                                           reinterpret_cast<long long*>(send_counts), st));
  return ZTVM_OK;
}

ztvm_status ztvm_moe_ep_dispatch(ztvm_ctx* ctx, const ztvm_moe_ep_layout* L, const uint32_t* ids, uint32_t tokens,
                                 uint32_t top_k, uint32_t has_shared, uint32_t ids_stride, const void* x, uint32_t d,
                                 uint32_t x_tok_stride, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!L || !ids || !x) return fail(ZTVM_ERR_NULL_POINTER, "layout/ids/x must be non-NULL");
  if (L->world == 0 || L->world > 8 || L->rank >= L->world) return fail(ZTVM_ERR_BAD_DIMS, "world=%u rank=%u: 1..8 ranks", L->world, L->rank);
  if (L->experts_per_rank == 0 || top_k == 0 || ids_stride < top_k + (has_shared ? 1u : 0u))
    return fail(ZTVM_ERR_BAD_DIMS, "experts_per_rank=%u top_k=%u ids_stride=%u", L->experts_per_rank, top_k, ids_stride);
  if (d == 0 || d % 8 || x_tok_stride % 8 || !aligned(x, 16)) return fail(ZTVM_ERR_ALIGNMENT, "rows are copied in 16-byte pieces: d, x_tok_stride multiples of 8, x 16-byte aligned");
  if ((uint64_t)tokens * top_k > L->seg_cap || tokens > L->seg_cap)
    return fail(ZTVM_ERR_TOO_LARGE, "tokens*top_k=%llu exceeds seg_cap=%u", (unsigned long long)tokens * top_k, L->seg_cap);
  if (!L->cursors) return fail(ZTVM_ERR_NULL_POINTER, "layout.cursors is NULL");
  for (uint32_t r = 0; r < L->world; ++r)
    if (!L->recv_x[r] || !L->recv_ids[r] || !L->recv_src[r] || !L->recv_cnt[r] || !aligned(L->recv_x[r], 16))
      return fail(ZTVM_ERR_NULL_POINTER, "receive buffers of rank %u missing or misaligned", r);
  if (tokens == 0) return ZTVM_OK;
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ztvm::EpDispatchParams p;
  memset(&p, 0, sizeof(p));
  p.ids = ids; p.x = static_cast<const __half*>(x);
  p.tokens = tokens; p.top_k = top_k; p.has_shared = has_shared ? 1u : 0u; p.ids_stride = ids_stride;
  p.slots_total = top_k + p.has_shared; p.d = d; p.x_tok_stride = x_tok_stride;
  p.epr = L->experts_per_rank; p.world = L->world; p.rank = L->rank; p.seg_cap = L->seg_cap;
  for (uint32_t r = 0; r < L->world; ++r) {
    p.recv_x[r] = static_cast<__half*>(L->recv_x[r]); p.recv_ids[r] = L->recv_ids[r];
    p.recv_src[r] = L->recv_src[r]; p.recv_cnt[r] = L->recv_cnt[r];
  }
  p.cursors = L->cursors; p.err = ctx->err_counter;
  ZTVM_CUDA(ztvm::launch_moe_ep_dispatch(p, ctx->sm_count, st));
  return ZTVM_OK;
}

ztvm_status ztvm_int4_matmul_moe_ep(ztvm_ctx* ctx, const ztvm_moe_desc* md, const ztvm_moe_ep_rows* rows, void* y,
                                    const void* x, const void* scales, const void* packed_w, const void* biases,
                                    const uint32_t* ids, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!md || !rows) return fail(ZTVM_ERR_NULL_POINTER, "desc/rows is NULL");
  const ztvm_mm_desc* d = &md->mm;
  if ((s = check_desc(d, false))) return s;
  if (!d->affine || d->out_f32 || d->M > 1) return fail(ZTVM_ERR_UNSUPPORTED, "MoE expert matmuls are affine, f16 out, one row per pair");
  if (md->slots != 1) return fail(ZTVM_ERR_BAD_DIMS, "a receive buffer holds one id per row: slots must be 1 (got %u)", md->slots);
  if (!rows->seg_counts || rows->seg_cap == 0 || rows->segments == 0 || rows->segments > 9 ||
      (uint64_t)rows->segments * rows->seg_cap != md->tokens)
    return fail(ZTVM_ERR_BAD_DIMS, "segments=%u x seg_cap=%u must equal tokens=%u (at most 9 regions)", rows->segments, rows->seg_cap, md->tokens);
  void* y_check = y;
  if (rows->dst_index) {
    for (uint32_t i = 0; i < rows->segments; ++i)
      if (!rows->y_seg[i]) return fail(ZTVM_ERR_NULL_POINTER, "y_seg[%u] is NULL", i);
    y_check = rows->y_seg[0];
  }
  if ((s = check_buffers(d, y_check, x, scales, packed_w, biases))) return s;
  if (!ids) return fail(ZTVM_ERR_NULL_POINTER, "ids is NULL");
  if (md->experts == 0 || md->ids_stride < 1) return fail(ZTVM_ERR_BAD_DIMS, "experts and ids_stride must be non-zero");
  if ((md->in_slot_stride | md->in_tok_stride) % 8)
    return fail(ZTVM_ERR_ALIGNMENT, "input strides must be multiples of 8 elements (16-byte activation loads)");
  if ((uint64_t)md->tokens >= (1ull << 31)) return fail(ZTVM_ERR_TOO_LARGE, "tokens=%u", md->tokens);
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ztvm::GemvParams p = moe_params(ctx, md, y_check, x, scales, packed_w, biases, ids);
  p.seg_counts = rows->seg_counts; p.seg_cap = rows->seg_cap; p.dst_index = rows->dst_index;
  for (uint32_t i = 0; i < rows->segments; ++i) p.y_seg[i] = rows->y_seg[i];
  const int pick = moe_pick(ctx, md, p, y_check);
  if (pick != 1 && pick != 2)
    return fail(ZTVM_ERR_UNSUPPORTED, "the expert-parallel form runs the grouped kernels only: bits=4, group=64, K %% 64 == 0 "
                "(got bits=%u group=%u K=%u N=%u)", d->bits, d->group, d->K, d->N);
  const size_t need = ztvm::moe_grouped_scratch_bytes(md->experts, md->tokens);
  if (ctx->d_ws_bytes < need) {
    ZTVM_CUDA(cudaDeviceSynchronize());
    if ((s = grow(&ctx->d_ws, &ctx->d_ws_bytes, need, false))) return s;
    ctx->plan_ids = nullptr;
  }
  const uint32_t tile_rows = pick == 1 ? ztvm::kMoeTaTileRows : ztvm::kMoeTcTileRows;
  const bool reuse = rows->reuse_plan && ctx->plan_ids == ids && ctx->plan_segs == rows->seg_counts &&
                     ctx->plan_tokens == md->tokens && ctx->plan_tile_rows == tile_rows && ctx->plan_experts == md->experts;
  uint32_t* ws = static_cast<uint32_t*>(ctx->d_ws);
  if (pick == 2) ZTVM_CUDA(ztvm::launch_moe_tc(p, md->tokens, 1, ws, ctx->sm_count, st, reuse));
  else ZTVM_CUDA(ztvm::launch_moe_ta(p, md->tokens, 1, ws, ctx->err_counter + 1, ctx->sm_count, st, reuse));
  ctx->plan_ids = ids; ctx->plan_segs = rows->seg_counts; ctx->plan_tokens = md->tokens; ctx->plan_slots = 1;
  ctx->plan_stride = md->ids_stride; ctx->plan_tile_rows = tile_rows; ctx->plan_experts = md->experts;
  return ZTVM_OK;
}

ztvm_status ztvm_silu_mul_rows(ztvm_ctx* ctx, const ztvm_moe_ep_rows* rows, uint32_t ffn, void* h, const void* gate_up,
                               void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!rows || !h || !gate_up) return fail(ZTVM_ERR_NULL_POINTER, "rows/h/gate_up must be non-NULL");
  if (ffn == 0 || !rows->seg_counts || rows->seg_cap == 0) return fail(ZTVM_ERR_BAD_DIMS, "ffn, seg_counts and seg_cap must be set");
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ZTVM_CUDA(ztvm::launch_silu_mul(static_cast<const __half*>(gate_up), static_cast<__half*>(h), rows->segments * rows->seg_cap,
                                  ffn, st, rows->seg_counts, rows->seg_cap));
  return ZTVM_OK;
}

ztvm_status ztvm_silu_mul(ztvm_ctx* ctx, uint32_t rows, uint32_t ffn, void* h, const void* gate_up, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!h || !gate_up) return fail(ZTVM_ERR_NULL_POINTER, "h/gate_up must be non-NULL");
  if (ffn == 0) return fail(ZTVM_ERR_BAD_DIMS, "ffn=0");
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ZTVM_CUDA(ztvm::launch_silu_mul(static_cast<const __half*>(gate_up), static_cast<__half*>(h), rows, ffn, st));
  return ZTVM_OK;
}

ztvm_status ztvm_moe_combine(ztvm_ctx* ctx, uint32_t tokens, uint32_t slots, uint32_t d, void* out,
                             const void* y_slots, const float* scores, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!out || !y_slots || !scores) return fail(ZTVM_ERR_NULL_POINTER, "out/y_slots/scores must be non-NULL");
  if (slots == 0 || d == 0) return fail(ZTVM_ERR_BAD_DIMS, "slots and d must be non-zero");
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ZTVM_CUDA(ztvm::launch_moe_combine(static_cast<const __half*>(y_slots), scores, static_cast<__half*>(out), tokens,
                                     slots, d, st));
  return ZTVM_OK;
}

ztvm_status ztvm_unpack_codes(ztvm_ctx* ctx, const ztvm_mm_desc* d, uint8_t* codes, const void* packed_w,
                              void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if ((s = check_desc(d, false))) return s;
  if (!codes || !packed_w) return fail(ZTVM_ERR_NULL_POINTER, "codes/packed_w must be non-NULL");
  if (!aligned(codes, 8) || !aligned(packed_w, 4)) return fail(ZTVM_ERR_ALIGNMENT, "codes need 8-byte alignment");
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ZTVM_CUDA(ztvm::launch_unpack_codes(static_cast<const uint32_t*>(packed_w), codes, d->N, d->K, (int)d->bits, st));
  return ZTVM_OK;
}

ztvm_status ztvm_unpack_codes_streamed(ztvm_ctx* ctx, const ztvm_mm_desc* d, uint8_t* codes, const void* packed_w,
                                       void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if ((s = check_desc(d, false))) return s;
  if (!codes || !packed_w) return fail(ZTVM_ERR_NULL_POINTER, "codes/packed_w must be non-NULL");
  if (!aligned(codes, 8) || !aligned(packed_w, 4)) return fail(ZTVM_ERR_ALIGNMENT, "codes need 8-byte alignment");
  if (d->bits == 8) return fail(ZTVM_ERR_UNSUPPORTED, "8-bit weights have no streaming matrix-unit kernel: use ztvm_unpack_codes");
  if (d->bits == 3 && d->K % 64) return fail(ZTVM_ERR_BAD_DIMS, "3-bit streams are unpacked per 64 codes: K=%u", d->K);
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ZTVM_CUDA(ztvm::launch_unpack_codes_streamed(static_cast<const uint32_t*>(packed_w), codes, d->N, d->K, (int)d->bits, st));
  return ZTVM_OK;
}

ztvm_status ztvm_dequant(ztvm_ctx* ctx, const ztvm_mm_desc* d, void* w_out, int32_t as_f16, const void* scales,
                         const void* packed_w, const void* biases, void* stream) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if ((s = check_desc(d, false))) return s;
  if (!w_out || !packed_w || !scales) return fail(ZTVM_ERR_NULL_POINTER, "w_out/scales/packed_w must be non-NULL");
  if (d->affine && !biases) return fail(ZTVM_ERR_NULL_POINTER, "affine weights need biases");
  if (!aligned(w_out, 16)) return fail(ZTVM_ERR_ALIGNMENT, "w_out needs 16-byte alignment");
  cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : ctx->stream;
  ZTVM_CUDA(ztvm::launch_dequant(static_cast<const uint32_t*>(packed_w), static_cast<const __half*>(scales),
                                 static_cast<const __half*>(biases), w_out, d->N, d->K, (int)d->bits,
                                 (uint32_t)log2_exact(d->group), d->affine != 0, as_f16 != 0, st));
  return ZTVM_OK;
}

ztvm_status ztvm_device_errors(ztvm_ctx* ctx, void* stream, uint32_t* count) {
  ztvm_status s = check_ctx(ctx);
  if (s) return s;
  if (!count) return fail(ZTVM_ERR_NULL_POINTER, "count is NULL");
  if (stream) ZTVM_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  ZTVM_CUDA(cudaStreamSynchronize(ctx->stream));
  uint32_t words[2] = {0, 0};
  ZTVM_CUDA(cudaMemcpy(words, ctx->err_counter, 8, cudaMemcpyDeviceToHost));
  ZTVM_CUDA(cudaMemset(ctx->err_counter, 0, 8));
  *count = words[0];
  if (words[1])
    return fail(ZTVM_ERR_CUDA, words[1] == 20u ? "a peer barrier gave up waiting for another rank (code %u); what followed it ran on incomplete data"
                                               : "a bounded wait inside a tensor-core kernel ran out (stage code %u); its output is invalid",
                words[1]);
  return ZTVM_OK;
}

}  // extern "C"
