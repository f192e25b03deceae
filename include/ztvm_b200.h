/* ztvm_b200.h — C ABI of libztvm_b200.so: CUDA (sm_100a) replacements for the Zero-TVM
 * int4 / int3 group-quantised dequant-matmul kernels and the MoE glue around them.
 *
 * The reference engine (TypeScript + WGSL over WebGPU) has no FFI today. Its seam for this
 * path is internal: a compute pipeline per kernel variant, a bind group
 * [out, in, scales, weights, PODArgs, biases?, ids?] per call site
 * (src/zero-tvm/engine-core.ts:76-92, :1699-1703) and
 * dispatch(enc, pipeline, bindGroup, wgX, wgY, wgZ, label) (src/zero-tvm/engine-core.ts:2151-2179).
 * Each entry point below takes exactly that tuple: raw device addresses for the buffers and a
 * small POD struct holding what the reference passes in PODArgs. Citations are file:line within
 * the reference project.
 *
 * Conventions
 *  - Every function returns a ztvm_status (0 = ok). Nothing throws, aborts or launches on
 *    invalid input (the reference's WebGPU validation silently SKIPS a bad dispatch; here the
 *    caller gets an error code before any launch).
 *  - Buffer arguments are device addresses (what cudaMalloc returns). The library never
 *    allocates or frees caller buffers. Unless stated otherwise a call is asynchronous on
 *    `stream` (a cudaStream_t; NULL = the context's own stream) and performs no host sync.
 *    The context's own stream is non-blocking: it is NOT ordered against the legacy default stream.
 *    A caller whose other work runs on the legacy default stream passes cudaStreamLegacy (handle 1),
 *    not NULL, to have the call ordered with that work.
 *  - Layouts: packed weights u32[N][K*bits/32], 4-bit code i of a word at bits [4i,4i+4)
 *    (src/compiler/shaders/int4_matmul.gen.ts:157-167); 3-bit code i of a row at bit 3i of the
 *    row's LSB-first bitstream (int4_matmul.gen.ts:115-131); scales / biases f16[N][K/group];
 *    x f16[M][K]; y f16[M][N] (f32 when out_f32). Expert stacks add a leading [experts] axis.
 *  - A context is bound to one GPU and is not re-entrant (the engine is single-threaded per
 *    device, src/zero-tvm/engine-lock.ts); distinct contexts are independent.
 */
#ifndef ZTVM_B200_H_
#define ZTVM_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The library is built with hidden visibility; only these entry points are exported. */
#if defined(__GNUC__)
#define ZTVM_API __attribute__((visibility("default")))
#else
#define ZTVM_API
#endif

typedef int32_t ztvm_status;
enum {
  ZTVM_OK = 0,
  ZTVM_ERR_NULL_POINTER = 1,  /* a required pointer is NULL */
  ZTVM_ERR_BAD_DIMS = 2,      /* K/N/M/group inconsistent with the layout rules */
  ZTVM_ERR_UNSUPPORTED = 3,   /* combination the kernel family does not have (e.g. 3-bit symmetric) */
  ZTVM_ERR_ALIGNMENT = 4,     /* buffer address not aligned as the kernel requires */
  ZTVM_ERR_CUDA = 5,          /* a CUDA runtime call failed; see ztvm_last_error */
  ZTVM_ERR_BAD_CONTEXT = 6,   /* NULL / destroyed context, or wrong device */
  ZTVM_ERR_TOO_LARGE = 7      /* size beyond a stated limit of the entry point */
};

typedef struct ztvm_ctx ztvm_ctx;

/* Library ABI version (major*100 + minor). */
ZTVM_API int32_t ztvm_version(void);
ZTVM_API const char* ztvm_status_string(ztvm_status s);

/* One context per GPU: owns a stream, pinned staging and device workspace.
 * Replaces compile(device, ...) creating the matmul pipelines (src/compiler/compiler.ts:319-454). */
ZTVM_API ztvm_status ztvm_init(int32_t device_ordinal, ztvm_ctx** out_ctx);
/* Replaces DecodeEngine.destroy() for the matmul resources (src/zero-tvm/engine-core.ts:5274-5313). */
ZTVM_API ztvm_status ztvm_destroy(ztvm_ctx* ctx);
/* Message of the last failing call on this thread (valid until the next call). ctx may be NULL. */
ZTVM_API const char* ztvm_last_error(ztvm_ctx* ctx);
/* Blocks until the context's own stream is idle. */
ZTVM_API ztvm_status ztvm_sync(ztvm_ctx* ctx);

/* What the reference passes as PODArgs {K_PACKED = K*bits/32, SCALES_PER_ROW = K/group, N, M_ROWS}
 * (src/zero-tvm/engine-core.ts:787-794, :1021-1022, :4033-4038), given as logical dims. */
typedef struct ztvm_mm_desc {
  uint32_t K;       /* reduction length; K % group == 0 */
  uint32_t N;       /* output features (weight rows) */
  uint32_t M;       /* activation rows (1 = decode) */
  uint32_t group;   /* 64 (MLX affine) or 32 (MLC symmetric) */
  uint32_t bits;    /* 4, 3 or 8 (8: K_PACKED = K/4, affine only: the int8_affine_* family) */
  uint32_t affine;  /* 1: w = scale*q + bias   0: w = scale*(q-7), biases ignored */
  uint32_t out_f32; /* 1: y is f32 (lm_head), 0: f16 */
} ztvm_mm_desc;

/* y = x * dequant(W)^T. Replaces every dispatch of an int4_matmul* pipeline on a dense projection (and, with
 * bits = 8, int8_affine_matvec / int8_affine_batched, src/compiler/shaders/int8_affine_matvec.wgsl,
 * int8_affine_batched.wgsl; selected at src/zero-tvm/variants.ts:370-388):
 * int4_matmul[_f32][_sg|_tiled|_tiled8][_vec4|_vec4h][_affine][_q3], int4_matmul_batched_m4,
 * int4_matmul_batched_dyn[_affine] and the tiled / subgroup-matrix prefill GEMMs
 * (src/compiler/shaders/int4_matmul.gen.ts:170-571, :580-695, :805-1456; call sites
 * src/zero-tvm/engine-core.ts:2290, :2312, :2517-2519, :2543-2549, :4280-4293).
 * M <= 8 runs the bandwidth-bound GEMV, M <= 16 two slabs of it; larger M runs the tensor-core GEMM (which multiplies
 * f16-rounded weights f16(s*q+b), like the reference's matrix-unit GEMMs). */
ZTVM_API ztvm_status ztvm_int4_matmul(ztvm_ctx* ctx, const ztvm_mm_desc* desc, void* y, const void* x,
                             const void* scales, const void* packed_w, const void* biases, void* stream);

/* The decode matmul (M <= 8) with its [M, N] result written to n_dst destinations at once, rows y_row_stride
 * elements apart. This is the primitive of the row-sharded form: rank r owns N of a projection's N_total output
 * rows and stores its shard straight into every rank's full output (the other ranks' buffers are peer-mapped
 * device addresses: the stores travel over NVLink from inside the kernel, there is no separate all-gather).
 * Each y_dsts[i] points at the shard's first column inside destination i. The reference runs on one device and
 * has no counterpart; single-device callers use ztvm_int4_matmul. Ordering between ranks (that every shard has
 * arrived before anyone reads the full row) is the caller's: a barrier after the call.
 * Only the persistent GEMV serves this form: bits 4, group 64, K % 256 == 0, else ZTVM_ERR_UNSUPPORTED. */
ZTVM_API ztvm_status ztvm_int4_matmul_multi(ztvm_ctx* ctx, const ztvm_mm_desc* desc, void* const* y_dsts,
                                   uint32_t n_dst, uint32_t y_row_stride, const void* x, const void* scales,
                                   const void* packed_w, const void* biases, void* stream);

/* Same call with HOST activations and HOST output: copies x to the device, runs, copies y back and
 * waits. Weights, scales and biases stay device-resident, as they are in the engine
 * (src/zero-tvm/engine-core.ts:5259-5267). Synchronous. */
ZTVM_API ztvm_status ztvm_int4_matmul_host(ztvm_ctx* ctx, const ztvm_mm_desc* desc, void* y_host, const void* x_host,
                                  const void* scales, const void* packed_w, const void* biases);

/* The host-buffer call without the wait, for callers that stream many matmuls: copy-in, matmul and copy-out are
 * queued on one of three internal lanes (round robin) and the call returns. Calls on different lanes overlap -- one
 * lane's kernel runs while another's activations arrive and a third's results leave. x_host and y_host must be
 * page-locked (else ZTVM_ERR_UNSUPPORTED) and belong to the call until ztvm_host_wait returns; calls in flight need
 * distinct y_host buffers. No counterpart in the reference (its activations never leave the device). */
ZTVM_API ztvm_status ztvm_int4_matmul_host_async(ztvm_ctx* ctx, const ztvm_mm_desc* desc, void* y_host, const void* x_host,
                                        const void* scales, const void* packed_w, const void* biases);
/* Waits for every ztvm_int4_matmul_host_async call made so far. */
ZTVM_API ztvm_status ztvm_host_wait(ztvm_ctx* ctx);

/* The MoE PODArgs (src/compiler/shaders/int4_matmul.gen.ts:216-225; built at
 * src/zero-tvm/engine-core.ts:1049-1056). Strides are in ELEMENTS of x / y. mm.M must be 1. */
typedef struct ztvm_moe_desc {
  ztvm_mm_desc mm;
  uint32_t experts;         /* rows of the stacks, including the shared expert if present */
  uint32_t slots;           /* top-K plus the shared slot (src/compiler/model-spec.ts:659-660) */
  uint32_t tokens;          /* grid y of the reference dispatch */
  uint32_t in_slot_stride;  /* 0 = every slot reads the same input (gate / up) */
  uint32_t out_slot_stride;
  uint32_t in_tok_stride;
  uint32_t out_tok_stride;
  uint32_t ids_stride;      /* ids[] entries per token */
} ztvm_moe_desc;

/* For every (token, slot): expert = ids[token*ids_stride + slot]; y[...] = x[...] * dequant(W[expert])^T.
 * Replaces int4_matmul_tiled[_vec4h]_affine[_q3]_moe (int4_matmul.gen.ts:229-254; call sites
 * src/zero-tvm/engine-core.ts:2342-2349, :4387-4390). ids outside [0, experts) make the pair a no-op
 * and raise the context's device-side error counter (see ztvm_device_errors). */
ZTVM_API ztvm_status ztvm_int4_matmul_moe(ztvm_ctx* ctx, const ztvm_moe_desc* desc, void* y, const void* x,
                                 const void* scales, const void* packed_w, const void* biases,
                                 const uint32_t* ids, void* stream);

/* The gate, up and down matmuls of one step walk the same id list, and each ztvm_int4_matmul_moe call sorts it by
 * expert again (the plan). With reuse enabled, a call whose ids address, tokens, slots, ids_stride and expert count
 * equal the previous call's uses that call's plan. The caller then promises that the id list changes only through
 * ztvm_moe_route_topk on this context (which drops the plan), or calls this function again after writing it by other
 * means (every call drops the plan). Off by default. The reference has no counterpart: its kernels read ids directly
 * (int4_matmul.gen.ts:229-254) and re-stream an expert's weights per pair. */
ZTVM_API ztvm_status ztvm_moe_plan_reuse(ztvm_ctx* ctx, int32_t enable);

/* ztvm_int4_matmul_moe for callers that must not let the call allocate. It has no counterpart in the reference
 * (WebGPU buffers are all created up front there); it exists for hosts whose device memory is entirely handed
 * to their own pool, or whose serving loop cannot take the device-wide synchronisation that growing a work
 * buffer costs. ztvm_int4_matmul_moe keeps its plan (expert histogram, tile table, sorted pair list) in a
 * buffer that grows on demand; this entry point keeps it in a fixed array inside the library's device image
 * and makes no allocating call at all.
 *  - Limits: tokens*slots <= ZTVM_MOE_NOALLOC_MAX_PAIRS and experts <= ZTVM_MOE_NOALLOC_MAX_EXPERTS, else
 *    ZTVM_ERR_TOO_LARGE. Only the grouped kernels run here (there is no fall-back to the per-pair kernel):
 *    bits 4, group 64, K % 64 == 0, N % 8 == 0, input strides multiples of 8 elements. Anything else is
 *    ZTVM_ERR_UNSUPPORTED / ZTVM_ERR_ALIGNMENT. From 128 pairs on
 *    (and with the ZTVM_MOE_GROUPED knob unset) the kernel is chosen exactly as ztvm_int4_matmul_moe chooses it, so
 *    the results are those of that call on the same inputs, bit for bit; below 128 pairs that call runs the per-pair
 *    GEMV instead, and the two agree within the path's tolerance only.
 *  - The first call on a device looks up the array's device address and loads the kernels: make one call
 *    per device at start-up, before any stream capture.
 *  - There is ONE array per device, shared by every context and stream: two calls that overlap in time on
 *    the same device race on it. Issue them on one stream, or order them with events. */
#define ZTVM_MOE_NOALLOC_MAX_PAIRS 65536u
#define ZTVM_MOE_NOALLOC_MAX_EXPERTS 1024u
ZTVM_API ztvm_status ztvm_int4_matmul_moe_noalloc(ztvm_ctx* ctx, const ztvm_moe_desc* desc, void* y, const void* x,
                                         const void* scales, const void* packed_w, const void* biases,
                                         const uint32_t* ids, void* stream);

/* Router logits: logits f32[tokens][rows] = x f16[tokens][D] * router^T, rows = experts (+ the shared expert's gate row).
 * bits 8 / 4: affine group-64 router (w u32[rows][D*bits/32], scales / biases f16[rows][D/64]); bits 16: w f16[rows][D],
 * scales / biases ignored. Replaces moe_router_logits, moe_router_logits_q4 (src/compiler/shaders/moe_router_logits.wgsl:44-140)
 * and moe_router_logits_f16 (moe_router_logits_f16.wgsl); bind group [logits, x, w, scales, biases, {D, rows}], grid
 * (rows, tokens) (src/zero-tvm/engine-core.ts:2031-2033, :2331, :4383). f32 accumulation over exact codes at every token
 * count (the logits feed a softmax and a top-k). */
ZTVM_API ztvm_status ztvm_moe_router_logits(ztvm_ctx* ctx, uint32_t D, uint32_t rows, uint32_t tokens, uint32_t bits,
                                   float* logits, const void* x, const void* w, const void* scales, const void* biases,
                                   void* stream);

/* Embedding rows of an affine-quantised table: out f16[seq_len][D], row t = dequantised row input_ids[t] of weights
 * u32[vocab][D*bits/32] with scales / biases f16[vocab][D/64]; bits 4 or 8. The values are the canonical f16 weights
 * (f16_rne(fl32(s*q + b)), what ztvm_dequant gives). Replaces embedding_affine (src/compiler/shaders/embedding_affine.wgsl:38-57)
 * and embedding_affine_int8 (embedding_affine_int8.wgsl); bind group [out, input_ids, scales, weights, {seq_len, ..}, biases].
 * An id outside [0, vocab) leaves its row untouched and is counted (ztvm_device_errors). */
ZTVM_API ztvm_status ztvm_embedding_affine(ztvm_ctx* ctx, uint32_t D, uint32_t bits, uint32_t vocab, uint32_t seq_len, void* out,
                                  const int32_t* input_ids, const void* scales, const void* weights, const void* biases,
                                  void* stream);

/* softmax over E routed experts -> top-K (ties to the lower index) -> optional renormalisation ->
 * slot K = expert E with sigmoid(logit[E]) when has_shared. logits f32[tokens][E+has_shared] ->
 * ids u32[tokens][K+has_shared], scores f32 same shape.
 * Replaces moe_router_topk (src/compiler/shaders/moe_router_topk.wgsl:66-136). E <= 1024, K <= 32. */
ZTVM_API ztvm_status ztvm_moe_route_topk(ztvm_ctx* ctx, uint32_t E, uint32_t K, uint32_t norm_topk, uint32_t has_shared,
                                uint32_t tokens, uint32_t* ids, float* scores, const float* logits,
                                void* stream);

/* Dispatch plan of the expert-parallel form (experts dealt to ranks in contiguous runs of experts_per_rank): sorts
 * the (token, slot) pairs of ids u32[tokens][ids_stride] (first `slots` entries of each row) by the rank that owns
 * their expert. order i64[tokens*slots] = pair indices (token*slots + slot) in destination order, local_expert
 * i32[...] = the pair's expert index inside its owner's stack, send_counts i64[world] = pairs per destination. Ids
 * outside [0, experts) are counted (ztvm_device_errors) and left out: the filled prefix of order / local_expert has
 * sum(send_counts) entries. The order inside one expert is not deterministic. No counterpart in the reference (it
 * runs on one device); uses the context's plan buffer like ztvm_int4_matmul_moe. */
ZTVM_API ztvm_status ztvm_moe_dispatch_plan(ztvm_ctx* ctx, const uint32_t* ids, uint32_t tokens, uint32_t slots,
                                   uint32_t ids_stride, uint32_t experts, uint32_t experts_per_rank, uint32_t world,
                                   int64_t* order, int32_t* local_expert, int64_t* send_counts, void* stream);

/* ---- expert-parallel form (experts dealt to `world` ranks in contiguous runs; one process per GPU) -------------------
 * The reference runs the whole block on one device and has no counterpart for these three entry points. They keep the
 * host out of the step: rows travel by stores to peer-mapped memory from inside the kernels, every count stays on
 * the device, and the step can be captured in a CUDA graph. Ordering between ranks is the caller's: a device-side
 * barrier after ztvm_moe_ep_dispatch (all rows have landed) and one after the down projection (all results are back).
 *
 * Receive buffers of a rank: world + 1 regions of seg_cap rows each. Region s < world is written by rank s only;
 * region `world` is local (one row per token for the replicated shared expert). recv_x f16[regions][seg_cap][d],
 * recv_ids u32[regions][seg_cap] (index of the row's expert inside the receiver's stack), recv_src u32[regions][seg_cap]
 * (token * (top_k + has_shared) + slot on the source rank: where the result row belongs there), recv_cnt
 * u32[regions]. The arrays below hold EVERY rank's buffers as mapped in this process (entry `rank` = its own). */
typedef struct ztvm_moe_ep_layout {
  uint32_t world, rank, experts_per_rank, seg_cap;
  void* recv_x[8];
  uint32_t* recv_ids[8];
  uint32_t* recv_src[8];
  uint32_t* recv_cnt[8];
  uint32_t* cursors;   /* this rank's own scratch: world + 2 words, zero before the first step (kept zero by the calls) */
} ztvm_moe_ep_layout;

/* Sends every routed pair (token, slot < top_k) of ids u32[tokens][ids_stride] to the owner of its expert: the token's
 * activation row x[token] (d f16, rows x_tok_stride apart; d % 8 == 0) plus the two index words, and publishes the
 * counts. With has_shared, each token's row also goes into the local region for the shared expert (stack index
 * experts_per_rank). seg_cap >= tokens * top_k (and >= tokens). Ids outside [0, world * experts_per_rank) are counted
 * (ztvm_device_errors) and dropped. */
ZTVM_API ztvm_status ztvm_moe_ep_dispatch(ztvm_ctx* ctx, const ztvm_moe_ep_layout* layout, const uint32_t* ids,
                                 uint32_t tokens, uint32_t top_k, uint32_t has_shared, uint32_t ids_stride, const void* x,
                                 uint32_t d, uint32_t x_tok_stride, void* stream);

/* How the rows of an expert-parallel id list are laid out, for ztvm_int4_matmul_moe_ep and ztvm_silu_mul_rows. */
typedef struct ztvm_moe_ep_rows {
  const uint32_t* seg_counts;  /* live rows of each region (recv_cnt) */
  uint32_t seg_cap;            /* rows per region */
  uint32_t segments;           /* regions: desc->tokens == segments * seg_cap */
  const uint32_t* dst_index;   /* NULL: results go to y as in ztvm_int4_matmul_moe. Else (recv_src) the result row of entry
                                  i goes to y_seg[i / seg_cap] + dst_index[i] * out_tok_stride elements */
  void* y_seg[9];              /* with dst_index: output base of every region's source rank, as mapped in this process */
  uint32_t reuse_plan;         /* 1: ids, tokens and seg_counts are those of the previous call on this context (gate, up
                                  and down of one step share one id list): its expert-sorted plan is used again */
} ztvm_moe_ep_rows;

/* ztvm_int4_matmul_moe over a receive buffer: one id per row (desc->slots must be 1), only the live prefix of each
 * region is computed; entries past it are skipped without being counted as bad ids. Runs the grouped kernels only
 * (bits 4, group 64, K % 64 == 0); with dst_index the tensor-core tiles, whose epilogue stores each result row
 * straight to the rank it came from. */
ZTVM_API ztvm_status ztvm_int4_matmul_moe_ep(ztvm_ctx* ctx, const ztvm_moe_desc* desc, const ztvm_moe_ep_rows* rows, void* y,
                                    const void* x, const void* scales, const void* packed_w, const void* biases,
                                    const uint32_t* ids, void* stream);

/* ztvm_silu_mul over the live rows of a receive buffer (rows == segments * seg_cap). */
ZTVM_API ztvm_status ztvm_silu_mul_rows(ztvm_ctx* ctx, const ztvm_moe_ep_rows* rows, uint32_t ffn, void* h, const void* gate_up,
                               void* stream);

/* Device-side barrier between the ranks of a sharded form, for hosts without one of their own. flags[r] = rank r's
 * flag words as mapped in this process, u32[world + 1], zero before the first use (entry `rank` is this rank's own).
 * The kernel bumps this rank's epoch (word `world` of its own array), stores it into word `rank` of every rank's array
 * and waits until every word of its own array has reached the epoch: whatever a rank queued on its stream before its
 * call -- stores to peer memory included -- is visible to a peer's work queued after that peer's call. Every rank makes
 * the same sequence of calls on the same flag arrays. Stream-ordered and capturable; the wait is bounded (about a
 * second), an expired wait is reported by ztvm_device_errors. No counterpart in the reference (one device). */
ZTVM_API ztvm_status ztvm_peer_barrier(ztvm_ctx* ctx, uint32_t* const* flags, uint32_t world, uint32_t rank, void* stream);

/* One expert-parallel FFN step in one call: ztvm_moe_ep_dispatch, barrier, gate and up projections and SiLU over what
 * arrived, down projection storing every result row into its source rank's y_slots, barrier. Afterwards y_slots of
 * this rank holds [tokens][top_k + has_shared][d] for its own tokens (ztvm_moe_combine finishes the block).
 * ids come from ztvm_moe_route_topk. Stacks are this rank's: experts_per_rank experts (+ the shared expert last when
 * has_shared). gate_up and h are scratch for (world + 1) * seg_cap rows. */
typedef struct ztvm_moe_ffn_ep_args {
  ztvm_moe_ep_layout layout;
  uint32_t tokens, top_k, has_shared, ids_stride, d, ffn, x_tok_stride;
  const uint32_t* ids;
  const void* x;
  const void* gate_w; const void* gate_scales; const void* gate_biases;   /* [experts][ffn][...], K = d */
  const void* up_w; const void* up_scales; const void* up_biases;
  const void* down_w; const void* down_scales; const void* down_biases;   /* [experts][d][...], K = ffn */
  void* gate_up;            /* f16 [(world + 1) * seg_cap][2 * ffn] */
  void* h;                  /* f16 [(world + 1) * seg_cap][ffn] */
  void* y_slots[8];         /* every rank's result buffer f16 [tokens_r][top_k + has_shared][d], as mapped here */
  uint32_t* flags[8];       /* ztvm_peer_barrier flag words of every rank */
} ztvm_moe_ffn_ep_args;
ZTVM_API ztvm_status ztvm_moe_ffn_ep(ztvm_ctx* ctx, const ztvm_moe_ffn_ep_args* args, void* stream);

/* Row-sharded decode projection in one call: ztvm_int4_matmul_multi (this rank's N rows stored into every rank's full
 * output) followed by ztvm_peer_barrier on `flags`, after which every rank holds the whole [M, N_total] row block. */
ZTVM_API ztvm_status ztvm_int4_matmul_nshard(ztvm_ctx* ctx, const ztvm_mm_desc* desc, void* const* y_dsts, uint32_t world,
                                    uint32_t rank, uint32_t y_row_stride, const void* x, const void* scales,
                                    const void* packed_w, const void* biases, uint32_t* const* flags, void* stream);

/* Fused FFN front half: h[m][i] = f16(up_i * gate_i / (1 + exp(-gate_i))) with gate_i = x[m] . W[i], up_i = x[m] . W[ffn + i],
 * both dot products and the activation in f32, one rounding at the store. `desc->N` is ffn (the output width); the
 * weight, scales and biases hold 2 * ffn rows, gate rows first. Replaces fused_ffn (src/compiler/shaders/fused_ffn.wgsl:
 * bindings [output, input, scales, weights, PODArgs]; symmetric group 32 there) and is the affine sibling the engine
 * lacks (src/zero-tvm/engine-core.ts:2513-2519 pays gate_up matmul + silu_mul on affine models).
 * 4-bit, group 64, K % 256 == 0, M <= 8: ONE launch of the persistent GEMV, whose CTAs own gate and up tiles of the
 * same output rows. Other shapes (group 32 / 128, 3-bit, 8-bit, M > 8): the 2 * ffn-row matmul into an f32 buffer of
 * the context (grown on demand: device synchronise + cudaMalloc when a call needs more than any before it), then the
 * activation -- same arithmetic, two launches. desc->out_f32 must be 0. */
ZTVM_API ztvm_status ztvm_fused_ffn(ztvm_ctx* ctx, const ztvm_mm_desc* desc, void* h, const void* x, const void* scales,
                           const void* packed_w, const void* biases, void* stream);

/* h[r][i] = f16(up * gate * 1/(1+exp(-gate))) over rows of [gate(ffn) | up(ffn)] f16.
 * Replaces silu_mul (src/compiler/shaders/silu_mul.wgsl:26-44). */
ZTVM_API ztvm_status ztvm_silu_mul(ztvm_ctx* ctx, uint32_t rows, uint32_t ffn, void* h, const void* gate_up, void* stream);

/* out[t][i] = f16(sum_s scores[t][s] * f32(y_slots[t][s][i])).
 * Replaces moe_combine (src/compiler/shaders/moe_combine.wgsl:32-44). */
ZTVM_API ztvm_status ztvm_moe_combine(ztvm_ctx* ctx, uint32_t tokens, uint32_t slots, uint32_t d, void* out,
                             const void* y_slots, const float* scores, void* stream);

/* Parity hooks: materialise what the fused kernels never store, each through the device function the corresponding
 * production kernel inlines (so "codes and dequantised weights bit-exact" is a statement about the kernels that run).
 *  - ztvm_unpack_codes: codes u8[N][K] through the arithmetic unpack (exact f16 integers for 4-bit, the 24-bit
 *    window walk of int4_matmul.gen.ts:409-448 for 3-bit) that the CUDA-core GEMV, the tensor-core GEMMs and the
 *    dequant hook use.
 *  - ztvm_unpack_codes_streamed: the same codes as the streaming matrix-unit kernels consume them (persistent GEMV,
 *    tiled GEMVs, streaming grouped MoE kernel, 3-bit GEMV): nibbles / 3-bit fields masked IN PLACE, which are f16
 *    subnormals q * 2^-24 .. q * 2^-19, produced by the kernels' own mask functions and scaled back to integers.
 *    Those kernels never form a dequantised weight: they multiply the in-place codes with the activations exactly and
 *    fold scale and bias per group in f32 (y = sum_g s_g * dot_g + b_g * xsum_g, int4_matmul.gen.ts:388-408).
 *    bits = 3 needs K % 64 == 0 (always true: K % group == 0).
 *  - ztvm_dequant: w_out f32[N][K] (as_f16 = 0: fl32(s*q+b), the f32-staged definition of int4_matmul.gen.ts:1001, what
 *    the CUDA-core GEMV multiplies) or f16[N][K] (as_f16 = 1: f16_rne of that value; equals
 *    scripts/make-dsv2-layer-ref.py:108-116). For 4-bit weights the f16 form is produced by the word dequantiser the
 *    tensor-core GEMMs (dense and grouped) inline. desc->M is ignored. */
ZTVM_API ztvm_status ztvm_unpack_codes(ztvm_ctx* ctx, const ztvm_mm_desc* desc, uint8_t* codes, const void* packed_w,
                              void* stream);
ZTVM_API ztvm_status ztvm_unpack_codes_streamed(ztvm_ctx* ctx, const ztvm_mm_desc* desc, uint8_t* codes,
                                       const void* packed_w, void* stream);
ZTVM_API ztvm_status ztvm_dequant(ztvm_ctx* ctx, const ztvm_mm_desc* desc, void* w_out, int32_t as_f16, const void* scales,
                         const void* packed_w, const void* biases, void* stream);

/* Number of device-side argument faults (out-of-range expert ids) seen since the last call of this
 * function; resets the counter. Synchronises the context's stream and `stream`. */
ZTVM_API ztvm_status ztvm_device_errors(ztvm_ctx* ctx, void* stream, uint32_t* count);

#ifdef __cplusplus
}
#endif
#endif /* ZTVM_B200_H_ */
