// Internal launch interfaces between the C-ABI layer (ztvm_api.cu) and the kernel files.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ztvm {

struct GemvParams {
  const uint32_t* W;   // packed codes [N][KP] (MoE: [experts][N][KP])
  const __half* S;     // scales [N][SPR]
  const __half* B;     // biases [N][SPR], nullptr for the symmetric flavour
  const __half* X;     // activations
  void* Y;             // f16 or f32 output
  uint32_t K, N, M;
  uint32_t KP;           // words per weight row = K*bits/32
  uint32_t SPR;          // scale groups per row = K/group
  uint32_t group_shift;  // log2(group)
  uint32_t out_f32;
  uint32_t x_row_stride, y_row_stride;  // elements between batch rows
  uint32_t tile_units;                  // set by the launcher
  // MoE indirection (int4_matmul.gen.ts:216-225)
  const uint32_t* ids;
  uint32_t experts, in_slot_stride, out_slot_stride, in_tok_stride, out_tok_stride, ids_stride;
  uint32_t* err_counter;
  // further destinations of the output (same layout as Y): peers' copies of a sharded projection's result
  void* y_more[7];
  uint32_t n_more;
  // Expert-parallel form of the grouped MoE matmuls (one entry of `ids` per row, slots = 1): the id list is made of
  // regions of seg_cap entries, one per source rank, of which only the first seg_counts[region] are live (the others
  // are skipped without being counted as bad ids); with dst_index set, the output row of entry i goes to
  // y_seg[i / seg_cap] + dst_index[i] * out_tok_stride (the buffers of the ranks the rows came from).
  const uint32_t* seg_counts;
  uint32_t seg_cap;
  const uint32_t* dst_index;
  void* y_seg[9];
  // Fused gate/up form of the persistent GEMV (fused_ffn.wgsl): the weight holds 2 * pair_rows rows, gate rows first
  // and up rows after them; the output has pair_rows columns, y[i] = f16(up[i] * silu(gate[i])) with both dot products
  // and the activation in f32. 0 = plain matmul.
  uint32_t pair_rows;
};

cudaError_t launch_gemv(GemvParams p, int bits, bool moe, uint32_t tokens, uint32_t slots, int sm_count,
                        cudaStream_t st);

// 4-bit weights on the warp-level matrix unit (ztvm_gemv_mma.cu); M <= 8.
bool gemv_mma_supported(int bits, uint32_t group);
cudaError_t launch_gemv_mma(GemvParams p, bool moe, uint32_t tokens, uint32_t slots, cudaStream_t st);

// 4-bit / group-64 weights, M <= 8, persistent matrix-unit GEMV (ztvm_gemv_tc.cu). `gemv_tc_supported` checks shape
// and alignment; anything it refuses goes to the kernels above.
bool gemv_tc_supported(const GemvParams& p, int bits, int sm_count);
cudaError_t launch_gemv_tc(const GemvParams& p, int sm_count, cudaStream_t st);

// 3-bit / group-64 weights, M = 1, persistent matrix-unit GEMV (ztvm_gemv_tc3.cu).
bool gemv_tc3_supported(const GemvParams& p, int bits, int sm_count);
cudaError_t launch_gemv_tc3(const GemvParams& p, int sm_count, cudaStream_t st);

// 4-bit weights, M > 8: tcgen05 GEMM with TMEM accumulators (ztvm_gemm.cu). status[0] receives a non-zero code
// if a pipeline wait inside the kernel ran out.
bool gemm_w4_supported(int bits, uint32_t group, uint32_t K);
cudaError_t launch_gemm_w4(const uint32_t* W, const __half* S, const __half* B, const __half* X, void* Y, uint32_t M,
                           uint32_t N, uint32_t K, uint32_t group_shift, bool out_f32, uint32_t* status, cudaStream_t st);

// Grouped MoE expert matmul (ztvm_moe_gemm.cu): pairs sorted by expert, tcgen05 tiles. `scratch` holds the plan
// (moe_grouped_scratch_bytes), `status[0]` receives a non-zero code if a bounded wait ran out.
size_t moe_grouped_scratch_bytes(uint32_t experts, uint32_t pairs);
bool moe_grouped_supported(int bits, uint32_t group, uint32_t K, uint32_t N, uint32_t experts);
cudaError_t launch_moe_grouped(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t* scratch, uint32_t* status,
                               cudaStream_t st);
// The same contract with the dequantised expert weights as the A operand in tensor memory, persistent over the units
// (ztvm_moe_ta.cu): the default tensor-core form; launch_moe_grouped stays selectable for comparison.
bool moe_ta_supported(int bits, uint32_t group, uint32_t K, uint32_t N, uint32_t experts);
cudaError_t launch_moe_ta(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t* scratch, uint32_t* status,
                          int sm_count, cudaStream_t st, bool reuse_plan = false);
constexpr uint32_t kMoeTaTileRows = 128, kMoeTcTileRows = 8;   // pairs per tile each kernel asks the plan for
// Streaming form of the grouped MoE matmul (ztvm_moe_tc.cu) for launches where an expert sees only a few pairs: bound
// by reading each active expert's weights once. Same scratch as launch_moe_grouped.
bool moe_tc_supported(const GemvParams& g, int bits);
cudaError_t launch_moe_tc(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t* scratch, int sm_count,
                          cudaStream_t st, bool reuse_plan = false);
// Dispatch plan of the expert-parallel form: pairs in owner-rank order, their local expert index, pairs per rank.
cudaError_t launch_moe_dispatch_plan(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t epr, uint32_t world,
                                     uint32_t* scratch, long long* order, int* local_expert, long long* send_counts,
                                     cudaStream_t st);
// The same launch with the planning scratch in a fixed array inside the module (no allocation anywhere on the path).
// `moe_static_scratch_fits` says whether a problem fits that array; the launcher refuses one that does not.
bool moe_static_scratch_fits(uint32_t experts, uint64_t pairs);
cudaError_t launch_moe_grouped_static(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t* status,
                                      cudaStream_t st);
cudaError_t launch_moe_tc_static(const GemvParams& g, uint32_t tokens, uint32_t slots, int sm_count, cudaStream_t st);
cudaError_t launch_moe_ta_static(const GemvParams& g, uint32_t tokens, uint32_t slots, uint32_t* status, int sm_count,
                                 cudaStream_t st);

// The same GEMM with the dequantised weights as the A operand in tensor memory and the activations as the only
// shared-memory operand (ztvm_gemm_ta.cu): the default for M > 8; launch_gemm_w4 stays selectable for comparison.
cudaError_t launch_gemm_w4_ta(const uint32_t* W, const __half* S, const __half* B, const __half* X, void* Y, uint32_t M,
                              uint32_t N, uint32_t K, uint32_t group_shift, bool out_f32, uint32_t* status, cudaStream_t st);

// Dispatch step of the expert-parallel MoE block (ztvm_moe_ep.cu): pair rows stored straight into the owners' receive
// buffers (peer-mapped addresses), one region per source rank.
struct EpDispatchParams {
  const uint32_t* ids;      // [tokens][ids_stride], first top_k entries of a row are the routed experts
  const __half* x;          // [tokens][x_tok_stride]
  uint32_t tokens, top_k, has_shared, ids_stride, slots_total, d, x_tok_stride;
  uint32_t epr, world, rank, seg_cap;
  __half* recv_x[8];
  uint32_t* recv_ids[8];
  uint32_t* recv_src[8];
  uint32_t* recv_cnt[8];
  uint32_t* cursors;        // this rank's own: world + 2 words, zero before the first step
  uint32_t* err;
};
cudaError_t launch_moe_ep_dispatch(const EpDispatchParams& p, int sm_count, cudaStream_t st);

struct PeerBarrierParams {
  uint32_t* flags[8];       // every rank's flag words (world + 1 each), as mapped in this process
  uint32_t world, rank;
  unsigned long long wait_cycles;
  uint32_t* status;
};
cudaError_t launch_peer_barrier(const PeerBarrierParams& p, cudaStream_t st);

cudaError_t launch_unpack_codes(const uint32_t* W, uint8_t* codes, uint32_t N, uint32_t K, int bits, cudaStream_t st);
// The codes as the streaming matrix-unit kernels consume them (in-place f16 subnormals, scaled back to integers).
cudaError_t launch_unpack_codes_streamed(const uint32_t* W, uint8_t* codes, uint32_t N, uint32_t K, int bits, cudaStream_t st);
cudaError_t launch_dequant(const uint32_t* W, const __half* S, const __half* B, void* out, uint32_t N, uint32_t K,
                           int bits, uint32_t group_shift, bool affine, bool as_f16, cudaStream_t st);

cudaError_t launch_embedding_affine(const int32_t* input_ids, const uint32_t* W, const __half* S, const __half* B, __half* out,
                                    uint32_t seq_len, uint32_t D, uint32_t vocab, int bits, uint32_t* err, cudaStream_t st);
cudaError_t launch_f16_matvec(const __half* x, const __half* w, float* y, uint32_t D, uint32_t rows, uint32_t tokens, cudaStream_t st);
cudaError_t launch_route_topk(const float* logits, uint32_t* ids, float* scores, uint32_t tokens, uint32_t E,
                              uint32_t K, bool norm_topk, bool has_shared, cudaStream_t st);
// seg_counts != nullptr: rows come in regions of seg_cap, only the first seg_counts[region] of each are computed
cudaError_t launch_silu_mul(const __half* gate_up, __half* h, uint32_t rows, uint32_t ffn, cudaStream_t st,
                            const uint32_t* seg_counts = nullptr, uint32_t seg_cap = 1);
cudaError_t launch_silu_mul_f32(const float* gate_up, __half* h, uint32_t rows, uint32_t ffn, cudaStream_t st);
cudaError_t launch_moe_combine(const __half* y_slots, const float* scores, __half* out, uint32_t tokens,
                               uint32_t slots, uint32_t d, cudaStream_t st);

}  // namespace ztvm
