// Plan scratch of the grouped MoE kernels (the tensor-core tiles of ztvm_moe_gemm.cu and the streaming kernel of
// ztvm_moe_tc.cu): layout in 32-bit words, and the launcher of the three planning kernels.
#pragma once
#include "ztvm_kernels.h"

namespace ztvm {

constexpr uint32_t kMoeMinTileRows = 8;   // smallest tile any grouped kernel asks for: sizes the tile table

struct MoeScratch {
  uint32_t* counts;   // [E]
  uint32_t* offsets;  // [E + 1]
  uint32_t* cursor;   // [E]
  uint32_t* ntiles;   // [1]
  uint32_t* tiles;    // [max_tiles][3]: expert, first sorted row, rows
  uint32_t* sorted;   // [P] pair index = token * slots + slot
};
__host__ __device__ constexpr size_t moe_max_tiles(uint32_t E, uint32_t P) {
  return (size_t)(P + kMoeMinTileRows - 1) / kMoeMinTileRows + E;
}
__host__ __device__ constexpr size_t moe_scratch_words(uint32_t E, uint32_t P) {
  return (size_t)E * 3 + 2 + 2 + moe_max_tiles(E, P) * 3 + P + 16;
}
__host__ __device__ inline MoeScratch moe_scratch_carve(uint32_t* base, uint32_t E, uint32_t P) {
  MoeScratch s;
  s.counts = base;
  s.offsets = s.counts + E;
  s.cursor = s.offsets + E + 1;
  s.ntiles = s.cursor + E;
  s.tiles = s.ntiles + 1;
  s.sorted = s.tiles + moe_max_tiles(E, P) * 3;
  return s;
}

cudaError_t launch_moe_plan(const GemvParams& g, uint32_t tokens, uint32_t slots, const MoeScratch& sc, uint32_t tile_rows,
                            cudaStream_t st);

}  // namespace ztvm
