// Structured attention masks shared by the forward and backward flash-attention kernels.
//
// Every query row attends the union of up to three key ranges [lo, hi) (block-causal windows with a sink, teacher
// forcing over [clean | noisy] halves, segment plans); the ranges are per row and the same for every head and batch
// entry.  A CTA does not walk all tiles of the streamed operand but a precomputed list of the tiles that interact with
// its stationary rows at all; bit 30 of a list entry marks a tile in which some (row, column) pair is masked -- only
// those tiles pay for element-wise masking.  The tables are built on the host (ops/attention_mask.py).
#pragma once

namespace solar {

struct AttnMask {
  const int* row_ranges;   // [S_queries][6]: lo0, hi0, lo1, hi1, lo2, hi2 (empty range: lo >= hi)
  const int* tile_list;    // [gridDim.x][stride] tile indices of the streamed operand
  const int* tile_count;   // [gridDim.x], >= 1
  int stride;
  const int* order;        // [gridDim.x] or null: the stationary tile that CTA x works on.  CTAs are dispatched in
                           // index order and own very different numbers of live tiles (a query tile of the first
                           // chunk sees one chunk of keys, one of the last sees the whole window); listing the
                           // heaviest tiles first keeps the end of the launch for the light ones
};
__device__ __forceinline__ int mask_tile_of_cta(const AttnMask& m, int cta) { return m.order ? m.order[cta] : cta; }
constexpr int kMaskPartialBit = 1 << 30;

__device__ __forceinline__ bool mask_sees(const int (&rg)[6], int key) {
  return (key >= rg[0] && key < rg[1]) || (key >= rg[2] && key < rg[3]) || (key >= rg[4] && key < rg[5]);
}

}  // namespace solar
