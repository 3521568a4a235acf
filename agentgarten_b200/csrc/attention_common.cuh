// Shared pieces of the segment-list flash-attention kernels (head_dim 128, bf16).
//
// Work description (all int32, built on the host once per forward):
//   q_tiles[t] = (q_row, rows, first_entry, entries)   one 128-row query tile
//   entries[e] = (source, k_row, k_len)                a key segment visible to the tile
//        source 0: text keys (valid length per sample = text_valid[b], prefix-valid)
//        source 1: visual keys (all k_len valid)
//        source 2: visual keys, causal against the tile's own chunk (key i visible to
//                  chunk-local query row r iff i <= r); q_local is q_row - chunk start,
//                  carried in the third field of the tile as rows | (q_local << 8)
// Key tiles are cut per segment from the segment start and never straddle two segments,
// so the softmax of a query row accumulates over the same tile partition no matter what
// else is processed in the launch.
#pragma once

#include "sm100.cuh"

namespace agb {

constexpr int ATT_D = 128;       // head dim
constexpr int ATT_BM = 128;      // query rows per tile
constexpr int ATT_BN = 128;      // keys per tile
constexpr int ATT_MAX_TILES = 1024;

struct KeyTile {
  int source;   // 0 text, 1 visual
  int row;      // first key row in its tensor
  int valid;    // number of valid keys in the tile (1..128)
  int causal0;  // -1: no causal mask; else key index (segment-local) of the tile's first key
};

// The work lists come from the host.  Every kernel checks the entries it is about to follow
// against the extents of its tensors before the first access (one thread, a few comparisons
// per CTA) and, instead of following a bad one, records kBadIndex and does nothing.
__device__ __forceinline__ bool rows_inside(int row, int rows, int64_t extent, int most) {
  return row >= 0 && rows >= 1 && rows <= most && int64_t(row) + rows <= extent;
}

// Expands the segment entries of one query tile into a list of key tiles in shared memory.
// Called by one thread.  Returns the tile count, -1 when the list would overflow, -2 when an
// entry does not lie inside its key tensor (nk visual keys, text_len text keys).
__device__ inline int build_key_tiles(const int* __restrict__ entries, int first, int count,
                                      const int* __restrict__ text_valid, int batch, int q_local,
                                      int q_rows, KeyTile* out, int64_t nk, int64_t text_len) {
  int n = 0;
  for (int e = first; e < first + count; ++e) {
    const int source = entries[3 * e + 0];
    const int k_row = entries[3 * e + 1];
    int len = entries[3 * e + 2];
    if (source < 0 || source > 2 || k_row < 0 || len < 0 ||
        int64_t(k_row) + len > (source == 0 ? text_len : nk)) {
      return -2;
    }
    if (source == 0 && text_valid) len = min(len, text_valid[batch]);
    const bool causal = source == 2;
    if (causal) len = min(len, q_local + q_rows);  // keys past the last query row are masked
    for (int t = 0; t * ATT_BN < len; ++t) {
      if (n >= ATT_MAX_TILES) return -1;
      out[n].source = source == 0 ? 0 : 1;
      out[n].row = k_row + t * ATT_BN;
      out[n].valid = min(ATT_BN, len - t * ATT_BN);
      out[n].causal0 = causal ? t * ATT_BN : -1;
      ++n;
    }
  }
  return n;
}

}  // namespace agb
