// Group-metadata kernel: prefix-sums group_sizes into the row-tile -> (group, tile-in-group)
// schedule the grouped GEMM kernels walk.  It produces the same five arrays, with the same
// values, as the reference's _make_gmm_group_metadata (gpu_ragged_dot.py:70-90) for
// chunk_m == tile_m, plus two small extras the kernels need (tile prefix per group, row total).
//
// Work is O(g + U log g) in one CTA instead of the reference's O(g * U) broadcast compare.
#pragma once

#include <stdint.h>

namespace rd {

// Layout of the int32 scratch region ("workspace") shared by the metadata kernel and the
// GEMM kernels.  All offsets are in int32 units from the start of the region.
struct WorkspaceLayout {
  int g;
  int max_tiles;  // U = ceil(m / tile_m) + g, the static upper bound on live row tiles
  __host__ __device__ int off_status() const { return 0; }        // [4]  device status words
  __host__ __device__ int off_totals() const { return 4; }        // [4]  {live tiles, row total, 0, 0}
  __host__ __device__ int off_group_offsets() const { return 8; }  // [g]
  __host__ __device__ int off_tile_prefix() const { return 8 + g; }            // [g + 1]
  __host__ __device__ int off_tile2group() const { return 8 + 2 * g + 1; }     // [U]
  __host__ __device__ int off_tile2idx() const { return 8 + 2 * g + 1 + max_tiles; }  // [U]
  // [U] records of 8 words, 32-byte aligned: everything a GEMM CTA needs to place a row tile
  __host__ __device__ int off_tile_rec() const { return (8 + 2 * g + 1 + 2 * max_tiles + 7) & ~7; }
  __host__ __device__ int total_words() const { return off_tile_rec() + 8 * max_tiles; }
};

// One record per live row tile (any tile of a group carries the group's facts).
struct __align__(16) TileRecord {
  int32_t group;         // group id
  int32_t weight;        // weight matrix the group multiplies by (group_to_weight or identity)
  int32_t group_offset;  // first row of the group
  int32_t group_size;    // rows of the group (clamped to >= 0)
  int32_t tile_base;     // number of row tiles in all earlier groups
  int32_t tiles;         // row tiles of this group
  int32_t idx;           // this tile's index inside the group
  int32_t pad;
};

constexpr int kMetaThreads = 1024;

__device__ __forceinline__ int warp_inclusive_scan(int v, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= d) v += t;
  }
  return v;
}

// One CTA.  Each output pointer may be null (then that array is not written).
//   group_offsets[g]   exclusive prefix sum of group_sizes            (reference :86)
//   tile2group[U]      row tile i -> group id, 0 past the live tiles  (reference :81)
//   tile2idx[U]        row tile i -> tile index inside its group      (reference :82)
//   total_tiles[1]     number of live row tiles                       (reference :89)
//   tile_prefix[g+1]   exclusive prefix sum of tiles per group (extra)
//   row_total[1]       min(sum(group_sizes), m) (extra)
//   status[1]          device status word, reset to 0 here at the start of every call (extra)
//   tile_rec[U]        one TileRecord per live row tile; needs tile_prefix and group_offsets (extra)
//   visit_group[g], visit_prefix[g+1]  scratch; when given (with group_to_weight and tile_rec), the
//                      tile records are laid out in VISITING order = groups sorted by the weight
//                      they use (stable), so that groups sharing a weight matrix are multiplied
//                      one after the other and the matrix leaves HBM once.  Rows, offsets and
//                      results are unchanged; only the order in which tiles are taken differs.
__global__ void __launch_bounds__(kMetaThreads, 1)
group_metadata_kernel(const int32_t* __restrict__ group_sizes, int g, int m, int tile_m,
                      int max_tiles, int32_t* group_offsets,
                      int32_t* __restrict__ tile2group, int32_t* __restrict__ tile2idx,
                      int32_t* __restrict__ total_tiles, int32_t* tile_prefix,
                      int32_t* __restrict__ row_total, int32_t* __restrict__ status,
                      TileRecord* __restrict__ tile_rec,
                      const int32_t* __restrict__ group_to_weight,
                      int32_t* visit_group = nullptr, int32_t* visit_prefix = nullptr) {
  __shared__ int warp_rows[32];
  __shared__ int warp_tiles[32];
  __shared__ int carry_rows;
  __shared__ int carry_tiles;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  if (tid == 0) {
    carry_rows = 0;
    carry_tiles = 0;
    if (status) {
      status[0] = 0;
      // words 1..3: timing counters of the expert-parallel kernels (microseconds; see rd_ep_send.cuh)
      status[1] = 0;
      status[2] = 0;
      status[3] = 0;
    }
  }
  __syncthreads();

  // Pass 1: blocked exclusive scan of rows and of tiles, kMetaThreads groups at a time.
  // For the GEMM kernels (tile_rec given) a group only counts the rows that exist below m, so a
  // caller whose group_sizes add up to more than m still gets every tile of the rows that are
  // there; the reference-shaped arrays alone follow the reference's formula (no clamp).
  const bool clamp_to_m = tile_rec != nullptr;
  for (int base = 0; base < g; base += kMetaThreads) {
    const int i = base + tid;
    int rows = 0;
    if (i < g) {
      rows = group_sizes[i];
      rows = rows < 0 ? 0 : rows;
    }
    int inc_rows = warp_inclusive_scan(rows, lane);
    if (lane == 31) warp_rows[warp] = inc_rows;
    __syncthreads();
    if (warp == 0) {
      int wr = warp_rows[lane];
      int ir = warp_inclusive_scan(wr, lane);
      warp_rows[lane] = ir - wr;  // exclusive prefix over warps
    }
    __syncthreads();
    const int ex_rows = carry_rows + warp_rows[warp] + inc_rows - rows;
    int live_rows = rows;
    if (clamp_to_m) {
      const int left = m - ex_rows;
      live_rows = left <= 0 ? 0 : (rows < left ? rows : left);
    }
    const int tiles = (live_rows + tile_m - 1) / tile_m;
    int inc_tiles = warp_inclusive_scan(tiles, lane);
    if (lane == 31) warp_tiles[warp] = inc_tiles;
    __syncthreads();
    if (warp == 0) {
      int wt = warp_tiles[lane];
      int it = warp_inclusive_scan(wt, lane);
      warp_tiles[lane] = it - wt;
    }
    __syncthreads();
    const int ex_tiles = carry_tiles + warp_tiles[warp] + inc_tiles - tiles;
    if (i < g) {
      if (group_offsets) group_offsets[i] = ex_rows;
      if (tile_prefix) tile_prefix[i] = ex_tiles;
    }
    __syncthreads();
    if (tid == kMetaThreads - 1) {
      carry_rows = ex_rows + rows;
      carry_tiles = ex_tiles + tiles;
    }
    __syncthreads();
  }

  const int all_tiles = carry_tiles;
  const int live_tiles = all_tiles < max_tiles ? all_tiles : max_tiles;
  if (tid == 0) {
    if (tile_prefix) tile_prefix[g] = all_tiles;
    if (total_tiles) total_tiles[0] = all_tiles;
    if (row_total) row_total[0] = carry_rows < m ? carry_rows : m;
  }
  if (tile2group == nullptr && tile2idx == nullptr && tile_rec == nullptr) return;

  const bool by_weight = visit_group != nullptr && visit_prefix != nullptr && group_to_weight != nullptr &&
                         tile_rec != nullptr && tile_prefix != nullptr;
  if (by_weight) {
    __syncthreads();
    for (int gi = tid; gi < g; gi += kMetaThreads) {  // rank of the group: by weight, then by index
      const int w = group_to_weight[gi];
      int rank = 0;
      for (int j = 0; j < g; ++j) {
        const int wj = group_to_weight[j];
        rank += (wj < w || (wj == w && j < gi)) ? 1 : 0;
      }
      visit_group[rank] = gi;
    }
    __syncthreads();
    if (tid == 0) {
      int acc = 0;
      for (int v = 0; v < g; ++v) {
        const int gi = visit_group[v];
        visit_prefix[v] = acc;
        acc += tile_prefix[gi + 1] - tile_prefix[gi];
      }
      visit_prefix[g] = acc;
    }
  }

  // Pass 2: every row tile finds its group by binary search over the per-group tile prefix
  // (recomputed from group_sizes when the caller did not ask for tile_prefix).
  __syncthreads();
  for (int u = tid; u < max_tiles; u += kMetaThreads) {
    int gi = 0, idx = 0;
    int visit_base = -1;
    if (u < live_tiles && by_weight) {
      int lo = 0, hi = g;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (visit_prefix[mid + 1] > u) hi = mid; else lo = mid + 1;
      }
      gi = visit_group[lo];
      visit_base = visit_prefix[lo];
      idx = u - visit_base;
    } else if (u < live_tiles) {
      if (tile_prefix) {
        int lo = 0, hi = g;  // first index with tile_prefix[index] > u lies in (lo, hi]
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (tile_prefix[mid + 1] > u) hi = mid; else lo = mid + 1;
        }
        gi = lo;
        idx = u - tile_prefix[gi];
      } else {
        int acc = 0;
        for (int i = 0; i < g; ++i) {
          int rows = group_sizes[i];
          rows = rows < 0 ? 0 : rows;
          const int t = (rows + tile_m - 1) / tile_m;
          if (u < acc + t) {
            gi = i;
            idx = u - acc;
            break;
          }
          acc += t;
        }
      }
    }
    if (tile2group) tile2group[u] = gi;
    if (tile2idx) tile2idx[u] = idx;
    if (tile_rec && tile_prefix && group_offsets && u < live_tiles) {
      TileRecord r;
      int rows = group_sizes[gi];
      r.group = gi;
      r.weight = group_to_weight ? group_to_weight[gi] : gi;
      r.group_offset = group_offsets[gi];
      rows = rows < 0 ? 0 : rows;
      const int left = m - r.group_offset;
      r.group_size = left <= 0 ? 0 : (rows < left ? rows : left);
      r.tile_base = by_weight ? visit_base : tile_prefix[gi];
      r.tiles = tile_prefix[gi + 1] - tile_prefix[gi];
      r.idx = idx;
      r.pad = 0;
      tile_rec[u] = r;
    }
  }
}

}  // namespace rd
