// Row gather: dst[i, :] = src[index[i], :].  The permute step that sits in front of ragged_dot
// in an MoE layer (tokens replicated per routed expert and sorted by expert).  Pure HBM traffic:
// one warp per output row, 16-byte vectors, four loads in flight per lane.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace rd {

constexpr int kGatherThreads = 256;

__global__ void __launch_bounds__(kGatherThreads)
gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ index,
                   uint4* __restrict__ dst, int rows_out, int rows_in, int vecs_per_row) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = kGatherThreads / 32;
  const int warp_global = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int warp_stride = gridDim.x * warps_per_block;
  for (int r = warp_global; r < rows_out; r += warp_stride) {
    const int s = index[r];
    uint4* d = dst + static_cast<size_t>(r) * vecs_per_row;
    if (s < 0 || s >= rows_in) {  // an index outside the source gives a zero row
      for (int v = lane; v < vecs_per_row; v += 32) d[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const uint4* p = src + static_cast<size_t>(s) * vecs_per_row;
    int v = lane;
    for (; v + 96 < vecs_per_row; v += 128) {
      const uint4 a = p[v], b = p[v + 32], c = p[v + 64], e = p[v + 96];
      d[v] = a;
      d[v + 32] = b;
      d[v + 64] = c;
      d[v + 96] = e;
    }
    for (; v < vecs_per_row; v += 32) d[v] = p[v];
  }
}

}  // namespace rd
