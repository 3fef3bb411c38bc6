// Expert-parallel dispatch without a host round trip: token rows go straight from the local
// token matrix into the receive buffers of the ranks that own their experts, through peer
// (NVLink) stores.  It replaces "sort by expert + gather + all-to-all with host-known split
// sizes" by three small stream-ordered kernels around one exchange of the per-expert counts:
//
//   ep_count_kernel     counts[e] = number of (token, slot) pairs routed to expert e
//   (all ranks exchange counts -> counts_all[W][E]; a tiny all-gather, done by the caller)
//   ep_plan_kernel      from counts_all: where this rank's rows for expert e start inside the
//                       owner's receive buffer, and the sizes of the W * El segments this rank
//                       will receive (they are the group_sizes of the local rd_gmm_indexed)
//   ep_dispatch_kernel  one warp per (token, slot): copies the row into
//                       peer_base[owner] + position * row_bytes with 16-byte stores
//
// Receive-buffer layout on every rank: segments ordered (source rank, local expert); segment
// (s, e) holds the rows source s routed to local expert e.  Rows inside a segment land in
// arrival order (an atomic counter per expert); dest_pos records where each (token, slot) went
// so results can be brought back.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rd_ptx.cuh"

namespace rd {

constexpr int kEpThreads = 256;

__global__ void __launch_bounds__(kEpThreads)
ep_count_kernel(const int32_t* __restrict__ routing, int entries, int num_experts,
                int32_t* __restrict__ counts) {
  extern __shared__ int32_t hist[];
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < entries; i += gridDim.x * blockDim.x) {
    const int e = routing[i];
    if (e >= 0 && e < num_experts) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x)
    if (hist[e]) atomicAdd(&counts[e], hist[e]);
}

// ep_count_kernel + the exchange of the counts, without a collective library: the last block to
// finish stores this rank's E counts into row `rank` of every rank's counts_all (peer stores; its
// own included), fences at system scope and stores `epoch` into word `rank` of every rank's count
// flags.  `counts` (E words) and `ticket` (1 word) are scratch that must be zero on entry and is
// left zero again.  The consumer is ep_plan_kernel with count_flags set, on every rank.
__global__ void __launch_bounds__(kEpThreads)
ep_count_share_kernel(const int32_t* __restrict__ routing, int entries, int num_experts, int32_t* counts,
                      int32_t* ticket, int world, int rank, const uint64_t* __restrict__ peer_counts,
                      const uint64_t* __restrict__ peer_flags, int epoch) {
  extern __shared__ int32_t hist[];
  __shared__ int last;
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < entries; i += gridDim.x * blockDim.x) {
    const int e = routing[i];
    if (e >= 0 && e < num_experts) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x)
    if (hist[e]) atomicAdd(&counts[e], hist[e]);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(ticket, 1) == static_cast<int>(gridDim.x) - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    const int c = atomicExch(&counts[e], 0);  // read the total and leave the scratch zero
    for (int r = 0; r < world; ++r)
      reinterpret_cast<int32_t*>(peer_counts[r])[rank * num_experts + e] = c;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) *ticket = 0;
  if (threadIdx.x < world) {
    int32_t* flag = reinterpret_cast<int32_t*>(peer_flags[threadIdx.x]) + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
  }
}

// One CTA.  counts_all[s * E + e]: rows source s routes to global expert e.
//   dest_offset[e]        first row, inside the receive buffer of e's owner, of MY rows for e
//   segment_sizes[s*El+j] rows I receive from source s for my local expert j
//   fill[e]               reset to 0 (arrival counters used by the dispatch kernel)
//   totals[0]             rows I receive in all
//
// ring != 0 selects the layout of the fused exchange (rd_gmm_ep_fused): on rank d the segments are ordered by
// "position" q = (d - source) mod W, i.e. d's own rows first, then those of d-1, d-2, ...; a
// source sends to d in phase q of its dispatch, so positions fill in the order the local GEMM
// reads them.  phase_done[W] (may be null) are the per-phase block counters, reset here.
__global__ void __launch_bounds__(kEpThreads)
ep_plan_kernel(const int32_t* __restrict__ counts_all, int world, int num_experts, int rank,
               int32_t* __restrict__ dest_offset, int32_t* __restrict__ segment_sizes,
               int32_t* __restrict__ fill, int32_t* __restrict__ totals, int ring,
               int32_t* __restrict__ phase_done, int32_t* __restrict__ send_start,
               int32_t* __restrict__ list_fill, const int32_t* count_flags, int epoch,
               uint32_t wait_limit_us, int32_t* status) {
  // With count_flags (ep_count_share_kernel's exchange): row s of counts_all is complete once
  // count_flags[s] >= epoch.  The waits are bounded like every wait in these kernels; on expiry
  // the status word is set and the plan is made from whatever is there.
  if (count_flags != nullptr) {
    __shared__ WaitCtl ctl;
    if (threadIdx.x == 0) {
      ctl.abort = 0;
      ctl.limit_us = wait_limit_us;
    }
    __syncthreads();
    if (threadIdx.x < world && !wait_flag_ge(count_flags + threadIdx.x, epoch, &ctl) && status != nullptr)
      atomicMax(status, 1);
    __syncthreads();
  }
  const int local = num_experts / world;
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    const int owner = e / local;
    const int first = owner * local;
    int off = 0;
    // Segments in front of mine in the owner's buffer: sources 0..rank-1, or (ring) the
    // sources at positions 0..my position-1, which are owner, owner-1, ...
    const int before = ring ? (owner - rank + world) % world : rank;
    for (int q = 0; q < before; ++q) {
      const int s = ring ? (owner - q + world) % world : q;
      for (int j = 0; j < local; ++j) off += counts_all[s * num_experts + first + j];
    }
    for (int j = first; j < e; ++j) off += counts_all[rank * num_experts + j];
    dest_offset[e] = off;
    fill[e] = 0;
  }
  for (int i = threadIdx.x; i < world * local; i += blockDim.x) {
    const int q = i / local, j = i - q * local;
    const int s = ring ? (rank - q + world) % world : q;
    segment_sizes[i] = counts_all[s * num_experts + rank * local + j];
  }
  if (phase_done != nullptr)
    for (int i = threadIdx.x; i < world; i += blockDim.x) phase_done[i] = 0;
  // Send lists (fused exchange): list positions [send_start[p], send_start[p+1]) hold the entries
  // this rank sends in phase p, i.e. to rank + p; list_fill[p] counts them as they are assigned.
  if (list_fill != nullptr)
    for (int i = threadIdx.x; i < world; i += blockDim.x) list_fill[i] = 0;
  if (send_start != nullptr && threadIdx.x == 0) {
    int acc = 0;
    for (int p = 0; p < world; ++p) {
      send_start[p] = acc;
      const int dest = (rank + p) % world;
      for (int j = 0; j < local; ++j) acc += counts_all[rank * num_experts + dest * local + j];
    }
    send_start[world] = acc;
  }
  if (threadIdx.x == 0) {
    int total = 0;
    for (int s = 0; s < world; ++s)
      for (int j = 0; j < local; ++j) total += counts_all[s * num_experts + rank * local + j];
    totals[0] = total;
  }
}

// peer_base[r]: address of rank r's receive buffer as seen from this GPU (its own buffer for
// r == rank).  capacity_rows: rows each receive buffer can hold; a position beyond it is
// dropped and reported as -1 in dest_pos.
__global__ void __launch_bounds__(kEpThreads)
ep_dispatch_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ routing, int tokens,
                   int top_k, int vecs_per_row, int num_experts, int experts_per_rank,
                   const int32_t* __restrict__ dest_offset, int32_t* __restrict__ fill,
                   const uint64_t* __restrict__ peer_base, int capacity_rows,
                   int32_t* __restrict__ dest_pos) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = kEpThreads / 32;
  const int warp_global = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int warp_stride = gridDim.x * warps_per_block;
  const int entries = tokens * top_k;
  for (int i = warp_global; i < entries; i += warp_stride) {
    const int e = routing[i];
    int pos = -1;
    if (e >= 0 && e < num_experts) {
      if (lane == 0) pos = dest_offset[e] + atomicAdd(&fill[e], 1);
      pos = __shfl_sync(0xffffffffu, pos, 0);
      if (pos >= capacity_rows) pos = -1;
    }
    if (lane == 0) dest_pos[i] = pos;
    if (pos < 0) continue;
    const int owner = e / experts_per_rank;
    const uint4* src = x + static_cast<size_t>(i / top_k) * vecs_per_row;
    uint4* dst = reinterpret_cast<uint4*>(peer_base[owner]) + static_cast<size_t>(pos) * vecs_per_row;
    int v = lane;
    for (; v + 96 < vecs_per_row; v += 128) {
      const uint4 a = src[v], b = src[v + 32], c = src[v + 64], d = src[v + 96];
      dst[v] = a;
      dst[v + 32] = b;
      dst[v + 64] = c;
      dst[v + 96] = d;
    }
    for (; v < vecs_per_row; v += 32) dst[v] = src[v];
  }
  __threadfence_system();  // rows must be visible to their owners before the ranks synchronise
}

// Fused exchange, step 1: one thread per (token, slot) entry, one pass per block.  Assigns the
// row its position at the expert's owner (dest_pos, as ep_dispatch_kernel does) and appends the
// entry to the send list of its phase p = (owner - rank) mod W.  Both counters are aggregated
// in shared memory first, so a block issues one global atomic per expert / phase it touches.
// Dynamic shared memory: 2 * (num_experts + world) ints.
__global__ void __launch_bounds__(kEpThreads)
ep_assign_kernel(const int32_t* __restrict__ routing, int entries, int num_experts,
                 int experts_per_rank, int world, int rank, const int32_t* __restrict__ dest_offset,
                 int32_t* __restrict__ fill, int capacity_rows, int32_t* __restrict__ dest_pos,
                 const int32_t* __restrict__ send_start, int32_t* __restrict__ list_fill,
                 int32_t* __restrict__ send_index) {
  extern __shared__ int32_t sm[];
  int32_t* cnt_e = sm;                       // [E]  entries of this block per expert
  int32_t* cnt_p = sm + num_experts;         // [W]  ... per phase
  int32_t* base_e = cnt_p + world;           // [E]  first slot of this block at the expert
  int32_t* base_p = base_e + num_experts;    // [W]  first list slot of this block in the phase
  for (int j = threadIdx.x; j < num_experts + world; j += blockDim.x) sm[j] = 0;
  __syncthreads();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  int e = -1, phase = -1, my_e = 0, my_p = 0;
  if (i < entries) {
    e = routing[i];
    if (e >= 0 && e < num_experts) {
      phase = (e / experts_per_rank - rank + world) % world;
      my_e = atomicAdd(&cnt_e[e], 1);
      my_p = atomicAdd(&cnt_p[phase], 1);
    } else {
      e = -1;
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < num_experts; j += blockDim.x)
    if (cnt_e[j] > 0) base_e[j] = atomicAdd(&fill[j], cnt_e[j]);
  for (int j = threadIdx.x; j < world; j += blockDim.x)
    if (cnt_p[j] > 0) base_p[j] = atomicAdd(&list_fill[j], cnt_p[j]);
  __syncthreads();
  if (i < entries) {
    if (e >= 0) {
      int pos = dest_offset[e] + base_e[e] + my_e;
      if (pos >= capacity_rows) pos = -1;
      dest_pos[i] = pos;
      send_index[send_start[phase] + base_p[phase] + my_p] = i;
    } else {
      dest_pos[i] = -1;
    }
  }
}

// Copies the rows of one phase's send list (one warp per row) into dest_base and raises the
// destination's flag when the last block is done.  Used for phase 0 (a rank's own rows, a local
// copy that runs before the fused kernel).
__global__ void __launch_bounds__(kEpThreads)
ep_send_list_kernel(const uint4* __restrict__ x, int top_k, int vecs_per_row,
                    const int32_t* __restrict__ send_index, const int32_t* __restrict__ send_start,
                    int phase, const int32_t* __restrict__ dest_pos, uint4* __restrict__ dest_base,
                    int capacity_rows, int32_t* __restrict__ phase_done, int32_t* ready_flag,
                    int epoch) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = kEpThreads / 32;
  const int warp_global = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int warp_stride = gridDim.x * warps_per_block;
  const int lo = send_start[phase], hi = send_start[phase + 1];
  for (int j = lo + warp_global; j < hi; j += warp_stride) {
    const int i = send_index[j];
    const int pos = dest_pos[i];
    if (pos < 0 || pos >= capacity_rows) continue;
    const uint4* src = x + static_cast<size_t>(i / top_k) * vecs_per_row;
    uint4* dst = dest_base + static_cast<size_t>(pos) * vecs_per_row;
    int v = lane;
    for (; v + 96 < vecs_per_row; v += 128) {
      const uint4 a = src[v], b = src[v + 32], c = src[v + 64], d = src[v + 96];
      dst[v] = a;
      dst[v + 32] = b;
      dst[v + 64] = c;
      dst[v + 96] = d;
    }
    for (; v < vecs_per_row; v += 32) dst[v] = src[v];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(phase_done + phase, 1) + 1;
    if (done == static_cast<int>(gridDim.x)) {
      __threadfence_system();
      *reinterpret_cast<volatile int32_t*>(ready_flag) = epoch;
      __threadfence_system();
    }
  }
}

// Reverse exchange of the expert-parallel backward pass, fused with the top-k combine: the
// gradient of token t is the sum, over its top_k routed copies, of the gradient rows the owners
// computed at the positions the forward dispatch recorded (dest_pos).  One warp per token pulls
// the top_k rows from the owners' buffers (peer loads over NVLink, or local memory), adds them in
// fp32 and writes one 16-bit row.  peer_base[r]: rank r's gradient buffer as seen from this GPU.
// The caller orders this kernel after every owner's dlhs GEMM (a cross-rank barrier).
template <bool kBf16>
__device__ __forceinline__ void add8(float (&acc)[8], const uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (kBf16) {
      acc[2 * i] += __uint_as_float(w[i] << 16);
      acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      const float2 f = __half22float2(h);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
}

template <bool kBf16, int kTopK>
__global__ void __launch_bounds__(kEpThreads)
ep_combine_pull_kernel(const int32_t* __restrict__ routing, const int32_t* __restrict__ dest_pos, int tokens,
                       int top_k, int vecs_per_row, int num_experts, int experts_per_rank,
                       const uint64_t* __restrict__ peer_base, int capacity_rows, uint4* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = kEpThreads / 32;
  const int warp_global = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int warp_stride = gridDim.x * warps_per_block;
  for (int t = warp_global; t < tokens; t += warp_stride) {
    const uint4* src[kTopK];
#pragma unroll
    for (int s = 0; s < kTopK; ++s) {
      src[s] = nullptr;
      if (s < top_k) {
        const int e = routing[t * top_k + s];
        const int pos = dest_pos[t * top_k + s];
        if (e >= 0 && e < num_experts && pos >= 0 && pos < capacity_rows)
          src[s] = reinterpret_cast<const uint4*>(peer_base[e / experts_per_rank]) +
                   static_cast<size_t>(pos) * vecs_per_row;
      }
    }
    uint4* dst = out + static_cast<size_t>(t) * vecs_per_row;
    for (int v = lane; v < vecs_per_row; v += 64) {
      const bool second = v + 32 < vecs_per_row;
      uint4 a[kTopK], b[kTopK];
#pragma unroll
      for (int s = 0; s < kTopK; ++s) {  // all loads first: 2 * top_k 16-byte loads in flight per lane
        a[s] = b[s] = make_uint4(0u, 0u, 0u, 0u);
        if (src[s] != nullptr) {
          a[s] = src[s][v];
          if (second) b[s] = src[s][v + 32];
        }
      }
      float fa[8] = {0, 0, 0, 0, 0, 0, 0, 0}, fb[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int s = 0; s < kTopK; ++s) {
        add8<kBf16>(fa, a[s]);
        add8<kBf16>(fb, b[s]);
      }
      auto pack = [](const float (&f)[8]) {
        uint4 o;
        uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (kBf16) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
          } else {
            __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        return o;
      };
      dst[v] = pack(fa);
      if (second) dst[v + 32] = pack(fb);
    }
  }
}

}  // namespace rd
