// Hardware-limit probes for the pipelines in rd_gemm*.cuh: what one SM of the GPU can do with the
// very instructions those kernels are made of, with everything else taken away.  Standalone
// program (python -m gpu_ragged_dot_b200.probe builds and runs it); nothing in the library uses it.
//
//   mma   clocks per tcgen05.mma (M = 128 per CTA, N = 256, K = 16, bf16) issued back to back by one
//         thread on operands that sit in shared memory, for every operand layout, for one CTA and
//         for a CTA pair, alone and while another thread streams TMA boxes into the same SM
//   tma   bytes per clock one thread can bring into shared memory with tiled TMA loads, by box
//         shape, and when several CTAs ask for the same boxes at the same time
//   sync  issue cost of the synchronisation instructions of the MMA loop
//   pair  signalling round trips between the two CTAs of a cluster, and the latency of a stage
//         load whose bytes are counted on the other CTA's barrier
//
// Every wait is bounded by an iteration count; a probe that gives up prints err != 0.
#include <cstdint>
#include <cstdio>
#include <cstring>

#include <cuda.h>
#include <cuda_runtime.h>

#include "rd_ptx.cuh"

using namespace rd;

namespace {

constexpr int kSpinLimit = 4000000;
constexpr int kRows = 8192, kCols = 2048;  // the bf16 tensor every TMA probe reads (32 MB: stays in L2)

__device__ __forceinline__ bool spin_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encoder() {
  EncodeFn fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", reinterpret_cast<void**>(&fn), cudaEnableDefault, &q);
  return fn;
}

// rank 2: (cols, rows) with boxes of 64 columns x box_rows.  rank 3: the column-blocked view
// (64 columns, rows, blocks of 64 columns) with boxes of 64 x box_rows x box_blocks.
bool encode(CUtensorMap* map, void* base, int rank, int box_rows, int box_blocks) {
  EncodeFn fn = encoder();
  if (!fn) return false;
  cuuint32_t es[3] = {1, 1, 1};
  if (rank == 2) {
    cuuint64_t d[2] = {kCols, kRows};
    cuuint64_t st[1] = {kCols * 2};
    cuuint32_t b[2] = {64, static_cast<cuuint32_t>(box_rows)};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  cuuint64_t d[3] = {64, kRows, kCols / 64};
  cuuint64_t st[2] = {kCols * 2, 128};
  cuuint32_t b[3] = {64, static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(box_blocks)};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// ---------------------------------------------------------------- mma
// Thread 0 of the (leader) CTA issues n_mma MMAs: two accumulators of 256 columns, four K steps
// each per 64-deep "stage", a commit per stage, stages taken round robin from `stages` slots.
// With stream_on, thread 64 of every CTA streams 32 KB boxes into a ring behind the operands.
template <int kCtas>
__global__ void __launch_bounds__(128, 1)
mma_probe(int a_mn, int b_mn, int n_mma, int stages, int bcols, const __grid_constant__ CUtensorMap map,
          int stream_on, long long* out, int* err) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ __align__(8) uint64_t bar_stage[4];
  __shared__ __align__(8) uint64_t bar_ring[2];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int mma_done;
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = kCtas == 2 ? static_cast<int>(cluster_cta_rank()) : 0;
  uint32_t* words = reinterpret_cast<uint32_t*>(smem_dyn + (base - smem_u32(smem_dyn)));
  for (int i = threadIdx.x; i < 48 * 1024; i += 128) words[i] = 0x3c003c00u;
  if (threadIdx.x == 0) {
    mma_done = 0;
    mbar_init(smem_u32(&bar_done), 1);
    for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&bar_stage[i]), 1);
    for (int i = 0; i < 2; ++i) mbar_init(smem_u32(&bar_ring[i]), 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<kCtas>(smem_u32(&tmem_slot), 512);
    tmem_relinquish<kCtas>();
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  if (kCtas == 2) cluster_sync();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 0 && lane == 0 && rank == 0) {
    const uint32_t idesc = make_idesc_f16(1, a_mn, b_mn, 128 * kCtas, 256);
    const uint32_t stage_bytes = 32768 + bcols * 128;
    const uint32_t a_step = (a_mn ? 2048u : 32u) >> 4, b_step = (b_mn ? 2048u : 32u) >> 4;
    const uint64_t ad = a_mn ? make_smem_desc(base, 8192, 1024) : make_smem_desc(base, 16, 1024);
    const uint64_t bd = b_mn ? make_smem_desc(base + 32768, 8192, 1024) : make_smem_desc(base + 32768, 16, 1024);
    const uint32_t a0 = static_cast<uint32_t>(ad), b0 = static_cast<uint32_t>(bd);
    const uint32_t hi = static_cast<uint32_t>(ad >> 32);
    const long long t0 = clock64();
    int s = 0;
    for (int i = 0; i < n_mma; i += 8) {
      const uint32_t al = a0 + s * (stage_bytes >> 4), bl = b0 + s * (stage_bytes >> 4);
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_f16<kCtas>(tmem_base + h * 256, make_desc64(al + h * 1024 + kk * a_step, hi),
                          make_desc64(bl + kk * b_step, hi), idesc, 1u);
      if (kCtas == 2) {
        umma_commit_pair(smem_u32(&bar_stage[s]), 0x3);
      } else {
        umma_commit(smem_u32(&bar_stage[s]));
      }
      s = s + 1 == stages ? 0 : s + 1;
    }
    if (kCtas == 2) {
      umma_commit_pair(smem_u32(&bar_done), 0x1);
    } else {
      umma_commit(smem_u32(&bar_done));
    }
    const long long t1 = clock64();
    if (!spin_wait(smem_u32(&bar_done), 0)) *err = 1;
    const long long t2 = clock64();
    mma_done = 1;
    if (blockIdx.x == 0) {
      out[0] = t1 - t0;
      out[1] = t2 - t0;
    }
  }
  if (warp == 2 && lane == 0 && stream_on) {
    const uint32_t ring = base + 128 * 1024;
    int r = (blockIdx.x * 448) % kRows, cb = (blockIdx.x * 4) % 32;
    long long n = 0;
    auto issue = [&](int sl) {
      mbar_arrive_expect_tx(smem_u32(&bar_ring[sl]), 32768);
      tma_load_3d(ring + sl * 32768, &map, smem_u32(&bar_ring[sl]), 0, r, cb);
      cb += 4;
      if (cb + 4 > 32) {
        cb = 0;
        r += 64;
        if (r + 64 > kRows) r = 0;
      }
    };
    issue(0);
    issue(1);
    for (int it = 0; it < 40000; ++it) {
      const int sl = it & 1;
      if (!spin_wait(smem_u32(&bar_ring[sl]), (it >> 1) & 1u)) {
        *err = 2;
        break;
      }
      ++n;
      if (mma_done || (rank != 0 && it > 6000)) {  // let the box still in flight land, then stop
        (void)spin_wait(smem_u32(&bar_ring[(it + 1) & 1]), ((it + 1) >> 1) & 1u);
        break;
      }
      issue(sl);
    }
    if (blockIdx.x == 0) out[2] = n;
  }
  __syncthreads();
  if (kCtas == 2) cluster_sync();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<kCtas>(tmem_base, 512);
  }
}

template <int kCtas>
void run_mma(int a_mn, int b_mn, const CUtensorMap& map, int stream_on, long long* out, int* err, int sms) {
  const int n_mma = 8 * 2000, stages = 2, bcols = 256 / kCtas;
  const int smem = 200 * 1024;
  auto k = mma_probe<kCtas>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaLaunchConfig_t lc = {};
  lc.blockDim = dim3(128);
  lc.dynamicSmemBytes = smem;
  lc.gridDim = dim3(kCtas == 2 ? (sms / 2) * 2 : sms);
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = kCtas;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  for (int rep = 0; rep < 2; ++rep) cudaLaunchKernelEx(&lc, k, a_mn, b_mn, n_mma, stages, bcols, map, stream_on, out, err);
  cudaDeviceSynchronize();
  long long h[3];
  int e;
  cudaMemcpy(h, out, 24, cudaMemcpyDeviceToHost);
  cudaMemcpy(&e, err, 4, cudaMemcpyDeviceToHost);
  printf("mma  cta_group %d  A %s  B %s  TMA ingest beside it %5.1f B/clk: issue %.1f clk/MMA, complete %.1f clk/MMA "
         "(M=%d N=256 K=16)  err %d %s\n",
         kCtas, a_mn ? "MN-major" : "K-major ", b_mn ? "MN-major" : "K-major ",
         stream_on ? double(h[2]) * 32768 / double(h[1]) : 0.0, double(h[0]) / n_mma, double(h[1]) / n_mma,
         128 * kCtas, e, cudaGetErrorString(cudaGetLastError()));
}

// ---------------------------------------------------------------- tma
// Thread 0 of every CTA keeps `slots` steps in flight; a step is per_iter boxes counted on one
// barrier.  CTAs in groups of `share` ask for the same boxes at the same time.
__global__ void __launch_bounds__(128, 1)
tma_probe(const __grid_constant__ CUtensorMap map, int rank, int box_bytes, int slots, int row_step, int cb_step,
          int iters, int per_iter, int share, long long* out, int* err) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar[8];
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&bar[i]), 1);
    fence_mbar_init();
    tma_prefetch_desc(&map);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const int cblocks = kCols / 64;
    const int grp = blockIdx.x / share;
    int r = (grp * 448) % kRows, cb = (grp * 3 * cb_step) % cblocks;
    if (cb + cb_step > cblocks) cb = 0;
    const long long t0 = clock64();
    for (int it = 0; it < iters + slots; ++it) {
      const int s = it % slots;
      if (it >= slots && !spin_wait(smem_u32(&bar[s]), ((it / slots) - 1) & 1u)) {
        *err = 1;
        return;
      }
      if (it < iters) {
        mbar_arrive_expect_tx(smem_u32(&bar[s]), box_bytes * per_iter);
        for (int j = 0; j < per_iter; ++j) {
          const uint32_t dst = base + s * 65536 + j * box_bytes;
          if (rank == 2) {
            tma_load_2d(dst, &map, smem_u32(&bar[s]), cb * 64, r);
          } else {
            tma_load_3d(dst, &map, smem_u32(&bar[s]), 0, r, cb);
          }
          cb += cb_step;
          if (cb + cb_step > cblocks) {
            cb = 0;
            r += row_step;
            if (r + row_step > kRows) r = 0;
          }
        }
      }
    }
    if (blockIdx.x == 0) out[0] = clock64() - t0;
  }
}

void run_tma(void* buf, long long* out, int* err, int sms) {
  struct Case {
    const char* name;
    int rank, rows, blocks, per_iter;
  };
  const Case cases[] = {
      {"2 KB boxes (64 cols x 16 rows), 8 per step", 2, 16, 1, 8},
      {"4 KB boxes (64 cols x 32 rows), 8 per step", 2, 32, 1, 8},
      {"8 KB boxes (64 cols x 64 rows), 8 per step", 2, 64, 1, 8},
      {"16 KB boxes (64 cols x 128 rows), 4 per step", 2, 128, 1, 4},
      {"32 KB boxes (64 cols x 256 rows), 2 per step", 2, 256, 1, 2},
      {"32 KB boxes (64 cols x 64 rows x 4 blocks), 2 per step", 3, 64, 4, 2},
      {"32 KB boxes (64 cols x 64 rows x 4 blocks), 1 per step", 3, 64, 4, 1},
  };
  cudaFuncSetAttribute(tma_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  for (const Case& c : cases) {
    CUtensorMap map;
    if (!encode(&map, buf, c.rank, c.rows, c.blocks)) {
      printf("tma  %s: tensor map could not be encoded\n", c.name);
      continue;
    }
    const int box_bytes = c.rows * 128 * c.blocks;
    for (int share : {1, 16}) {
      const int slots = 3;
      const int iters = (64 << 20) / (box_bytes * c.per_iter);
      for (int rep = 0; rep < 2; ++rep) {
        cudaEventRecord(e0);
        tma_probe<<<sms, 128, 200 * 1024>>>(map, c.rank, box_bytes, slots, c.rows, c.blocks, iters, c.per_iter, share,
                                            out, err);
        cudaEventRecord(e1);
        cudaDeviceSynchronize();
      }
      float ms;
      cudaEventElapsedTime(&ms, e0, e1);
      long long clk;
      int e;
      cudaMemcpy(&clk, out, 8, cudaMemcpyDeviceToHost);
      cudaMemcpy(&e, err, 4, cudaMemcpyDeviceToHost);
      const double bytes = double(iters) * box_bytes * c.per_iter;
      printf("tma  %-56s 3 steps in flight, %2d CTAs per address: %5.1f B/clk, %5.1f GB/s per SM, %5.2f TB/s all SMs "
             "(%.0f ns per step)  err %d %s\n",
             c.name, share, bytes / clk, bytes / ms / 1e6, sms * bytes / ms / 1e9, ms * 1e6 / iters, e,
             cudaGetErrorString(cudaGetLastError()));
    }
  }
}

// ---------------------------------------------------------------- sync
__global__ void __launch_bounds__(128, 1) sync_probe(long long* out) {
  __shared__ __align__(8) uint64_t bar[4];
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&bar[i]), 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(&tmem_slot), 64);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) {
    const int n = 2000;
    long long t0 = clock64();
    for (int i = 0; i < n; ++i) tc_fence_after_sync();
    if (lane == 0) out[0] = clock64() - t0;
    t0 = clock64();
    if (lane == 0)
      for (int i = 0; i < n; ++i) umma_commit(smem_u32(&bar[0]));
    if (lane == 0) out[1] = clock64() - t0;
    __syncwarp();
    t0 = clock64();
    if (lane == 0) {
      uint32_t ph = 0;
      for (int i = 0; i < n; ++i) {
        umma_commit(smem_u32(&bar[1]));
        (void)spin_wait(smem_u32(&bar[1]), ph);
        ph ^= 1u;
      }
      out[2] = clock64() - t0;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&bar[2]));
    __syncwarp();
    t0 = clock64();
    int acc = 0;
    for (int i = 0; i < n; ++i) acc += mbar_try_wait(smem_u32(&bar[2]), 0) ? 1 : 0;
    if (lane == 0) out[3] = clock64() - t0 + (acc == -1);
    t0 = clock64();
    for (int i = 0; i < n; ++i) __syncwarp();
    if (lane == 0) out[4] = clock64() - t0;
    t0 = clock64();
    if (lane == 0) {
      uint32_t ph = 0;
      for (int i = 0; i < n; ++i) {
        mbar_arrive(smem_u32(&bar[3]));
        (void)spin_wait(smem_u32(&bar[3]), ph);
        ph ^= 1u;
      }
      out[5] = clock64() - t0;
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_slot, 64);
  }
}

void run_sync(long long* out) {
  for (int rep = 0; rep < 2; ++rep) {
    sync_probe<<<1, 128>>>(out);
    cudaDeviceSynchronize();
  }
  long long h[6];
  cudaMemcpy(h, out, 48, cudaMemcpyDeviceToHost);
  const char* names[6] = {"tcgen05.fence::after_thread_sync (whole warp)",
                          "tcgen05.commit, nothing pending, issue only",
                          "tcgen05.commit + wait for its arrival",
                          "mbarrier.try_wait on a completed phase (whole warp)",
                          "__syncwarp after a divergent section",
                          "mbarrier.arrive + try_wait on the same barrier"};
  for (int i = 0; i < 6; ++i) printf("sync %-52s %6.1f clk each\n", names[i], h[i] / 2000.0);
}

// ---------------------------------------------------------------- pair
// mode 0: leader -> peer by remote mbarrier.arrive, peer answers the same way.
// mode 1: leader -> peer by tcgen05.commit (multicast form, peer only).
// mode 2: tcgen05.commit to both; the leader also times its own copy.
__global__ void __launch_bounds__(128, 1) pair_signal_probe(long long* out, int* err) {
  __shared__ __align__(8) uint64_t bar_a, bar_b;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_cta_rank());
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_a), 1);
    mbar_init(smem_u32(&bar_b), 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<2>(smem_u32(&tmem_slot), 64);
    tmem_relinquish<2>();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync();
  tc_fence_after_sync();
  const int n = 1000;
  for (int mode = 0; mode < 3; ++mode) {
    if (warp == 0 && lane == 0) {
      uint32_t ph = 0;
      if (rank == 0) {
        const long long t0 = clock64();
        long long own = 0;
        for (int i = 0; i < n; ++i) {
          if (mode == 0) {
            mbar_arrive_cluster(smem_u32(&bar_a), 1);
          } else if (mode == 1) {
            umma_commit_pair(smem_u32(&bar_a), 0x2);
          } else {
            const long long q = clock64();
            umma_commit_pair(smem_u32(&bar_a), 0x3);
            (void)spin_wait(smem_u32(&bar_a), ph);
            own += clock64() - q;
          }
          if (!spin_wait(smem_u32(&bar_b), ph)) {
            *err = 1;
            break;
          }
          ph ^= 1u;
        }
        out[mode] = clock64() - t0;
        if (mode == 2) out[3] = own;
      } else {
        for (int i = 0; i < n; ++i) {
          if (!spin_wait(smem_u32(&bar_a), ph)) {
            *err = 2;
            break;
          }
          mbar_arrive_cluster(smem_u32(&bar_b), 0);
          ph ^= 1u;
        }
      }
    }
    __syncthreads();
    cluster_sync();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<2>(tmem_slot, 64);
  }
}

// A stage load of 48 KB per CTA (32 KB + 16 KB boxes), `inflight` stages at a time.  mode 0: own
// barrier.  mode 1: the peer's bytes are counted on the leader's barrier (.cta_group::2 form); the
// leader waits for both and frees the peer's slot with a remote arrive.
__global__ void __launch_bounds__(128, 1)
pair_load_probe(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, int mode,
                int inflight, int iters, long long* out, int* err) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t full[4];
  __shared__ __align__(8) uint64_t go[4];
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int rank = static_cast<int>(cluster_cta_rank());
  if (threadIdx.x == 0) {
    for (int i = 0; i < 4; ++i) {
      mbar_init(smem_u32(&full[i]), 1);
      mbar_init(smem_u32(&go[i]), 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  cluster_sync();
  if (threadIdx.x == 0) {
    int r = ((blockIdx.x >> 1) * 448) % kRows;
    const int cb = ((blockIdx.x >> 1) * 8 + rank * 4) % 32;
    const long long t0 = clock64();
    for (int it = 0; it < iters + inflight; ++it) {
      const int s = it % inflight;
      if (it >= inflight) {
        const uint32_t php = ((it / inflight) - 1) & 1u;
        if (mode == 0 || rank == 0) {
          if (!spin_wait(smem_u32(&full[s]), php)) {
            *err = 1;
            break;
          }
          if (mode == 1) mbar_arrive_cluster(smem_u32(&go[s]), 1);
        } else if (!spin_wait(smem_u32(&go[s]), php)) {
          *err = 2;
          break;
        }
      }
      if (it < iters) {
        const uint32_t dst = base + s * 49152;
        if (mode == 0 || rank == 0) {
          mbar_arrive_expect_tx(smem_u32(&full[s]), mode == 0 ? 49152 : 2 * 49152);
          tma_load_3d(dst, &map_a, smem_u32(&full[s]), 0, r, cb);
          tma_load_3d(dst + 32768, &map_b, smem_u32(&full[s]), 0, r, (cb + 8) % 32);
        } else {
          const uint32_t remote = map_to_cta(smem_u32(&full[s]), 0);
          tma_load_3d_pair(dst, &map_a, remote, 0, r, cb);
          tma_load_3d_pair(dst + 32768, &map_b, remote, 0, r, (cb + 8) % 32);
        }
        r += 64;
        if (r + 64 > kRows) r = 0;
      }
    }
    if (blockIdx.x == 0) out[0] = clock64() - t0;
  }
  __syncthreads();
  cluster_sync();
}

void run_pair(void* buf, long long* out, int* err, int sms) {
  cudaLaunchConfig_t lc = {};
  lc.blockDim = dim3(128);
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  lc.gridDim = dim3(2);
  for (int rep = 0; rep < 2; ++rep) {
    cudaLaunchKernelEx(&lc, pair_signal_probe, out, err);
    cudaDeviceSynchronize();
  }
  long long h[4];
  int e;
  cudaMemcpy(h, out, 32, cudaMemcpyDeviceToHost);
  cudaMemcpy(&e, err, 4, cudaMemcpyDeviceToHost);
  printf("pair remote arrive -> peer sees it -> remote arrive back -> leader sees it: %.0f clk\n", h[0] / 1000.0);
  printf("pair tcgen05.commit to the peer -> peer sees it -> remote arrive back:       %.0f clk\n", h[1] / 1000.0);
  printf("pair tcgen05.commit to both: own copy seen after %.0f clk, peer's answer after %.0f clk  err %d\n",
         h[3] / 1000.0, h[2] / 1000.0, e);
  CUtensorMap ma, mb;
  if (!encode(&ma, buf, 3, 64, 4) || !encode(&mb, buf, 3, 64, 2)) {
    printf("pair tensor maps could not be encoded\n");
    return;
  }
  cudaFuncSetAttribute(pair_load_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  lc.dynamicSmemBytes = 200 * 1024;
  lc.gridDim = dim3((sms / 2) * 2);
  for (int mode = 0; mode < 2; ++mode)
    for (int inflight : {1, 2, 4}) {
      const int iters = 4000;
      for (int rep = 0; rep < 2; ++rep) {
        cudaLaunchKernelEx(&lc, pair_load_probe, ma, mb, mode, inflight, iters, out, err);
        cudaDeviceSynchronize();
      }
      long long clk;
      cudaMemcpy(&clk, out, 8, cudaMemcpyDeviceToHost);
      cudaMemcpy(&e, err, 4, cudaMemcpyDeviceToHost);
      printf("pair 48 KB stage load, %s, %d in flight: %.0f clk per stage per CTA (%.1f B/clk)  err %d %s\n",
             mode ? "peer's bytes on the leader's barrier" : "every CTA on its own barrier       ", inflight,
             double(clk) / iters, 49152.0 * iters / clk, e, cudaGetErrorString(cudaGetLastError()));
    }
}

}  // namespace

int main(int argc, char** argv) {
  const char* which = argc > 1 ? argv[1] : "all";
  auto want = [&](const char* name) { return !strcmp(which, "all") || !strcmp(which, name); };
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  void* buf = nullptr;
  const size_t bytes = size_t(kRows) * kCols * 2;
  long long* out = nullptr;
  int* err = nullptr;
  if (cudaMalloc(&buf, bytes) != cudaSuccess || cudaMalloc(&out, 64) != cudaSuccess ||
      cudaMalloc(&err, 4) != cudaSuccess) {
    printf("no device memory\n");
    return 1;
  }
  cudaMemset(buf, 1, bytes);
  cudaMemset(out, 0, 64);
  cudaMemset(err, 0, 4);
  if (want("mma")) {
    CUtensorMap map;
    if (!encode(&map, buf, 3, 64, 4)) {
      printf("mma  tensor map could not be encoded\n");
    } else {
      for (int stream_on = 0; stream_on < 2; ++stream_on)
        for (int a = 0; a < 2; ++a)
          for (int b = 0; b < 2; ++b) {
            run_mma<1>(a, b, map, stream_on, out, err, sms);
            run_mma<2>(a, b, map, stream_on, out, err, sms);
          }
    }
  }
  if (want("tma")) run_tma(buf, out, err, sms);
  if (want("sync")) run_sync(out);
  if (want("pair")) run_pair(buf, out, err, sms);
  cudaDeviceSynchronize();
  printf("%s\n", cudaGetErrorString(cudaGetLastError()));
  return 0;
}
