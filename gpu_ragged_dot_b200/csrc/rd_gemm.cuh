// Grouped ("ragged") GEMM kernels for sm_100a.
//
//   gmm  : y[rows of group i, :] = x[rows of group i, :] @ W[i]        (reference
//          gpu_ragged_dot.py:93-165; W[i] is [k,n], or [n,k] with trans_rhs)
//   tgmm : out[i] = x[rows of group i, :]^T @ dout[rows of group i, :]   (reference :231-281)
//
// One persistent, warp-specialised CTA per SM:
//   warp 0      TMA producer   -- cp.async.bulk.tensor tiles into a kStages-deep smem ring
//   warp 1      MMA issuer     -- tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM accumulators
//   warps 2..5  epilogue       -- tcgen05.ld, fp32 -> bf16/fp16, row/column-masked 16-byte stores
// The two TMEM accumulators let the epilogue of tile t overlap the main loop of tile t+1.
//
// Operand layouts (all 128-byte-swizzled, written by TMA, read through UMMA descriptors):
//   K-major  operand tile [rows][64 k]  : one box, 8-row groups 1024 B apart
//   MN-major operand tile [64 k][64 mn] : boxes of 8 KB; K-groups of 8 rows 1024 B apart,
//                                         next 64 M/N elements in the next box (8192 B)
//
// Every mbarrier wait is bounded (rd_ptx.cuh: mbar_wait); on expiry the CTA records a status
// word, drains and frees its TMEM instead of spinning.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "rd_ptx.cuh"

namespace rd {

constexpr int kTileM = 128;  // UMMA M per CTA == output rows per tile
constexpr int kTileK = 64;   // elements per 128-byte swizzle row == contraction depth per stage
constexpr int kUmmaK = 16;   // contraction depth of one tcgen05.mma for 16-bit inputs
constexpr int kBoxBytes = 64 * 128;  // one [64 rows][128 B] TMA box
constexpr int kGemmThreads = 192;

enum DeviceStatus : int32_t {
  kStatusOk = 0,
  kStatusWaitExpired = 1,  // a bounded mbarrier wait gave up
};

struct GemmArgs {
  int m, k, n, g;   // gmm: x[m,k] . W[g] -> y[m,n]      tgmm: x[m,k], dout[m,n] -> out[g,k,n]
  int n_tiles;      // ceil(n / BN)
  int k_tiles;      // tgmm: ceil(k / 128) tiles of the output's k axis; gmm: unused
  int max_m_tiles;  // static upper bound on live row tiles (gmm)
  int ab_format;    // 0 = fp16, 1 = bf16
  const int32_t* group_sizes;
  const int32_t* group_offsets;
  const int32_t* tile2group;
  const int32_t* tile2idx;
  const int32_t* tile_prefix;
  const int32_t* totals;  // {live row tiles, min(sum(group_sizes), m)}
  const int32_t* group_to_weight;  // gmm: weight matrix used by each group, or null (identity)
  int32_t* status;
  void* out;
};

struct TileCoord {
  int group;   // group index
  int weight;  // gmm: index of the weight matrix this group multiplies by
  int row0;    // gmm: first row of x / y;  tgmm: first row of the group
  int rows;    // gmm: valid rows in this tile (<=128);  tgmm: rows of the group (contraction)
  int n0;      // first output column
  int k0;      // tgmm: first row of out[group] covered by this tile
};

__device__ __forceinline__ int imin(int a, int b) { return a < b ? a : b; }
__device__ __forceinline__ int imax(int a, int b) { return a > b ? a : b; }

// gmm tile order: group-major; inside a group the n-tiles are outer and the group's row
// tiles inner, so CTAs running concurrently share one [k, BN] weight panel through L2 and an
// expert's weights stream from HBM once.
__device__ __forceinline__ TileCoord decode_gmm_tile(const GemmArgs& p, int tile) {
  const int mt = tile / p.n_tiles;
  const int gi = p.tile2group[mt];
  const int base = p.tile_prefix[gi];
  const int tiles_g = p.tile_prefix[gi + 1] - base;
  const int local = tile - base * p.n_tiles;
  const int nt = local / tiles_g;
  const int mi = local - nt * tiles_g;
  TileCoord t;
  t.group = gi;
  t.weight = p.group_to_weight ? p.group_to_weight[gi] : gi;
  t.row0 = p.group_offsets[gi] + mi * kTileM;
  t.rows = imin(kTileM, imax(p.group_sizes[gi], 0) - mi * kTileM);
  t.rows = imin(t.rows, p.m - t.row0);  // never touch rows past m
  t.n0 = 0;
  t.k0 = 0;
  t.n0 = nt;  // caller scales by BN
  return t;
}

__device__ __forceinline__ TileCoord decode_tgmm_tile(const GemmArgs& p, int tile) {
  const int per_group = p.k_tiles * p.n_tiles;
  const int gi = tile / per_group;
  const int rem = tile - gi * per_group;
  const int kt = rem / p.n_tiles;
  const int nt = rem - kt * p.n_tiles;
  TileCoord t;
  t.group = gi;
  t.weight = gi;
  t.row0 = p.group_offsets[gi];
  t.rows = imax(imin(imax(p.group_sizes[gi], 0), p.m - t.row0), 0);
  t.n0 = nt;
  t.k0 = kt * kTileM;
  return t;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int ab_format) {
  if (ab_format == 1) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int BN, bool kTgmm>
constexpr int stage_bytes() {
  return kTileM * kTileK * 2 + BN * kTileK * 2;
}

// kTgmm == false : gmm.   A operand = x tile, K-major.  B operand = W tile, K-major when
//                  kBKMajor (trans_rhs: W[g] is [n,k]) else MN-major (W[g] is [k,n]).
// kTgmm == true  : tgmm.  A operand = x^T tile (MN-major), B operand = dout tile (MN-major);
//                  kBKMajor must be false.
template <int BN, bool kBKMajor, int kStages, bool kTgmm>
__global__ void __launch_bounds__(kGemmThreads, 1)
ragged_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                   const __grid_constant__ CUtensorMap tmap_b, const GemmArgs p) {
  static_assert(BN == 64 || BN == 128 || BN == 256, "BN must be 64, 128 or 256");
  static_assert(!(kTgmm && kBKMajor), "tgmm reads both operands MN-major");
  constexpr uint32_t kABytes = kTileM * kTileK * 2;
  constexpr uint32_t kBBytes = BN * kTileK * 2;
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;  // two fp32 accumulators of BN columns
  constexpr uint32_t kIdesc =
      0;  // built at run time (ab_format is a run-time value); see make_idesc_f16 below

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  (void)kIdesc;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t stage_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_acc_full[a]), 1);
      mbar_init(smem_u32(&bar_acc_empty[a]), 4);  // one arrival per epilogue warp
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(&tmem_slot), kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abort_ptr = &abort_flag;

  int num_tiles;
  if (kTgmm) {
    num_tiles = p.g * p.k_tiles * p.n_tiles;
  } else {
    num_tiles = imin(p.totals[0], p.max_m_tiles) * p.n_tiles;
  }
  const int k_blocks_gmm = (p.k + kTileK - 1) / kTileK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileCoord t = kTgmm ? decode_tgmm_tile(p, tile) : decode_gmm_tile(p, tile);
        const int n0 = t.n0 * BN;
        const int kb_count = kTgmm ? (t.rows + kTileK - 1) / kTileK : k_blocks_gmm;
        for (int kb = 0; kb < kb_count; ++kb, ++it) {
          const uint32_t s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_ptr)) {
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t sa = stage_base + s * kStageBytes;
          const uint32_t sb = sa + kABytes;
          mbar_arrive_expect_tx(full, kStageBytes);
          if (kTgmm) {
            const int r = t.row0 + kb * kTileK;
            tma_load_2d(sa, &tmap_a, full, t.k0, r);
            tma_load_2d(sa + kBoxBytes, &tmap_a, full, t.k0 + 64, r);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * kBoxBytes, &tmap_b, full, n0 + j * 64, r);
          } else {
            tma_load_2d(sa, &tmap_a, full, kb * kTileK, t.row0);
            if (kBKMajor) {
              tma_load_3d(sb, &tmap_b, full, kb * kTileK, n0, t.weight);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(sb + j * kBoxBytes, &tmap_b, full, n0 + j * 64, kb * kTileK, t.weight);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc_f16(p.ab_format, kTgmm ? 1 : 0, kBKMajor ? 0 : 1, kTileM, BN);
    uint32_t it = 0;
    uint32_t local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      const TileCoord t = kTgmm ? decode_tgmm_tile(p, tile) : decode_gmm_tile(p, tile);
      const int kb_count = kTgmm ? (t.rows + kTileK - 1) / kTileK : k_blocks_gmm;
      const uint32_t acc = local_tile & 1u;
      const uint32_t acc_ph = (local_tile >> 1) & 1u;
      if (!mbar_wait(smem_u32(&bar_acc_empty[acc]), acc_ph ^ 1u, abort_ptr)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + acc * BN;
      for (int kb = 0; kb < kb_count; ++kb, ++it) {
        const uint32_t s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_ptr)) {
          ok = false;
          break;
        }
        const uint32_t sa = stage_base + s * kStageBytes;
        const uint32_t sb = sa + kABytes;
        if (kTgmm) {
          // Rows past the end of the group belong to the next group (or to nobody): clear
          // them in every box of this stage so they add nothing to the reduction.
          const int live = t.rows - kb * kTileK;
          if (live < kTileK) {
            constexpr int kBoxes = (kABytes + kBBytes) / kBoxBytes;
            const int dead = kTileK - live;
            const int chunks = kBoxes * dead * 8;  // 16-byte chunks
            for (int c = lane; c < chunks; c += 32) {
              const int box = c / (dead * 8);
              const int rem = c - box * (dead * 8);
              const uint32_t addr = sa + box * kBoxBytes + (live * 128) + rem * 16;
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u)
                           : "memory");
            }
            fence_proxy_async_smem();
          }
          __syncwarp();
        }
        tc_fence_after_sync();
        if (lane == 0) {
#pragma unroll
          for (int kk = 0; kk < kTileK / kUmmaK; ++kk) {
            uint64_t adesc, bdesc;
            if (kTgmm) {
              adesc = make_smem_desc(sa + kk * 2048, kBoxBytes, 1024);
            } else {
              adesc = make_smem_desc(sa + kk * 32, 16, 1024);
            }
            if (kBKMajor) {
              bdesc = make_smem_desc(sb + kk * 32, 16, 1024);
            } else {
              bdesc = make_smem_desc(sb + kk * 2048, kBoxBytes, 1024);
            }
            umma_f16<1>(tmem_d, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&bar_empty[s]));  // frees the smem stage when these MMAs retire
        }
        __syncwarp();
      }
      if (!ok) break;
      if (lane == 0) {
        if (kb_count > 0) {
          umma_commit(smem_u32(&bar_acc_full[acc]));
        } else {
          mbar_arrive(smem_u32(&bar_acc_full[acc]));  // empty group: nothing to wait for
        }
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const int r_in_tile = quarter * 32 + lane;
    uint32_t local_tile = 0;
    bool ok = true;
    uint16_t* out16 = reinterpret_cast<uint16_t*>(p.out);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      const TileCoord t = kTgmm ? decode_tgmm_tile(p, tile) : decode_gmm_tile(p, tile);
      const int n0 = t.n0 * BN;
      const uint32_t acc = local_tile & 1u;
      const uint32_t acc_ph = (local_tile >> 1) & 1u;
      if (!mbar_wait(smem_u32(&bar_acc_full[acc]), acc_ph, abort_ptr)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();

      bool row_ok;
      size_t row_off;  // element offset of this thread's output row
      bool warp_has_rows;
      bool zero_only = false;
      if (kTgmm) {
        const int kr = t.k0 + r_in_tile;
        row_ok = kr < p.k;
        warp_has_rows = (t.k0 + quarter * 32) < p.k;
        row_off = (static_cast<size_t>(t.group) * p.k + kr) * static_cast<size_t>(p.n);
        zero_only = t.rows <= 0;
      } else {
        row_ok = r_in_tile < t.rows;
        warp_has_rows = quarter * 32 < t.rows;
        row_off = static_cast<size_t>(t.row0 + r_in_tile) * static_cast<size_t>(p.n);
      }

      if (warp_has_rows) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col = n0 + c * 32;
          if (col >= p.n) break;
          uint32_t v[32];
          if (!zero_only) {
            const uint32_t taddr =
                tmem_base + acc * BN + c * 32 + (static_cast<uint32_t>(quarter * 32) << 16);
            tmem_ld_32x32(taddr, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
          if (row_ok) {
            uint16_t* dst = out16 + row_off + col;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (col + q * 8 < p.n) {  // n is a multiple of 8: a chunk is all in or all out
                uint4 o;
                o.x = pack2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]), p.ab_format);
                o.y = pack2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]), p.ab_format);
                o.z = pack2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]), p.ab_format);
                o.w = pack2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]), p.ab_format);
                *reinterpret_cast<uint4*>(dst + q * 8) = o;
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[acc]));
    }

    if (!kTgmm) {
      // Rows past sum(group_sizes) belong to no group: jax.lax.ragged_dot defines them as 0
      // (the reference writes them from its last live program, gpu_ragged_dot.py:155-165).
      const int first = imin(imax(p.totals[1], 0), p.m);
      const size_t chunks_per_row = static_cast<size_t>(p.n) / 8;
      const size_t total = static_cast<size_t>(p.m - first) * chunks_per_row;
      const size_t tid = static_cast<size_t>(blockIdx.x) * 128 + (threadIdx.x - 64);
      const size_t stride = static_cast<size_t>(gridDim.x) * 128;
      uint4* dst = reinterpret_cast<uint4*>(out16 + static_cast<size_t>(first) * p.n);
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      for (size_t i = tid; i < total; i += stride) dst[i] = z;
    }
  }

  // ------------------------------------------------------------ tear-down
  __syncthreads();
  if (abort_flag) {
    if (threadIdx.x == 0) atomicMax(p.status, static_cast<int32_t>(kStatusWaitExpired));
    // Give copies and MMAs that are still in flight time to land before smem/TMEM go away.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
}

}  // namespace rd
