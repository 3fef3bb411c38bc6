// fp32-input grouped GEMM kernels: gmm / gmm trans_rhs / tgmm with float32 operands multiplied
// on the tensor cores as TF32 (tcgen05.mma.kind::tf32, fp32 accumulation in TMEM) and float32
// output.  This is the precision the reference gets for float32 inputs: its Triton `tl.dot` and
// the jax.lax.ragged_dot it is tested against both run float32 matmuls as TF32 on NVIDIA GPUs
// by default (reference tolerance for float32: relative L2 5e-4, tests.py:127).
//
// Same structure as the 16-bit kernel in rd_gemm.cuh (one persistent CTA per SM; TMA producer
// warp, MMA warp, four epilogue warps; two TMEM accumulators; bounded waits), with the geometry
// of 4-byte elements: a 128-byte swizzle row holds 32 elements, so a stage is 32 deep in the
// contraction, one MMA is 8 deep, an MN-major box is [32 k][32 mn] = 4 KB, and the epilogue
// moves 32 fp32 columns (one 128-byte row) per staging box.  MN-major 32-bit operands must use
// the 128-byte swizzle with 32-byte atoms (TMA: SWIZZLE_128B_ATOM_32B; descriptor layout type
// 1); with the ordinary 16-byte-atom swizzle the tensor core returns zeros.
#pragma once

#include "rd_gemm.cuh"

namespace rd {

constexpr int kF32TileK = 32;             // fp32 elements per 128-byte row == stage depth
constexpr int kF32UmmaK = 8;              // contraction depth of one kind::tf32 MMA
constexpr int kF32BoxBytes = kF32TileK * 128;  // one [32 rows][128 B] box

__host__ __device__ constexpr uint32_t make_idesc_tf32(int a_mn_major, int b_mn_major, int mma_m,
                                                       int mma_n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(mma_n >> 3) << 17) |
         (static_cast<uint32_t>(mma_m >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ bool tail_needs_clearing_f32(int group_rows) {
  const int live = group_rows % kF32TileK;
  return live != 0 && (live % kF32UmmaK) != 0;
}

template <int kBoxes>
__device__ __forceinline__ void clear_tail_rows_f32(uint32_t stage_addr, int live, int lane) {
  const int n_mma = (live + kF32UmmaK - 1) / kF32UmmaK;
  const int dead = n_mma * kF32UmmaK - live;
  if (dead <= 0) return;
  const int chunks = kBoxes * dead * 8;  // 16-byte chunks
  for (int c = lane; c < chunks; c += 32) {
    const int box = c / (dead * 8);
    const int rem = c - box * (dead * 8);
    const uint32_t addr = stage_addr + box * kF32BoxBytes + (live * 128) + rem * 16;
    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
  }
  fence_proxy_async_smem();
}

template <int BN>
constexpr int f32_stage_bytes() {
  return kTileM * 128 + BN * 128;
}

template <int BN, bool kBKMajor, int kStages, bool kTgmm>
__global__ void __launch_bounds__(kGemmThreads, 1)
ragged_gemm_f32_kernel(const __grid_constant__ CUtensorMap tmap_a,
                       const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_out, const GemmArgs p) {
  static_assert(BN == 64 || BN == 128 || BN == 256, "BN must be 64, 128 or 256");
  static_assert(!(kTgmm && kBKMajor), "tgmm reads both operands MN-major");
  constexpr uint32_t kABytes = kTileM * 128;  // [128 rows][128 B] or four [32 k][32 m] boxes
  constexpr uint32_t kBBytes = BN * 128;
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;
  constexpr int kChunkCols = 32;  // fp32 columns per 128-byte output row

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ WaitCtl wait_ctl;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t stage_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;

  if (threadIdx.x == 0) {
    wait_ctl.abort = 0;
    wait_ctl.limit_us = p.wait_limit_us;
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_out);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_acc_full[a]), 1);
      mbar_init(smem_u32(&bar_acc_empty[a]), 4);
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
  volatile WaitCtl* abort_ptr = &wait_ctl;

  const int num_tiles =
      kTgmm ? p.g * p.k_tiles * p.n_tiles : imin(p.totals[0], p.max_m_tiles) * p.n_tiles;
  const int tile_step = static_cast<int>(gridDim.x);
  const int k_blocks_gmm = (p.k + kF32TileK - 1) / kF32TileK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += tile_step) {
        const TileCoord t = kTgmm ? decode_tgmm_tile<BN, 1>(p, tile, 0) : decode_gmm_tile<BN, 1>(p, tile, 0);
        const int kb_count = kTgmm ? (t.rows + kF32TileK - 1) / kF32TileK : k_blocks_gmm;
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
            const int r = t.row0 + kb * kF32TileK;
#pragma unroll
            for (int j = 0; j < kTileM / 32; ++j)
              tma_load_2d(sa + j * kF32BoxBytes, &tmap_a, full, t.k0 + j * 32, r);
#pragma unroll
            for (int j = 0; j < BN / 32; ++j)
              tma_load_2d(sb + j * kF32BoxBytes, &tmap_b, full, t.n0 + j * 32, r);
          } else {
            tma_load_2d(sa, &tmap_a, full, kb * kF32TileK, t.row0);
            if (kBKMajor) {
              tma_load_3d(sb, &tmap_b, full, kb * kF32TileK, t.n0, t.weight);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 32; ++j)
                tma_load_3d(sb + j * kF32BoxBytes, &tmap_b, full, t.n0 + j * 32, kb * kF32TileK, t.weight);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc_tf32(kTgmm ? 1 : 0, kBKMajor ? 0 : 1, kTileM, BN);
    constexpr uint32_t kAStep = (kTgmm ? 1024u : 32u) >> 4;     // 8 k-rows of 128 B, or 8 k-elements
    constexpr uint32_t kBStep = (kBKMajor ? 32u : 1024u) >> 4;
    // MN-major fp32 operands use the 32-byte-atom swizzle: boxes of [32 k][128 B], K-groups of
    // 4 rows (512 B apart), next 32 M/N elements in the next box.
    const uint64_t adesc0 = kTgmm ? make_smem_desc(stage_base, kF32BoxBytes, 512, 1)
                                  : make_smem_desc(stage_base, 16, 1024, 2);
    const uint64_t bdesc0 = kBKMajor ? make_smem_desc(stage_base + kABytes, 16, 1024, 2)
                                     : make_smem_desc(stage_base + kABytes, kF32BoxBytes, 512, 1);
    const uint32_t adesc0_lo = static_cast<uint32_t>(adesc0);
    const uint32_t bdesc0_lo = static_cast<uint32_t>(bdesc0);
    const uint32_t a_hi = static_cast<uint32_t>(adesc0 >> 32);
    const uint32_t b_hi = static_cast<uint32_t>(bdesc0 >> 32);
    uint32_t it = 0;
    uint32_t local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += tile_step, ++local_tile) {
      const TileCoord t = kTgmm ? decode_tgmm_tile<BN, 1>(p, tile, 0) : decode_gmm_tile<BN, 1>(p, tile, 0);
      const int kb_count = kTgmm ? (t.rows + kF32TileK - 1) / kF32TileK : k_blocks_gmm;
      const bool tail_stage = kTgmm && kb_count > 0 && tail_needs_clearing_f32(t.rows);
      const uint32_t acc = local_tile & 1u;
      const uint32_t acc_ph = (local_tile >> 1) & 1u;
      if (!mbar_wait(smem_u32(&bar_acc_empty[acc]), acc_ph ^ 1u, abort_ptr)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t tmem_d = tmem_base + acc * BN;
      uint32_t s = it % kStages;
      uint32_t ph = (it / kStages) & 1u;
      for (int kb = 0; kb < kb_count; ++kb, ++it, s = (s + 1 == kStages ? 0 : s + 1), ph ^= (s == 0)) {
        if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_ptr)) {
          ok = false;
          break;
        }
        const uint32_t sa = stage_base + s * kStageBytes;
        const int live = kTgmm ? t.rows - kb * kF32TileK : kF32TileK;
        const int n_mma = live >= kF32TileK ? kF32TileK / kF32UmmaK : (live + kF32UmmaK - 1) / kF32UmmaK;
        if (kTgmm && tail_stage && kb == kb_count - 1) {
          clear_tail_rows_f32<kStageBytes / kF32BoxBytes>(sa, live, lane);
          __syncwarp();
        }
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_lo = adesc0_lo + s * (kStageBytes >> 4);
          const uint32_t b_lo = bdesc0_lo + s * (kStageBytes >> 4);
          if (kTgmm && n_mma < kF32TileK / kF32UmmaK) {
            for (int kk = 0; kk < n_mma; ++kk) {
              umma_tf32(tmem_d, make_desc64(a_lo + kk * kAStep, a_hi),
                        make_desc64(b_lo + kk * kBStep, b_hi), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
          } else {
            umma_tf32(tmem_d, make_desc64(a_lo, a_hi), make_desc64(b_lo, b_hi), idesc,
                      kb > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < kF32TileK / kF32UmmaK; ++kk) {
              umma_tf32(tmem_d, make_desc64(a_lo + kk * kAStep, a_hi),
                        make_desc64(b_lo + kk * kBStep, b_hi), idesc, 1u);
            }
          }
          umma_commit(smem_u32(&bar_empty[s]));
        }
        __syncwarp();
      }
      if (!ok) break;
      if (lane == 0) {
        const uint32_t bar = smem_u32(&bar_acc_full[acc]);
        if (kb_count > 0) {
          umma_commit(bar);
        } else {
          mbar_arrive(bar);  // empty group: nothing to wait for
        }
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    const int r_in_tile = quarter * 32 + lane;
    const uint32_t staging = stage_base + kStages * kStageBytes + (warp - 2) * 2 * kOutBoxBytes;
    uint32_t local_tile = 0;
    uint32_t boxes_stored = 0;
    bool ok = true;
    float* out32 = reinterpret_cast<float*>(p.out);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += tile_step, ++local_tile) {
      const TileCoord t = kTgmm ? decode_tgmm_tile<BN, 1>(p, tile, 0) : decode_gmm_tile<BN, 1>(p, tile, 0);
      const int n0 = t.n0;
      const uint32_t acc = local_tile & 1u;
      const uint32_t acc_ph = (local_tile >> 1) & 1u;
      if (!mbar_wait(smem_u32(&bar_acc_full[acc]), acc_ph, abort_ptr)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();

      bool row_ok, warp_has_rows, slab_by_tma, zero_only = false;
      size_t row_off;
      int out_row0;
      if (kTgmm) {
        const int kr = t.k0 + r_in_tile;
        out_row0 = t.k0 + quarter * 32;
        row_ok = kr < p.k;
        warp_has_rows = out_row0 < p.k;
        slab_by_tma = true;
        row_off = (static_cast<size_t>(t.group) * p.k + kr) * static_cast<size_t>(p.n);
        zero_only = t.rows <= 0;
      } else {
        out_row0 = t.row0 + quarter * 32;
        row_ok = r_in_tile < t.rows;
        warp_has_rows = quarter * 32 < t.rows;
        slab_by_tma = quarter * 32 + 32 <= t.rows;
        row_off = static_cast<size_t>(t.row0 + r_in_tile) * static_cast<size_t>(p.n);
      }

      const int n_chunks =
          warp_has_rows ? imin(BN / kChunkCols, (p.n - n0 + kChunkCols - 1) / kChunkCols) : 0;
      const uint32_t acc_empty_bar = smem_u32(&bar_acc_empty[acc]);
#pragma unroll 1
      for (int c = 0; c < n_chunks; ++c) {
        const int col = n0 + c * kChunkCols;
        uint32_t v[32];
        if (!zero_only) {
          const uint32_t taddr =
              tmem_base + acc * BN + c * kChunkCols + (static_cast<uint32_t>(quarter * 32) << 16);
          tmem_ld_32x32(taddr, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
        if (c == n_chunks - 1) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty_bar);
        }
        if (slab_by_tma) {
          const uint32_t buf = staging + (boxes_stored & 1u) * kOutBoxBytes;
          if (lane == 0) bulk_wait_group_read<1>();
          __syncwarp();
          const uint32_t row_addr = buf + lane * 128;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t a = row_addr + (((q ^ (lane & 7)) & 7) << 4);  // 128-byte swizzle
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(v[q * 4 + 0]),
                         "r"(v[q * 4 + 1]), "r"(v[q * 4 + 2]), "r"(v[q * 4 + 3])
                         : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (kTgmm) {
              tma_store_3d(&tmap_out, buf, col, out_row0, t.group);
            } else {
              tma_store_2d(&tmap_out, buf, col, out_row0);
            }
            bulk_commit_group();
          }
          ++boxes_stored;
        } else if (row_ok) {
          float* dst = out32 + row_off + col;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (col + q * 4 < p.n) {  // n is a multiple of 4: a chunk is all in or all out
              *reinterpret_cast<uint4*>(dst + q * 4) =
                  make_uint4(v[q * 4 + 0], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            }
          }
        }
      }
      if (n_chunks == 0) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar);
      }
    }
    if (lane == 0) bulk_wait_group<0>();
    __syncwarp();

    if (!kTgmm && p.zero_tail) {
      const int first = imin(imax(p.totals[1], 0), p.m);
      const size_t chunks_per_row = static_cast<size_t>(p.n) / 4;
      const size_t total = static_cast<size_t>(p.m - first) * chunks_per_row;
      const size_t tid = static_cast<size_t>(blockIdx.x) * 128 + (threadIdx.x - 64);
      const size_t stride = static_cast<size_t>(gridDim.x) * 128;
      uint4* dst = reinterpret_cast<uint4*>(out32 + static_cast<size_t>(first) * p.n);
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      for (size_t i = tid; i < total; i += stride) dst[i] = z;
    }
  }

  // ------------------------------------------------------------ tear-down
  __syncthreads();
  if (wait_ctl.abort) {
    if (threadIdx.x == 0) atomicMax(p.status, static_cast<int32_t>(kStatusWaitExpired));
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
