// Grouped GEMM with the row permutation of a mixture-of-experts layer fused in.
//
// A caller of gmm in an MoE layer sorts token rows by expert first (x_sorted = x[row_index]),
// and un-sorts the result afterwards; the reference leaves both passes to the caller
// (gpu_ragged_dot.py takes rows that are already grouped).  These kernels read and write the
// un-sorted tensors directly:
//
//   gmm  : y[out_rows[r], :] = x[a_rows[r], :] @ W[group of r]      for r < sum(group_sizes)
//   tgmm : out[i] = x[a_rows[rows of group i], :]^T @ dout[b_rows[rows of group i], :]
//
// Any of the index arrays may be null (identity).  An operand with an index array is fetched by
// four gather warps with 16-byte cp.async copies, 8 lanes per 128-byte row, written straight
// into the 128-byte-swizzled layout a TMA tile load would produce; their completion is counted
// on the stage's "full" barrier (cp.async.mbarrier.arrive.noinc) next to the TMA bytes of the
// operands that need no gather.  (TMA's own row gather, tile::gather4, was measured at about
// 40 ns per four rows per SM: a third of the rate the tensor core consumes A tiles at.)
// With out_rows the epilogue stores each row at its own destination and nothing else of y is
// touched (no zero tail).
//
// Barriers, MMA issue, epilogue and bounded waits are those of the 128-row single-CTA kernel
// in rd_gemm.cuh, whose helpers are reused.
#pragma once

#include "rd_gemm.cuh"

namespace rd {

struct PermArgs {
  const int32_t* a_rows;    // gmm: x row of sorted row r;  tgmm: same for x.   null = identity
  const int32_t* b_rows;    // tgmm: dout row of sorted row r.                  null = identity
  const int32_t* out_rows;  // gmm: y row of sorted row r.                      null = identity
  const void* a_base;       // x (the tensor a_rows indexes), row-major, p.k elements per row
  const void* b_base;       // tgmm: dout, p.n elements per row
  int a_rows_in;            // rows of the tensor a_rows points into
  int b_rows_in;
  int out_rows_n;           // rows of y when out_rows is given
};

constexpr int kPermGatherWarps = 4;
constexpr int kPermGatherThreads = 32 * kPermGatherWarps;
constexpr int kPermPassRows = kPermGatherThreads / 8;  // rows covered per pass: 8 lanes per row
constexpr int kPermThreads = kGemmThreads + kPermGatherThreads;

// 16-byte asynchronous copy global -> shared; src_bytes == 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
// One arrival on `bar` (part of its expected count) once this thread's copies so far are done.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// Byte offset of source row `r` (a sorted row, valid when r < r_end) of a [rows_in, ld] 16-bit
// tensor, or -1 when the row does not exist (sorted row past the end, index out of range).
__device__ __forceinline__ long long gather_row_offset(const int32_t* index, int rows_in, int ld,
                                                       int r, int r_end) {
  if (r >= r_end) return -1;
  const int src = index ? index[r] : r;
  if (src < 0 || src >= rows_in) return -1;
  return static_cast<long long>(src) * ld * 2;
}

template <int BN, bool kBKMajor, int kStages, bool kTgmm>
__global__ void __launch_bounds__(kPermThreads, 1)
ragged_gemm_perm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                        const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_out, const GemmArgs p,
                        const PermArgs q) {
  static_assert(BN == 64 || BN == 128 || BN == 256, "BN must be 64, 128 or 256");
  static_assert(!(kTgmm && kBKMajor), "tgmm reads both operands MN-major");
  constexpr uint32_t kABytes = kTileM * kTileK * 2;
  constexpr uint32_t kBBytes = BN * kTileK * 2;
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;

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
      // producer lane (TMA bytes) + one deferred arrival per gather thread
      mbar_init(smem_u32(&bar_full[s]), 1 + kPermGatherThreads);
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
  const int k_blocks_gmm = (p.k + kTileK - 1) / kTileK;

  const bool gather_a = q.a_rows != nullptr;
  const bool gather_b = kTgmm && q.b_rows != nullptr;
  const uint8_t* a_base = static_cast<const uint8_t*>(q.a_base);
  const uint8_t* b_base = static_cast<const uint8_t*>(q.b_base);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // Posts each stage's TMA byte count and loads the operands that need no gather.
    if (lane == 0) {
      const uint32_t tma_bytes = (gather_a ? 0u : kABytes) + (gather_b ? 0u : kBBytes);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += tile_step) {
        const TileCoord t = kTgmm ? decode_tgmm_tile<BN, 1>(p, tile, 0) : decode_gmm_tile<BN, 1>(p, tile, 0);
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
          if (tma_bytes != 0) {
            mbar_arrive_expect_tx(full, tma_bytes);
          } else {
            mbar_arrive(full);
          }
          if (kTgmm) {
            const int r = t.row0 + kb * kTileK;
            if (!gather_a) {
              tma_load_2d(sa, &tmap_a, full, t.k0, r);
              tma_load_2d(sa + kBoxBytes, &tmap_a, full, t.k0 + 64, r);
            }
            if (!gather_b) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * kBoxBytes, &tmap_b, full, t.n0 + j * 64, r);
            }
          } else {
            if (!gather_a) tma_load_2d(sa, &tmap_a, full, kb * kTileK, t.row0);
            if (kBKMajor) {
              tma_load_3d(sb, &tmap_b, full, kb * kTileK, t.n0, t.weight);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_3d(sb + j * kBoxBytes, &tmap_b, full, t.n0 + j * 64, kb * kTileK, t.weight);
            }
          }
        }
      }
    }
  } else if (warp >= kGemmThreads / 32) {
    // ------------------------------------------------------------ gather warps
    // Thread (rg, sub): 16-byte chunk `sub` of rows rg, rg+R, rg+2R, ... (R = kPermPassRows) of
    // each gathered box.
    constexpr int R = kPermPassRows;
    constexpr int kGmmRows = kTileM / R;   // rows per thread of a gmm A tile
    constexpr int kTgmmRows = kTileK / R;  // rows per thread of a tgmm stage
    static_assert(R % 8 == 0 && kTileK % R == 0, "gather passes must keep a row's swizzle phase");
    const int gt = threadIdx.x - kGemmThreads;
    const int sub = gt & 7;
    const int rg = gt >> 3;
    const uint32_t swz = static_cast<uint32_t>((sub ^ (rg & 7)) << 4);  // rows rg+R*i share rg&7
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += tile_step) {
      const TileCoord t = kTgmm ? decode_tgmm_tile<BN, 1>(p, tile, 0) : decode_gmm_tile<BN, 1>(p, tile, 0);
      const int kb_count = kTgmm ? (t.rows + kTileK - 1) / kTileK : k_blocks_gmm;
      long long arow[kGmmRows];  // gmm: byte offsets of this thread's rows of the tile (-1: no row)
      if (!kTgmm && gather_a) {
        const int r_end = t.row0 + imax(t.rows, 0);
#pragma unroll
        for (int i = 0; i < kGmmRows; ++i)
          arow[i] = gather_row_offset(q.a_rows, q.a_rows_in, p.k, t.row0 + rg + R * i, r_end);
      }
      // tgmm: a stage's 64 sorted rows, 4 per thread.  The row indices of stage kb+1 are
      // loaded while stage kb is copied and not looked at until then, so the loads' latency
      // stays off the loop.
      int xi[kTgmmRows], di[kTgmmRows], xi_next[kTgmmRows], di_next[kTgmmRows];
      const int r_end = t.row0 + t.rows;
      if (kTgmm && kb_count > 0) {
#pragma unroll
        for (int i = 0; i < kTgmmRows; ++i) {
          const int r = imin(t.row0 + rg + R * i, p.m - 1);
          xi[i] = gather_a ? q.a_rows[r] : 0;
          di[i] = gather_b ? q.b_rows[r] : 0;
        }
      }
      for (int kb = 0; kb < kb_count; ++kb, ++it) {
        const uint32_t s = it % kStages;
        const uint32_t ph = (it / kStages) & 1u;
        if (kTgmm && kb + 1 < kb_count) {
#pragma unroll
          for (int i = 0; i < kTgmmRows; ++i) {
            const int r = imin(t.row0 + (kb + 1) * kTileK + rg + R * i, p.m - 1);
            xi_next[i] = gather_a ? q.a_rows[r] : 0;
            di_next[i] = gather_b ? q.b_rows[r] : 0;
          }
        }
        if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_ptr)) {
          ok = false;
          break;
        }
        const uint32_t sa = stage_base + s * kStageBytes;
        const uint32_t sb = sa + kABytes;
        if (!kTgmm) {
          if (gather_a) {
            const int col = kb * kTileK + sub * 8;
            const bool col_ok = col < p.k;
#pragma unroll
            for (int i = 0; i < kGmmRows; ++i) {
              const bool okr = col_ok && arow[i] >= 0;
              const uint8_t* src = a_base + (okr ? arow[i] + col * 2 : 0);
              cp_async16(sa + (rg + R * i) * 128 + swz, src, okr ? 16u : 0u);
            }
          }
        } else {
          // Per stage and operand: four row pointers (column of this thread's chunk in the
          // operand's first box), then one copy per box and row with constant strides.
          const int r0 = t.row0 + kb * kTileK + rg;
          if (gather_a) {
            const int col0 = t.k0 + sub * 8;
            const uint32_t dst0 = sa + rg * 128 + swz;
#pragma unroll
            for (int i = 0; i < kTgmmRows; ++i) {
              const bool okr = r0 + R * i < r_end &&
                               static_cast<unsigned>(xi[i]) < static_cast<unsigned>(q.a_rows_in);
              const uint8_t* rp = a_base + (static_cast<long long>(okr ? xi[i] : 0) * p.k + col0) * 2;
#pragma unroll
              for (int b = 0; b < 2; ++b) {
                const bool okc = okr && col0 + b * 64 < p.k;
                cp_async16(dst0 + b * kBoxBytes + i * (R * 128), okc ? rp + b * 128 : a_base, okc ? 16u : 0u);
              }
            }
          }
          if (gather_b) {
            const int col0 = t.n0 + sub * 8;
            const uint32_t dst0 = sb + rg * 128 + swz;
#pragma unroll
            for (int i = 0; i < kTgmmRows; ++i) {
              const bool okr = r0 + R * i < r_end &&
                               static_cast<unsigned>(di[i]) < static_cast<unsigned>(q.b_rows_in);
              const uint8_t* rp = b_base + (static_cast<long long>(okr ? di[i] : 0) * p.n + col0) * 2;
#pragma unroll
              for (int b = 0; b < BN / 64; ++b) {
                const bool okc = okr && col0 + b * 64 < p.n;
                cp_async16(dst0 + b * kBoxBytes + i * (R * 128), okc ? rp + b * 128 : b_base, okc ? 16u : 0u);
              }
            }
          }
        }
        cp_async_arrive(smem_u32(&bar_full[s]));
        if (kTgmm) {
#pragma unroll
          for (int i = 0; i < kTgmmRows; ++i) {
            xi[i] = xi_next[i];
            di[i] = di_next[i];
          }
        }
      }
    }
    // Copies still in flight must land before shared memory is given up.
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc_f16(p.ab_format, kTgmm ? 1 : 0, kBKMajor ? 0 : 1, kTileM, BN);
    constexpr uint32_t kAStep = (kTgmm ? 2048u : 32u) >> 4;
    constexpr uint32_t kBStep = (kBKMajor ? 32u : 2048u) >> 4;
    const uint64_t adesc0 = kTgmm ? make_smem_desc(stage_base, kBoxBytes, 1024)
                                  : make_smem_desc(stage_base, 16, 1024);
    const uint64_t bdesc0 = kBKMajor ? make_smem_desc(stage_base + kABytes, 16, 1024)
                                     : make_smem_desc(stage_base + kABytes, kBoxBytes, 1024);
    const uint32_t adesc0_lo = static_cast<uint32_t>(adesc0);
    const uint32_t bdesc0_lo = static_cast<uint32_t>(bdesc0);
    const uint32_t desc_hi = static_cast<uint32_t>(adesc0 >> 32);
    uint32_t it = 0;
    uint32_t local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += tile_step, ++local_tile) {
      const TileCoord t = kTgmm ? decode_tgmm_tile<BN, 1>(p, tile, 0) : decode_gmm_tile<BN, 1>(p, tile, 0);
      const int kb_count = kTgmm ? (t.rows + kTileK - 1) / kTileK : k_blocks_gmm;
      const bool tail_stage = kTgmm && kb_count > 0 && tail_needs_clearing(t.rows);
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
        // The gather warps wrote this stage through the generic proxy; the tensor core reads it
        // through the async proxy.
        fence_proxy_async_smem();
        const uint32_t sa = stage_base + s * kStageBytes;
        const int live = kTgmm ? t.rows - kb * kTileK : kTileK;
        const int n_mma = live >= kTileK ? kTileK / kUmmaK : (live + kUmmaK - 1) / kUmmaK;
        if (kTgmm && tail_stage && kb == kb_count - 1) {
          clear_tail_rows<(kABytes + kBBytes) / kBoxBytes>(sa, live, lane);
          __syncwarp();
        }
        tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_lo = adesc0_lo + s * (kStageBytes >> 4);
          const uint32_t b_lo = bdesc0_lo + s * (kStageBytes >> 4);
          if (kTgmm && n_mma < kTileK / kUmmaK) {
            for (int kk = 0; kk < n_mma; ++kk) {
              umma_f16<1>(tmem_d, make_desc64(a_lo + kk * kAStep, desc_hi),
                          make_desc64(b_lo + kk * kBStep, desc_hi), idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
          } else {
            umma_f16<1>(tmem_d, make_desc64(a_lo, desc_hi), make_desc64(b_lo, desc_hi), idesc,
                        kb > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < kTileK / kUmmaK; ++kk) {
              umma_f16<1>(tmem_d, make_desc64(a_lo + kk * kAStep, desc_hi),
                          make_desc64(b_lo + kk * kBStep, desc_hi), idesc, 1u);
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
          mbar_arrive(bar);
        }
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    const int r_in_tile = quarter * 32 + lane;
    const uint32_t staging = stage_base + kStages * kStageBytes + (warp - 2) * 2 * kOutBoxBytes;
    const bool scatter = !kTgmm && q.out_rows != nullptr;
    uint32_t local_tile = 0;
    uint32_t boxes_stored = 0;
    bool ok = true;
    uint16_t* out16 = reinterpret_cast<uint16_t*>(p.out);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += tile_step, ++local_tile) {
      const TileCoord t = kTgmm ? decode_tgmm_tile<BN, 1>(p, tile, 0) : decode_gmm_tile<BN, 1>(p, tile, 0);
      const int n0 = t.n0;
      const uint32_t acc = local_tile & 1u;
      const uint32_t acc_ph = (local_tile >> 1) & 1u;

      bool row_ok;
      size_t row_off;
      bool warp_has_rows;
      bool slab_by_tma;
      bool zero_only = false;
      int out_row0;
      int scatter_row = -1;  // scatter mode: this thread's destination row, -1 = none
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
        slab_by_tma = !scatter && quarter * 32 + 32 <= t.rows;
        int dst_row = t.row0 + r_in_tile;
        if (scatter && row_ok) {
          // The destination row is fetched before the wait on the accumulator, off the
          // critical path.  A row outside y is dropped.
          dst_row = q.out_rows[dst_row];
          row_ok = dst_row >= 0 && dst_row < q.out_rows_n;
        }
        row_off = static_cast<size_t>(dst_row) * static_cast<size_t>(p.n);
        scatter_row = row_ok ? dst_row : -1;
      }

      if (!mbar_wait(smem_u32(&bar_acc_full[acc]), acc_ph, abort_ptr)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();

      const int n_chunks = warp_has_rows ? imin(BN / 64, (p.n - n0 + 63) / 64) : 0;
      const uint32_t acc_empty_bar = smem_u32(&bar_acc_empty[acc]);
#pragma unroll 1
      for (int c = 0; c < n_chunks; ++c) {
        const int col = n0 + c * 64;
        uint32_t v[64];
        if (!zero_only) {
          const uint32_t taddr =
              tmem_base + acc * BN + c * 64 + (static_cast<uint32_t>(quarter * 32) << 16);
          tmem_ld_32x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
          tmem_ld_32x32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 64; ++j) v[j] = 0u;
        }
        if (c == n_chunks - 1) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty_bar);
        }
        uint4 o[8];
#pragma unroll
        for (int qq = 0; qq < 8; ++qq) {
          o[qq].x = pack2(__uint_as_float(v[qq * 8 + 0]), __uint_as_float(v[qq * 8 + 1]), p.ab_format);
          o[qq].y = pack2(__uint_as_float(v[qq * 8 + 2]), __uint_as_float(v[qq * 8 + 3]), p.ab_format);
          o[qq].z = pack2(__uint_as_float(v[qq * 8 + 4]), __uint_as_float(v[qq * 8 + 5]), p.ab_format);
          o[qq].w = pack2(__uint_as_float(v[qq * 8 + 6]), __uint_as_float(v[qq * 8 + 7]), p.ab_format);
        }
        if (slab_by_tma) {
          const uint32_t buf = staging + (boxes_stored & 1u) * kOutBoxBytes;
          if (lane == 0) bulk_wait_group_read<1>();
          __syncwarp();
          const uint32_t row_addr = buf + lane * 128;
#pragma unroll
          for (int qq = 0; qq < 8; ++qq) {
            const uint32_t a = row_addr + (((qq ^ (lane & 7)) & 7) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(o[qq].x),
                         "r"(o[qq].y), "r"(o[qq].z), "r"(o[qq].w)
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
        } else if (scatter) {
          // Rows go to destinations of their own: stage the 32 x 64 block in shared memory, then
          // 8 lanes write one row's 128 bytes (4 rows per pass), so every store instruction
          // covers whole 128-byte lines.
          const uint32_t buf = staging;
          __syncwarp();  // the previous chunk has been read out
          const uint32_t row_addr = buf + lane * 128;
#pragma unroll
          for (int qq = 0; qq < 8; ++qq) {
            const uint32_t a = row_addr + (((qq ^ (lane & 7)) & 7) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(o[qq].x),
                         "r"(o[qq].y), "r"(o[qq].z), "r"(o[qq].w)
                         : "memory");
          }
          __syncwarp();
          const int sub = lane & 7;
          const bool col_in = col + sub * 8 < p.n;
#pragma unroll
          for (int pass = 0; pass < 8; ++pass) {
            const int rr = (lane >> 3) + 4 * pass;
            const int drow = __shfl_sync(0xffffffffu, scatter_row, rr);
            uint4 val;
            const uint32_t a = buf + rr * 128 + (((sub ^ (rr & 7)) & 7) << 4);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                         : "r"(a)
                         : "memory");
            if (drow >= 0 && col_in) {
              *reinterpret_cast<uint4*>(out16 + static_cast<size_t>(drow) * p.n + col + sub * 8) = val;
            }
          }
        } else if (row_ok) {
          uint16_t* dst = out16 + row_off + col;
#pragma unroll
          for (int qq = 0; qq < 8; ++qq) {
            if (col + qq * 8 < p.n) *reinterpret_cast<uint4*>(dst + qq * 8) = o[qq];
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

    if (!kTgmm && p.zero_tail && !scatter) {
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
