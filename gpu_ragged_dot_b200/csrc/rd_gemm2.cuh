// Grouped GEMM kernels with 256-row tiles on ONE CTA ("two-half" tiles).
//
// The 128 x 256 kernel in rd_gemm.cuh is bound by how fast shared memory can be refilled:
// every 64-deep stage moves 16 KB of A and 32 KB of B for 128 x 256 x 64 MMAs, and with four
// 48 KB stages in flight the load -> MMA -> free-the-stage loop (about 1.6 us) caps the tensor
// pipe near 75 %.  Here a CTA owns a 256 x 256 tile as two 128-row halves that share each B
// stage: per stage 32 KB of A + 32 KB of B feed twice the MMAs, a third less traffic per flop,
// which three 64 KB stages can sustain.  The price is TMEM: the two halves use both 256-column
// accumulators, so a tile's epilogue no longer overlaps the next tile's main loop by double
// buffering; instead eight epilogue warps drain the two halves at once and each half's
// accumulator is handed back as soon as it has been read.
//
// A half that has no rows (the last tile of a group with <= 128 rows left; the last 128 rows
// of k in tgmm) is skipped entirely -- no loads, no MMAs -- so nothing is wasted beyond the
// 128-row granularity of the other kernel.
//
// Same roles, operand layouts, barrier discipline (bounded waits) and epilogue (swizzled smem
// staging + TMA stores, row-masked stores where a gmm slab crosses its group's end) as
// rd_gemm.cuh; the helpers of that file are reused.
//
// kPair (tgmm only): two CTAs of a cluster own a 512 x 256 tile, CTA c its rows [256 c, 256 c +
// 256).  Half h is ONE tcgen05.mma.cta_group::2 product of 256 rows, rows [128 h, 128 h + 128) of
// either CTA; each CTA loads its own rows of the A operand (32 KB) and HALF of the B operand's
// columns (16 KB), so a stage is 48 KB for the same MMAs per SM, a quarter less L2 -> SM traffic
// per flop, and four stages fit.  The hand-shakes between the two CTAs are those of the 128-row
// pair kernel in rd_gemm.cuh.  Measured on the Mixtral-shaped weight gradient it moves 5.8 GB
// instead of 7.75 GB from L2 and takes 0.71-0.73 ms against 0.72-0.74 ms for one CTA per tile.
//
// Blocked operand maps (GemmArgs::blocked_maps, tgmm): x and dout are described to TMA as
// (64 columns, rows, blocks of 64 columns), so ONE box of (64, 64 rows, 4 blocks) = 32 KB lands as
// the same four [64 rows][128 B] slabs that four 2-D boxes would write: two TMA instructions per
// stage instead of eight (about 1 % on the Mixtral-shaped weight gradient).  Needs k and n to be
// multiples of 64; otherwise one 2-D box per 64 columns, as in rd_gemm.cuh.
#pragma once

#include "rd_gemm.cuh"

namespace rd {

constexpr int kG2EpilogueWarps = 8;
constexpr int kG2FixerWarp = 2 + kG2EpilogueWarps;  // warp 10: clears tail rows of tgmm stages
constexpr int kG2Threads = 64 + 32 * kG2EpilogueWarps + 32;
constexpr int kG2Stages = 3;
constexpr int kG2PairStages = 4;  // 48 KB stages when a CTA pair shares the B operand
constexpr int kG2TileN = 256;
constexpr int kG2TileRows = 2 * kTileM;
constexpr int kG2TgmmBand = 8;  // column tiles per band of the tgmm tile order
constexpr uint32_t kG2ABytes = 2 * kTileM * kTileK * 2;   // two 128-row halves
constexpr uint32_t kG2BBytes = kG2TileN * kTileK * 2;
constexpr uint32_t kG2StageBytes = kG2ABytes + kG2BBytes;  // 64 KB
constexpr int kG2SmemBytes = kG2Stages * kG2StageBytes + kG2EpilogueWarps * kOutBoxBytes + 1024;
constexpr uint32_t kG2PairStageBytes = kG2ABytes + kG2BBytes / 2;  // 48 KB
constexpr int kG2PairSmemBytes = kG2PairStages * kG2PairStageBytes + kG2EpilogueWarps * kOutBoxBytes + 1024;

// rows: valid rows of the whole 256-row tile (gmm) / rows of the group (tgmm).
__device__ __forceinline__ TileCoord decode_gmm_tile256(const GemmArgs& p, int tile) {
  const int mt = tile / p.n_tiles;
  const int4* rp = reinterpret_cast<const int4*>(p.tile_rec + mt);
  const int4 a = rp[0];  // group, weight, group_offset, group_size
  const int4 b = rp[1];  // tile_base, tiles, idx, pad
  const int local = tile - b.x * p.n_tiles;
  const int nt = local / b.y;
  const int mi = local - nt * b.y;
  TileCoord t;
  t.group = a.x;
  t.weight = a.y;
  t.row0 = a.z + mi * kG2TileRows;
  t.rows = imin(kG2TileRows, a.w - mi * kG2TileRows);
  t.rows = imin(t.rows, p.m - t.row0);
  t.n0 = nt * kG2TileN;
  t.k0 = 0;
  return t;
}

template <int kRows = kG2TileRows>
__device__ __forceinline__ TileCoord decode_tgmm_tile256(const GemmArgs& p, int tile) {
  const int per_group = p.k_tiles * p.n_tiles;
  const int gi = tile / per_group;
  const int rem = tile - gi * per_group;
  // Column tiles are taken in bands of kG2TgmmBand: consecutive tiles (= CTAs running at the same
  // time) walk all k tiles of one band before the next band, so a wave of CTAs shares about
  // k_tiles + band operand panels instead of n_tiles + a few.
  const int band_tiles = p.k_tiles * kG2TgmmBand;
  const int band = rem / band_tiles;
  const int in_band = rem - band * band_tiles;
  const int width = imin(kG2TgmmBand, p.n_tiles - band * kG2TgmmBand);
  const int kt = in_band / width;
  const int nt = band * kG2TgmmBand + (in_band - kt * width);
  TileCoord t;
  t.group = gi;
  t.weight = gi;
  t.row0 = p.group_offsets[gi];
  t.rows = imax(imin(imax(p.group_sizes[gi], 0), p.m - t.row0), 0);
  t.n0 = nt * kG2TileN;
  t.k0 = kt * kRows;
  return t;
}

// kVariant selects a second instantiation of either product, kept apart from the plain one because
// this kernel's main loop is sensitive to code generation (merely routing the tile loops through
// `cta_index` / `gemm_ctas` variables cost the plain kernel 3-5 %):
//   gmm:  the expert-parallel variant (ready flags in the loader, sender CTAs in the grid);
//   tgmm: strided segments (a block contracts over several row ranges, rd_tgmm_strided).
template <bool kBKMajor, bool kTgmm, bool kVariant = false, bool kPair = false>
__global__ void __launch_bounds__(kG2Threads, 1)
ragged_gemm2_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_out, const GemmArgs p) {
  static_assert(!(kTgmm && kBKMajor), "tgmm reads both operands MN-major");
  static_assert(!kPair || (kTgmm && !kVariant), "CTA pairs: plain tgmm only");
  constexpr bool kEp = !kTgmm && kVariant;
  constexpr bool kSeg = kTgmm && kVariant;
  constexpr int kCtas = kPair ? 2 : 1;
  constexpr int BN = kG2TileN;
  constexpr int kBCols = BN / kCtas;  // B-operand columns this CTA loads
  constexpr int kStages = kPair ? kG2PairStages : kG2Stages;
  constexpr uint32_t kHalfABytes = kTileM * kTileK * 2;  // 16 KB
  constexpr uint32_t kBBytes = kBCols * kTileK * 2;
  constexpr uint32_t kStageBytes = kG2ABytes + kBBytes;  // 64 KB, 48 KB in a pair
  constexpr uint32_t kTmemCols = 2 * BN;                 // accumulator of half h at column h * BN
  constexpr int kCtaRows = 2 * kTileM;                   // output rows of one CTA (both halves)

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_acc_full[2];   // per half
  __shared__ __align__(8) uint64_t bar_acc_empty[2];  // per half (pair: the leader's is used)
  __shared__ __align__(8) uint64_t bar_tail_go;    // MMA thread -> fixer warp(s): a stage with tail rows has landed
  __shared__ __align__(8) uint64_t bar_tail_done;  // fixer warp(s) -> MMA thread: its tail rows are cleared
  __shared__ uint32_t tmem_slot;
  __shared__ WaitCtl wait_ctl;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t stage_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int cta_rank = kPair ? static_cast<int>(cluster_cta_rank()) : 0;
  const bool leader = cta_rank == 0;

  // Fused expert-parallel exchange: some CTAs of the grid send rows instead of multiplying.
  // The senders are the FIRST CTAs of the grid, so they are resident before any CTA that may wait
  // for another GPU's senders.
  int sender_ctas = 0;
  if constexpr (kEp) {
    sender_ctas = p.send.world > 0 ? p.send.sender_ctas : 0;
    if (static_cast<int>(blockIdx.x) < sender_ctas) {
      ep_sender_role(p.send, p.ready_epoch, static_cast<int>(blockIdx.x), stage_base, &wait_ctl, p.wait_limit_us,
                     p.status);
      return;
    }
  }

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
    for (int h = 0; h < 2; ++h) {
      mbar_init(smem_u32(&bar_acc_full[h]), 1);
      mbar_init(smem_u32(&bar_acc_empty[h]), 4 * kCtas);  // the four epilogue warps of that half (per CTA)
    }
    mbar_init(smem_u32(&bar_tail_go), 1);
    mbar_init(smem_u32(&bar_tail_done), kCtas);  // one arrival per CTA's fixer warp (pair: the leader's is used)
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<kCtas>(smem_u32(&tmem_slot), kTmemCols);
    tmem_relinquish<kCtas>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) cluster_sync();  // the peer's barriers exist before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  volatile WaitCtl* abort_ptr = &wait_ctl;

  const int num_tiles =
      kTgmm ? p.g * p.k_tiles * p.n_tiles : imin(p.totals[0], p.max_m_tiles) * p.n_tiles;
  const int k_blocks_gmm = (p.k + kTileK - 1) / kTileK;
  const int tile_step = kPair ? static_cast<int>(gridDim.x >> 1)
                        : kEp ? static_cast<int>(gridDim.x) - sender_ctas : static_cast<int>(gridDim.x);
  auto first_tile = [&]() -> int {
    if constexpr (kPair) return static_cast<int>(blockIdx.x >> 1);
    if constexpr (kEp) return static_cast<int>(blockIdx.x) - sender_ctas;
    return static_cast<int>(blockIdx.x);
  };
  auto decode = [&](int tile) -> TileCoord {
    if constexpr (kPair) return decode_tgmm_tile256<2 * kG2TileRows>(p, tile);
    if constexpr (kTgmm) return decode_tgmm_tile256(p, tile);
    return decode_gmm_tile256(p, tile);
  };

  // Number of halves of a tile that exist.
  auto halves_of = [&](const TileCoord& t) -> int {
    if (kTgmm) return (t.k0 + kTileM < p.k) ? 2 : 1;
    return t.rows > kTileM ? 2 : 1;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      const uint64_t keep = l2_policy_evict_last();
      int ready_slot = -1;  // last ready flag this producer has seen set
      uint64_t waited_ns = 0;
      const uint64_t t_start = kEp ? global_timer_ns() : 0;
      for (int tile = first_tile(); tile < num_tiles && ok; tile += tile_step) {
        const TileCoord t = decode(tile);
        const int halves = halves_of(t);
        const int kb_count = kTgmm ? tgmm_block_count<kSeg>(p, t) : k_blocks_gmm;
        RowBlocks blocks = first_block(t);
        if (kEp && p.ready_flags != nullptr) {
          const int slot = t.group / p.groups_per_flag;
          if (slot != ready_slot) {
            const uint64_t w0 = global_timer_ns();
            if (!wait_flag_ge(p.ready_flags + slot, p.ready_epoch, abort_ptr)) {
              ok = false;
              break;
            }
            waited_ns += global_timer_ns() - w0;
            ready_slot = slot;
          }
        }
        for (int kb = 0; kb < kb_count; ++kb, ++it) {
          const uint32_t s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_ptr)) {
            ok = false;
            break;
          }
          uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t sa = stage_base + s * kStageBytes;
          const uint32_t sb = sa + kG2ABytes;
          const uint32_t own_bytes = halves * kHalfABytes + kBBytes;
          if constexpr (kPair) {
            // The peer's bytes are counted on the leader's barrier, except for the stage whose tail
            // rows the peer has to clear first (it then needs to see its own data land).
            const bool local_stage = kb == kb_count - 1 && tail_needs_clearing(t.rows);
            int r, live;
            tgmm_block<false>(p, t, blocks, kb, r, live);
            const int ka = t.k0 + cta_rank * kCtaRows;
            const int nb = t.n0 + cta_rank * kBCols;
            const uint32_t bytes = p.blocked_maps ? kStageBytes : own_bytes;  // a blocked A box always has both halves
            if (leader || local_stage) {
              mbar_arrive_expect_tx(full, (leader && !local_stage) ? 2 * bytes : bytes);
              if (p.blocked_maps) {
                tma_load_3d_hint(sa, &tmap_a, full, 0, r, ka >> 6, keep);
                tma_load_3d_hint(sb, &tmap_b, full, 0, r, nb >> 6, keep);
              } else {
                for (int h = 0; h < halves; ++h) {
                  tma_load_2d_hint(sa + h * kHalfABytes, &tmap_a, full, ka + h * kTileM, r, keep);
                  tma_load_2d_hint(sa + h * kHalfABytes + kBoxBytes, &tmap_a, full, ka + h * kTileM + 64, r, keep);
                }
#pragma unroll
                for (int j = 0; j < kBCols / 64; ++j)
                  tma_load_2d_hint(sb + j * kBoxBytes, &tmap_b, full, nb + j * 64, r, keep);
              }
            } else {
              full = map_to_cta(full, 0);
              if (p.blocked_maps) {
                tma_load_3d_pair_hint(sa, &tmap_a, full, 0, r, ka >> 6, keep);
                tma_load_3d_pair_hint(sb, &tmap_b, full, 0, r, nb >> 6, keep);
              } else {
                for (int h = 0; h < halves; ++h) {
                  tma_load_2d_pair_hint(sa + h * kHalfABytes, &tmap_a, full, ka + h * kTileM, r, keep);
                  tma_load_2d_pair_hint(sa + h * kHalfABytes + kBoxBytes, &tmap_a, full, ka + h * kTileM + 64, r, keep);
                }
#pragma unroll
                for (int j = 0; j < kBCols / 64; ++j)
                  tma_load_2d_pair_hint(sb + j * kBoxBytes, &tmap_b, full, nb + j * 64, r, keep);
              }
            }
            continue;
          }
          if (kTgmm) {
            int r, live;
            tgmm_block<kSeg>(p, t, blocks, kb, r, live);
            if (p.blocked_maps) {  // one box per operand; the A box always has both halves
              mbar_arrive_expect_tx(full, kStageBytes);
              tma_load_3d_hint(sa, &tmap_a, full, 0, r, t.k0 >> 6, keep);
              tma_load_3d_hint(sb, &tmap_b, full, 0, r, t.n0 >> 6, keep);
              continue;
            }
            mbar_arrive_expect_tx(full, own_bytes);
            for (int h = 0; h < halves; ++h) {
              tma_load_2d_hint(sa + h * kHalfABytes, &tmap_a, full, t.k0 + h * kTileM, r, keep);
              tma_load_2d_hint(sa + h * kHalfABytes + kBoxBytes, &tmap_a, full, t.k0 + h * kTileM + 64, r, keep);
            }
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d_hint(sb + j * kBoxBytes, &tmap_b, full, t.n0 + j * 64, r, keep);
          } else {
            mbar_arrive_expect_tx(full, own_bytes);
            for (int h = 0; h < halves; ++h)
              tma_load_2d(sa + h * kHalfABytes, &tmap_a, full, kb * kTileK, t.row0 + h * kTileM);
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
      if (kEp) {
        // status[2]: longest total wait of a loader for remote rows; status[3]: longest loader
        // lifetime (microseconds).  Read back by the expert-parallel harness.
        atomicMax(p.status + 2, static_cast<int32_t>(waited_ns / 1000ull));
        atomicMax(p.status + 3, static_cast<int32_t>((global_timer_ns() - t_start) / 1000ull));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // ONE thread runs the whole loop (in a pair: of the leader CTA).  The loop sits on the ring's
    // critical path -- a stage can be refilled only after its MMAs, and they only start after
    // this thread has seen the stage land -- and warp-wide steps are expensive there (a
    // __syncwarp costs about 160 clocks on B200, a stage's MMAs take 1024).  The one warp-wide
    // job, clearing the rows past a group's end in a tgmm stage, belongs to the fixer warp.
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc_f16(p.ab_format, kTgmm ? 1 : 0, kBKMajor ? 0 : 1, kTileM * kCtas, BN);
      constexpr uint32_t kAStep = (kTgmm ? 2048u : 32u) >> 4;
      constexpr uint32_t kBStep = (kBKMajor ? 32u : 2048u) >> 4;
      const uint64_t adesc0 = kTgmm ? make_smem_desc(stage_base, kBoxBytes, 1024)
                                    : make_smem_desc(stage_base, 16, 1024);
      const uint64_t bdesc0 = kBKMajor ? make_smem_desc(stage_base + kG2ABytes, 16, 1024)
                                       : make_smem_desc(stage_base + kG2ABytes, kBoxBytes, 1024);
      const uint32_t adesc0_lo = static_cast<uint32_t>(adesc0);
      const uint32_t bdesc0_lo = static_cast<uint32_t>(bdesc0);
      const uint32_t desc_hi = static_cast<uint32_t>(adesc0 >> 32);
      uint32_t it = 0;
      uint32_t uses[2] = {0u, 0u};  // how often each half's accumulator has been used
      uint32_t tail_events = 0;     // stages handed to the fixer warp so far
      bool ok = true;
      for (int tile = first_tile(); tile < num_tiles && ok; tile += tile_step) {
        const TileCoord t = decode(tile);
        const int halves = halves_of(t);
        const int kb_count = kTgmm ? tgmm_block_count<kSeg>(p, t) : k_blocks_gmm;
        RowBlocks blocks = first_block(t);
        const bool tail_stage = kTgmm && kb_count > 0 && tail_needs_clearing(t.rows);

        if (kb_count == 0) {  // tgmm, empty group: the epilogue writes zeros, nothing to compute
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (h < halves) {
              if (!mbar_wait(smem_u32(&bar_acc_empty[h]), (uses[h] & 1u) ^ 1u, abort_ptr)) {
                ok = false;
                break;
              }
              ++uses[h];
              mbar_arrive(smem_u32(&bar_acc_full[h]));
              if constexpr (kPair) mbar_arrive_cluster(smem_u32(&bar_acc_full[h]), 1);
            }
          }
          continue;
        }

        uint32_t s = it % kStages;
        uint32_t ph = (it / kStages) & 1u;
        for (int kb = 0; kb < kb_count; ++kb, ++it, s = (s + 1 == kStages ? 0 : s + 1), ph ^= (s == 0)) {
          if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_ptr)) {
            ok = false;
            break;
          }
          int live = kTileK;
          if (kTgmm) {
            int r;
            tgmm_block<kSeg>(p, t, blocks, kb, r, live);
          }
          const int n_mma = live >= kTileK ? kTileK / kUmmaK : (live + kUmmaK - 1) / kUmmaK;
          if (kTgmm && (kSeg ? block_needs_clearing(live) : (tail_stage && kb == kb_count - 1))) {
            // Rows past the end of the group belong to the next group (or to nobody): the fixer
            // warp (of either CTA in a pair) clears them before the MMAs read the stage.
            mbar_arrive(smem_u32(&bar_tail_go));
            if constexpr (kPair) mbar_arrive_cluster(smem_u32(&bar_tail_go), 1);
            if (!mbar_wait<kPair>(smem_u32(&bar_tail_done), tail_events & 1u, abort_ptr)) {
              ok = false;
              break;
            }
            ++tail_events;
          }
          const bool last = kb == kb_count - 1;
          const uint32_t b_lo = bdesc0_lo + s * (kStageBytes >> 4);
          tc_fence_after_sync();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (h < halves) {
              if (kb == 0) {  // the half's accumulator must have been drained by the epilogue
                if (!mbar_wait(smem_u32(&bar_acc_empty[h]), (uses[h] & 1u) ^ 1u, abort_ptr)) {
                  ok = false;
                  break;
                }
                ++uses[h];
                tc_fence_after_sync();
              }
              const uint32_t tmem_d = tmem_base + h * BN;
              const uint32_t a_lo = adesc0_lo + s * (kStageBytes >> 4) + h * (kHalfABytes >> 4);
              if (kTgmm && n_mma < kTileK / kUmmaK) {
                for (int kk = 0; kk < n_mma; ++kk) {
                  umma_f16<kCtas>(tmem_d, make_desc64(a_lo + kk * kAStep, desc_hi),
                                  make_desc64(b_lo + kk * kBStep, desc_hi), idesc,
                                  (kb > 0 || kk > 0) ? 1u : 0u);
                }
              } else {
                umma_f16<kCtas>(tmem_d, make_desc64(a_lo, desc_hi), make_desc64(b_lo, desc_hi), idesc,
                                kb > 0 ? 1u : 0u);
#pragma unroll
                for (int kk = 1; kk < kTileK / kUmmaK; ++kk) {
                  umma_f16<kCtas>(tmem_d, make_desc64(a_lo + kk * kAStep, desc_hi),
                                  make_desc64(b_lo + kk * kBStep, desc_hi), idesc, 1u);
                }
              }
              if (last) {  // this half is complete
                if constexpr (kPair) {
                  umma_commit_pair(smem_u32(&bar_acc_full[h]), 0x3);
                } else {
                  umma_commit(smem_u32(&bar_acc_full[h]));
                }
              }
            }
          }
          if (!ok) break;
          // both halves have read the stage (in both CTAs of a pair)
          if constexpr (kPair) {
            umma_commit_pair(smem_u32(&bar_empty[s]), 0x3);
          } else {
            umma_commit(smem_u32(&bar_empty[s]));
          }
        }
      }
    }
  } else if (warp == kG2FixerWarp) {
    // ------------------------------------------------------------ tail fixer (tgmm)
    // Walks the tiles like the MMA thread and, for every stage whose last 16-deep MMA reaches past
    // the end of its group, waits for the MMA thread's go (the stage has landed), clears those
    // rows in every box of the stage in THIS CTA's shared memory and reports back.
    if constexpr (kTgmm) {
      uint32_t it = 0;
      uint32_t events = 0;
      uint32_t own_parity = 0;  // peer of a pair, bit s: parity of the next landing on its own barrier of slot s
      bool ok = true;
      for (int tile = first_tile(); tile < num_tiles && ok; tile += tile_step) {
        const TileCoord t = decode(tile);
        const int kb_count = tgmm_block_count<kSeg>(p, t);
        RowBlocks blocks = first_block(t);
        const bool tail_stage = kb_count > 0 && tail_needs_clearing(t.rows);
        for (int kb = kSeg ? 0 : imax(kb_count - 1, 0); kb < kb_count; ++kb) {
          int r, live;
          tgmm_block<kSeg>(p, t, blocks, kb, r, live);
          if (!(kSeg ? block_needs_clearing(live) : tail_stage)) continue;
          const uint32_t s = (it + kb) % kStages;
          if (!mbar_wait<kPair>(smem_u32(&bar_tail_go), events & 1u, abort_ptr)) {
            ok = false;
            break;
          }
          if constexpr (kPair) {
            // The peer's bytes of such a stage are counted on its own barrier of that slot (see
            // the producer), which is used for nothing else.
            if (!leader) {
              const uint32_t par = (own_parity >> s) & 1u;
              own_parity ^= 1u << s;
              if (!mbar_wait(smem_u32(&bar_full[s]), par, abort_ptr)) {
                ok = false;
                break;
              }
            }
          }
          ++events;
          clear_tail_rows<kStageBytes / kBoxBytes>(stage_base + s * kStageBytes, live, lane);
          __syncwarp();
          if (lane == 0) {
            if constexpr (kPair) {
              mbar_arrive_cluster(smem_u32(&bar_tail_done), 0);
            } else {
              mbar_arrive(smem_u32(&bar_tail_done));
            }
          }
        }
        it += kb_count;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9)
    // Warps 2..5 drain half 0, warps 6..9 half 1; within a half a warp owns the 32 TMEM lanes
    // of its quarter (warp index mod 4).
    const int half = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int r_in_tile = cta_rank * kCtaRows + half * kTileM + quarter * 32 + lane;
    const uint32_t buf = stage_base + kStages * kStageBytes + (warp - 2) * kOutBoxBytes;
    uint32_t uses = 0;
    bool ok = true;
    const uint64_t stream_out = l2_policy_evict_first();
    uint16_t* out16 = reinterpret_cast<uint16_t*>(p.out);
    for (int tile = first_tile(); tile < num_tiles && ok; tile += tile_step) {
      const TileCoord t = decode(tile);
      if (half >= halves_of(t)) continue;  // this half does not exist in this tile
      const int n0 = t.n0;
      if (!mbar_wait(smem_u32(&bar_acc_full[half]), uses & 1u, abort_ptr)) {
        ok = false;
        break;
      }
      ++uses;
      tc_fence_after_sync();

      bool row_ok, warp_has_rows, slab_by_tma, zero_only = false;
      size_t row_off;
      int out_row0;
      const int slab0 = cta_rank * kCtaRows + half * kTileM + quarter * 32;  // first tile row of this warp's slab
      if (kTgmm) {
        const int kr = t.k0 + r_in_tile;
        out_row0 = t.k0 + slab0;
        row_ok = kr < p.k;
        warp_has_rows = out_row0 < p.k;
        slab_by_tma = true;
        row_off = (static_cast<size_t>(t.group) * p.k + kr) * static_cast<size_t>(p.n);
        zero_only = kSeg ? tgmm_block_count<kSeg>(p, t) == 0 : t.rows <= 0;
      } else {
        out_row0 = t.row0 + slab0;
        row_ok = r_in_tile < t.rows;
        warp_has_rows = slab0 < t.rows;
        slab_by_tma = slab0 + 32 <= t.rows;
        row_off = static_cast<size_t>(t.row0 + r_in_tile) * static_cast<size_t>(p.n);
      }

      const int n_chunks = warp_has_rows ? imin(BN / 64, (p.n - n0 + 63) / 64) : 0;
      const uint32_t acc_empty_bar = smem_u32(&bar_acc_empty[half]);
      // First the whole accumulator slab leaves TMEM (packed to 16 bits, 32 registers per 64
      // columns) and the half is handed back to the MMA warp; only chunk 0 is stored on the way,
      // so that its TMA store runs under the remaining loads.  The other chunks are stored after
      // the hand-back: the waits for the staging buffer no longer hold up the next tile's MMAs.
      uint4 o[BN / 64][8];
      auto load_chunk = [&](int c) {
        uint32_t v[64];
        if (!zero_only) {
          const uint32_t taddr =
              tmem_base + half * BN + c * 64 + (static_cast<uint32_t>(quarter * 32) << 16);
          tmem_ld_32x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
          tmem_ld_32x32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 64; ++j) v[j] = 0u;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          o[c][q].x = pack2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]), p.ab_format);
          o[c][q].y = pack2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]), p.ab_format);
          o[c][q].z = pack2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]), p.ab_format);
          o[c][q].w = pack2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]), p.ab_format);
        }
      };
      auto store_chunk = [&](int c) {
        const int col = n0 + c * 64;
        if (slab_by_tma) {
          if (lane == 0) bulk_wait_group_read<0>();  // the previous box has left this buffer
          __syncwarp();
          const uint32_t row_addr = buf + lane * 128;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t a = row_addr + (((q ^ (lane & 7)) & 7) << 4);  // 128-byte swizzle
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(o[c][q].x),
                         "r"(o[c][q].y), "r"(o[c][q].z), "r"(o[c][q].w)
                         : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (kTgmm) {
              tma_store_3d_hint(&tmap_out, buf, col, out_row0, t.group, stream_out);
            } else {
              tma_store_2d(&tmap_out, buf, col, out_row0);
            }
            bulk_commit_group();
          }
        } else if (row_ok) {
          uint16_t* dst = out16 + row_off + col;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (col + q * 8 < p.n) *reinterpret_cast<uint4*>(dst + q * 8) = o[c][q];
          }
        }
      };
#pragma unroll
      for (int c = 0; c < BN / 64; ++c) {
        if (c < n_chunks) {
          load_chunk(c);
          if (c == 0) store_chunk(0);
        }
      }
      if (n_chunks > 0) {  // the accumulator is in registers: hand it back
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kPair) {
            mbar_arrive_cluster(acc_empty_bar, 0);
          } else {
            mbar_arrive(acc_empty_bar);
          }
        }
      }
#pragma unroll
      for (int c = 1; c < BN / 64; ++c) {
        if (c < n_chunks) store_chunk(c);
      }
      if (n_chunks == 0) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kPair) {
            mbar_arrive_cluster(acc_empty_bar, 0);
          } else {
            mbar_arrive(acc_empty_bar);
          }
        }
      }
    }
    if (lane == 0) bulk_wait_group<0>();
    __syncwarp();

    if (!kTgmm && p.zero_tail) {
      // Rows past sum(group_sizes) belong to no group and are defined as zero.
      constexpr int kEpiThreads = 32 * kG2EpilogueWarps;
      const int first = imin(imax(p.totals[1], 0), p.m);
      const size_t chunks_per_row = static_cast<size_t>(p.n) / 8;
      const size_t total = static_cast<size_t>(p.m - first) * chunks_per_row;
      const size_t tid = static_cast<size_t>(kEp ? blockIdx.x - sender_ctas : blockIdx.x) * kEpiThreads +
                         (threadIdx.x - 64);
      const size_t stride = static_cast<size_t>(kEp ? gridDim.x - sender_ctas : gridDim.x) * kEpiThreads;
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
  // Neither CTA of a pair may leave while the other can still reach its barriers or smem.
  if constexpr (kPair) cluster_sync();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<kCtas>(tmem_base, kTmemCols);
  }
}

}  // namespace rd
