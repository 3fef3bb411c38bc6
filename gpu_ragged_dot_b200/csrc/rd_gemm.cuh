// Grouped ("ragged") GEMM kernels for sm_100a.
//
//   gmm  : y[rows of group i, :] = x[rows of group i, :] @ W[i]        (reference
//          gpu_ragged_dot.py:93-165; W[i] is [k,n], or [n,k] with trans_rhs)
//   tgmm : out[i] = x[rows of group i, :]^T @ dout[rows of group i, :]   (reference :231-281)
//
// One persistent, warp-specialised CTA per SM:
//   warp 0      TMA producer   -- one thread: cp.async.bulk.tensor tiles into a kStages-deep smem ring
//   warp 1      MMA issuer     -- one thread: tcgen05.mma (K=16) into one of two TMEM accumulators
//   warp 6      tail fixer     -- tgmm: clears the rows past a group's end in a stage
//   warps 2..5  epilogue       -- tcgen05.ld, fp32 -> bf16/fp16, staged through swizzled smem and
//                                 written with TMA stores ([32 rows][64 cols] boxes, clipped at the
//                                 tensor's edges); a gmm slab that crosses the end of its group
//                                 is written with row-masked 16-byte stores instead
// The two TMEM accumulators let the epilogue of tile t overlap the main loop of tile t+1.
//
// kCtas == 1: each CTA owns a 128 x BN output tile (tcgen05.mma.cta_group::1, M=128).
// kCtas == 2: two CTAs of a cluster own a 256 x BN tile (cta_group::2, M=256).  Each CTA loads
//             its own 128 rows of the A operand and HALF of the B operand's BN columns; the
//             leader CTA (cluster rank 0) issues the MMAs, which read B from both CTAs' shared
//             memory.  Per SM this cuts the shared-memory fill per flop by a third, which is
//             what bounds the 1-CTA kernel.  Every CTA loads only its own tiles (nothing is
//             broadcast); the peer's loads count their bytes on the LEADER's "full" barrier
//             (cta_group::2 TMA form), so the leader sees one barrier per stage, and
//             tcgen05.commit frees the stage in both CTAs.  The one stage per tgmm tile whose
//             tail rows must be cleared goes through a slower hand-shake (the peer's bytes
//             land on its own barrier, either CTA's fixer warp clears its rows and arrives on
//             the leader's tail_done barrier).
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

#include "rd_ep_send.cuh"
#include "rd_metadata.cuh"
#include "rd_ptx.cuh"

namespace rd {

constexpr int kTileM = 128;  // UMMA M per CTA == output rows per CTA tile
constexpr int kTileK = 64;   // elements per 128-byte swizzle row == contraction depth per stage
constexpr int kUmmaK = 16;   // contraction depth of one tcgen05.mma for 16-bit inputs
constexpr int kBoxBytes = 64 * 128;  // one [64 rows][128 B] TMA box
constexpr int kGemmThreads = 192;       // TMA warp, MMA warp, four epilogue warps
constexpr int kGemmFixerWarp = 6;       // ragged_gemm_kernel only: clears tail rows of tgmm stages
constexpr int kGemmFixerThreads = kGemmThreads + 32;
constexpr int kOutBoxBytes = 32 * 128;                  // one [32 rows][64 cols] output box
constexpr int kOutStagingBytes = 4 * 2 * kOutBoxBytes;  // 4 epilogue warps x 2 buffers

enum DeviceStatus : int32_t {
  kStatusOk = 0,
  kStatusWaitExpired = 1,  // a bounded mbarrier wait gave up
};

struct GemmArgs {
  int m, k, n, g;   // gmm: x[m,k] . W[g] -> y[m,n]      tgmm: x[m,k], dout[m,n] -> out[g,k,n]
  int n_tiles;      // ceil(n / BN)
  // tgmm over strided segments (seg_count > 1): output block i contracts over the rows of the
  // groups i, i + seg_stride, ..., i + (seg_count - 1) * seg_stride of group_sizes, one after
  // the other; g is then the number of output blocks.  seg_count <= 1: block i = group i.
  int seg_count, seg_stride;
  int k_tiles;      // tgmm: tiles along the output's k axis (128 * kCtas rows each); gmm: unused
  int max_m_tiles;  // static upper bound on live row tiles (gmm)
  int ab_format;    // 0 = fp16, 1 = bf16
  int zero_tail;    // gmm: write zeros to the rows past sum(group_sizes)
  // tgmm on 256-row tiles: the operand maps are "column-blocked" views (64 columns, rows, blocks
  // of 64 columns), so that ONE box fetches all the 64-column slabs an operand has in a stage.
  int blocked_maps;
  uint32_t wait_limit_us;  // how long a bounded wait inside the kernel may last (microseconds)
  const float* weight_scale;  // 8-bit inputs: scale of weight matrix w, applied to the accumulator (null: 1)
  const int32_t* group_sizes;
  const int32_t* group_offsets;
  const TileRecord* tile_rec;  // gmm: one record per live row tile (of 128 * kCtas rows)
  const int32_t* totals;       // {live row tiles, min(sum(group_sizes), m)}
  int32_t* status;
  void* out;
  // gmm, optional: rows of group i may be read once ready_flags[i / groups_per_flag] >=
  // ready_epoch (the rows are being written by other kernels, possibly on other GPUs, while
  // this kernel runs).  Null: all rows are there at launch.
  const int32_t* ready_flags;
  int groups_per_flag;
  int ready_epoch;
  // gmm on one CTA per tile, optional (send.world > 0): the first send.sender_ctas CTAs of the
  // grid run the expert-parallel sender role (rd_ep_send.cuh) instead of multiplying.
  EpSendArgs send;
};

// Coordinates of one CTA's share of a tile.
struct TileCoord {
  int group;   // group index
  int weight;  // gmm: index of the weight matrix this group multiplies by
  int row0;    // gmm: first row of x / y for this CTA;  tgmm: first row of the group
  int rows;    // gmm: valid rows for this CTA (<=128, may be <= 0);  tgmm: rows of the group
  int n0;      // first output column of the tile
  int k0;      // tgmm: first row of out[group] written by this CTA
};

__device__ __forceinline__ int imin(int a, int b) { return a < b ? a : b; }
__device__ __forceinline__ int imax(int a, int b) { return a > b ? a : b; }

// gmm tile order: group-major; inside a group the n-tiles are outer and the group's row
// tiles inner, so CTAs running concurrently share one [k, BN] weight panel through L2 and an
// expert's weights stream from HBM once.  One 32-byte record load per tile, no dependent loads.
template <int BN, int kCtas>
__device__ __forceinline__ TileCoord decode_gmm_tile(const GemmArgs& p, int tile, int cta_rank) {
  constexpr int kRows = kTileM * kCtas;
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
  t.row0 = a.z + mi * kRows + cta_rank * kTileM;
  t.rows = imin(kTileM, a.w - mi * kRows - cta_rank * kTileM);
  t.rows = imin(t.rows, p.m - t.row0);  // never touch rows past m
  t.n0 = nt * BN;
  t.k0 = 0;
  return t;
}

template <int BN, int kCtas>
__device__ __forceinline__ TileCoord decode_tgmm_tile(const GemmArgs& p, int tile, int cta_rank) {
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
  t.n0 = nt * BN;
  t.k0 = (kt * kCtas + cta_rank) * kTileM;
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

// tgmm: does the group's last 64-row stage need rows cleared before its MMAs (rows past the end
// of the group that fall inside the last 16-deep MMA issued)?
__device__ __forceinline__ bool tail_needs_clearing(int group_rows) {
  const int live = group_rows % kTileK;
  return live != 0 && (live % kUmmaK) != 0;
}

// tgmm: the 64-row blocks one output block contracts over.  A block never crosses the end of a
// segment (a group of group_sizes); its rows past the segment's end are cleared or skipped by
// the fixer warp and the MMA thread.  Plain tgmm has one segment per output block, the rows of group t.group.
struct RowBlocks {
  int q;     // segments opened so far
  int row;   // first row of the next block
  int left;  // rows of the current segment from `row` on
};

__device__ __forceinline__ void segment_rows(const GemmArgs& p, int group, int& row0, int& rows) {
  row0 = p.group_offsets[group];
  rows = imax(imin(imax(p.group_sizes[group], 0), p.m - row0), 0);
}

template <bool kSeg>
__device__ __forceinline__ int tgmm_block_count(const GemmArgs& p, const TileCoord& t) {
  if constexpr (!kSeg) return (t.rows + kTileK - 1) / kTileK;
  int blocks = 0;
  for (int q = 0; q < p.seg_count; ++q) {
    int row0, rows;
    segment_rows(p, t.group + q * p.seg_stride, row0, rows);
    blocks += (rows + kTileK - 1) / kTileK;
  }
  return blocks;
}

__device__ __forceinline__ RowBlocks first_block(const TileCoord& t) {
  RowBlocks it;
  it.q = 1;
  it.row = t.row0;
  it.left = t.rows;
  return it;
}

// First row and live rows (1..64) of the next block.  Call at most tgmm_block_count() times.
__device__ __forceinline__ void next_block(const GemmArgs& p, const TileCoord& t, RowBlocks& it, int& row,
                                           int& live) {
  while (it.left <= 0 && it.q < p.seg_count) {
    segment_rows(p, t.group + it.q * p.seg_stride, it.row, it.left);
    ++it.q;
  }
  row = it.row;
  live = imin(it.left, kTileK);
  it.row += kTileK;
  it.left -= kTileK;
}

// Does a block with `live` rows need rows cleared before its MMAs?
__device__ __forceinline__ bool block_needs_clearing(int live) {
  return live < kTileK && (live % kUmmaK) != 0;
}

// First row and live rows of block kb of a tile.  Plain tgmm (kSeg false) computes them from the
// group's row range, as cheaply as can be: this sits in the producer's and the MMA thread's loops.
template <bool kSeg>
__device__ __forceinline__ void tgmm_block(const GemmArgs& p, const TileCoord& t, RowBlocks& it, int kb,
                                           int& row, int& live) {
  if constexpr (kSeg) {
    next_block(p, t, it, row, live);
  } else {
    row = t.row0 + kb * kTileK;
    live = t.rows - kb * kTileK;
  }
}

// Zero rows [live, end of the last 16-deep MMA) of every [64 rows][128 B] box of one stage and
// make the writes visible to the tensor core (async proxy).  Whole warp.
template <int kBoxes>
__device__ __forceinline__ void clear_tail_rows(uint32_t stage_addr, int live, int lane) {
  const int n_mma = (live + kUmmaK - 1) / kUmmaK;
  const int dead = n_mma * kUmmaK - live;  // 0..15 rows
  if (dead <= 0) return;
  // Row r of a box is the 128 bytes at box + r * 128 (the swizzle only permutes 16-byte chunks
  // inside a row), so the dead rows of a box are one contiguous range of at most 1920 bytes:
  // four 512-byte warp stores per box, no index arithmetic in the loop.
  const int bytes = dead * 128;
  const uint32_t first = stage_addr + live * 128 + lane * 16;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (i * 512 + lane * 16 < bytes) {
#pragma unroll
      for (int box = 0; box < kBoxes; ++box) {
        const uint32_t addr = first + box * kBoxBytes + i * 512;
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
      }
    }
  }
  fence_proxy_async_smem();
}

// TMA load whose bytes are counted on this CTA's own barrier, or (remote_bar) on a barrier of
// the other CTA of the pair.
__device__ __forceinline__ void load_2d(bool remote_bar, uint32_t dst, const CUtensorMap* map,
                                        uint32_t bar, int c0, int c1) {
  if (remote_bar) {
    tma_load_2d_pair(dst, map, bar, c0, c1);
  } else {
    tma_load_2d(dst, map, bar, c0, c1);
  }
}
__device__ __forceinline__ void load_3d(bool remote_bar, uint32_t dst, const CUtensorMap* map,
                                        uint32_t bar, int c0, int c1, int c2) {
  if (remote_bar) {
    tma_load_3d_pair(dst, map, bar, c0, c1, c2);
  } else {
    tma_load_3d(dst, map, bar, c0, c1, c2);
  }
}

template <int BN, int kCtas>
constexpr int stage_bytes() {
  return kTileM * kTileK * 2 + (BN / kCtas) * kTileK * 2;
}

// kTgmm == false : gmm.   A operand = x tile, K-major.  B operand = W tile, K-major when
//                  kBKMajor (trans_rhs: W[g] is [n,k]) else MN-major (W[g] is [k,n]).
// kTgmm == true  : tgmm.  A operand = x^T tile (MN-major), B operand = dout tile (MN-major);
//                  kBKMajor must be false.
template <int BN, bool kBKMajor, int kStages, bool kTgmm, int kCtas, bool kSeg = false, bool kFp8 = false>
__global__ void __launch_bounds__(kGemmFixerThreads, 1)
ragged_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                   const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_out, const GemmArgs p) {
  static_assert(BN == 64 || BN == 128 || BN == 256, "BN must be 64, 128 or 256");
  static_assert(!(kTgmm && kBKMajor), "tgmm reads both operands MN-major");
  static_assert(kCtas == 1 || (kCtas == 2 && BN >= 128), "a CTA pair needs BN >= 128");
  static_assert(!kSeg || (kTgmm && kCtas == 1), "strided segments: tgmm on one CTA per tile");
  // 8-bit inputs (e4m3): both operands K-major (x[m,k], W[g,n,k]), so the tiles are byte for byte
  // those of a 16-bit problem with k/2 elements per row (which is what the tensor maps and
  // GemmArgs::k describe); only the MMA kind differs, 32 elements = 32 bytes per instruction, and
  // the epilogue multiplies by the weight matrix's scale.  Output is bf16.
  static_assert(!kFp8 || (kBKMajor && !kTgmm && kCtas == 1), "8-bit inputs: gmm with K-major weights, one CTA");
  constexpr bool kPair = kCtas == 2;
  constexpr int kBCols = BN / kCtas;  // B-operand columns this CTA loads
  constexpr uint32_t kABytes = kTileM * kTileK * 2;
  constexpr uint32_t kBBytes = kBCols * kTileK * 2;
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;  // two fp32 accumulators of BN columns

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) uint64_t bar_full[kStages];        // TMA data of this CTA landed
  __shared__ __align__(8) uint64_t bar_empty[kStages];       // MMAs reading the stage retired
  __shared__ __align__(8) uint64_t bar_tail_go;    // MMA thread -> fixer warp(s): a stage with tail rows has landed
  __shared__ __align__(8) uint64_t bar_tail_done;  // fixer warp(s) -> MMA thread (pair: the leader's is used)
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];  // leader only when paired
  __shared__ uint32_t tmem_slot;
  __shared__ WaitCtl wait_ctl;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta_rank = kPair ? static_cast<int>(cluster_cta_rank()) : 0;
  const bool leader = cta_rank == 0;
  const uint32_t stage_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;

  // Fused expert-parallel exchange: some CTAs of the grid send rows instead of multiplying.
  const int sender_ctas = (!kTgmm && !kPair && p.send.world > 0) ? p.send.sender_ctas : 0;
  const int gemm_ctas = static_cast<int>(gridDim.x) - sender_ctas;
  // The senders are the FIRST CTAs of the grid, so they are resident before any CTA that may wait
  // for another GPU's senders.
  if (static_cast<int>(blockIdx.x) < sender_ctas) {
    ep_sender_role(p.send, p.ready_epoch, static_cast<int>(blockIdx.x), stage_base, &wait_ctl, p.wait_limit_us,
                   p.status);
    return;
  }
  const int cta_index = static_cast<int>(blockIdx.x) - sender_ctas;  // among the multiplying CTAs

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
    mbar_init(smem_u32(&bar_tail_go), 1);
    mbar_init(smem_u32(&bar_tail_done), kCtas);  // one arrival per CTA's fixer warp
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bar_acc_full[a]), 1);
      mbar_init(smem_u32(&bar_acc_empty[a]), 4 * kCtas);  // one arrival per epilogue warp
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<kCtas>(smem_u32(&tmem_slot), kTmemCols);
    tmem_relinquish<kCtas>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (kPair) cluster_sync();  // the peer's barriers exist before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  volatile WaitCtl* abort_ptr = &wait_ctl;

  int num_tiles;
  if (kTgmm) {
    num_tiles = p.g * p.k_tiles * p.n_tiles;
  } else {
    num_tiles = imin(p.totals[0], p.max_m_tiles) * p.n_tiles;
  }
  const int tile_start = cta_index / kCtas;
  const int tile_step = gemm_ctas / kCtas;
  const int k_blocks_gmm = (p.k + kTileK - 1) / kTileK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int ready_slot = -1;  // last ready flag this producer has seen set
      for (int tile = tile_start; tile < num_tiles && ok; tile += tile_step) {
        const TileCoord t = kTgmm ? decode_tgmm_tile<BN, kCtas>(p, tile, cta_rank)
                                  : decode_gmm_tile<BN, kCtas>(p, tile, cta_rank);
        const int nb = t.n0 + cta_rank * kBCols;  // first B column this CTA loads
        const int kb_count = kTgmm ? tgmm_block_count<kSeg>(p, t) : k_blocks_gmm;
        RowBlocks blocks = first_block(t);
        if (!kTgmm && p.ready_flags != nullptr) {
          const int slot = t.group / p.groups_per_flag;
          if (slot != ready_slot) {
            if (!wait_flag_ge(p.ready_flags + slot, p.ready_epoch, abort_ptr)) {
              ok = false;
              break;
            }
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
          const uint32_t sb = sa + kABytes;
          // In a pair the peer's bytes are counted on the leader's barrier, except for a stage
          // whose tail rows the peer has to clear first (it then needs to see its own data land).
          const bool local_stage = !kPair || (kTgmm && kb == kb_count - 1 && tail_needs_clearing(t.rows));
          bool remote_bar = false;
          if (leader) {
            mbar_arrive_expect_tx(full, local_stage ? kStageBytes : 2 * kStageBytes);
          } else if (local_stage) {
            mbar_arrive_expect_tx(full, kStageBytes);
          } else {
            full = map_to_cta(full, 0);
            remote_bar = true;
          }
          if (kTgmm) {
            int r, live;
            tgmm_block<kSeg>(p, t, blocks, kb, r, live);
            load_2d(remote_bar, sa, &tmap_a, full, t.k0, r);
            load_2d(remote_bar, sa + kBoxBytes, &tmap_a, full, t.k0 + 64, r);
#pragma unroll
            for (int j = 0; j < kBCols / 64; ++j)
              load_2d(remote_bar, sb + j * kBoxBytes, &tmap_b, full, nb + j * 64, r);
          } else {
            load_2d(remote_bar, sa, &tmap_a, full, kb * kTileK, t.row0);
            if (kBKMajor) {
              load_3d(remote_bar, sb, &tmap_b, full, kb * kTileK, nb, t.weight);
            } else {
#pragma unroll
              for (int j = 0; j < kBCols / 64; ++j)
                load_3d(remote_bar, sb + j * kBoxBytes, &tmap_b, full, nb + j * 64, kb * kTileK,
                        t.weight);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // ONE thread runs the whole loop (in a pair: of the leader CTA): the loop sits on the ring's
    // critical path and warp-wide steps are expensive there (a __syncwarp costs about 160 clocks
    // on B200, the MMAs of a stage take 512).  The one warp-wide job, clearing the rows past a
    // group's end in a tgmm stage, belongs to the fixer warp.
    if (lane == 0 && leader) {
      const uint32_t idesc_full =
          make_idesc_f16(kFp8 ? 0 : p.ab_format, kTgmm ? 1 : 0, kBKMajor ? 0 : 1, kTileM * kCtas, BN);
      // A gmm row tile with at most 64 rows (the short last tile of a group, a small expert) is
      // multiplied with M = 64: half the tensor-core time for a tile that is mostly padding.
      // Its accumulator rows live in lanes 0-15 of each 32-lane quarter of tensor memory.
      const uint32_t idesc_half = make_idesc_f16(kFp8 ? 0 : p.ab_format, 0, kBKMajor ? 0 : 1, 64, BN);
      // Stage-0 operand descriptors; later stages / k-steps only add to the 16-byte-unit address.
      constexpr uint32_t kAStep = (kTgmm ? 2048u : 32u) >> 4;       // A: MN-major (tgmm) or K-major
      constexpr uint32_t kBStep = (kBKMajor ? 32u : 2048u) >> 4;    // B: K-major or MN-major
      const uint64_t adesc0 = kTgmm ? make_smem_desc(stage_base, kBoxBytes, 1024)
                                    : make_smem_desc(stage_base, 16, 1024);
      const uint64_t bdesc0 = kBKMajor ? make_smem_desc(stage_base + kABytes, 16, 1024)
                                       : make_smem_desc(stage_base + kABytes, kBoxBytes, 1024);
      const uint32_t adesc0_lo = static_cast<uint32_t>(adesc0);
      const uint32_t bdesc0_lo = static_cast<uint32_t>(bdesc0);
      const uint32_t desc_hi = static_cast<uint32_t>(adesc0 >> 32);  // same for A and B (SBO, version, swizzle)
      uint32_t it = 0;
      uint32_t local_tile = 0;
      uint32_t tail_events = 0;  // stages handed to the fixer warp so far
      bool ok = true;
      for (int tile = tile_start; tile < num_tiles && ok; tile += tile_step, ++local_tile) {
        const TileCoord t = kTgmm ? decode_tgmm_tile<BN, kCtas>(p, tile, cta_rank)
                                  : decode_gmm_tile<BN, kCtas>(p, tile, cta_rank);
        const int kb_count = kTgmm ? tgmm_block_count<kSeg>(p, t) : k_blocks_gmm;
        const bool tail_stage = kTgmm && kb_count > 0 && tail_needs_clearing(t.rows);
        RowBlocks blocks = first_block(t);
        const uint32_t idesc = (!kTgmm && !kPair && t.rows <= 64) ? idesc_half : idesc_full;

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
          // tgmm: contraction depth that is really there in this stage (the group's last rows);
          // whole 16-deep MMAs past it are skipped.  gmm always issues all four: columns past k
          // are zero-filled by TMA in both operands.
          int live = kTileK;
          if (kTgmm) {
            int r;
            tgmm_block<kSeg>(p, t, blocks, kb, r, live);
          }
          const int n_mma = live >= kTileK ? kTileK / kUmmaK : (live + kUmmaK - 1) / kUmmaK;
          if (kTgmm && (kSeg ? block_needs_clearing(live) : (tail_stage && kb == kb_count - 1))) {
            // Rows past the end of the group belong to the next group (or to nobody): the fixer
            // warp (of either CTA in a pair) clears them, up to the end of the last MMA that is
            // issued, in every box of this stage, so they add nothing to the reduction.  (In gmm
            // the columns past k are zero-filled by TMA.)
            mbar_arrive(smem_u32(&bar_tail_go));
            if constexpr (kPair) mbar_arrive_cluster(smem_u32(&bar_tail_go), 1);
            if (!mbar_wait<kPair>(smem_u32(&bar_tail_done), tail_events & 1u, abort_ptr)) {
              ok = false;
              break;
            }
            ++tail_events;
          }
          tc_fence_after_sync();
          // Descriptors are the stage-0 descriptors plus a stage / k-step offset added to their
          // address field, and only a tgmm tile's last stage looks at n_mma.
          const uint32_t a_lo = adesc0_lo + s * (kStageBytes >> 4);
          const uint32_t b_lo = bdesc0_lo + s * (kStageBytes >> 4);
          if (kTgmm && n_mma < kTileK / kUmmaK) {
            for (int kk = 0; kk < n_mma; ++kk) {
              umma_ab<kCtas, kFp8>(tmem_d, make_desc64(a_lo + kk * kAStep, desc_hi),
                                   make_desc64(b_lo + kk * kBStep, desc_hi), idesc,
                                   (kb > 0 || kk > 0) ? 1u : 0u);
            }
          } else {
            umma_ab<kCtas, kFp8>(tmem_d, make_desc64(a_lo, desc_hi), make_desc64(b_lo, desc_hi), idesc,
                                 kb > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < kTileK / kUmmaK; ++kk) {
              umma_ab<kCtas, kFp8>(tmem_d, make_desc64(a_lo + kk * kAStep, desc_hi),
                                   make_desc64(b_lo + kk * kBStep, desc_hi), idesc, 1u);
            }
          }
          // Frees the smem stage (in both CTAs of a pair) when these MMAs retire.
          if (kPair) {
            umma_commit_pair(smem_u32(&bar_empty[s]), 0x3);
          } else {
            umma_commit(smem_u32(&bar_empty[s]));
          }
        }
        if (!ok) break;
        const uint32_t bar = smem_u32(&bar_acc_full[acc]);
        if (kb_count > 0) {
          if (kPair) {
            umma_commit_pair(bar, 0x3);
          } else {
            umma_commit(bar);
          }
        } else {  // empty group: nothing to wait for
          mbar_arrive(bar);
          if (kPair) mbar_arrive_cluster(bar, 1);
        }
      }
    }
  } else if (warp == kGemmFixerWarp) {
    // ------------------------------------------------------------ tail fixer (tgmm)
    // Walks the tiles like the MMA thread and, for every stage whose last 16-deep MMA reaches past
    // the end of its group, waits for the MMA thread's go (the stage has landed), clears those
    // rows in every box of the stage in THIS CTA's shared memory and reports back.
    if constexpr (kTgmm) {
      uint32_t it = 0;
      uint32_t events = 0;
      uint32_t own_parity = 0;  // peer of a pair, bit s: parity of the next landing on its own barrier of slot s
      bool ok = true;
      for (int tile = tile_start; tile < num_tiles && ok; tile += tile_step) {
        const TileCoord t = decode_tgmm_tile<BN, kCtas>(p, tile, cta_rank);
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
          clear_tail_rows<(kABytes + kBBytes) / kBoxBytes>(stage_base + s * kStageBytes, live, lane);
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
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const int r_in_tile = quarter * 32 + lane;
    const uint32_t staging = stage_base + kStages * kStageBytes + (warp - 2) * 2 * kOutBoxBytes;
    uint32_t local_tile = 0;
    uint32_t boxes_stored = 0;
    bool ok = true;
    uint16_t* out16 = reinterpret_cast<uint16_t*>(p.out);
    for (int tile = tile_start; tile < num_tiles && ok; tile += tile_step, ++local_tile) {
      const TileCoord t = kTgmm ? decode_tgmm_tile<BN, kCtas>(p, tile, cta_rank)
                                : decode_gmm_tile<BN, kCtas>(p, tile, cta_rank);
      const int n0 = t.n0;
      const uint32_t acc = local_tile & 1u;
      const uint32_t acc_ph = (local_tile >> 1) & 1u;
      if (!mbar_wait<kPair>(smem_u32(&bar_acc_full[acc]), acc_ph, abort_ptr)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();

      bool row_ok;         // this thread's output row exists
      size_t row_off;      // element offset of this thread's output row
      bool warp_has_rows;  // any row of this warp's 32-row slab exists
      bool slab_by_tma;    // the whole slab may be written as one box per 64 columns
      bool zero_only = false;
      int out_row0;        // first output row of the slab (TMA coordinate)
      if (kTgmm) {
        const int kr = t.k0 + r_in_tile;
        out_row0 = t.k0 + quarter * 32;
        row_ok = kr < p.k;
        warp_has_rows = out_row0 < p.k;
        slab_by_tma = true;  // rows >= k are outside the map and dropped by the store
        row_off = (static_cast<size_t>(t.group) * p.k + kr) * static_cast<size_t>(p.n);
        zero_only = kSeg ? tgmm_block_count<kSeg>(p, t) == 0 : t.rows <= 0;
      } else if (!kPair && t.rows <= 64) {
        // M = 64 tile: row 16 * quarter + lane sits in lane `lane` (< 16) of this warp's quarter
        const int r64 = quarter * 16 + lane;
        out_row0 = t.row0 + quarter * 16;
        row_ok = lane < 16 && r64 < t.rows;
        warp_has_rows = quarter * 16 < t.rows;
        slab_by_tma = false;
        row_off = static_cast<size_t>(t.row0 + r64) * static_cast<size_t>(p.n);
      } else {
        out_row0 = t.row0 + quarter * 32;
        row_ok = r_in_tile < t.rows;
        warp_has_rows = quarter * 32 < t.rows;
        slab_by_tma = quarter * 32 + 32 <= t.rows;  // else the box would overwrite the next group
        row_off = static_cast<size_t>(t.row0 + r_in_tile) * static_cast<size_t>(p.n);
      }

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
        if constexpr (kFp8) {  // dequantise: one scale per weight matrix (1 when none is given)
          const float sc = p.weight_scale != nullptr ? p.weight_scale[t.weight] : 1.0f;
#pragma unroll
          for (int j = 0; j < 64; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * sc);
        }
        if (c == n_chunks - 1) {
          // Everything this warp needs from the accumulator is in registers: hand it back.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if (kPair) {
              mbar_arrive_cluster(acc_empty_bar, 0);
            } else {
              mbar_arrive(acc_empty_bar);
            }
          }
        }
        uint4 o[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          o[q].x = pack2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]), p.ab_format);
          o[q].y = pack2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]), p.ab_format);
          o[q].z = pack2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]), p.ab_format);
          o[q].w = pack2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]), p.ab_format);
        }
        if (slab_by_tma) {
          const uint32_t buf = staging + (boxes_stored & 1u) * kOutBoxBytes;
          // The box stored two boxes ago used this buffer: wait until TMA has read it out.
          if (lane == 0) bulk_wait_group_read<1>();
          __syncwarp();
          const uint32_t row_addr = buf + lane * 128;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const uint32_t a = row_addr + (((q ^ (lane & 7)) & 7) << 4);  // 128-byte swizzle
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(o[q].x),
                         "r"(o[q].y), "r"(o[q].z), "r"(o[q].w)
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
          uint16_t* dst = out16 + row_off + col;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (col + q * 8 < p.n) {  // n is a multiple of 8: a chunk is all in or all out
              *reinterpret_cast<uint4*>(dst + q * 8) = o[q];
            }
          }
        }
      }
      if (n_chunks == 0) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (kPair) {
            mbar_arrive_cluster(acc_empty_bar, 0);
          } else {
            mbar_arrive(acc_empty_bar);
          }
        }
      }
    }
    // All boxes must have left shared memory (and reached global memory) before the CTA goes.
    if (lane == 0) bulk_wait_group<0>();
    __syncwarp();

    if (!kTgmm && p.zero_tail) {
      // Rows past sum(group_sizes) belong to no group: jax.lax.ragged_dot defines them as 0
      // (the reference writes them from its last live program, gpu_ragged_dot.py:155-165).
      const int first = imin(imax(p.totals[1], 0), p.m);
      const size_t chunks_per_row = static_cast<size_t>(p.n) / 8;
      const size_t total = static_cast<size_t>(p.m - first) * chunks_per_row;
      const size_t tid = static_cast<size_t>(cta_index) * 128 + (threadIdx.x - 64);
      const size_t stride = static_cast<size_t>(gemm_ctas) * 128;
      uint4* dst = reinterpret_cast<uint4*>(out16 + static_cast<size_t>(first) * p.n);
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      for (size_t i = tid; i < total; i += stride) dst[i] = z;
    }
  }

  // ------------------------------------------------------------ tear-down
  __syncthreads();
  if (wait_ctl.abort) {
    if (threadIdx.x == 0) atomicMax(p.status, static_cast<int32_t>(kStatusWaitExpired));
    // Give copies and MMAs that are still in flight time to land before smem/TMEM go away.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  // Neither CTA of a pair may leave while the other can still reach its barriers or smem.
  if (kPair) cluster_sync();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<kCtas>(tmem_base, kTmemCols);
  }
}

}  // namespace rd
