// C ABI of the ragged-dot library (declared in include/ragged_dot_b200.h): argument checks,
// TMA descriptor encoding, tile selection and kernel launches.  No torch / XLA types here;
// the XLA-FFI and Python layers sit on top of these entry points.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>

#include "../../include/ragged_dot_b200.h"
#include "rd_gemm.cuh"
#include "rd_dispatch.cuh"
#include "rd_gemm2.cuh"
#include "rd_gemm_f32.cuh"
#include "rd_gemm_perm.cuh"
#include "rd_metadata.cuh"
#include "rd_rows.cuh"

namespace {

using rd::GemmArgs;
using rd::WorkspaceLayout;

// ------------------------------------------------------------------ driver entry point
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

// rank-2 or rank-3 tiled map over a dense row-major 16-bit or 32-bit float tensor, 128-byte swizzle,
// zero fill outside the bounds.  dims / box are innermost first.
int encode_map(CUtensorMap* map, const void* base, int dtype, int rank, const uint64_t* dims,
               const uint32_t* box, bool atom32 = false) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return RD_ERR_DRIVER;
  cuuint64_t gdims[3];
  cuuint64_t gstrides[2];
  cuuint32_t gbox[3];
  cuuint32_t estr[3] = {1, 1, 1};
  uint64_t stride = dtype == RD_DTYPE_F32 ? 4 : 2;
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    stride *= dims[i];
    if (i + 1 < rank) gstrides[i] = stride;
  }
  const CUtensorMapDataType dt = dtype == RD_DTYPE_BF16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : dtype == RD_DTYPE_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                         : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides,
                  gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "ragged_dot_b200: cuTensorMapEncodeTiled failed (CUresult %d): base=%p rank=%d "
            "dims={%llu,%llu,%llu} box={%u,%u,%u}\n",
            static_cast<int>(r), base, rank, (unsigned long long)gdims[0],
            (unsigned long long)gdims[1], (unsigned long long)(rank > 2 ? gdims[2] : 0), gbox[0],
            gbox[1], rank > 2 ? gbox[2] : 0u);
    return RD_ERR_TENSOR_MAP;
  }
  return RD_OK;
}

// "Column-blocked" view of a dense row-major 16-bit [rows, cols] tensor, cols a multiple of 64:
// (64 columns, rows, cols / 64 blocks).  A box of (64, box_rows, box_blocks) lands in shared memory
// as box_blocks slabs of [box_rows][128 B], block after block -- what box_blocks separate 2-D boxes
// of 64 columns would write -- in ONE TMA instruction.
int encode_blocked_map(CUtensorMap* map, const void* base, int dtype, int cols, int rows, int box_rows,
                       int box_blocks) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return RD_ERR_DRIVER;
  cuuint64_t gdims[3] = {64, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(cols / 64)};
  cuuint64_t gstrides[2] = {static_cast<cuuint64_t>(cols) * 2, 128};
  cuuint32_t gbox[3] = {64, static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(box_blocks)};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt =
      dtype == RD_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUresult r = fn(map, dt, 3, const_cast<void*>(base), gdims, gstrides, gbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "ragged_dot_b200: cuTensorMapEncodeTiled failed (CUresult %d): blocked map base=%p "
            "rows=%d cols=%d box=(64,%d,%d)\n", static_cast<int>(r), base, rows, cols, box_rows, box_blocks);
    return RD_ERR_TENSOR_MAP;
  }
  return RD_OK;
}

// ------------------------------------------------------------------ device properties
int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

bool aligned16(const void* p) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int max_row_tiles(int m, int g) { return (m + rd::kTileM - 1) / rd::kTileM + g; }

struct Workspace {
  WorkspaceLayout layout;
  int32_t* base;
  int32_t* status() const { return base + layout.off_status(); }
  int32_t* totals() const { return base + layout.off_totals(); }
  int32_t* group_offsets() const { return base + layout.off_group_offsets(); }
  int32_t* tile_prefix() const { return base + layout.off_tile_prefix(); }
  int32_t* tile2group() const { return base + layout.off_tile2group(); }
  int32_t* tile2idx() const { return base + layout.off_tile2idx(); }
  rd::TileRecord* tile_rec() const {
    return reinterpret_cast<rd::TileRecord*>(base + layout.off_tile_rec());
  }
};

int bind_workspace(void* ws, size_t ws_bytes, int m, int g, Workspace* out) {
  if (!aligned16(ws)) return RD_ERR_BAD_POINTER;
  out->layout.g = g;
  out->layout.max_tiles = max_row_tiles(m, g);
  if (ws_bytes < static_cast<size_t>(out->layout.total_words()) * sizeof(int32_t))
    return RD_ERR_WORKSPACE;
  out->base = static_cast<int32_t*>(ws);
  return RD_OK;
}

void launch_internal_metadata(const int32_t* group_sizes, const int32_t* group_to_weight, int g,
                              int m, int tile_m, const Workspace& w, cudaStream_t stream,
                              bool by_weight = false) {
  if (by_weight && group_to_weight != nullptr && m > 0) {
    // the two reference-shaped arrays are not needed by the kernels: their space (U >= g + 1
    // words each) serves as the scratch of the visiting order
    rd::group_metadata_kernel<<<1, rd::kMetaThreads, 0, stream>>>(
        group_sizes, g, m, tile_m, w.layout.max_tiles, w.group_offsets(), nullptr, nullptr, w.totals(),
        w.tile_prefix(), w.totals() + 1, w.status(), w.tile_rec(), group_to_weight, w.tile2group(),
        w.tile2idx());
    return;
  }
  rd::group_metadata_kernel<<<1, rd::kMetaThreads, 0, stream>>>(
      group_sizes, g, m, tile_m, w.layout.max_tiles, w.group_offsets(), w.tile2group(),
      w.tile2idx(), w.totals(), w.tile_prefix(), w.totals() + 1, w.status(), w.tile_rec(),
      group_to_weight);
}

// ------------------------------------------------------------------ tile selection
// The committed replacement for the reference's run-time tune-jax search.  Measured on B200:
// the 256-wide tile wins at every benchmark shape, compute-bound or bandwidth-bound (decode m=256: 93 % of copy bandwidth at 256, 67 % at 128, 39 % at 64), so
// narrower tiles are only used when n itself is narrow.
int choose_tile_n(long long /*row_tiles*/, int n, int /*sms*/) {
  if (n <= 64) return 64;
  if (n <= 128) return 128;
  return 256;
}

template <int BN, bool kBKMajor, bool kTgmm, int kCtas, bool kSeg = false, bool kFp8 = false>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tout,
                const GemmArgs& args, int ctas, cudaStream_t stream) {
  constexpr int kStageBytes = rd::stage_bytes<BN, kCtas>();
  constexpr int kStages = (196608 / kStageBytes) > 8 ? 8 : (196608 / kStageBytes);
  constexpr int kSmem = kStages * kStageBytes + rd::kOutStagingBytes + 1024;
  auto kernel = rd::ragged_gemm_kernel<BN, kBKMajor, kStages, kTgmm, kCtas, kSeg, kFp8>;
  // The attribute is per device; setting it again is cheap, so do it on every call rather
  // than track which devices have seen it.
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
      cudaSuccess)
    return RD_ERR_LAUNCH;
  cudaLaunchConfig_t lc = {};
  lc.blockDim = dim3(rd::kGemmFixerThreads, 1, 1);
  lc.dynamicSmemBytes = kSmem;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  lc.attrs = attr;
  lc.numAttrs = 0;
  if (kCtas == 2) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    lc.numAttrs = 1;
    // A persistent grid must be fully co-resident: ask how many CTA pairs fit at once.
    lc.gridDim = dim3(2, 1, 1);
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &lc) != cudaSuccess || clusters <= 0)
      return RD_ERR_LAUNCH;
    int pairs = ctas / 2;
    if (pairs > clusters) pairs = clusters;
    if (pairs < 1) pairs = 1;
    lc.gridDim = dim3(2 * pairs, 1, 1);
  } else {
    lc.gridDim = dim3(ctas, 1, 1);
  }
  if (cudaLaunchKernelEx(&lc, kernel, ta, tb, tout, args) != cudaSuccess) {
    (void)cudaGetLastError();
    return RD_ERR_LAUNCH;
  }
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

template <int BN, bool kBKMajor, bool kTgmm>
int launch_gemm_f32(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tout,
                    const GemmArgs& args, int ctas, cudaStream_t stream) {
  constexpr int kStageBytes = rd::f32_stage_bytes<BN>();
  constexpr int kStages = (196608 / kStageBytes) > 8 ? 8 : (196608 / kStageBytes);
  constexpr int kSmem = kStages * kStageBytes + rd::kOutStagingBytes + 1024;
  auto kernel = rd::ragged_gemm_f32_kernel<BN, kBKMajor, kStages, kTgmm>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
      cudaSuccess)
    return RD_ERR_LAUNCH;
  kernel<<<ctas, rd::kGemmThreads, kSmem, stream>>>(ta, tb, tout, args);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

template <int BN, bool kBKMajor, bool kTgmm>
int launch_gemm_perm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tout,
                     const GemmArgs& args, const rd::PermArgs& perm, int ctas, cudaStream_t stream) {
  constexpr int kStageBytes = rd::stage_bytes<BN, 1>();
  constexpr int kStages = (196608 / kStageBytes) > 8 ? 8 : (196608 / kStageBytes);
  constexpr int kSmem = kStages * kStageBytes + rd::kOutStagingBytes + 1024;
  auto kernel = rd::ragged_gemm_perm_kernel<BN, kBKMajor, kStages, kTgmm>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) !=
      cudaSuccess)
    return RD_ERR_LAUNCH;
  kernel<<<ctas, rd::kPermThreads, kSmem, stream>>>(ta, tb, tout, args, perm);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

// Tile-load map over a [rows, cols] 16-bit tensor with boxes of [box_rows][64 columns].  The
// permuted kernels use it for an operand without a row index; with one they read the tensor
// through its base pointer and the map is only prefetched.
int encode_rows_map(CUtensorMap* map, const void* base, int dtype, int cols, int rows, int box_rows) {
  const uint64_t dims[2] = {static_cast<uint64_t>(cols), static_cast<uint64_t>(rows)};
  const uint32_t box[2] = {64, static_cast<uint32_t>(box_rows)};
  return encode_map(map, base, dtype, 2, dims, box);
}

template <bool kBKMajor, bool kTgmm, bool kVariant = false>
int launch_gemm2(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tout,
                 const GemmArgs& args, int ctas, cudaStream_t stream) {
  if constexpr (!kTgmm && !kVariant) {
    // ready flags / sender CTAs live in a separate instantiation (see rd_gemm2.cuh)
    if (args.ready_flags != nullptr || args.send.world > 0)
      return launch_gemm2<kBKMajor, false, true>(ta, tb, tout, args, ctas, stream);
  }
  if constexpr (kTgmm && !kVariant) {
    if (args.seg_count > 1) return launch_gemm2<false, true, true>(ta, tb, tout, args, ctas, stream);
  }
  auto kernel = rd::ragged_gemm2_kernel<kBKMajor, kTgmm, kVariant>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, rd::kG2SmemBytes) !=
      cudaSuccess)
    return RD_ERR_LAUNCH;
  kernel<<<ctas, rd::kG2Threads, rd::kG2SmemBytes, stream>>>(ta, tb, tout, args);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

// tgmm with 512 x 256 tiles on CTA pairs (rd_gemm2.cuh, kPair).
int launch_gemm2_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tout,
                      const GemmArgs& args, int ctas, cudaStream_t stream) {
  auto kernel = rd::ragged_gemm2_kernel<false, true, false, true>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, rd::kG2PairSmemBytes) !=
      cudaSuccess)
    return RD_ERR_LAUNCH;
  cudaLaunchConfig_t lc = {};
  lc.blockDim = dim3(rd::kG2Threads, 1, 1);
  lc.dynamicSmemBytes = rd::kG2PairSmemBytes;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  // A persistent grid must be fully co-resident: ask how many CTA pairs fit at once.
  lc.gridDim = dim3(2, 1, 1);
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &lc) != cudaSuccess || clusters <= 0)
    return RD_ERR_LAUNCH;
  int pairs = ctas / 2;
  if (pairs > clusters) pairs = clusters;
  if (pairs < 1) pairs = 1;
  lc.gridDim = dim3(2 * pairs, 1, 1);
  if (cudaLaunchKernelEx(&lc, kernel, ta, tb, tout, args) != cudaSuccess) {
    (void)cudaGetLastError();
    return RD_ERR_LAUNCH;
  }
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

// 256-row tiles on one CTA (rd_gemm2.cuh) move a third less data per flop than 128-row tiles.
// They pay off when a tile's second half usually exists: tgmm with k >= 256, and gmm when the
// groups are long (mean rows per group >= 512; a half without rows is skipped, so the cost of a
// wrong guess is only a shallower smem ring).  At exactly 512 rows per group the picture is mixed:
// 16 ragged groups over m 8192, k 4096, n 14336 are 5-13 % faster on 128-row tiles, the
// expert-parallel step (64 segments of about 512 rows over 32 weight matrices) 4 % slower.
bool choose_two_half(bool tgmm, long long m, int k, int g, int bn) {
  if (bn != 256) return false;
  if (tgmm) return k >= 256;
  return g > 0 && m / g >= 512;
}

// tgmm with 256-row tiles: 512 x 256 tiles on CTA pairs (a quarter less L2 -> SM traffic, a
// fourth stage) were 0.6-2.4 % faster than one CTA per tile on every compute-bound shape swept
// (m/g 512 to 2048; k 4096 and 7168; n 1536 to 14336).  Short groups make tgmm output-bound and
// were not measured: they stay on one CTA.
bool choose_pair_512(long long m, int k, int g) { return k >= 512 && g > 0 && m / g >= 512; }

// CTA pairs (256 x 256 tiles, B operand split between the two CTAs) pay off where the
// 256-row granularity wastes nothing: tgmm, whose tile rows are the dense k axis.  For gmm the
// tile rows are a group's ragged token rows and the wider tile wastes more than the pair
// saves at the benchmark group sizes, so gmm pairs only on request (rd_tile_cfg.cta_group).
bool choose_pair(bool tgmm, long long tiles256, int bn, int sms) {
  if (!tgmm || bn != 256) return false;
  return tiles256 >= 2LL * (sms / 2);
}

// Limit of every bounded wait inside a kernel, in microseconds: rd_tile_cfg.wait_limit_ms if
// set, else the environment variable RD_WAIT_LIMIT_MS (read once), else two seconds.
uint32_t wait_limit_us(const rd_tile_cfg* cfg) {
  static const long env_ms = [] {
    const char* v = getenv("RD_WAIT_LIMIT_MS");
    const long ms = v ? strtol(v, nullptr, 10) : 0;
    return ms > 0 ? ms : 0;
  }();
  long ms = (cfg && cfg->wait_limit_ms > 0) ? cfg->wait_limit_ms : env_ms;
  if (ms <= 0) return rd::kDefaultWaitLimitUs;
  if (ms > 4000000) ms = 4000000;
  return static_cast<uint32_t>(ms) * 1000u;
}

int pick_ctas(const rd_tile_cfg* cfg) {
  int ctas = sm_count();
  if (cfg && cfg->max_ctas > 0 && cfg->max_ctas < ctas) ctas = cfg->max_ctas;
  return ctas;
}

}  // namespace

extern "C" {

int rd_version(void) { return RD_VERSION; }

const char* rd_status_string(int code) {
  switch (code) {
    case RD_OK: return "ok";
    case RD_ERR_BAD_SHAPE: return "bad shape: sizes must be >= 0 and rows of k, n elements multiples of 16 bytes";
    case RD_ERR_BAD_DTYPE: return "unsupported dtype: f16, bf16 or f32";
    case RD_ERR_BAD_POINTER: return "null or misaligned pointer (16-byte alignment required)";
    case RD_ERR_WORKSPACE: return "workspace too small (see rd_workspace_bytes)";
    case RD_ERR_BAD_CONFIG: return "unsupported tile configuration";
    case RD_ERR_TENSOR_MAP: return "driver rejected a TMA tensor map";
    case RD_ERR_LAUNCH: return "kernel launch failed";
    case RD_ERR_DRIVER: return "cuTensorMapEncodeTiled entry point not available";
    case RD_ERR_DEVICE_WAIT: return "a bounded wait inside a kernel expired";
    case RD_ERR_TOO_LARGE:
      return "problem too large for the built-in scratch of rd_gmm_static_scratch "
             "(needs 12*g + 10*ceil(m/128) + 16 <= 16384 words); use rd_gmm with a workspace";
    case RD_ERR_SCRATCH_SETUP: return "could not resolve the address of the built-in scratch array";
    default: return "unknown status";
  }
}

int rd_workspace_bytes(int m, int g, size_t* bytes) {
  if (m < 0 || g < 0 || bytes == nullptr) return RD_ERR_BAD_SHAPE;
  WorkspaceLayout l;
  l.g = g;
  l.max_tiles = max_row_tiles(m, g);
  size_t b = static_cast<size_t>(l.total_words()) * sizeof(int32_t);
  *bytes = (b + 255) & ~static_cast<size_t>(255);
  return RD_OK;
}

int rd_metadata(const int32_t* group_sizes, int g, int m, int chunk_m, int32_t* group_offsets,
                int32_t* row_it2group, int32_t* row_it2it_in_group, int32_t* total_row_its,
                void* stream) {
  if (g < 0 || m < 0 || chunk_m <= 0) return RD_ERR_BAD_SHAPE;
  if (g == 0) {
    // U = ceil(m / chunk_m) rows of zeros and a zero total.
    const int u = (m + chunk_m - 1) / chunk_m;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (row_it2group && u) cudaMemsetAsync(row_it2group, 0, sizeof(int32_t) * u, s);
    if (row_it2it_in_group && u) cudaMemsetAsync(row_it2it_in_group, 0, sizeof(int32_t) * u, s);
    if (total_row_its) cudaMemsetAsync(total_row_its, 0, sizeof(int32_t), s);
    return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
  }
  if (group_sizes == nullptr) return RD_ERR_BAD_POINTER;
  const int u = (m + chunk_m - 1) / chunk_m + g;
  rd::group_metadata_kernel<<<1, rd::kMetaThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      group_sizes, g, m, chunk_m, u, group_offsets, row_it2group, row_it2it_in_group,
      total_row_its, nullptr, nullptr, nullptr, nullptr, nullptr);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

// Shared body of rd_gmm / rd_gmm_indexed.  `num_weights` is A's leading dimension;
// `group_to_weight` (device, [g]) is null when group i uses A[i].
struct ReadyFlags {
  const int32_t* flags;  // null: no waiting
  int groups_per_flag;
  int epoch;
};

static int gmm_impl(const void* x, const void* A, const int32_t* group_sizes,
                    const int32_t* group_to_weight, int num_weights, void* y, void* workspace,
                    size_t workspace_bytes, int m, int k, int n, int g, int trans_rhs, int dtype,
                    const rd_tile_cfg* cfg, void* stream_v, ReadyFlags ready = {nullptr, 1, 0},
                    const rd::EpSendArgs* send = nullptr) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (dtype != RD_DTYPE_F16 && dtype != RD_DTYPE_BF16 && dtype != RD_DTYPE_F32) return RD_ERR_BAD_DTYPE;
  const bool f32 = dtype == RD_DTYPE_F32;
  const int esize = f32 ? 4 : 2;            // bytes per element
  const int amask = f32 ? 3 : 7;            // rows must be multiples of 16 bytes
  const int row_elems = 128 / esize;        // elements per 128-byte swizzle row
  if (m < 0 || k < 0 || n < 0 || g < 0 || num_weights < 0 || (k & amask) || (n & amask))
    return RD_ERR_BAD_SHAPE;
  if (m == 0 || n == 0) return RD_OK;
  if (!aligned16(y)) return RD_ERR_BAD_POINTER;
  if (g == 0 || k == 0 || num_weights == 0) {  // nothing contributes: every row is a zero row
    cudaMemsetAsync(y, 0, static_cast<size_t>(m) * n * esize, stream);
    return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
  }
  if (!aligned16(x) || !aligned16(A) || group_sizes == nullptr) return RD_ERR_BAD_POINTER;
  Workspace w;
  int rc = bind_workspace(workspace, workspace_bytes, m, g, &w);
  if (rc != RD_OK) return rc;

  const int sms = sm_count();
  int bn = cfg && cfg->tile_n ? cfg->tile_n : choose_tile_n((m + rd::kTileM - 1) / rd::kTileM, n, sms);
  if (bn != 64 && bn != 128 && bn != 256) return RD_ERR_BAD_CONFIG;
  int cta_group = cfg ? cfg->cta_group : 0;
  if (cta_group < 0 || cta_group > 2 || (cta_group == 2 && bn != 256)) return RD_ERR_BAD_CONFIG;
  if (cta_group == 0) cta_group = choose_pair(false, 0, bn, sms) ? 2 : 1;
  int tile_m = cfg ? cfg->tile_m : 0;
  if (tile_m != 0 && tile_m != 128 && tile_m != 256) return RD_ERR_BAD_CONFIG;
  if (tile_m == 256 && (bn != 256 || cta_group != 1)) return RD_ERR_BAD_CONFIG;
  if (f32) {  // the float32 (TF32) kernels exist as single-CTA 128-row tiles only
    if (cta_group == 2 || tile_m == 256) return RD_ERR_BAD_CONFIG;
    cta_group = 1;
    tile_m = 128;
  }
  if (tile_m == 0) tile_m = (cta_group == 1 && choose_two_half(false, m, k, g, bn)) ? 256 : 128;
  const bool two_half = tile_m == 256;

  // Launch the metadata kernel before encoding the tensor maps: besides being the first step
  // of the call, a runtime launch binds the device's primary context to the calling thread,
  // which the driver's tensor-map encoder needs (threads such as torch's autograd workers
  // arrive here without one).
  launch_internal_metadata(group_sizes, group_to_weight, g, m,
                           two_half ? rd::kG2TileRows : rd::kTileM * cta_group, w, stream,
                           cfg != nullptr && (cfg->flags & RD_CFG_GROUP_BY_WEIGHT) != 0);
  if (cudaGetLastError() != cudaSuccess) return RD_ERR_LAUNCH;

  CUtensorMap ta, tb;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m)};
    const uint32_t box[2] = {static_cast<uint32_t>(row_elems), rd::kTileM};
    rc = encode_map(&ta, x, dtype, 2, dims, box);
    if (rc != RD_OK) return rc;
  }
  if (trans_rhs) {  // A[g, n, k]: rows of k, K-major operand, one [BN][128 B] box per stage
    const uint64_t dims[3] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n),
                              static_cast<uint64_t>(num_weights)};
    const uint32_t box[3] = {static_cast<uint32_t>(row_elems), static_cast<uint32_t>(bn / cta_group), 1};
    rc = encode_map(&tb, A, dtype, 3, dims, box);
  } else {  // A[g, k, n]: rows of n, MN-major operand, [stage-depth k][128 B of n] boxes
    const uint64_t dims[3] = {static_cast<uint64_t>(n), static_cast<uint64_t>(k),
                              static_cast<uint64_t>(num_weights)};
    const uint32_t box[3] = {static_cast<uint32_t>(row_elems), static_cast<uint32_t>(row_elems), 1};
    rc = encode_map(&tb, A, dtype, 3, dims, box, /*atom32=*/f32);  // MN-major fp32: 32-byte atoms
  }
  if (rc != RD_OK) return rc;
  CUtensorMap tout;
  {  // y[m, n] written as [32 rows][128 B] boxes
    const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(m)};
    const uint32_t box[2] = {static_cast<uint32_t>(row_elems), 32};
    rc = encode_map(&tout, y, dtype, 2, dims, box);
    if (rc != RD_OK) return rc;
  }

  GemmArgs args = {};
  args.m = m; args.k = k; args.n = n; args.g = g;
  args.n_tiles = (n + bn - 1) / bn;
  args.k_tiles = 0;
  args.max_m_tiles = w.layout.max_tiles;
  args.ab_format = dtype;
  args.wait_limit_us = wait_limit_us(cfg);
  args.zero_tail = (cfg && (cfg->flags & RD_CFG_NO_ZERO_TAIL)) ? 0 : 1;
  args.group_sizes = group_sizes;
  args.group_offsets = w.group_offsets();
  args.tile_rec = w.tile_rec();
  args.totals = w.totals();
  args.status = w.status();
  args.out = y;
  args.ready_flags = ready.flags;
  args.groups_per_flag = ready.groups_per_flag > 0 ? ready.groups_per_flag : 1;
  args.ready_epoch = ready.epoch;
  if (send != nullptr) {
    if (f32 || cta_group == 2) return RD_ERR_BAD_CONFIG;  // the sender role lives in the 16-bit 1-CTA kernels
    args.send = *send;
  }

  const int ctas = pick_ctas(cfg);
  if (send != nullptr && send->sender_ctas >= ctas) return RD_ERR_BAD_CONFIG;
  if (f32) {
    if (ready.flags != nullptr) return RD_ERR_BAD_DTYPE;  // the float32 kernels do not wait on flags
    if (trans_rhs) {
      if (bn == 256) return launch_gemm_f32<256, true, false>(ta, tb, tout, args, ctas, stream);
      if (bn == 128) return launch_gemm_f32<128, true, false>(ta, tb, tout, args, ctas, stream);
      return launch_gemm_f32<64, true, false>(ta, tb, tout, args, ctas, stream);
    }
    if (bn == 256) return launch_gemm_f32<256, false, false>(ta, tb, tout, args, ctas, stream);
    if (bn == 128) return launch_gemm_f32<128, false, false>(ta, tb, tout, args, ctas, stream);
    return launch_gemm_f32<64, false, false>(ta, tb, tout, args, ctas, stream);
  }
  if (two_half) {
    return trans_rhs ? launch_gemm2<true, false>(ta, tb, tout, args, ctas, stream)
                     : launch_gemm2<false, false>(ta, tb, tout, args, ctas, stream);
  }
  if (trans_rhs) {
    if (cta_group == 2) return launch_gemm<256, true, false, 2>(ta, tb, tout, args, ctas, stream);
    if (bn == 256) return launch_gemm<256, true, false, 1>(ta, tb, tout, args, ctas, stream);
    if (bn == 128) return launch_gemm<128, true, false, 1>(ta, tb, tout, args, ctas, stream);
    return launch_gemm<64, true, false, 1>(ta, tb, tout, args, ctas, stream);
  }
  if (cta_group == 2) return launch_gemm<256, false, false, 2>(ta, tb, tout, args, ctas, stream);
  if (bn == 256) return launch_gemm<256, false, false, 1>(ta, tb, tout, args, ctas, stream);
  if (bn == 128) return launch_gemm<128, false, false, 1>(ta, tb, tout, args, ctas, stream);
  return launch_gemm<64, false, false, 1>(ta, tb, tout, args, ctas, stream);
}

int rd_gmm(const void* x, const void* A, const int32_t* group_sizes, void* y, void* workspace,
           size_t workspace_bytes, int m, int k, int n, int g, int trans_rhs, int dtype,
           const rd_tile_cfg* cfg, void* stream) {
  return gmm_impl(x, A, group_sizes, nullptr, g, y, workspace, workspace_bytes, m, k, n, g, trans_rhs,
                  dtype, cfg, stream);
}

int rd_gmm_indexed(const void* x, const void* A, int num_weights, const int32_t* group_sizes,
                   const int32_t* group_to_weight, void* y, void* workspace, size_t workspace_bytes,
                   int m, int k, int n, int g, int trans_rhs, int dtype, const rd_tile_cfg* cfg,
                   void* stream) {
  if (g > 0 && group_to_weight == nullptr) return RD_ERR_BAD_POINTER;
  return gmm_impl(x, A, group_sizes, group_to_weight, num_weights, y, workspace, workspace_bytes, m, k,
                  n, g, trans_rhs, dtype, cfg, stream);
}

int rd_gather_rows(const void* src, const int32_t* row_index, void* dst, int rows_out, int rows_in,
                   int row_bytes, void* stream) {
  if (rows_out < 0 || rows_in < 0 || row_bytes < 0 || (row_bytes & 15)) return RD_ERR_BAD_SHAPE;
  if (rows_out == 0 || row_bytes == 0) return RD_OK;
  if (!aligned16(src) || !aligned16(dst) || row_index == nullptr) return RD_ERR_BAD_POINTER;
  const int warps_per_block = rd::kGatherThreads / 32;
  int blocks = (rows_out + warps_per_block - 1) / warps_per_block;
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  rd::gather_rows_kernel<<<blocks, rd::kGatherThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), row_index, static_cast<uint4*>(dst), rows_out, rows_in,
      row_bytes / 16);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

int rd_ep_count(const int32_t* routing, int entries, int num_experts, int32_t* counts, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (entries < 0 || num_experts <= 0 || num_experts > 8192) return RD_ERR_BAD_SHAPE;
  if (counts == nullptr || (entries > 0 && routing == nullptr)) return RD_ERR_BAD_POINTER;
  if (cudaMemsetAsync(counts, 0, sizeof(int32_t) * num_experts, stream) != cudaSuccess)
    return RD_ERR_LAUNCH;
  if (entries == 0) return RD_OK;
  int blocks = (entries + rd::kEpThreads - 1) / rd::kEpThreads;
  if (blocks > sm_count()) blocks = sm_count();
  rd::ep_count_kernel<<<blocks, rd::kEpThreads, sizeof(int32_t) * num_experts, stream>>>(
      routing, entries, num_experts, counts);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

int rd_ep_plan(const int32_t* counts_all, int world, int num_experts, int rank, int32_t* dest_offset,
               int32_t* segment_sizes, int32_t* fill, int32_t* totals, void* stream) {
  if (world <= 0 || num_experts <= 0 || num_experts % world != 0 || rank < 0 || rank >= world)
    return RD_ERR_BAD_SHAPE;
  if (!counts_all || !dest_offset || !segment_sizes || !fill || !totals) return RD_ERR_BAD_POINTER;
  rd::ep_plan_kernel<<<1, rd::kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      counts_all, world, num_experts, rank, dest_offset, segment_sizes, fill, totals, 0, nullptr, nullptr,
      nullptr, nullptr, 0, 0u, nullptr);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

int rd_ep_plan_ring(const int32_t* counts_all, int world, int num_experts, int rank,
                    int32_t* dest_offset, int32_t* segment_sizes, int32_t* fill, int32_t* totals,
                    int32_t* phase_done, int32_t* send_start, int32_t* list_fill, void* stream) {
  if (world <= 0 || num_experts <= 0 || num_experts % world != 0 || rank < 0 || rank >= world)
    return RD_ERR_BAD_SHAPE;
  if (!counts_all || !dest_offset || !segment_sizes || !fill || !totals || !phase_done)
    return RD_ERR_BAD_POINTER;
  if ((send_start == nullptr) != (list_fill == nullptr)) return RD_ERR_BAD_POINTER;
  rd::ep_plan_kernel<<<1, rd::kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      counts_all, world, num_experts, rank, dest_offset, segment_sizes, fill, totals, 1, phase_done,
      send_start, list_fill, nullptr, 0, 0u, nullptr);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

int rd_ep_count_share(const int32_t* routing, int entries, int num_experts, int32_t* counts_scratch,
                      int32_t* ticket, int world, int rank, const uint64_t* peer_counts,
                      const uint64_t* peer_flags, int epoch, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (entries < 0 || num_experts <= 0 || num_experts > 8192 || world <= 0 || world > rd::kEpThreads ||
      rank < 0 || rank >= world)
    return RD_ERR_BAD_SHAPE;
  if (!counts_scratch || !ticket || !peer_counts || !peer_flags || (entries > 0 && routing == nullptr))
    return RD_ERR_BAD_POINTER;
  int blocks = (entries + rd::kEpThreads - 1) / rd::kEpThreads;
  if (blocks > sm_count()) blocks = sm_count();
  if (blocks < 1) blocks = 1;  // the counts (zeros) and the flag go out even without entries
  rd::ep_count_share_kernel<<<blocks, rd::kEpThreads, sizeof(int32_t) * num_experts, stream>>>(
      routing, entries, num_experts, counts_scratch, ticket, world, rank, peer_counts, peer_flags, epoch);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

int rd_ep_plan_ring_when_counted(const int32_t* counts_all, const int32_t* count_flags, int epoch,
                                 int world, int num_experts, int rank, int32_t* dest_offset,
                                 int32_t* segment_sizes, int32_t* fill, int32_t* totals,
                                 int32_t* phase_done, int32_t* send_start, int32_t* list_fill,
                                 int32_t* status, int wait_limit_ms, void* stream) {
  if (world <= 0 || world > rd::kEpThreads || num_experts <= 0 || num_experts % world != 0 || rank < 0 ||
      rank >= world)
    return RD_ERR_BAD_SHAPE;
  if (!counts_all || !count_flags || !dest_offset || !segment_sizes || !fill || !totals || !phase_done)
    return RD_ERR_BAD_POINTER;
  if ((send_start == nullptr) != (list_fill == nullptr)) return RD_ERR_BAD_POINTER;
  rd_tile_cfg cfg = {};
  cfg.wait_limit_ms = wait_limit_ms;
  rd::ep_plan_kernel<<<1, rd::kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      counts_all, world, num_experts, rank, dest_offset, segment_sizes, fill, totals, 1, phase_done,
      send_start, list_fill, count_flags, epoch, wait_limit_us(&cfg), status);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

int rd_ep_assign(const int32_t* routing, int entries, int num_experts, int world, int rank,
                 const int32_t* dest_offset, int32_t* fill, int capacity_rows, int32_t* dest_pos,
                 const int32_t* send_start, int32_t* list_fill, int32_t* send_index, void* stream) {
  if (entries < 0 || world <= 0 || num_experts <= 0 || num_experts % world != 0 || rank < 0 ||
      rank >= world || capacity_rows < 0)
    return RD_ERR_BAD_SHAPE;
  if (entries == 0) return RD_OK;
  if (!routing || !dest_offset || !fill || !dest_pos || !send_start || !list_fill || !send_index)
    return RD_ERR_BAD_POINTER;
  if (num_experts + world > 5000) return RD_ERR_BAD_SHAPE;  // shared-memory counters of the kernel
  const int blocks = (entries + rd::kEpThreads - 1) / rd::kEpThreads;
  const size_t smem = 2 * static_cast<size_t>(num_experts + world) * sizeof(int32_t);
  rd::ep_assign_kernel<<<blocks, rd::kEpThreads, smem, static_cast<cudaStream_t>(stream)>>>(
      routing, entries, num_experts, num_experts / world, world, rank, dest_offset, fill, capacity_rows,
      dest_pos, send_start, list_fill, send_index);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

int rd_ep_send_list(const void* x, int top_k, int row_bytes, const int32_t* send_index,
                    const int32_t* send_start, int phase, int world, int max_rows,
                    const int32_t* dest_pos, void* dest_base, int capacity_rows, int32_t* phase_done,
                    int32_t* dest_ready_flag, int epoch, void* stream) {
  if (top_k <= 0 || row_bytes <= 0 || (row_bytes & 15) || world <= 0 || phase < 0 || phase >= world ||
      max_rows < 0 || capacity_rows < 0)
    return RD_ERR_BAD_SHAPE;
  if (!aligned16(dest_base) || !send_index || !send_start || !dest_pos || !phase_done ||
      !dest_ready_flag || (max_rows > 0 && !aligned16(x)))
    return RD_ERR_BAD_POINTER;
  const int warps_per_block = rd::kEpThreads / 32;
  int blocks = (max_rows + warps_per_block - 1) / warps_per_block;
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;  // the flag is raised even when the list is empty
  rd::ep_send_list_kernel<<<blocks, rd::kEpThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), top_k, row_bytes / 16, send_index, send_start, phase, dest_pos,
      static_cast<uint4*>(dest_base), capacity_rows, phase_done, dest_ready_flag, epoch);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

int rd_ep_combine_pull(const int32_t* routing, const int32_t* dest_pos, int tokens, int top_k,
                       int row_bytes, int num_experts, int world, const uint64_t* peer_base,
                       int capacity_rows, int dtype, void* out, int max_blocks, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (dtype != RD_DTYPE_F16 && dtype != RD_DTYPE_BF16) return RD_ERR_BAD_DTYPE;
  if (tokens < 0 || top_k <= 0 || top_k > 8 || row_bytes <= 0 || (row_bytes & 15) || world <= 0 ||
      num_experts <= 0 || num_experts % world != 0 || capacity_rows < 0)
    return RD_ERR_BAD_SHAPE;
  if (tokens == 0) return RD_OK;
  if (!routing || !dest_pos || !peer_base || !aligned16(out)) return RD_ERR_BAD_POINTER;
  const int warps_per_block = rd::kEpThreads / 32;
  int blocks = (tokens + warps_per_block - 1) / warps_per_block;
  const int cap = max_blocks > 0 ? max_blocks : sm_count() * 8;
  if (blocks > cap) blocks = cap;
  const int vecs = row_bytes / 16, local = num_experts / world;
  uint4* o = static_cast<uint4*>(out);
#define RD_COMBINE(BF, TK)                                                                          \
  rd::ep_combine_pull_kernel<BF, TK><<<blocks, rd::kEpThreads, 0, stream>>>(                        \
      routing, dest_pos, tokens, top_k, vecs, num_experts, local, peer_base, capacity_rows, o)
  const bool bf = dtype == RD_DTYPE_BF16;
  if (top_k <= 2) { if (bf) RD_COMBINE(true, 2); else RD_COMBINE(false, 2); }
  else if (top_k <= 4) { if (bf) RD_COMBINE(true, 4); else RD_COMBINE(false, 4); }
  else { if (bf) RD_COMBINE(true, 8); else RD_COMBINE(false, 8); }
#undef RD_COMBINE
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

int rd_gmm_indexed_when_ready(const void* x, const void* A, int num_weights, const int32_t* group_sizes,
                              const int32_t* group_to_weight, void* y, void* workspace,
                              size_t workspace_bytes, int m, int k, int n, int g, int trans_rhs,
                              int dtype, const rd_tile_cfg* cfg, const int32_t* ready_flags,
                              int groups_per_flag, int epoch, void* stream) {
  if (g > 0 && group_to_weight == nullptr) return RD_ERR_BAD_POINTER;
  if (ready_flags == nullptr) return RD_ERR_BAD_POINTER;
  if (groups_per_flag <= 0) return RD_ERR_BAD_SHAPE;
  if (cfg && cfg->cta_group == 2) return RD_ERR_BAD_CONFIG;  // CTA pairs do not wait on flags
  return gmm_impl(x, A, group_sizes, group_to_weight, num_weights, y, workspace, workspace_bytes, m, k,
                  n, g, trans_rhs, dtype, cfg, stream, ReadyFlags{ready_flags, groups_per_flag, epoch});
}

int rd_ep_dispatch(const void* x, const int32_t* routing, int tokens, int top_k, int row_bytes,
                   int num_experts, int world, const int32_t* dest_offset, int32_t* fill,
                   const uint64_t* peer_base, int capacity_rows, int32_t* dest_pos, void* stream) {
  if (tokens < 0 || top_k <= 0 || row_bytes <= 0 || (row_bytes & 15) || world <= 0 ||
      num_experts <= 0 || num_experts % world != 0 || capacity_rows < 0)
    return RD_ERR_BAD_SHAPE;
  if (tokens == 0) return RD_OK;
  if (!aligned16(x) || !routing || !dest_offset || !fill || !peer_base || !dest_pos)
    return RD_ERR_BAD_POINTER;
  const long long entries = static_cast<long long>(tokens) * top_k;
  const int warps_per_block = rd::kEpThreads / 32;
  long long blocks = (entries + warps_per_block - 1) / warps_per_block;
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  rd::ep_dispatch_kernel<<<static_cast<int>(blocks), rd::kEpThreads, 0,
                           static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), routing, tokens, top_k, row_bytes / 16, num_experts,
      num_experts / world, dest_offset, fill, peer_base, capacity_rows, dest_pos);
  return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
}

// Shared body of rd_tgmm / rd_tgmm_strided: `g` output blocks, block i contracting over the rows
// of groups i, i + g, ..., i + (seg_count - 1) * g of group_sizes (seg_count * g entries).
static int tgmm_impl(const void* x, const void* dout, const int32_t* group_sizes, void* out,
                     void* workspace, size_t workspace_bytes, int m, int k, int n, int g, int seg_count,
                     int dtype, const rd_tile_cfg* cfg, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (seg_count < 1 || (seg_count > 1 && g > 0 && seg_count > 0x7fffffff / g)) return RD_ERR_BAD_SHAPE;
  const int g_fine = g * seg_count;
  if (dtype != RD_DTYPE_F16 && dtype != RD_DTYPE_BF16 && dtype != RD_DTYPE_F32) return RD_ERR_BAD_DTYPE;
  const bool f32 = dtype == RD_DTYPE_F32;
  const int esize = f32 ? 4 : 2;
  const int amask = f32 ? 3 : 7;
  const int row_elems = 128 / esize;
  if (m < 0 || k < 0 || n < 0 || g < 0 || (k & amask) || (n & amask)) return RD_ERR_BAD_SHAPE;
  if (g == 0 || k == 0 || n == 0) return RD_OK;
  if (!aligned16(out)) return RD_ERR_BAD_POINTER;
  if (m == 0) {  // every group is empty
    cudaMemsetAsync(out, 0, static_cast<size_t>(g) * k * n * esize, stream);
    return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
  }
  if (!aligned16(x) || !aligned16(dout) || group_sizes == nullptr) return RD_ERR_BAD_POINTER;
  Workspace w;
  int rc = bind_workspace(workspace, workspace_bytes, m, g_fine, &w);
  if (rc != RD_OK) return rc;

  const int sms = sm_count();
  int bn = cfg && cfg->tile_n
               ? cfg->tile_n
               : choose_tile_n(static_cast<long long>((k + rd::kTileM - 1) / rd::kTileM) * g, n, sms);
  if (bn != 64 && bn != 128 && bn != 256) return RD_ERR_BAD_CONFIG;
  int cta_group = cfg ? cfg->cta_group : 0;
  int tile_m = cfg ? cfg->tile_m : 0;
  if (cta_group < 0 || cta_group > 2 || (cta_group == 2 && bn != 256)) return RD_ERR_BAD_CONFIG;
  if (tile_m != 0 && tile_m != 128 && tile_m != 256) return RD_ERR_BAD_CONFIG;
  if (tile_m == 256 && bn != 256) return RD_ERR_BAD_CONFIG;
  if (f32) {  // the float32 (TF32) kernels exist as single-CTA 128-row tiles only
    if (cta_group == 2 || tile_m == 256 || seg_count > 1) return RD_ERR_BAD_CONFIG;
    cta_group = 1;
    tile_m = 128;
  }
  if (seg_count > 1) {  // strided segments: one CTA per tile
    if (cta_group == 2) return RD_ERR_BAD_CONFIG;
    cta_group = 1;
  }
  // Preference order when nothing is forced: 256-row tiles on one CTA, then a CTA pair, then
  // plain 128-row tiles.
  if (tile_m == 0 && cta_group != 2) tile_m = choose_two_half(true, m, k, g, bn) ? 256 : 128;
  if (tile_m == 0) tile_m = 128;
  if (cta_group == 0) {
    if (tile_m == 256) {
      cta_group = (seg_count == 1 && choose_pair_512(m, k, g)) ? 2 : 1;
    } else {
      cta_group = choose_pair(true, static_cast<long long>((k + 255) / 256) * g * ((n + 255) / 256), bn, sms)
                      ? 2
                      : 1;
    }
  }
  const bool two_half = tile_m == 256;
  const int tile_rows = two_half ? rd::kG2TileRows * cta_group : rd::kTileM * cta_group;
  const long long k_tiles = (k + tile_rows - 1) / tile_rows;

  // Launch the metadata kernel before encoding the tensor maps: besides being the first step
  // of the call, a runtime launch binds the device's primary context to the calling thread,
  // which the driver's tensor-map encoder needs (threads such as torch's autograd workers
  // arrive here without one).
  launch_internal_metadata(group_sizes, nullptr, g_fine, m, rd::kTileM, w, stream);
  if (cudaGetLastError() != cudaSuccess) return RD_ERR_LAUNCH;

  // 256-row tiles fetch each operand of a stage with one box when the 64-column blocks tile the
  // rows exactly (see rd_gemm2.cuh); otherwise one 2-D box per 64 columns.
  const bool blocked = two_half && !f32 && k % 64 == 0 && n % 64 == 0;
  CUtensorMap ta, tb;
  if (blocked) {
    rc = encode_blocked_map(&ta, x, dtype, k, m, rd::kTileK, rd::kG2TileRows / 64);
    if (rc != RD_OK) return rc;
    rc = encode_blocked_map(&tb, dout, dtype, n, m, rd::kTileK, rd::kG2TileN / 64 / cta_group);
    if (rc != RD_OK) return rc;
  } else {
    {
      const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(m)};
      const uint32_t box[2] = {static_cast<uint32_t>(row_elems), static_cast<uint32_t>(row_elems)};
      rc = encode_map(&ta, x, dtype, 2, dims, box, /*atom32=*/f32);
      if (rc != RD_OK) return rc;
    }
    {
      const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(m)};
      const uint32_t box[2] = {static_cast<uint32_t>(row_elems), static_cast<uint32_t>(row_elems)};
      rc = encode_map(&tb, dout, dtype, 2, dims, box, /*atom32=*/f32);
      if (rc != RD_OK) return rc;
    }
  }

  CUtensorMap tout;
  {  // out[g, k, n] written as [32 rows][128 B] boxes of one group
    const uint64_t dims[3] = {static_cast<uint64_t>(n), static_cast<uint64_t>(k),
                              static_cast<uint64_t>(g)};
    const uint32_t box[3] = {static_cast<uint32_t>(row_elems), 32, 1};
    rc = encode_map(&tout, out, dtype, 3, dims, box);
    if (rc != RD_OK) return rc;
  }

  GemmArgs args = {};
  args.m = m; args.k = k; args.n = n; args.g = g;
  args.n_tiles = (n + bn - 1) / bn;
  args.k_tiles = static_cast<int>(k_tiles);
  args.seg_count = seg_count;
  args.seg_stride = g;
  args.blocked_maps = blocked ? 1 : 0;
  args.max_m_tiles = w.layout.max_tiles;
  args.ab_format = dtype;
  args.wait_limit_us = wait_limit_us(cfg);
  args.zero_tail = 0;
  args.group_sizes = group_sizes;
  args.group_offsets = w.group_offsets();
  args.tile_rec = w.tile_rec();
  args.totals = w.totals();
  args.status = w.status();
  args.out = out;

  const int ctas = pick_ctas(cfg);
  if (f32) {
    if (bn == 256) return launch_gemm_f32<256, false, true>(ta, tb, tout, args, ctas, stream);
    if (bn == 128) return launch_gemm_f32<128, false, true>(ta, tb, tout, args, ctas, stream);
    return launch_gemm_f32<64, false, true>(ta, tb, tout, args, ctas, stream);
  }
  if (two_half && cta_group == 2) return launch_gemm2_pair(ta, tb, tout, args, ctas, stream);
  if (two_half) return launch_gemm2<false, true>(ta, tb, tout, args, ctas, stream);
  if (seg_count > 1) {
    if (bn == 256) return launch_gemm<256, false, true, 1, true>(ta, tb, tout, args, ctas, stream);
    if (bn == 128) return launch_gemm<128, false, true, 1, true>(ta, tb, tout, args, ctas, stream);
    return launch_gemm<64, false, true, 1, true>(ta, tb, tout, args, ctas, stream);
  }
  if (cta_group == 2) return launch_gemm<256, false, true, 2>(ta, tb, tout, args, ctas, stream);
  if (bn == 256) return launch_gemm<256, false, true, 1>(ta, tb, tout, args, ctas, stream);
  if (bn == 128) return launch_gemm<128, false, true, 1>(ta, tb, tout, args, ctas, stream);
  return launch_gemm<64, false, true, 1>(ta, tb, tout, args, ctas, stream);
}

int rd_tgmm(const void* x, const void* dout, const int32_t* group_sizes, void* out,
            void* workspace, size_t workspace_bytes, int m, int k, int n, int g, int dtype,
            const rd_tile_cfg* cfg, void* stream) {
  return tgmm_impl(x, dout, group_sizes, out, workspace, workspace_bytes, m, k, n, g, 1, dtype, cfg, stream);
}

int rd_tgmm_strided(const void* x, const void* dout, const int32_t* group_sizes, void* out,
                    void* workspace, size_t workspace_bytes, int m, int k, int n, int g, int seg_count,
                    int dtype, const rd_tile_cfg* cfg, void* stream) {
  return tgmm_impl(x, dout, group_sizes, out, workspace, workspace_bytes, m, k, n, g, seg_count, dtype, cfg,
                   stream);
}

int rd_gmm_permuted(const void* x, int x_rows, const int32_t* in_rows, const void* A, int num_weights,
                    const int32_t* group_sizes, const int32_t* group_to_weight, void* y, int y_rows,
                    const int32_t* out_rows, void* workspace, size_t workspace_bytes, int m, int k,
                    int n, int g, int trans_rhs, int dtype, const rd_tile_cfg* cfg, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (dtype != RD_DTYPE_F16 && dtype != RD_DTYPE_BF16) return RD_ERR_BAD_DTYPE;
  if (m < 0 || k < 0 || n < 0 || g < 0 || num_weights < 0 || x_rows < 0 || y_rows < 0 || (k & 7) ||
      (n & 7))
    return RD_ERR_BAD_SHAPE;
  if (in_rows == nullptr && x_rows < m) return RD_ERR_BAD_SHAPE;
  if (out_rows == nullptr && y_rows != m) return RD_ERR_BAD_SHAPE;
  if (m == 0 || n == 0 || y_rows == 0) return RD_OK;
  if (!aligned16(y)) return RD_ERR_BAD_POINTER;
  if (g == 0 || k == 0 || num_weights == 0 || x_rows == 0) {
    // Nothing contributes.  Without out_rows every row of y is a zero row; with out_rows the
    // rows that would have been written are not known without reading the indices, and the
    // call leaves y alone only if there is no group at all.
    if (out_rows == nullptr || g == 0) {
      if (out_rows == nullptr) cudaMemsetAsync(y, 0, static_cast<size_t>(m) * n * 2, stream);
      return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
    }
    return RD_ERR_BAD_SHAPE;
  }
  if (!aligned16(x) || !aligned16(A) || group_sizes == nullptr) return RD_ERR_BAD_POINTER;
  if (group_to_weight == nullptr && num_weights != g) return RD_ERR_BAD_SHAPE;
  Workspace w;
  int rc = bind_workspace(workspace, workspace_bytes, m, g, &w);
  if (rc != RD_OK) return rc;
  int bn = cfg && cfg->tile_n ? cfg->tile_n : choose_tile_n(0, n, 0);
  if (bn != 64 && bn != 128 && bn != 256) return RD_ERR_BAD_CONFIG;
  if (cfg && (cfg->cta_group == 2 || cfg->tile_m == 256)) return RD_ERR_BAD_CONFIG;

  launch_internal_metadata(group_sizes, group_to_weight, g, m, rd::kTileM, w, stream);
  if (cudaGetLastError() != cudaSuccess) return RD_ERR_LAUNCH;

  CUtensorMap ta, tb, tout;
  rc = encode_rows_map(&ta, x, dtype, k, x_rows, rd::kTileM);
  if (rc != RD_OK) return rc;
  if (trans_rhs) {
    const uint64_t dims[3] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n),
                              static_cast<uint64_t>(num_weights)};
    const uint32_t box[3] = {64, static_cast<uint32_t>(bn), 1};
    rc = encode_map(&tb, A, dtype, 3, dims, box);
  } else {
    const uint64_t dims[3] = {static_cast<uint64_t>(n), static_cast<uint64_t>(k),
                              static_cast<uint64_t>(num_weights)};
    const uint32_t box[3] = {64, 64, 1};
    rc = encode_map(&tb, A, dtype, 3, dims, box);
  }
  if (rc != RD_OK) return rc;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(y_rows)};
    const uint32_t box[2] = {64, 32};
    rc = encode_map(&tout, y, dtype, 2, dims, box);
    if (rc != RD_OK) return rc;
  }

  GemmArgs args = {};
  args.m = m; args.k = k; args.n = n; args.g = g;
  args.n_tiles = (n + bn - 1) / bn;
  args.k_tiles = 0;
  args.max_m_tiles = w.layout.max_tiles;
  args.ab_format = dtype;
  args.wait_limit_us = wait_limit_us(cfg);
  args.zero_tail = (cfg && (cfg->flags & RD_CFG_NO_ZERO_TAIL)) ? 0 : 1;
  args.group_sizes = group_sizes;
  args.group_offsets = w.group_offsets();
  args.tile_rec = w.tile_rec();
  args.totals = w.totals();
  args.status = w.status();
  args.out = y;
  rd::PermArgs perm;
  perm.a_rows = in_rows;
  perm.a_base = x;
  perm.a_rows_in = x_rows;
  perm.b_rows = nullptr;
  perm.b_base = nullptr;
  perm.b_rows_in = 0;
  perm.out_rows = out_rows;
  perm.out_rows_n = y_rows;

  const int ctas = pick_ctas(cfg);
  if (trans_rhs) {
    if (bn == 256) return launch_gemm_perm<256, true, false>(ta, tb, tout, args, perm, ctas, stream);
    if (bn == 128) return launch_gemm_perm<128, true, false>(ta, tb, tout, args, perm, ctas, stream);
    return launch_gemm_perm<64, true, false>(ta, tb, tout, args, perm, ctas, stream);
  }
  if (bn == 256) return launch_gemm_perm<256, false, false>(ta, tb, tout, args, perm, ctas, stream);
  if (bn == 128) return launch_gemm_perm<128, false, false>(ta, tb, tout, args, perm, ctas, stream);
  return launch_gemm_perm<64, false, false>(ta, tb, tout, args, perm, ctas, stream);
}

int rd_tgmm_permuted(const void* x, int x_rows, const int32_t* x_row_index, const void* dout,
                     int dout_rows, const int32_t* dout_row_index, const int32_t* group_sizes,
                     void* out, void* workspace, size_t workspace_bytes, int m, int k, int n, int g,
                     int dtype, const rd_tile_cfg* cfg, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (dtype != RD_DTYPE_F16 && dtype != RD_DTYPE_BF16) return RD_ERR_BAD_DTYPE;
  if (m < 0 || k < 0 || n < 0 || g < 0 || x_rows < 0 || dout_rows < 0 || (k & 7) || (n & 7))
    return RD_ERR_BAD_SHAPE;
  if ((x_row_index == nullptr && x_rows < m) || (dout_row_index == nullptr && dout_rows < m))
    return RD_ERR_BAD_SHAPE;
  if (g == 0 || k == 0 || n == 0) return RD_OK;
  if (!aligned16(out)) return RD_ERR_BAD_POINTER;
  if (m == 0 || x_rows == 0 || dout_rows == 0) {
    cudaMemsetAsync(out, 0, static_cast<size_t>(g) * k * n * 2, stream);
    return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
  }
  if (!aligned16(x) || !aligned16(dout) || group_sizes == nullptr) return RD_ERR_BAD_POINTER;
  Workspace w;
  int rc = bind_workspace(workspace, workspace_bytes, m, g, &w);
  if (rc != RD_OK) return rc;
  int bn = cfg && cfg->tile_n ? cfg->tile_n : choose_tile_n(0, n, 0);
  if (bn != 64 && bn != 128 && bn != 256) return RD_ERR_BAD_CONFIG;
  if (cfg && (cfg->cta_group == 2 || cfg->tile_m == 256)) return RD_ERR_BAD_CONFIG;

  launch_internal_metadata(group_sizes, nullptr, g, m, rd::kTileM, w, stream);
  if (cudaGetLastError() != cudaSuccess) return RD_ERR_LAUNCH;

  CUtensorMap ta, tb, tout;
  rc = encode_rows_map(&ta, x, dtype, k, x_rows, 64);
  if (rc != RD_OK) return rc;
  rc = encode_rows_map(&tb, dout, dtype, n, dout_rows, 64);
  if (rc != RD_OK) return rc;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(n), static_cast<uint64_t>(k),
                              static_cast<uint64_t>(g)};
    const uint32_t box[3] = {64, 32, 1};
    rc = encode_map(&tout, out, dtype, 3, dims, box);
    if (rc != RD_OK) return rc;
  }

  GemmArgs args = {};
  args.m = m; args.k = k; args.n = n; args.g = g;
  args.n_tiles = (n + bn - 1) / bn;
  args.k_tiles = (k + rd::kTileM - 1) / rd::kTileM;
  args.max_m_tiles = w.layout.max_tiles;
  args.ab_format = dtype;
  args.wait_limit_us = wait_limit_us(cfg);
  args.zero_tail = 0;
  args.group_sizes = group_sizes;
  args.group_offsets = w.group_offsets();
  args.tile_rec = w.tile_rec();
  args.totals = w.totals();
  args.status = w.status();
  args.out = out;
  rd::PermArgs perm;
  perm.a_rows = x_row_index;
  perm.a_base = x;
  perm.a_rows_in = x_rows;
  perm.b_rows = dout_row_index;
  perm.b_base = dout;
  perm.b_rows_in = dout_rows;
  perm.out_rows = nullptr;
  perm.out_rows_n = 0;

  const int ctas = pick_ctas(cfg);
  if (bn == 256) return launch_gemm_perm<256, false, true>(ta, tb, tout, args, perm, ctas, stream);
  if (bn == 128) return launch_gemm_perm<128, false, true>(ta, tb, tout, args, perm, ctas, stream);
  return launch_gemm_perm<64, false, true>(ta, tb, tout, args, perm, ctas, stream);
}

int rd_gmm_ep_fused(const void* x, const void* A, int num_weights, const int32_t* group_sizes,
                    const int32_t* group_to_weight, void* y, void* workspace, size_t workspace_bytes,
                    int m, int k, int n, int g, int trans_rhs, int dtype, const rd_tile_cfg* cfg,
                    const int32_t* ready_flags, int groups_per_flag, int epoch, const rd_ep_send* send,
                    void* stream) {
  if (g > 0 && group_to_weight == nullptr) return RD_ERR_BAD_POINTER;
  if (ready_flags == nullptr || send == nullptr) return RD_ERR_BAD_POINTER;
  if (groups_per_flag <= 0 || send->world <= 0 || send->rank < 0 ||
      send->rank >= send->world || send->row_bytes <= 0 || (send->row_bytes & 15) || send->top_k <= 0 ||
      send->sender_ctas <= 0 || send->capacity_rows < 0)
    return RD_ERR_BAD_SHAPE;
  if (m == 0 || n == 0 || g == 0 || k == 0) return RD_ERR_BAD_SHAPE;  // the sender role needs a launch
  if (!aligned16(send->x_tokens) || !send->send_index || !send->send_start || !send->dest_pos ||
      !send->phase_done || !send->peer_base || !send->peer_flags)
    return RD_ERR_BAD_POINTER;
  rd::EpSendArgs a = {};
  a.x = static_cast<const uint8_t*>(send->x_tokens);
  a.send_index = send->send_index;
  a.send_start = send->send_start;
  a.dest_pos = send->dest_pos;
  a.phase_done = send->phase_done;
  a.peer_base = send->peer_base;
  a.peer_flags = send->peer_flags;
  a.row_bytes = send->row_bytes;
  a.top_k = send->top_k;
  a.world = send->world;
  a.rank = send->rank;
  a.capacity_rows = send->capacity_rows;
  a.sender_ctas = send->sender_ctas;
  return gmm_impl(x, A, group_sizes, group_to_weight, num_weights, y, workspace, workspace_bytes, m, k,
                  n, g, trans_rhs, dtype, cfg, stream, ReadyFlags{ready_flags, groups_per_flag, epoch}, &a);
}

int rd_ep_fused_forward(const rd_ep_step* st, const void* recv, const void* A, int num_weights,
                        const int32_t* group_to_weight, void* y, void* workspace, size_t workspace_bytes,
                        int capacity_rows, int k, int n, int dtype, const rd_tile_cfg* cfg,
                        const int32_t* ready_flags, const rd_ep_send* send, void* stream) {
  if (st == nullptr || send == nullptr) return RD_ERR_BAD_POINTER;
  const int world = send->world, rank = send->rank;
  if (world < 2 || st->tokens < 0 || st->top_k <= 0 || st->num_experts <= 0 || st->num_experts % world != 0)
    return RD_ERR_BAD_SHAPE;
  const int entries = st->tokens * st->top_k;
  const int local = st->num_experts / world;
  int rc = rd_ep_count_share(st->routing, entries, st->num_experts, st->counts_scratch, st->ticket, world,
                             rank, st->peer_counts, st->peer_count_flags, st->epoch, stream);
  if (rc != RD_OK) return rc;
  rc = rd_ep_plan_ring_when_counted(st->counts_all, st->count_flags, st->epoch, world, st->num_experts, rank,
                                    st->dest_offset, st->segment_sizes, st->fill, st->totals,
                                    send->phase_done, st->send_start, st->list_fill, st->plan_status,
                                    st->wait_limit_ms, stream);
  if (rc != RD_OK) return rc;
  rc = rd_ep_assign(st->routing, entries, st->num_experts, world, rank, st->dest_offset, st->fill,
                    capacity_rows, st->dest_pos, st->send_start, st->list_fill, st->send_index, stream);
  if (rc != RD_OK) return rc;
  rc = rd_ep_send_list(send->x_tokens, st->top_k, send->row_bytes, st->send_index, st->send_start, 0, world,
                       entries, st->dest_pos, st->own_buffer, capacity_rows, send->phase_done,
                       st->own_ready_flag, st->epoch, stream);
  if (rc != RD_OK) return rc;
  return rd_gmm_ep_fused(recv, A, num_weights, st->segment_sizes, group_to_weight, y, workspace,
                         workspace_bytes, capacity_rows, k, n, world * local, 0, dtype, cfg, ready_flags, local,
                         st->epoch, send, stream);
}

int rd_gmm_fp8(const void* x, const void* A, int num_weights, const int32_t* group_sizes,
               const int32_t* group_to_weight, const float* weight_scale, void* y, void* workspace,
               size_t workspace_bytes, int m, int k, int n, int g, const rd_tile_cfg* cfg, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  // rows of k one-byte elements and of n two-byte results must be multiples of 16 bytes
  if (m < 0 || k < 0 || n < 0 || g < 0 || num_weights < 0 || (k & 15) || (n & 7)) return RD_ERR_BAD_SHAPE;
  if (group_to_weight == nullptr && num_weights != g) return RD_ERR_BAD_SHAPE;
  if (m == 0 || n == 0) return RD_OK;
  if (!aligned16(y)) return RD_ERR_BAD_POINTER;
  if (g == 0 || k == 0 || num_weights == 0) {
    cudaMemsetAsync(y, 0, static_cast<size_t>(m) * n * 2, stream);
    return cudaGetLastError() == cudaSuccess ? RD_OK : RD_ERR_LAUNCH;
  }
  if (!aligned16(x) || !aligned16(A) || group_sizes == nullptr) return RD_ERR_BAD_POINTER;
  Workspace w;
  int rc = bind_workspace(workspace, workspace_bytes, m, g, &w);
  if (rc != RD_OK) return rc;
  int bn = cfg && cfg->tile_n ? cfg->tile_n : choose_tile_n(0, n, 0);
  if (bn != 64 && bn != 128 && bn != 256) return RD_ERR_BAD_CONFIG;
  if (cfg && (cfg->cta_group == 2 || cfg->tile_m == 256)) return RD_ERR_BAD_CONFIG;  // 128-row tiles only

  launch_internal_metadata(group_sizes, group_to_weight, g, m, rd::kTileM, w, stream,
                           cfg != nullptr && (cfg->flags & RD_CFG_GROUP_BY_WEIGHT) != 0);
  if (cudaGetLastError() != cudaSuccess) return RD_ERR_LAUNCH;

  // Both operands are K-major, so a row of k one-byte elements is described to TMA as k/2
  // two-byte elements: the bytes that land in shared memory are the same.
  const int k2 = k / 2;
  CUtensorMap ta, tb, tout;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(k2), static_cast<uint64_t>(m)};
    const uint32_t box[2] = {64, rd::kTileM};
    rc = encode_map(&ta, x, RD_DTYPE_BF16, 2, dims, box);
    if (rc != RD_OK) return rc;
  }
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(k2), static_cast<uint64_t>(n),
                              static_cast<uint64_t>(num_weights)};
    const uint32_t box[3] = {64, static_cast<uint32_t>(bn), 1};
    rc = encode_map(&tb, A, RD_DTYPE_BF16, 3, dims, box);
    if (rc != RD_OK) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(m)};
    const uint32_t box[2] = {64, 32};
    rc = encode_map(&tout, y, RD_DTYPE_BF16, 2, dims, box);
    if (rc != RD_OK) return rc;
  }
  GemmArgs args = {};
  args.m = m; args.k = k2; args.n = n; args.g = g;
  args.n_tiles = (n + bn - 1) / bn;
  args.max_m_tiles = w.layout.max_tiles;
  args.ab_format = RD_DTYPE_BF16;  // type of the output
  args.wait_limit_us = wait_limit_us(cfg);
  args.weight_scale = weight_scale;
  args.zero_tail = (cfg && (cfg->flags & RD_CFG_NO_ZERO_TAIL)) ? 0 : 1;
  args.group_sizes = group_sizes;
  args.group_offsets = w.group_offsets();
  args.tile_rec = w.tile_rec();
  args.totals = w.totals();
  args.status = w.status();
  args.out = y;
  args.groups_per_flag = 1;
  const int ctas = pick_ctas(cfg);
  if (bn == 256) return launch_gemm<256, true, false, 1, false, true>(ta, tb, tout, args, ctas, stream);
  if (bn == 128) return launch_gemm<128, true, false, 1, false, true>(ta, tb, tout, args, ctas, stream);
  return launch_gemm<64, true, false, 1, false, true>(ta, tb, tout, args, ctas, stream);
}

int rd_device_status(const void* workspace, void* stream) {
  if (workspace == nullptr) return RD_ERR_BAD_POINTER;
  int32_t word = 0;
  cudaError_t e = cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost,
                                  static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return RD_ERR_LAUNCH;
  e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return RD_ERR_LAUNCH;
  return word == 0 ? RD_OK : RD_ERR_DEVICE_WAIT;
}

}  // extern "C"

// ------------------------------------------------------------------ entry point that allocates nothing
//
// Some hosts of this library can neither hand over a workspace nor create one: an operator slot
// whose argument list is frozen to "inputs and outputs" (a legacy custom-call interface, a
// plugin ABI defined by someone else), running inside a framework that has reserved the whole
// device for its own allocator -- there a cudaMalloc from inside the call may fail, and where it
// succeeds it synchronises the device and stalls every stream.  For them rd_gmm_static_scratch
// keeps the group-metadata scratch in a fixed array inside this library's device image.
//
// The array costs kStaticScratchBytes (64 KiB) on every GPU that loads the library, until the
// process exits.  It is one array per device, shared by every call: it still holds whatever the
// previous call left there, so the header words the kernels accumulate into are cleared at the
// start of each call, and two calls that overlap on the GPU (different streams, no ordering
// between them) race on it -- serialise them, or use rd_gmm with separate workspaces.
namespace {

constexpr size_t kStaticScratchWords = 16384;
constexpr size_t kStaticScratchBytes = kStaticScratchWords * sizeof(int32_t);

static __device__ __align__(256) int32_t g_static_scratch[kStaticScratchWords];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the
// address a kernel can use has to be asked for, per device, with that device current.
int static_scratch_address(int32_t** out) {
  static std::mutex mu;
  static int32_t* per_device[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return RD_ERR_SCRATCH_SETUP;
  std::lock_guard<std::mutex> lock(mu);
  if (per_device[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      fprintf(stderr, "ragged_dot_b200: cudaGetSymbolAddress(scratch) failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return RD_ERR_SCRATCH_SETUP;
    }
    per_device[dev] = static_cast<int32_t*>(ptr);
  }
  *out = per_device[dev];
  return RD_OK;
}

}  // namespace

extern "C" int rd_gmm_static_scratch(const void* x, const void* A, const int32_t* group_sizes,
                                     void* y, int m, int k, int n, int g, int trans_rhs, int dtype,
                                     const rd_tile_cfg* cfg, void* stream) {
  if (m < 0 || g < 0) return RD_ERR_BAD_SHAPE;
  WorkspaceLayout layout;
  layout.g = g;
  layout.max_tiles = max_row_tiles(m, g);
  if (static_cast<size_t>(layout.total_words()) > kStaticScratchWords) return RD_ERR_TOO_LARGE;
  int32_t* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc != RD_OK) return rc;
  // The array keeps the last call's contents: start this call's status and totals from zero.
  if (cudaMemsetAsync(scratch, 0, 8 * sizeof(int32_t), static_cast<cudaStream_t>(stream)) !=
      cudaSuccess)
    return RD_ERR_LAUNCH;
  return rd_gmm(x, A, group_sizes, y, scratch, kStaticScratchBytes, m, k, n, g, trans_rhs, dtype, cfg,
                stream);
}
