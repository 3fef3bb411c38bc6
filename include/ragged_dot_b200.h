/* ragged_dot_b200.h -- C ABI of the B200 (sm_100a) ragged-dot library.
 *
 * Every entry point is stream-ordered and asynchronous: it validates its arguments on the
 * host, enqueues kernels on `stream` and returns.  Nothing here allocates or frees device
 * memory, synchronises the device or copies group_sizes to the host (group_sizes is a
 * run-time device value, as in the reference where the metadata is computed inside the jit,
 * gpu_ragged_dot.py:203).  All buffers, the workspace included, are owned by the caller.
 *
 * Return value: RD_OK (0) when the work was enqueued, otherwise one of the RD_ERR_* codes;
 * rd_status_string() gives the text.  Nothing throws, exits or traps.  Conditions only the
 * device can see (a bounded wait that expired) are recorded in the workspace and read back
 * with rd_device_status().
 *
 * Shapes follow the reference's signature (gpu_ragged_dot.py:362-376, README.md:52-67):
 *   x            [m, k]      row-major, f16 / bf16 / f32 (all tensors of a call share the type)
 *   A            [g, k, n]   (trans_rhs == 0)  or  [g, n, k]  (trans_rhs != 0)
 *   group_sizes  [g]         int32, sum <= m; rows past the sum are written as zeros
 *   y            [m, n]
 * Rows of k and of n elements must be multiples of 16 bytes (k, n multiples of 8 for 16-bit
 * types, of 4 for f32) and every pointer 16-byte aligned (TMA strides); the Python host layer
 * pads other shapes before calling.
 */
#ifndef RAGGED_DOT_B200_H_
#define RAGGED_DOT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RD_VERSION 2

enum rd_error {
  RD_OK = 0,
  RD_ERR_BAD_SHAPE = 1,       /* negative size, or k / n rows not a multiple of 16 bytes */
  RD_ERR_BAD_DTYPE = 2,       /* dtype is not one of rd_dtype */
  RD_ERR_BAD_POINTER = 3,     /* null or not 16-byte aligned */
  RD_ERR_WORKSPACE = 4,       /* workspace smaller than rd_workspace_bytes() */
  RD_ERR_BAD_CONFIG = 5,      /* rd_tile_cfg names a tile the kernels do not have */
  RD_ERR_TENSOR_MAP = 6,      /* the driver rejected a TMA descriptor */
  RD_ERR_LAUNCH = 7,          /* cudaGetLastError() after a launch */
  RD_ERR_DRIVER = 8,          /* driver entry point for tensor-map encoding not found */
  RD_ERR_DEVICE_WAIT = 9,     /* device status: a bounded wait inside a kernel expired */
  RD_ERR_TOO_LARGE = 10,      /* rd_gmm_static_scratch: problem exceeds the built-in scratch */
  RD_ERR_SCRATCH_SETUP = 11   /* rd_gmm_static_scratch: scratch address could not be resolved */
};

/* F32: float32 in and out, multiplied on the tensor cores as TF32 with fp32 accumulation (what
 * the reference's Triton kernel and jax.lax.ragged_dot do for float32 on NVIDIA GPUs). */
enum rd_dtype { RD_DTYPE_F16 = 0, RD_DTYPE_BF16 = 1, RD_DTYPE_F32 = 2 };

/* Tile choice for one call; replaces the reference's block_m/block_k/block_n + tune-jax
 * search (tuning.py:49-58).  Pass NULL to let the library choose.
 *   tile_n    : output columns per tile, one of 64, 128, 256; 0 = library's choice
 *               (the contraction step is always 64).
 *   max_ctas  : cap on the persistent grid (0 = one CTA per SM).
 *   cta_group : 1 = one CTA per tile; 2 = a pair of CTAs per tile, each with half of the B operand
 *               (tile_n must be 256); 0 = library's choice.
 *   tile_m    : 128, or 256 = one CTA computes 256-row tiles as two 128-row halves sharing
 *               each B stage (tile_n must be 256); 0 = library's choice.  With cta_group 2,
 *               tile_m 256 (512-row tiles on a CTA pair) exists for rd_tgmm only.
 *   flags     : RD_CFG_NO_ZERO_TAIL = rd_gmm leaves the rows past sum(group_sizes) unwritten
 *               (for callers that pass an upper bound as m and never read those rows).
 *               RD_CFG_GROUP_BY_WEIGHT = rd_gmm_indexed takes the groups in the order of the weight
 *               matrix they use (stable) instead of in row order, so groups that share a matrix
 *               are multiplied one after the other and it leaves HBM once: for many small
 *               groups over few matrices (the decode-sized expert-parallel step).  Results are
 *               the same; with ready flags a late group may be waited for early.
 *   wait_limit_ms : how long a wait inside a kernel (on a pipeline barrier, on a ready flag of
 *               rd_gmm_indexed_when_ready) may last before the kernel gives up, records
 *               RD_ERR_DEVICE_WAIT in the status word and returns; 0 = the environment variable
 *               RD_WAIT_LIMIT_MS if set, else 2000. */
#define RD_CFG_NO_ZERO_TAIL 1
#define RD_CFG_GROUP_BY_WEIGHT 2
typedef struct rd_tile_cfg {
  int32_t tile_n;
  int32_t max_ctas;
  int32_t cta_group;
  int32_t tile_m;
  int32_t flags;
  int32_t wait_limit_ms;
} rd_tile_cfg;

int rd_version(void);
const char* rd_status_string(int code);

/* Bytes of workspace rd_gmm / rd_tgmm need for a problem with m rows and g groups. */
int rd_workspace_bytes(int m, int g, size_t* bytes);

/* Group metadata: replaces _make_gmm_group_metadata (gpu_ragged_dot.py:70-90).  Writes the
 * reference's arrays for chunk size `chunk_m`, all int32 and all on the device:
 *   group_offsets[g], row_it2group[U], row_it2it_in_group[U], total_row_its[1],
 *   U = ceil(m / chunk_m) + g; entries past total_row_its are 0.  Any output may be NULL. */
int rd_metadata(const int32_t* group_sizes, int g, int m, int chunk_m, int32_t* group_offsets,
                int32_t* row_it2group, int32_t* row_it2it_in_group, int32_t* total_row_its,
                void* stream);

/* Forward grouped GEMM; replaces _gpu_gmm_fwd + _gpu_gmm_kernel (gpu_ragged_dot.py:93-228).
 * With trans_rhs it is also the dlhs half of the backward pass (gpu_ragged_dot.py:400).
 * k is x's second dimension (the contraction), n the output's. */
int rd_gmm(const void* x, const void* A, const int32_t* group_sizes, void* y, void* workspace,
           size_t workspace_bytes, int m, int k, int n, int g, int trans_rhs, int dtype,
           const rd_tile_cfg* cfg, void* stream);

/* rd_gmm with an indirection on the weights: group i multiplies by A[group_to_weight[i]], A is
 * [num_weights, k, n] (or [num_weights, n, k]).  No counterpart in the reference; it serves the
 * expert-parallel path, where the rows received from W source ranks form W * (experts per rank)
 * consecutive segments that share the local experts' weights, so no re-sort is needed after
 * the all-to-all.  group_to_weight is an int32 device array of g entries in [0, num_weights). */
int rd_gmm_indexed(const void* x, const void* A, int num_weights, const int32_t* group_sizes,
                   const int32_t* group_to_weight, void* y, void* workspace, size_t workspace_bytes,
                   int m, int k, int n, int g, int trans_rhs, int dtype, const rd_tile_cfg* cfg,
                   void* stream);

/* rd_gmm_indexed for 8-bit floating-point inputs (e4m3), a Blackwell extension with no counterpart
 * in the reference: x [m, k] and A [num_weights, n, k] (the trans_rhs layout: both operands
 * contiguous along k) hold one-byte e4m3 values, products are exact, accumulation is fp32, and
 * y [m, n] = weight_scale[w] * (x_rows . A[w]^T) is written as bf16 (w = group_to_weight[i], or i
 * when group_to_weight is NULL and num_weights == g; weight_scale NULL = 1; a scale for x is a
 * factor the caller folds into weight_scale).  k must be a multiple of 16, n of 8.  128-row tiles. */
int rd_gmm_fp8(const void* x, const void* A, int num_weights, const int32_t* group_sizes,
               const int32_t* group_to_weight, const float* weight_scale, void* y, void* workspace,
               size_t workspace_bytes, int m, int k, int n, int g, const rd_tile_cfg* cfg, void* stream);

/* dst[i, :] = src[row_index[i], :] for rows of row_bytes (a multiple of 16) bytes: the permute
 * that precedes ragged_dot in an MoE layer (rows replicated per routed expert, sorted by
 * expert).  The reference leaves this step to its caller.  An index outside [0, rows_in)
 * yields a zero row. */
int rd_gather_rows(const void* src, const int32_t* row_index, void* dst, int rows_out, int rows_in,
                   int row_bytes, void* stream);

/* Expert-parallel dispatch without a host round trip (no counterpart in the reference, which
 * has no multi-device code).  E experts are sharded E / world per rank; every rank runs, on
 * its stream:
 *   rd_ep_count     counts[e] = number of (token, slot) pairs of routing[tokens, top_k] that
 *                   name expert e (counts is zeroed first);
 *   (the caller all-gathers the counts of all ranks into counts_all[world][E]);
 *   rd_ep_plan      dest_offset[E], segment_sizes[world * E/world] (the group sizes of the local
 *                   rd_gmm_indexed, segment (s, j) = rows from source s for local expert j),
 *                   totals[0] = rows this rank receives, fill[E] reset;
 *   rd_ep_dispatch  copies every routed row of x straight into the receive buffer of the rank
 *                   that owns its expert: peer_base[r] (a device array of `world` addresses) is
 *                   rank r's buffer as seen from this GPU (peer memory over NVLink, or local
 *                   memory for r == rank); dest_pos[tokens * top_k] records the row position.
 * The caller synchronises the ranks after rd_ep_dispatch (all rows have landed) before the
 * local rd_gmm_indexed reads the buffer, and must not dispatch into a buffer its owner is
 * still reading.  Plain peer stores only: no multicast, no TMA from or to peer memory. */
int rd_ep_count(const int32_t* routing, int entries, int num_experts, int32_t* counts, void* stream);
int rd_ep_plan(const int32_t* counts_all, int world, int num_experts, int rank, int32_t* dest_offset,
               int32_t* segment_sizes, int32_t* fill, int32_t* totals, void* stream);
int rd_ep_dispatch(const void* x, const int32_t* routing, int tokens, int top_k, int row_bytes,
                   int num_experts, int world, const int32_t* dest_offset, int32_t* fill,
                   const uint64_t* peer_base, int capacity_rows, int32_t* dest_pos, void* stream);

/* Expert-parallel exchange running under the local GEMM (no counterpart in the reference).  The
 * receive buffer of rank d is laid out by "position" q = (d - source) mod world: d's own rows
 * first, then those of d-1, d-2, ...; a source sends to rank + p in phase p, so in every phase the
 * ranks form a permutation and each NVLink port carries one flow.
 *   rd_ep_plan_ring       as rd_ep_plan for that layout (segment q*El + j = rows from source
 *                         (rank - q) mod world for local expert j); resets phase_done[world].
 *   rd_gmm_indexed_when_ready  rd_gmm_indexed whose loader, before it reads the rows of group i,
 *                         waits (bounded: expiry gives RD_ERR_DEVICE_WAIT through the status word)
 *                         until ready_flags[i / groups_per_flag] >= epoch.  It multiplies position
 *                         q while positions q+1.. are still arriving.  Epochs must increase from
 *                         call to call; flags start at 0.
 * Whoever raises the flags must be certain to run while this kernel waits: kernels launched
 * separately on the same GPU are NOT (a persistent grid that fills every SM can keep them from
 * ever being placed), which is why the senders of rd_gmm_ep_fused below are CTAs of the same
 * launch.  The caller keeps one exchange in flight per buffer: a rank may start the next exchange
 * only when every rank has finished reading its buffer (e.g. the all-gather of the next counts,
 * issued after the GEMM in stream order).  Plain peer stores and loads of flags only. */
int rd_ep_plan_ring(const int32_t* counts_all, int world, int num_experts, int rank,
                    int32_t* dest_offset, int32_t* segment_sizes, int32_t* fill, int32_t* totals,
                    int32_t* phase_done, int32_t* send_start, int32_t* list_fill, void* stream);
int rd_gmm_indexed_when_ready(const void* x, const void* A, int num_weights, const int32_t* group_sizes,
                              const int32_t* group_to_weight, void* y, void* workspace,
                              size_t workspace_bytes, int m, int k, int n, int g, int trans_rhs,
                              int dtype, const rd_tile_cfg* cfg, const int32_t* ready_flags,
                              int groups_per_flag, int epoch, void* stream);

/* The exchange of the per-expert counts without a collective library (no counterpart in the
 * reference): a small all-gather costs more in launch latency than in bytes.
 *   rd_ep_count_share            rd_ep_count whose last block stores this rank's E counts into row
 *                                `rank` of EVERY rank's counts_all[world][E] (peer_counts[r] = that
 *                                array on rank r as seen from this GPU, its own included) and then
 *                                `epoch` into word `rank` of every rank's count flags (peer_flags[r]).
 *                                counts_scratch[E] and ticket[1] must be zero before the first call;
 *                                every call leaves them zero.
 *   rd_ep_plan_ring_when_counted rd_ep_plan_ring that first waits (bounded; expiry sets *status,
 *                                the workspace status word of the GEMM that follows) until
 *                                count_flags[s] >= epoch for every source s.
 * The pair also orders the buffers' reuse, as the all-gather did: a rank's counts of step t+1
 * leave only after its kernels of step t.  Callers alternate between two counts_all arrays by
 * epoch parity so that a fast rank cannot overwrite counts a slow rank has not planned from. */
int rd_ep_count_share(const int32_t* routing, int entries, int num_experts, int32_t* counts_scratch,
                      int32_t* ticket, int world, int rank, const uint64_t* peer_counts,
                      const uint64_t* peer_flags, int epoch, void* stream);
int rd_ep_plan_ring_when_counted(const int32_t* counts_all, const int32_t* count_flags, int epoch,
                                 int world, int num_experts, int rank, int32_t* dest_offset,
                                 int32_t* segment_sizes, int32_t* fill, int32_t* totals,
                                 int32_t* phase_done, int32_t* send_start, int32_t* list_fill,
                                 int32_t* status, int wait_limit_ms, void* stream);

/* The same exchange with the sending done INSIDE the GEMM kernel (one launch does both): 
 * `sender_ctas` CTAs of the persistent grid push this rank's rows of phases 1 .. world-1 to
 * their owners (bulk async copies global -> shared, plain stores shared -> peer memory, then the
 * owner's ready flag), the other CTAs multiply the positions that have arrived.
 *   rd_ep_plan_ring  with send_start[world + 1] and list_fill[world] (both non-NULL) also sizes the
 *                    per-phase send lists;
 *   rd_ep_assign     dest_pos[i] for every (token, slot) entry and the send lists: entries of phase
 *                    p at send_index[send_start[p] .. send_start[p+1]);
 *   rd_ep_send_list  copies one phase's list with an ordinary kernel and raises the flag; used for
 *                    phase 0 (the rank's own rows), before the fused launch; max_rows bounds the
 *                    list length for the grid size;
 *   rd_gmm_ep_fused  rd_gmm_indexed_when_ready + the sender role.  peer_base[r] / peer_flags[r]
 *                    (device arrays of `world` addresses) are rank r's receive buffer and flag array
 *                    as seen from this GPU.  16-bit types, one CTA per tile (cta_group != 2). */
typedef struct rd_ep_send {
  const void* x_tokens;        /* [tokens, row_bytes] */
  const int32_t* send_index;   /* from rd_ep_assign */
  const int32_t* send_start;   /* from rd_ep_plan_ring */
  const int32_t* dest_pos;     /* from rd_ep_assign */
  int32_t* phase_done;         /* [world], reset by rd_ep_plan_ring */
  const uint64_t* peer_base;   /* device array [world] */
  const uint64_t* peer_flags;  /* device array [world] */
  int32_t row_bytes, top_k, world, rank, capacity_rows, sender_ctas;
} rd_ep_send;
int rd_ep_assign(const int32_t* routing, int entries, int num_experts, int world, int rank,
                 const int32_t* dest_offset, int32_t* fill, int capacity_rows, int32_t* dest_pos,
                 const int32_t* send_start, int32_t* list_fill, int32_t* send_index, void* stream);
int rd_ep_send_list(const void* x, int top_k, int row_bytes, const int32_t* send_index,
                    const int32_t* send_start, int phase, int world, int max_rows,
                    const int32_t* dest_pos, void* dest_base, int capacity_rows, int32_t* phase_done,
                    int32_t* dest_ready_flag, int epoch, void* stream);
int rd_gmm_ep_fused(const void* x, const void* A, int num_weights, const int32_t* group_sizes,
                    const int32_t* group_to_weight, void* y, void* workspace, size_t workspace_bytes,
                    int m, int k, int n, int g, int trans_rhs, int dtype, const rd_tile_cfg* cfg,
                    const int32_t* ready_flags, int groups_per_flag, int epoch, const rd_ep_send* send,
                    void* stream);

/* One call for the whole fused expert-parallel forward step (no counterpart in the reference):
 * rd_ep_count_share, rd_ep_plan_ring_when_counted, rd_ep_assign, rd_ep_send_list (phase 0, the
 * rank's own rows) and rd_gmm_ep_fused, enqueued back to back on `stream` with exactly the
 * arguments those entry points take.  It exists because a decode-sized step is bound by the
 * host's cost of five separate calls, not by the GPU.  world == 1 is not served (nothing to
 * exchange: use rd_ep_count / rd_ep_plan_ring).  Returns the first non-zero status. */
typedef struct rd_ep_step {
  const int32_t* routing;        /* [tokens, top_k] expert ids */
  int32_t tokens, top_k, num_experts, epoch;
  int32_t* counts_scratch;       /* rd_ep_count_share */
  int32_t* ticket;
  const uint64_t* peer_counts;   /* this epoch's table on every rank */
  const uint64_t* peer_count_flags;
  const int32_t* counts_all;     /* this rank's own copy of this epoch's table, [world, num_experts] */
  const int32_t* count_flags;    /* this rank's count flags */
  int32_t* dest_offset;          /* rd_ep_plan_ring outputs */
  int32_t* segment_sizes;
  int32_t* fill;
  int32_t* totals;
  int32_t* send_start;
  int32_t* list_fill;
  int32_t* plan_status;          /* status word of the plan kernel's wait */
  int32_t* dest_pos;             /* rd_ep_assign outputs, [tokens * top_k] */
  int32_t* send_index;
  void* own_buffer;              /* this rank's receive buffer (destination of phase 0) */
  int32_t* own_ready_flag;       /* word 0 of this rank's ready flags */
  int32_t wait_limit_ms;
} rd_ep_step;
int rd_ep_fused_forward(const rd_ep_step* step, const void* recv, const void* A, int num_weights,
                        const int32_t* group_to_weight, void* y, void* workspace, size_t workspace_bytes,
                        int capacity_rows, int k, int n, int dtype, const rd_tile_cfg* cfg,
                        const int32_t* ready_flags, const rd_ep_send* send, void* stream);

/* Transposed grouped GEMM out[g,k,n] = x_g^T . dout_g; replaces _gpu_tgmm_fwd +
 * _gpu_tgmm_kernel (gpu_ragged_dot.py:231-342), the drhs half of the backward pass
 * (gpu_ragged_dot.py:401).  Empty groups produce zero blocks. */
int rd_tgmm(const void* x, const void* dout, const int32_t* group_sizes, void* out,
            void* workspace, size_t workspace_bytes, int m, int k, int n, int g, int dtype,
            const rd_tile_cfg* cfg, void* stream);

/* rd_tgmm over strided segments: group_sizes has g * seg_count entries and output block i
 * (of g) is the sum over q < seg_count of x_s^T . dout_s for the rows of group s = i + q * g.
 * No counterpart in the reference.  It is the drhs of the expert-parallel layout, where the
 * rows received from seg_count source ranks form seg_count * g consecutive segments and segment
 * (q, i) belongs to local expert i: the per-expert weight gradient sums over the sources without
 * re-sorting the rows.  16-bit types; seg_count == 1 is rd_tgmm. */
int rd_tgmm_strided(const void* x, const void* dout, const int32_t* group_sizes, void* out,
                    void* workspace, size_t workspace_bytes, int m, int k, int n, int g, int seg_count,
                    int dtype, const rd_tile_cfg* cfg, void* stream);

/* Reverse exchange of the expert-parallel backward pass fused with the top-k combine (no
 * counterpart in the reference): out[t, :] = sum over the top_k slots s of row
 * dest_pos[t * top_k + s] of the buffer of the rank that owns expert routing[t * top_k + s].
 * peer_base[r] (device array of `world` addresses) is rank r's [capacity_rows, row_bytes] buffer
 * of gradient rows (its rd_gmm_indexed(dout, A, trans_rhs) result over the received layout) as
 * seen from this GPU; rows are pulled with plain peer loads, summed in fp32 and written as one
 * 16-bit row per token.  Slots with an expert outside [0, num_experts) or a position outside
 * [0, capacity_rows) add nothing.  top_k <= 8.  max_blocks caps the grid (0 = eight blocks of
 * 256 threads per SM), for a caller that runs the pull beside another kernel on SMs it has left
 * free.  The caller orders this call after every owner's GEMM (a cross-rank barrier) and keeps
 * the buffers unchanged until every rank has pulled. */
int rd_ep_combine_pull(const int32_t* routing, const int32_t* dest_pos, int tokens, int top_k,
                       int row_bytes, int num_experts, int world, const uint64_t* peer_base,
                       int capacity_rows, int dtype, void* out, int max_blocks, void* stream);

/* Grouped GEMMs with the row permutation of a mixture-of-experts layer fused in.  The
 * reference takes rows that are already sorted by group (gpu_ragged_dot.py:362-376) and leaves
 * x_sorted = x[row_index] and the inverse permutation of the result to its caller; these entry
 * points read and write the un-sorted tensors, so the sorted copies never exist (16-bit types).
 *
 *   rd_gmm_permuted   for r < sum(group_sizes):  y[out_rows[r], :] = x[in_rows[r], :] . W(r)
 *     x        [x_rows, k];  in_rows  [m] int32, values in [0, x_rows), NULL = identity
 *                            (then x_rows >= m);  A / num_weights / group_to_weight as for
 *                            rd_gmm_indexed (group_to_weight NULL = group i uses A[i])
 *     y        [y_rows, n];  out_rows [m] int32, NULL = identity (then y_rows == m and rows past
 *                            sum(group_sizes) are zeroed as in rd_gmm).  With out_rows only the
 *                            rows named are written (entries outside [0, y_rows) are dropped);
 *                            rows named twice hold one of the results.
 *   rd_tgmm_permuted  out[i] = x[x_row_index[rows of group i], :]^T . dout[dout_row_index[...], :]
 *     either index may be NULL (identity).
 * m is the static bound on the sorted rows (sum(group_sizes) <= m sizes the workspace). */
int rd_gmm_permuted(const void* x, int x_rows, const int32_t* in_rows, const void* A, int num_weights,
                    const int32_t* group_sizes, const int32_t* group_to_weight, void* y, int y_rows,
                    const int32_t* out_rows, void* workspace, size_t workspace_bytes, int m, int k,
                    int n, int g, int trans_rhs, int dtype, const rd_tile_cfg* cfg, void* stream);
int rd_tgmm_permuted(const void* x, int x_rows, const int32_t* x_row_index, const void* dout,
                     int dout_rows, const int32_t* dout_row_index, const int32_t* group_sizes,
                     void* out, void* workspace, size_t workspace_bytes, int m, int k, int n, int g,
                     int dtype, const rd_tile_cfg* cfg, void* stream);

/* rd_gmm for callers that cannot supply a workspace and cannot allocate one.  It has no
 * counterpart in the reference (there XLA allocates every buffer).  Meant for an operator slot
 * whose argument list is fixed to inputs and outputs, inside a framework that owns all device
 * memory: a cudaMalloc made from inside such a call can fail, and when it works it synchronises
 * the whole device.  This entry point allocates and frees nothing; the group-metadata scratch
 * lives in a 64 KiB array built into the library's device image (held on every GPU that loads
 * the library until the process exits).
 *   Limit: 12*g + 10*ceil(m/128) + 16 <= 16384 words (e.g. g = 256 with m up to 170,000 rows);
 *          beyond it the call returns RD_ERR_TOO_LARGE and does nothing.
 *   First call on each device resolves the array's device address (cudaGetSymbolAddress, with
 *          that device current); make that first call outside any stream capture.
 *   The array is shared by all calls on a device and keeps the previous call's contents; the
 *          words that must start at zero are cleared on `stream` at the start of every call.
 *          Calls that can overlap on the GPU race on it: keep them on one stream or order them.
 * Arguments and results otherwise exactly as rd_gmm; the device status is not readable through
 * rd_device_status (there is no caller-visible workspace). */
int rd_gmm_static_scratch(const void* x, const void* A, const int32_t* group_sizes, void* y, int m,
                          int k, int n, int g, int trans_rhs, int dtype, const rd_tile_cfg* cfg,
                          void* stream);

/* Synchronises `stream`, reads the device status word of `workspace` and returns RD_OK or
 * RD_ERR_DEVICE_WAIT.  For tests and debugging; the hot path never calls it. */
int rd_device_status(const void* workspace, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* RAGGED_DOT_B200_H_ */
