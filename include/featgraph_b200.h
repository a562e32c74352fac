/*
 * featgraph_b200 -- C ABI of the sm_100a SpMM / SDDMM backend.
 *
 * Every entry point returns an int status (FG_OK == 0) and never throws or
 * aborts; fg_last_error_string() gives the message of the calling thread's
 * last failure.  Pointers whose name ends in _dev are device pointers on the
 * device the call (or the plan) names, pointers ending in _host are ordinary
 * host memory.  `stream` is a cudaStream_t passed as void* (NULL = the legacy
 * default stream).  No torch types appear in any signature.
 *
 * Each declaration cites the interface of the reference implementation
 * (amazon-science/FeatGraph, paths relative to that project) that it stands
 * in for.
 */
#ifndef FEATGRAPH_B200_H_
#define FEATGRAPH_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum fg_status {
  FG_OK = 0,
  FG_ERR_INVALID_ARGUMENT = 1, /* bad shape, null pointer, inconsistent indptr */
  FG_ERR_CUDA = 2,             /* a CUDA runtime call failed                 */
  FG_ERR_UNSUPPORTED = 3,      /* size beyond what the ABI can index         */
  FG_ERR_OUT_OF_MEMORY = 4
};

/* Operators of the generalised kernels (fg_spmm_csr_f32_general,
 * fg_sddmm_coo_f32_general): a message msg(lhs, rhs) per nonzero and feature, and the
 * reducer that folds the messages, in order, into one accumulator.  max / min start
 * from the lowest / highest finite float, keep the accumulator on a tie and never take
 * a NaN message.  The reference hard-codes FG_MSG_MUL with FG_REDUCE_SUM
 * (python/featgraph/op/vanilla_spmm.py:53, 121; vanilla_sddmm.py:47). */
enum fg_msg_op {
  FG_MSG_MUL = 0,      /* lhs * rhs */
  FG_MSG_ADD = 1,      /* lhs + rhs */
  FG_MSG_SUB = 2,      /* lhs - rhs */
  FG_MSG_DIV = 3,      /* lhs / rhs */
  FG_MSG_COPY_LHS = 4, /* lhs       */
  FG_MSG_COPY_RHS = 5  /* rhs       */
};
enum fg_reduce_op { FG_REDUCE_SUM = 0, FG_REDUCE_MAX = 1, FG_REDUCE_MIN = 2 };

/* Message of the last failure on the calling thread ("" if none). */
const char* fg_last_error_string(void);

/* Library version, "major.minor.patch". */
const char* fg_version(void);

/* Options for the NEXT fg_spmm_csr_f32* / fg_sddmm_coo_f32* call of the calling host
 * thread; that call consumes them.  They let a caller put an SpMM and an SDDMM that do
 * not depend on each other into one stream so that the second fills the machine under
 * the tail of the first (the SpMM's giant rows: a few whole-SM CTAs that outlast the rest):
 *     fg_spmm_csr_f32(...);
 *     fg_next_launch_options(FG_LAUNCH_PROGRAMMATIC, 0);     fg_sddmm_coo_f32(...);
 * or, with the SpMM cut in two around the SDDMM:
 *     fg_next_launch_options(FG_SPMM_GIANT_ROWS_ONLY, 0);            fg_spmm_csr_f32(...);
 *     fg_next_launch_options(FG_LAUNCH_PROGRAMMATIC, 0);             fg_sddmm_coo_f32(...);
 *     fg_next_launch_options(FG_SPMM_SKIP_GIANT_ROWS | FG_LAUNCH_PROGRAMMATIC, 0);
 *                                                                    fg_spmm_csr_f32(...);
 * FG_LAUNCH_PROGRAMMATIC: the call's first kernel may be dispatched as soon as every CTA
 *   of the kernel before it in the stream is resident, instead of when that kernel has
 *   completed (programmatic dependent launch).  The caller asserts that this call reads
 *   nothing that kernel writes.  The last CTA of each of this library's kernels waits
 *   for the grid before it, so a later, ordinary launch still sees all of them complete.
 * FG_SPMM_GIANT_ROWS_ONLY / FG_SPMM_SKIP_GIANT_ROWS: the SpMM call computes only the
 *   plan's giant rows / everything but them; the two calls together are one SpMM.
 * FG_SPMM_LONG_ROWS_ONLY / FG_SPMM_SKIP_LONG_ROWS: the same cut one class further down:
 *   the giant AND the heavy rows (every row that is one long dependent chain) / the light
 *   rows only.
 * max_ctas > 0 (SDDMM): at most this many CTAs, each walking more edges, so that the whole
 *   grid is resident at once and the kernel behind it can be dispatched beside it.
 * FG_SDDMM_TMA_STAGING (SDDMM, multiply / sum, feat_len a multiple of 32): the gathered
 *   feature segments are brought into shared memory by the tensor memory accelerator
 *   (cp.async.bulk.tensor tile::gather4 copies, 128-byte swizzle, mbarriers with bounded
 *   waits; see fg_sddmm_status) instead of by the lanes' cp.async copies.  Same results
 *   bit for bit.  Measured slower on B200 for 128-byte segments (3.57 against 2.82 ms at
 *   feat_len 64 on 114.6 M edges: the TMA unit takes about 16 cycles per four-row gather),
 *   so it is not the default.
 * FG_SDDMM_ROW_REGISTERS (SDDMM, one head, feat_len a multiple of 32; a hint, ignored
 *   where it does not apply): the kernel that keeps the dst operand in registers
 *   (sddmm_rowreg_kernel) -- faster when nearly every run of 32 consecutive edges shares
 *   one row index, as in a row-sorted list of a graph with long rows (2.64 against 2.82
 *   ms at feat_len 64, 25.1 against 29.1 at 512, on 114.6 M edges); a tile that crosses
 *   a row boundary reads its dst segments from global memory, so lists of short rows are
 *   better served without it.  Same results bit for bit.  The Python module sets it by
 *   itself from the edge list (module/sddmm.py).
 * The reference has no counterpart (one kernel, one stream). */
enum fg_launch_flags {
  FG_LAUNCH_PROGRAMMATIC = 1,
  FG_SPMM_GIANT_ROWS_ONLY = 2,
  FG_SPMM_SKIP_GIANT_ROWS = 4,
  FG_SDDMM_TMA_STAGING = 8,
  FG_SPMM_LONG_ROWS_ONLY = 16,
  FG_SPMM_SKIP_LONG_ROWS = 32,
  FG_SDDMM_ROW_REGISTERS = 64
};
int fg_next_launch_options(int32_t flags, int32_t max_ctas);

/* ------------------------------------------------------------------ SpMM -- */

/* Opaque launch plan of one CSR matrix: the rows sorted by degree and cut into
 * three classes (light rows served by sub-warp groups, heavy rows by staged
 * single-warp CTAs, the few giant rows by producer/consumer CTAs), the
 * feature-slab width chosen from the device's L2 size, and the status word of
 * the giant-row kernel's bounded waits.  A call launches its (up to three)
 * kernels back to back on the caller's stream, once per feature slab when
 * feat_len is wider than the slab; the plan is read-only during a call apart
 * from that status word, which all calls of one plan share. */
typedef struct fg_spmm_plan fg_spmm_plan;

/* Builds the plan from the HOST copy of indptr (n_rows + 1 int32 entries).
 * Stands in for the specialisation step of SpMMbase.build
 * (python/featgraph/module/spmm.py:81-111) together with the schedule
 * schedule_vanilla_spmm_csr_cuda (python/featgraph/op/vanilla_spmm.py:128-146).
 * heavy_threshold <= 0 selects the built-in default. */
int fg_spmm_plan_create(const int32_t* indptr_host, int64_t n_rows,
                        int64_t n_cols, int32_t feat_len, int32_t device,
                        int32_t heavy_threshold, fg_spmm_plan** out_plan);

int fg_spmm_plan_destroy(fg_spmm_plan* plan);

/* Writes a one-line human readable description of the plan (bins, slab width,
 * launch shapes) into buf.  Stands in for SpMMbase.lower_to_ir
 * (python/featgraph/module/spmm.py:113-140). */
int fg_spmm_plan_describe(const fg_spmm_plan* plan, char* buf, int64_t buf_len);

/* Synchronises the plan's device and reads the status word its kernels write:
 * 0 = fine; non-zero = a bounded wait inside the giant-row kernel gave up since
 * the last time this function was called (1: a producer warp, 2: the consumer
 * warp).  In that case this function also returns FG_ERR_CUDA, the rows that
 * kernel was summing hold NaN in Y, and the word is cleared, so the next SpMM
 * call is judged on its own.  The reference has no counterpart (TVM kernels
 * have no device-side waits). */
int fg_spmm_plan_status(const fg_spmm_plan* plan, int32_t* device_status);

/* Sets how many times a wait inside the giant-row kernel polls before it gives
 * up (default 2^20; polls < 0 restores the default; 0 = never wait).  A hook
 * for tests of the give-up path: with a tiny limit the kernel still returns,
 * reports through fg_spmm_plan_status and fills the affected rows with NaN.
 * No counterpart in the reference. */
int fg_spmm_plan_set_poll_limit(fg_spmm_plan* plan, int64_t polls);

/* Number of kernels one fg_spmm_csr_f32 call launches with this plan. */
int fg_spmm_plan_num_launches(const fg_spmm_plan* plan);

/* Y[r, f] = sum over e in [indptr[r], indptr[r+1]) of vals[e] * X[indices[e], f],
 * e ascending, one fp32 accumulator per (r, f), product and sum rounded
 * separately.  X is (n_cols, feat_len) row-major, Y is (n_rows, feat_len)
 * row-major and every element of Y is overwritten.  Stands in for the
 * compiled function that SpMMbase.run calls
 * (python/featgraph/module/spmm.py:142-161), i.e. vanilla_spmm_csr_cuda
 * (python/featgraph/op/vanilla_spmm.py:83-125). */
int fg_spmm_csr_f32(const fg_spmm_plan* plan, const int32_t* indptr_dev,
                    const int32_t* indices_dev, const float* vals_dev,
                    const float* x_dev, float* y_dev, void* stream);

/* Generalised SpMM: Y[r, f] = reduce, over the row's nonzeros in CSR order, of
 * msg(X[indices[e], f], vals[e]) -- lhs is the source vertex's feature, rhs the
 * edge's value; one fp32 accumulator per (r, f) that starts from the reducer's
 * identity (so an empty row holds the identity: 0, or the lowest / highest finite
 * float for max / min).  FG_MSG_MUL with FG_REDUCE_SUM is fg_spmm_csr_f32, bit
 * for bit.  The reference calls its kernels "generalized" (README.md:6) but ships
 * only this pair (python/featgraph/op/vanilla_spmm.py:53, 121); the other
 * operator pairs have no counterpart there. */
int fg_spmm_csr_f32_general(const fg_spmm_plan* plan, const int32_t* indptr_dev,
                            const int32_t* indices_dev, const float* vals_dev,
                            const float* x_dev, float* y_dev, int32_t msg_op,
                            int32_t reduce_op, void* stream);

/* The same SpMM with its result written to n_ys buffers at once (1 <= n_ys <= 8):
 * ys_host_array[0] is normally the caller's own Y block, the others the same block
 * inside the Y of peer GPUs (peer-mapped device pointers).  The kernels store every
 * finished row to all of them (plain stores over NVLink), so on a multi-GPU run the
 * all-gather of the row blocks happens in the kernels' epilogue; the caller still
 * has to synchronise the GPUs before the peers read.  No counterpart in the
 * reference (single device, python/featgraph/module/spmm.py:218). */
int fg_spmm_csr_f32_multi(const fg_spmm_plan* plan, const int32_t* indptr_dev,
                          const int32_t* indices_dev, const float* vals_dev,
                          const float* x_dev, float* const* ys_host_array, int32_t n_ys,
                          void* stream);

/* The same SpMM with every finished row stored ONCE through an NVLink-switch
 * multicast address: y_mcast_dev is the position of this call's first row inside
 * a multicast mapping of an output buffer that every GPU of the group holds (e.g.
 * torch symmetric memory's multicast_ptr); the switch writes the row into every
 * GPU's copy, this GPU's included (multimem.st; a store, never a multicast load).
 * The caller still has to synchronise the GPUs before anyone reads (fg_peer_barrier).
 * No counterpart in the reference (single device, python/featgraph/module/spmm.py:218). */
int fg_spmm_csr_f32_mcast(const fg_spmm_plan* plan, const int32_t* indptr_dev,
                          const int32_t* indices_dev, const float* vals_dev,
                          const float* x_dev, float* y_mcast_dev, void* stream);

/* Same computation from HOST buffers: uploads X, launches, downloads Y and
 * synchronises the stream.  The adjacency stays resident on the device, as it
 * does in the reference after SpMMbase.__init__
 * (python/featgraph/module/spmm.py:67-69); x_stage_dev / y_stage_dev are
 * caller-provided device buffers of the sizes of X and Y. */
int fg_spmm_csr_f32_host(const fg_spmm_plan* plan, const int32_t* indptr_dev,
                         const int32_t* indices_dev, const float* vals_dev,
                         const float* x_host, float* y_host,
                         float* x_stage_dev, float* y_stage_dev, void* stream);

/* The same SpMM for callers that must not allocate device memory (a plug-in
 * inside a server that owns the whole device pool, a loop in which cudaMalloc
 * and cudaFree are banned after start-up because they synchronise the device,
 * a process whose memory budget is already spent).  It has no counterpart in
 * the reference.  No plan is needed and nothing is allocated, by this library
 * or by any library it calls: the degree-ordered row list lives in a fixed
 * array inside the library image, sized for fg_spmm_noalloc_max_rows() rows
 * (1 048 576; about 4 MiB held by every GPU that loads the library until the
 * process exits) and rebuilt on the device by every call.  More rows than that,
 * feat_len not a multiple of 32, or x_dev / y_dev not 16-byte aligned return
 * FG_ERR_UNSUPPORTED with a message.  The first call on a device looks up the
 * array's device address; make that call before starting any stream capture.
 * All calls share the one array, so two calls that overlap on the same GPU
 * (different streams or threads) race; issue them one after the other.  Long
 * rows take the same group-per-row kernel as short ones, so graphs with very
 * long rows run slower here than through a plan.  Results are bit-identical to
 * fg_spmm_csr_f32. */
int fg_spmm_csr_f32_noalloc(const int32_t* indptr_dev, const int32_t* indices_dev,
                            const float* vals_dev, const float* x_dev, float* y_dev,
                            int64_t n_rows, int64_t n_cols, int32_t feat_len,
                            int32_t device, void* stream);

/* Largest n_rows fg_spmm_csr_f32_noalloc accepts. */
int fg_spmm_noalloc_max_rows(void);

/* ------------------------------------------- SpMM over column blocks (DDS) -- */

/* The reference's 1-D source-vertex partitioning: vanilla_spmm_dds_x86 and its
 * schedule (python/featgraph/op/vanilla_spmm.py:149-246), reached there through
 * VanillaSpMMx86(adj, num_col_partitions > 1) (python/featgraph/module/spmm.py:41-56,
 * 95-103).  The adjacency comes in the dense-dense-sparse form that
 * util_convert_csr_to_dds makes (python/featgraph/util/adj_partitioning.py:7-57):
 * the columns cut into P = num_col_partitions blocks of width ceil(n_cols / P),
 * s1_pos holding P row-pointer arrays of n_rows + 1 entries each (positions into
 * the arrays below, block after block), s1_idx block-local column indices.
 *   S_p[row, f] = sum of vals[e] * X[s1_idx[e] + p * width, f] over the entries of
 *                 block p's row, e ascending, accumulator starting at 0;
 *   Y[row, f]   = ((0 + S_0) + S_1) + ... + S_(P-1), as the reference sums its
 *                 Intermediate tensor over the block axis.
 * Bit-identical to that order; NOT to fg_spmm_csr_f32's for P > 1 (different
 * association; both agree with an exact sum to rounding).  The reference has this
 * path for x86 only.
 *
 * The plan holds one CSR plan per block (s1_pos on the host); the call runs the
 * blocks one after the other on the stream with the CSR kernels, each adding to
 * Y, so that block p's gathers stay within its width * feat_len * 4 bytes of X. */
typedef struct fg_spmm_dds_plan fg_spmm_dds_plan;
int fg_spmm_dds_plan_create(const int32_t* s1_pos_host, int64_t n_rows, int64_t n_cols,
                            int32_t feat_len, int32_t num_col_partitions, int32_t device,
                            fg_spmm_dds_plan** out_plan);
int fg_spmm_dds_plan_destroy(fg_spmm_dds_plan* plan);
/* Kernels one fg_spmm_dds_f32 call launches. */
int fg_spmm_dds_plan_num_launches(const fg_spmm_dds_plan* plan);
/* fg_spmm_plan_status over every block's plan. */
int fg_spmm_dds_plan_status(const fg_spmm_dds_plan* plan, int32_t* device_status);
/* Y = A @ X from the DDS arrays on the device; asynchronous on `stream`.
 * Launch options set by fg_next_launch_options are dropped, not applied. */
int fg_spmm_dds_f32(const fg_spmm_dds_plan* plan, const int32_t* s1_pos_dev,
                    const int32_t* s1_idx_dev, const float* vals_dev, const float* x_dev,
                    float* y_dev, void* stream);

/* ----------------------------------------------------------------- SDDMM -- */

/* out[e, h] = sum over d < D of src[col[e], h*D + d] * dst[row[e], h*D + d],
 * d ascending, one fp32 accumulator per (e, h), product and sum rounded
 * separately; D = feat_len / num_heads.  src is (n_cols, feat_len) row-major
 * and is indexed by COL, dst is (n_rows, feat_len) row-major and is indexed
 * by ROW; out is (nnz, num_heads) row-major in the given edge order.
 * num_heads == 1 is the reference's vanilla_sddmm
 * (python/featgraph/op/vanilla_sddmm.py:6-63) as run by SDDMMbase.run
 * (python/featgraph/module/sddmm.py:115-129); num_heads > 1 is the multi-head
 * extension, which has no counterpart in the reference. */
int fg_sddmm_coo_f32(const int32_t* row_dev, const int32_t* col_dev,
                     const float* src_dev, const float* dst_dev, float* out_dev,
                     int64_t nnz, int64_t n_rows, int64_t n_cols,
                     int32_t feat_len, int32_t num_heads, int32_t device,
                     void* stream);

/* Generalised SDDMM: out[e, h] = reduce over d ascending of
 * msg(src[col[e], h*D + d], dst[row[e], h*D + d]) -- lhs is the src element, rhs
 * the dst element.  FG_MSG_MUL with FG_REDUCE_SUM is fg_sddmm_coo_f32, bit for bit
 * (the reference's only pair, python/featgraph/op/vanilla_sddmm.py:47); the other
 * pairs have no counterpart in the reference. */
int fg_sddmm_coo_f32_general(const int32_t* row_dev, const int32_t* col_dev,
                             const float* src_dev, const float* dst_dev, float* out_dev,
                             int64_t nnz, int64_t n_rows, int64_t n_cols, int32_t feat_len,
                             int32_t num_heads, int32_t msg_op, int32_t reduce_op,
                             int32_t device, void* stream);

/* The same SDDMM with its result written to n_outs buffers at once (see
 * fg_spmm_csr_f32_multi): outs_host_array[i] points at the position of this call's
 * first edge inside output buffer i.  No counterpart in the reference. */
int fg_sddmm_coo_f32_multi(const int32_t* row_dev, const int32_t* col_dev,
                           const float* src_dev, const float* dst_dev,
                           float* const* outs_host_array, int32_t n_outs, int64_t nnz,
                           int64_t n_rows, int64_t n_cols, int32_t feat_len,
                           int32_t num_heads, int32_t device, void* stream);

/* The same SDDMM with every result stored once through an NVLink-switch multicast
 * address (see fg_spmm_csr_f32_mcast): out_mcast_dev is the position of this call's
 * first edge inside the multicast mapping of the output.  No counterpart in the
 * reference. */
int fg_sddmm_coo_f32_mcast(const int32_t* row_dev, const int32_t* col_dev,
                           const float* src_dev, const float* dst_dev, float* out_mcast_dev,
                           int64_t nnz, int64_t n_rows, int64_t n_cols, int32_t feat_len,
                           int32_t num_heads, int32_t device, void* stream);

/* SDDMM of this GPU's edge range with the result also delivered to peers (multi-GPU; no
 * counterpart in the reference, which is single-device: module/sddmm.py:185).  The edge
 * list is cut into pieces; piece k is copied into the same position of every peer's
 * buffer (peer-mapped device pointers, plain 16-byte stores over NVLink by a copy kernel
 * on an internal second stream) while piece k+1 is computed on `stream`.  `stream` waits
 * for the last copy before the call's work counts as done on it.  Asynchronous.
 * n_peers = 0 is fg_sddmm_coo_f32. */
int fg_sddmm_coo_f32_push(const int32_t* row_dev, const int32_t* col_dev, const float* src_dev,
                          const float* dst_dev, float* out_dev, float* const* peer_outs,
                          int32_t n_peers, int64_t nnz, int64_t n_rows, int64_t n_cols,
                          int32_t feat_len, int32_t num_heads, int32_t device, void* stream);

/* Same computation from HOST feature buffers (edge lists stay resident, as in
 * SDDMMbase.__init__, python/featgraph/module/sddmm.py:59-60). */
int fg_sddmm_coo_f32_host(const int32_t* row_dev, const int32_t* col_dev,
                          const float* src_host, const float* dst_host,
                          float* out_host, float* src_stage_dev,
                          float* dst_stage_dev, float* out_stage_dev,
                          int64_t nnz, int64_t n_rows, int64_t n_cols,
                          int32_t feat_len, int32_t num_heads, int32_t device,
                          void* stream);

/* Synchronises `device` and reads the status word of the SDDMM kernel that stages
 * its tiles with TMA copies: 0 = fine; non-zero = a bounded wait for a copy gave up
 * since the last call of this function (the function then returns FG_ERR_CUDA, the
 * results of the edges behind that wait were not written, and the word is cleared).
 * No counterpart in the reference (TVM kernels have no device-side waits). */
int fg_sddmm_status(int32_t device, int32_t* device_status);

/* Number of kernels one fg_sddmm_coo_f32 call launches for this shape. */
int fg_sddmm_num_launches(int64_t nnz, int32_t feat_len, int32_t num_heads);

/* One-line description of the launch chosen for this shape; stands in for
 * SDDMMbase.lower_to_ir (python/featgraph/module/sddmm.py:94-113). */
int fg_sddmm_describe(int64_t nnz, int32_t feat_len, int32_t num_heads,
                      char* buf, int64_t buf_len);

/* ------------------------------------------------- multi-GPU partitioning -- */

/* Splits the rows of a CSR matrix into `world` contiguous blocks holding about
 * nnz / world nonzeros each; a row is never split.  bounds receives world + 1
 * row indices, bounds[0] = 0, bounds[world] = n_rows.  Pure host code.  The
 * reference is single-device (python/featgraph/module/spmm.py:218), so this
 * has no counterpart there. */
int fg_shard_rows_by_nnz(const int32_t* indptr_host, int64_t n_rows,
                         int32_t world, int64_t* bounds);

/* Splits nnz edges into `world` contiguous ranges of equal length, the length
 * rounded up to a multiple of 32 edges (so every range starts on a 128-byte
 * boundary of a float output and one even all-gather assembles the padded
 * result); trailing ranges may be short or empty.  bounds receives world + 1
 * edge indices, bounds[world] = nnz.  Pure host code; no counterpart in the
 * reference (python/featgraph/module/sddmm.py:185 is single-device). */
int fg_shard_edges(int64_t nnz, int32_t world, int64_t* bounds);

/* Device-side barrier between the `world` (at most 8) GPUs of one box, enqueued on
 * `stream`: flag_arrays_host_array[r] is rank r's array of `world` 32-bit counters
 * as THIS rank addresses it (peer-mapped; all zero before the first barrier), `epoch`
 * counts the barriers (1, 2, 3, ... on every rank alike).  The kernel announces the
 * epoch in this rank's slot of every array and waits, at most max_polls polls per
 * peer (about a microsecond each; < 0 selects the default, a few seconds), until
 * every peer has announced it.  A wait that runs out writes 1 + the missing rank to
 * *status_dev (an int32 the caller zeroed; the first code sticks) and the kernel
 * returns -- nothing hangs, the host reads the word when it next synchronises.
 * Brackets the multi-GPU calls whose kernels store into peers' outputs.  No
 * counterpart in the reference (single device). */
int fg_peer_barrier(uint32_t* const* flag_arrays_host_array, int32_t rank, int32_t world,
                    uint32_t epoch, int32_t* status_dev, int64_t max_polls, int32_t device,
                    void* stream);

/* ------------------------------------------------------------ measurement -- */

/* Launches a gather-only kernel: n_blocks CTAs of 256 threads, groups of
 * row_floats / 4 lanes (row_floats = 32, 64 or 128) each read rows_per_group
 * whole rows of table_dev (n_rows x row_floats fp32) at pseudo-random row
 * indices, eight 16-byte loads in flight per lane.  Timed by the caller, it gives
 * the rate at which the L2 -> SM path delivers gathered rows from a table that
 * fits L2: the denominator of the benchmark's L2 roofline.  sink_dev is one
 * float that is practically never written.  No counterpart in the reference. */
int fg_gather_probe(const float* table_dev, int64_t n_rows, int32_t row_floats,
                    int64_t rows_per_group, int32_t n_blocks, float* sink_dev,
                    int32_t device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FEATGRAPH_B200_H_ */
