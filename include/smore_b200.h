/*
 * smore_b200 — C ABI of the B200 (sm_100a) distance-op and sparse-row-update library.
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; every pointer is DEVICE memory owned by the caller unless
 *     a parameter is documented as a host pointer.  The library never allocates or frees device
 *     memory (scratch is passed in; see smore_unique_rows_workspace_bytes).
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it and the call returns
 *     without synchronising.  The device that is current when the call is made must own the
 *     pointers.
 *   - return value: SMORE_OK (0) or a negative SMORE_ERR_* code.  The library never exits the
 *     process and never prints; smore_last_error() gives a thread-local message for the last
 *     failing call.  (The reference prints and calls exit(), extlib_cuda.cpp:26-49, or silently
 *     ignores an unknown distance name, ext_cuda_kernel.cu:48-49; both become error codes here.)
 *   - all arithmetic is IEEE fp32 unless the name ends in _f64.
 *
 * Shapes follow the reference's op contract (extlib_cuda.cpp:172-196): an entity operand
 * [be, ne, mul*dim], query operands [bc, nc, dim], an output [bsize, num] with
 * bsize = max(be, bc), num = max(ne, nc); cell (i, j) pairs entity row (i % be, j % ne) with
 * query row (i % bc, j % nc).  mul is 2 for the distances whose entity rows hold two parts
 * ([part0 | part1], each `dim` long: rotate, complex) and 1 otherwise.
 */
#ifndef SMORE_B200_H_
#define SMORE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SMORE_API __attribute__((visibility("default")))
#else
#define SMORE_API
#endif

#define SMORE_OK 0
#define SMORE_ERR_BAD_DIST (-1)   /* unknown distance / optimizer id */
#define SMORE_ERR_BAD_SHAPE (-2)  /* sizes violate the broadcast contract or a documented limit */
#define SMORE_ERR_NULL (-3)       /* a required pointer is NULL */
#define SMORE_ERR_CUDA (-4)       /* the CUDA runtime reported an error (see smore_last_error) */
#define SMORE_ERR_WORKSPACE (-5)  /* scratch buffer missing, misaligned or too small */
#define SMORE_ERR_TOO_LARGE (-6)  /* size beyond what an entry point supports */

/* Distance ids.  Same set and order as the name dispatch of the reference
 * (ext_cuda_kernel.cu:27-46) without the beta family. */
enum smore_dist {
  SMORE_DIST_BOX_OUT = 0,  /* sum relu(|e - c| - o)                 dist_kernel.h:58-79   */
  SMORE_DIST_BOX_IN = 1,   /* sum |min(|e - c|, o)|                 dist_kernel.h:82-105  */
  SMORE_DIST_ROTATE = 2,   /* sum sqrt((e0-re)^2 + (e1-im)^2 + eps) dist_kernel.h:108-126 */
  SMORE_DIST_L1 = 3,       /* sum |e - c|                           dist_kernel.h:129-155 */
  SMORE_DIST_L2 = 4,       /* sum (e - c)^2  (no root)              dist_kernel.h:158-184 */
  SMORE_DIST_COMPLEX = 5,  /* sum e0*re + e1*im                     dist_kernel.h:187-204 */
  SMORE_DIST_DISTMULT = 6, /* sum e*c                               dist_kernel.h:324-349 */
  SMORE_DIST_COUNT = 7,
  SMORE_DIST_BOX_BOTH = 7  /* box_out and box_in of the same operands; smore_union_* entry points only */
};

enum smore_opt {
  SMORE_OPT_SGD = 0,     /* embed_optimizer.py:166-185 */
  SMORE_OPT_ADAM = 1,    /* embed_optimizer.py:188-252 */
  SMORE_OPT_ADAGRAD = 2  /* embed_optimizer.py:312-349 */
};

SMORE_API const char* smore_last_error(void);
/* Library build tag, e.g. "smore_b200 sm_100a". */
SMORE_API const char* smore_version(void);
/* Number of this library's kernels enqueued by the calling process so far (all threads, all
 * streams); memsets are not counted.  For accounting in benchmarks. */
SMORE_API unsigned long long smore_kernel_launch_count(void);

/* Measurement aid (no counterpart in the reference): enqueues one kernel in which every thread of a
 * grid that fills the GPU runs eight independent chains of `iters` dependent fp32 fused
 * multiply-adds, and returns in *fma_count (host) how many FMAs that is in all.  Timed with CUDA
 * events it gives the non-tensor fp32 instruction rate of the device, the bound of the kernels that
 * are limited by arithmetic rather than by memory (shared-candidate scoring).  `out` is one device
 * float that is never written in practice. */
SMORE_API int smore_alu_probe(float* out, size_t iters, double* fma_count, void* stream);

/* ------------------------------------------------------------------------------------------
 * Distance ops on materialised operands.
 * Replace DistImpl<float>::forward / ::backward (ext_cuda_kernel.h:24-32, ext_cuda_kernel.cu:25-77)
 * and the dist_forward / dist_backward bindings above them (extlib_cuda.cpp:172-196, 233-262).
 * `second` / `g_second` may be NULL for l1, l2, distmult.  Every element of dst, g_ent, g_first
 * and g_second is written; the caller need not clear them.
 * ------------------------------------------------------------------------------------------ */
SMORE_API int smore_dist_forward(int dist_id, const float* ent, const float* first, const float* second,
                       float* dst, size_t bsize, size_t num, size_t be, size_t ne, size_t bc,
                       size_t nc, size_t dim, void* stream);

SMORE_API int smore_dist_backward(int dist_id, const float* gout, const float* ent, const float* first,
                        const float* second, float* g_ent, float* g_first, float* g_second,
                        size_t bsize, size_t num, size_t be, size_t ne, size_t bc, size_t nc,
                        size_t dim, void* stream);

/* fp64 instantiation (the reference dispatches over float and double,
 * extlib_cuda.cpp:187,249; ext_cuda_kernel.cu:79-80). */
SMORE_API int smore_dist_forward_f64(int dist_id, const double* ent, const double* first,
                           const double* second, double* dst, size_t bsize, size_t num, size_t be,
                           size_t ne, size_t bc, size_t nc, size_t dim, void* stream);

SMORE_API int smore_dist_backward_f64(int dist_id, const double* gout, const double* ent,
                            const double* first, const double* second, double* g_ent,
                            double* g_first, double* g_second, size_t bsize, size_t num, size_t be,
                            size_t ne, size_t bc, size_t nc, size_t dim, void* stream);

/* ------------------------------------------------------------------------------------------
 * Distance ops that read entity rows straight from the table.
 * The entity operand is (table[n_table_rows, mul*dim], idx[be*ne] int64) instead of the gathered
 * copy that SparseEmbedding.forward -> EmbeddingRW.read materialises (sparse_embed.py:56-67,
 * embed_rw.py:74-77) before the op runs; results equal smore_dist_forward on table[idx].
 *
 * Backward does not produce a [be, ne, mul*dim] gradient.  It adds each row's gradient into
 * g_rows[slot[p], :] (p = position in idx), the compact per-step buffer that
 * merge_grad_indices / merge_grad_list (embed_optimizer.py:39-48) would build afterwards:
 * `slot` is the inverse map of the step's sorted-unique row list and slot_count[s] the number
 * of positions of the whole step that map to s (see smore_unique_rows).  A row with
 * slot_count == 1 is stored, others are accumulated with atomics, so g_rows rows with
 * slot_count > 1 must be zero beforehand (smore_zero_shared_rows).
 * slot_count == NULL means "accumulate everywhere": every row gradient is added atomically.
 * Use it for the second and later backward calls over the same positions in one step (a union
 * query scores the same candidate rows once per branch): the first call may store, the others
 * must add.
 * g_first / g_second are fully written as in smore_dist_backward.
 *
 * Row ids are the caller's data and are checked against n_table_rows in every entry point that
 * takes (table, idx): an id outside [0, n_table_rows) is never dereferenced.  The forward result of
 * a pair with such an id is NaN, the backward pass takes no gradient from it and writes none for
 * it, a gathered row is NaN, and bit 2 (value 4) of the status word of smore_async_status is set.
 * (The reference indexes with torch, which raises a device-side assertion instead,
 * embed_rw.py:74-77.)  n_table_rows == 0 switches the check off.
 * ------------------------------------------------------------------------------------------ */
SMORE_API int smore_dist_forward_rows(int dist_id, const float* table, const int64_t* idx,
                            size_t n_table_rows, const float* first, const float* second, float* dst,
                            size_t bsize, size_t num, size_t be, size_t ne, size_t bc, size_t nc,
                            size_t dim, void* stream);

SMORE_API int smore_dist_backward_rows(int dist_id, const float* gout, const float* table,
                             const int64_t* idx, size_t n_table_rows, const float* first,
                             const float* second, const int32_t* slot, const int32_t* slot_count,
                             float* g_rows, float* g_first, float* g_second, size_t bsize, size_t num,
                             size_t be, size_t ne, size_t bc, size_t nc, size_t dim, void* stream);

/* Query2box scores both box distances of the same operands (box.py:157-164 calls box_dist_out
 * and box_dist_in back to back).  These two entry points read every entity row once and return
 * / consume both: dst_out, dst_in and gout_out, gout_in are [bsize, num].
 * idx == NULL means `ent` is a materialised [be, ne, dim] operand; then g_ent ([be, ne, dim])
 * receives the entity gradient and slot / slot_count / g_rows must be NULL.  With idx != NULL
 * the rules of the _rows entry points apply (n_table_rows included) and g_ent must be NULL. */
SMORE_API int smore_box_forward(const float* ent, const int64_t* idx, size_t n_table_rows,
                      const float* center, const float* offset, float* dst_out, float* dst_in,
                      size_t bsize, size_t num, size_t be, size_t ne, size_t bc, size_t nc, size_t dim,
                      void* stream);

SMORE_API int smore_box_backward(const float* gout_out, const float* gout_in, const float* ent,
                       const int64_t* idx, size_t n_table_rows, const float* center,
                       const float* offset, float* g_ent, const int32_t* slot,
                       const int32_t* slot_count, float* g_rows, float* g_center, float* g_offset,
                       size_t bsize, size_t num, size_t be, size_t ne, size_t bc, size_t nc, size_t dim,
                       void* stream);

/* Device-side status word.  Kernels that stage table rows through shared memory with bulk
 * asynchronous copies wait for each copy with a time limit (about a second); a wait that runs out
 * sets bit 0 (distance kernels) or bit 1 (background row pull), the kernel stops early and its
 * results are invalid.  Bit 2 is set when a kernel met a row id outside its table (see the _rows
 * entry points).  Nothing else reports either condition: hosts should read the word where they
 * synchronise anyway (when they read the loss, before a checkpoint).  This call synchronises the
 * current device and returns that device's word (0 = nothing happened so far); the bits stay set
 * until smore_async_status_clear.  No counterpart in the reference. */
SMORE_API int smore_async_status(int* status);
/* Synchronises the current device and sets its status word back to 0 (a host that has dealt with
 * what the word reported, e.g. dropped the offending batch). */
SMORE_API int smore_async_status_clear(void);

/* Union queries (query operand [B, U, 1, dim]): the reference front-ends loop over the U branches
 * in Python, call the op once per branch on the same entity operand and stack the results to
 * [B, U, num] (box_dist.py:60-68, l1_dist.py:52-60, rotate_dist.py:54-63).  These entry points score
 * all branches of a query in one pass over the table rows and, in backward, add the sum of the
 * branches' row gradients to g_rows once (slot / slot_count / g_rows as for the _rows entry points).
 *   first, second      [bsize, branches, dim]           g_first, g_second the same
 *   dst0 (dst1)        [bsize, branches, num]           gout0 (gout1) the same
 * Shape: every query has its own `num` candidate rows (idx is [bsize, num]).
 * dist_id: a SMORE_DIST_* id (dst1 / gout1 unused), or SMORE_DIST_BOX_BOTH: dst0 / gout0 belong to
 * box_out, dst1 / gout1 to box_in.  Results equal the per-branch calls.
 * `branches` must be 2 (the union structures of the reference, 2u and up, have two branches);
 * callers run other counts branch by branch.  SMORE_ERR_BAD_SHAPE if dim is not a multiple of 4,
 * exceeds 1024, an operand is not 16-byte aligned or num < 4. */
SMORE_API int smore_union_forward_rows(int dist_id, const float* table, const int64_t* idx,
                             size_t n_table_rows, const float* first, const float* second, float* dst0,
                             float* dst1, size_t branches, size_t bsize, size_t num, size_t dim,
                             void* stream);

SMORE_API int smore_union_backward_rows(int dist_id, const float* gout0, const float* gout1,
                              const float* table, const int64_t* idx, size_t n_table_rows,
                              const float* first, const float* second, const int32_t* slot,
                              const int32_t* slot_count, float* g_rows, float* g_first, float* g_second,
                              size_t branches, size_t bsize, size_t num, size_t dim, void* stream);

/* ------------------------------------------------------------------------------------------
 * Row gather, per-step gradient merge and row-wise optimizers.
 * ------------------------------------------------------------------------------------------ */

/* out[p, :] = table[idx[p], :]   (embed_rw.py:74-77: self.embed[indices]); ids are checked against
 * n_table_rows as described for the _rows entry points (a bad id gives a NaN row). */
SMORE_API int smore_gather_rows(const float* table, const int64_t* idx, size_t n_table_rows, float* out,
                      size_t n, size_t width, void* stream);

/* Sorted-unique of a step's row ids with inverse map — the result of
 * torch.unique(cat(idx_list), return_inverse=True) in merge_grad_indices
 * (embed_optimizer.py:39-42), bit for bit: uniq ascending, inverse[p] = rank of idx[p].
 *   idx[n] int64, every value in [0, n_table_rows)   (values outside are reported, see below)
 *   uniq[n] int64 (first *n_unique entries valid), inverse[n] int32, counts[n] int32
 *   n_unique: device int32[2]; [0] = number of distinct ids, [1] = number of out-of-range ids
 *             (those positions get inverse -1 and are ignored everywhere else)
 *   workspace: device scratch of at least smore_unique_rows_workspace_bytes(n_table_rows) bytes,
 *              256-byte aligned; contents are scratch on entry and exit.
 * Cost is O(n_table_rows / 32 + n): a presence bitmap over the id space and a popcount scan,
 * not a sort. */
SMORE_API size_t smore_unique_rows_workspace_bytes(size_t n_table_rows);
SMORE_API int smore_unique_rows(const int64_t* idx, size_t n, size_t n_table_rows, int64_t* uniq,
                      int32_t* inverse, int32_t* counts, int32_t* n_unique, void* workspace,
                      size_t workspace_bytes, void* stream);

/* smore_unique_rows for callers that cannot provide scratch memory.  (No counterpart in the
 * reference: it exists for hosts that cannot allocate when they call — a server whose memory
 * manager reserved the whole GPU at start-up, so that a later cudaMalloc fails, or a steady-state
 * training loop that must avoid cudaMalloc because it synchronises the device.)
 * Same arguments and results as smore_unique_rows minus the workspace: the scratch is a fixed
 * array inside the library, about 4 MiB per GPU that loads the library, held until the process
 * exits.  Limits and rules:
 *   - n_table_rows <= SMORE_UNIQUE_STATIC_MAX_ROWS, otherwise SMORE_ERR_TOO_LARGE (use
 *     smore_unique_rows with your own workspace for larger tables);
 *   - neither this call nor anything it uses calls cudaMalloc / cudaFree;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress,
 *     with the calling thread's current device); make that first call outside any stream
 *     capture;
 *   - all calls on a device share the one array, which still holds the previous call's bitmap:
 *     the entry point clears what has to start at zero, but two calls whose kernels overlap on
 *     the GPU (different streams, no ordering between them) race on it and give wrong results.
 *     Order such calls, or use smore_unique_rows with separate workspaces. */
#define SMORE_UNIQUE_STATIC_MAX_ROWS ((size_t)1 << 24)
SMORE_API int smore_unique_rows_static(const int64_t* idx, size_t n, size_t n_table_rows, int64_t* uniq,
                                       int32_t* inverse, int32_t* counts, int32_t* n_unique,
                                       void* stream);

/* Zero the rows of g_rows[capacity, width] whose slot_count > 1 (see smore_dist_backward_rows).
 * n_unique is the device counter written by smore_unique_rows. */
SMORE_API int smore_zero_shared_rows(float* g_rows, const int32_t* slot_count, const int32_t* n_unique,
                           size_t capacity, size_t width, void* stream);

/* g_rows[slot[p], :] (+)= grad[p, :] for p < n — merge_grad_list's scatter-sum
 * (embed_optimizer.py:45-48) for gradients that autograd delivers as a dense [n, width]
 * block (anchor and positive-entity lookups).  Store when slot_count == 1, atomic add
 * otherwise (always, when slot_count is NULL); positions with slot < 0 are skipped. */
SMORE_API int smore_scatter_add_rows(const float* grad, const int32_t* slot, const int32_t* slot_count,
                           float* g_rows, size_t n, size_t width, void* stream);

/* Row-wise optimizer step on the touched rows: for u < *n_unique, row = uniq[u], g = g_rows[u,:].
 *   SGD      table[row] += -lr * g
 *   Adam     m, v moments (v is [N, width], or [N] row-wise mean of g^2 when squeeze != 0),
 *            beta1, beta2, eps, one optimizer-wide `step` (>= 1) for the bias corrections
 *            (embed_optimizer.py:208-252)
 *   Adagrad  v accumulates g^2 (or its row mean)          (embed_optimizer.py:328-349)
 * m may be NULL for SGD/Adagrad, v NULL for SGD. */
SMORE_API int smore_sparse_update_rows(int opt_id, float* table, float* m, float* v, const int64_t* uniq,
                             const float* g_rows, const int32_t* n_unique, size_t capacity,
                             size_t width, double lr, double beta1, double beta2, double eps,
                             int64_t step, int squeeze, void* stream);

/* Entries of uniq that are negative are skipped (smore_rows_backward_fused_adam marks the rows it
 * has already updated by complementing their id). */

/* Backward of a distance over table rows (per-query candidates, as smore_dist_backward_rows /
 * smore_box_backward / smore_union_backward_rows; dist_id may be SMORE_DIST_BOX_BOTH, branches 1 or 2)
 * WITH the Adam step of every row that has a single contributor in the step folded in (row-wise
 * second moment only: v is [n_table_rows]).  No counterpart in the reference, where the gradient of
 * such a row is written to the gathered-gradient tensor, merged, and read back by the optimizer
 * together with the row (embed_optimizer.py:39-48, 208-252); here the warp that has the row in
 * shared memory for its gradient also brings in the first-moment row, updates both in place and
 * writes them back: per such row 1.6 KB less written and 3.2 KB less read (Query2box, dim 400).
 *   - slot_count is required: a row with slot_count == 1 is updated here and uniq[slot] becomes
 *     ~row (negative); rows with more contributors get their gradient added into g_rows (zeroed
 *     beforehand, smore_zero_shared_rows) and are updated by the smore_sparse_update_rows call that
 *     follows, which skips the negative entries;
 *   - lr, beta1, beta2, eps, step / step_scalars: those of that update call;
 *   - use it for a lookup that exactly ONE distance op consumes in the step (a second backward over
 *     the same positions would add to rows that are already updated) and only after every forward
 *     read of the step is done;
 *   - SMORE_ERR_BAD_SHAPE when the shape is not covered (then nothing was enqueued: call the
 *     ordinary backward). */
SMORE_API int smore_rows_backward_fused_adam(int dist_id, const float* gout0, const float* gout1, float* table,
                                   const int64_t* idx, size_t n_table_rows, const float* first,
                                   const float* second, const int32_t* slot, const int32_t* slot_count,
                                   float* g_rows, float* g_first, float* g_second, size_t branches,
                                   size_t bsize, size_t num, size_t dim, float* m, float* v, int64_t* uniq,
                                   double lr, double beta1, double beta2, double eps, int64_t step,
                                   const float* step_scalars, void* stream);

/* The same update with the optimizer's step counter on the device, for hosts that replay a
 * captured CUDA graph step after step (kernel arguments are frozen in a graph, the step is not).
 * smore_adam_step_scalars increments *step (device int64) and writes the two step-dependent
 * scalars {-lr / (1 - beta1^step), sqrt(1 - beta2^step)} to step_scalars (device float[2]);
 * smore_sparse_update_rows_dev reads them instead of taking `step`.  Enqueue both on one stream,
 * scalars first. */
SMORE_API int smore_adam_step_scalars(int64_t* step, double lr, double beta1, double beta2, float* step_scalars,
                            void* stream);
SMORE_API int smore_sparse_update_rows_dev(int opt_id, float* table, float* m, float* v, const int64_t* uniq,
                                 const float* g_rows, const int32_t* n_unique, size_t capacity,
                                 size_t width, double lr, double beta1, double beta2, double eps,
                                 const float* step_scalars, int squeeze, void* stream);

/* ------------------------------------------------------------------------------------------
 * Relation projection of path queries for the additive geometries (GQE, Query2box): all hops of
 * a batch in one kernel each way, in place of the per-hop lookups and additions of
 * kg_reasoning.py:229-236 with vec.py:58-60 / box.py:126-129.
 *   center[b, :] = start_center[b, :] + sum_h rel_table[ids[b, h], :]        (hop order)
 *   offset[b, :] = start_offset[b, :] + sum_h act(off_table[ids[b, h], :])   (off_table != NULL)
 * ids[b, h] = rel_ids[b * id_stride + h] (a column block of the reference's query matrix);
 * start_offset NULL = zeros (box.py:138-139); act = relu if relu_offset else identity (box.py:76-85).
 * Backward overwrites g_rel_table [n_relations, dim] (and g_off_table) with the dense gradients
 * of the tables; the gradient of start_center / start_offset is g_center / g_offset unchanged. */
SMORE_API int smore_path_project_forward(const float* start_center, const float* start_offset,
                               const float* rel_table, const float* off_table, size_t n_relations,
                               const int64_t* rel_ids, size_t id_stride, size_t n_queries, size_t hops,
                               size_t dim, int relu_offset, float* center, float* offset, void* stream);
SMORE_API int smore_path_project_backward(const float* g_center, const float* g_offset, const float* off_table,
                                size_t n_relations, const int64_t* rel_ids, size_t id_stride,
                                size_t n_queries, size_t hops, size_t dim, int relu_offset,
                                float* g_rel_table, float* g_off_table, void* stream);

/* The general form of the two calls above: every geometry, and a path may start from table rows.
 *   geometry 0  additive (as above; out0 = center, out1 = offset when off_table != NULL)
 *   geometry 1  rotation: rel_table [n_relations, dim] holds phases; each hop multiplies the complex
 *               state (re, im) by cos(p) + i sin(p), p = row * phase_scale (rotate.py:101-109, where
 *               phase_scale = pi / embedding_range); out0 = re, out1 = im
 *   geometry 2  complex product: rel_table [n_relations, 2*dim] rows [re | im] (complex.py:108-117 with
 *               the identity normaliser); out0 = re, out1 = im
 *   geometry 3  product: rel_table [n_relations, dim] (distmult.py:106-111, identity normaliser); out0
 * start: [n_queries, W] state rows (W = dim, or 2*dim = [re | im] for geometries 1 and 2) - or, with
 * start_idx != NULL, the entity table [n_start_rows, W] whose rows start_idx[b] the paths start from
 * (kg_reasoning.py:217-250 looks the anchors up first, box.py:131-139 / rotate.py:111-119): the anchor
 * rows are then read in place and never gathered.  Ids outside the table: see the _rows entry points.
 * At most 8 hops per call for geometries 1-3.
 * Backward overwrites g_rel_table (and g_off_table) with the dense gradients of the relation tables
 * and delivers the gradient of the start rows either as g_start [n_queries, W] (start given as a
 * tensor; may be NULL if not wanted) or, for table rows, into g_rows[slot[b], :] under the rules of
 * smore_dist_backward_rows (store when slot_count == 1, atomic add otherwise, always with slot_count
 * NULL).  Geometry 0: the start rows' gradient is g_out0 itself. */
SMORE_API int smore_path_embed_forward(int geometry, const float* start, const int64_t* start_idx,
                             size_t n_start_rows, const float* start_offset, const float* rel_table,
                             const float* off_table, size_t n_relations, const int64_t* rel_ids,
                             size_t id_stride, size_t n_queries, size_t hops, size_t dim, int relu_offset,
                             double phase_scale, float* out0, float* out1, void* stream);
SMORE_API int smore_path_embed_backward(int geometry, const float* g_out0, const float* g_out1,
                              const float* start, const int64_t* start_idx, size_t n_start_rows,
                              const float* rel_table, const float* off_table, size_t n_relations,
                              const int64_t* rel_ids, size_t id_stride, size_t n_queries, size_t hops,
                              size_t dim, int relu_offset, double phase_scale, float* g_rel_table,
                              float* g_off_table, float* g_start, const int32_t* slot,
                              const int32_t* slot_count, float* g_rows, void* stream);

/* ------------------------------------------------------------------------------------------
 * Evaluation: filtered ranks of the answers of each query among all candidates.
 * The reference (train_process.py:113-146) argsorts the [1, N] logits of a query, scatters the
 * permutation into a rank per entity, takes the ranks of the easy and hard answers, sorts them and
 * subtracts each one's position in that sorted list ("filtered setting").  Only the answers' ranks
 * are used, so this entry point counts instead of sorting N values:
 *   ranks[p] = 1 + #{candidates ahead of answer p} - #{answers of the same query ahead of it}
 * where "ahead" means a higher logit, or an equal logit and a lower candidate id (the order of a
 * stable descending sort; torch.argsort leaves ties unspecified).
 *   logits      [n_queries, n_candidates] fp32 (ordered as torch.sort does: NaN largest, -0 == +0)
 *   answer_ptr  [n_queries + 1] int64, CSR offsets into answer_ids (device memory)
 *   answer_ids  [n_answers] candidate ids: per query the easy and the hard answers in any order;
 *               the caller keeps the ranks of the hard ones
 *   ranks       [n_answers] int64, in the order of answer_ids
 *   max_answers the longest answer list (host value, <= 8192; SMORE_ERR_TOO_LARGE beyond)
 * workspace: smore_filtered_ranks_workspace_bytes(n_answers) bytes, 256-byte aligned. */
SMORE_API size_t smore_filtered_ranks_workspace_bytes(size_t n_answers);
SMORE_API int smore_filtered_ranks(const float* logits, size_t n_queries, size_t n_candidates,
                         const int64_t* answer_ptr, const int64_t* answer_ids, size_t n_answers,
                         size_t max_answers, int64_t* ranks, void* workspace, size_t workspace_bytes,
                         void* stream);

/* The evaluation step in one call: the n_queries queries are scored against every row of `table`
 * ([n_candidates, mul*dim], the whole entity table) and the filtered ranks of their answers are
 * counted from the scoring tiles directly; the [n_queries, n_candidates] logits are never written.
 * Replaces the model call of train_process.py:117 (custom_cal_logit on all entities) together with
 * the ranking block :120-141.  first / second: [n_queries, dim] query operands.
 * dist_id selects the model's logit: SMORE_DIST_BOX_BOTH gamma - d_out - cen * d_in (box.py:157-164);
 * SMORE_DIST_L1 / SMORE_DIST_ROTATE gamma - d (vec.py:85-90, rotate.py:137-142); SMORE_DIST_L2
 * gamma - sqrt(d); SMORE_DIST_COMPLEX / SMORE_DIST_DISTMULT the similarity itself (complex.py:140-149),
 * each with the roundings of the separate torch operations.  Ranks equal smore_filtered_ranks on the
 * logits the distance ops and those torch operations would have produced.  answer_* / ranks /
 * max_answers as for smore_filtered_ranks; at least 8 queries, 8 candidates and 8 answers in all,
 * dim a multiple of 4 (SMORE_ERR_BAD_SHAPE otherwise: score and rank separately).
 * workspace: smore_score_filtered_ranks_workspace_bytes(n_queries, n_answers) bytes, 256-byte aligned. */
SMORE_API size_t smore_score_filtered_ranks_workspace_bytes(size_t n_queries, size_t n_answers);
SMORE_API int smore_score_filtered_ranks(int dist_id, const float* table, size_t n_candidates, const float* first,
                               const float* second, size_t n_queries, size_t dim, double gamma, double cen,
                               const int64_t* answer_ptr, const int64_t* answer_ids, size_t n_answers,
                               size_t max_answers, int64_t* ranks, void* workspace, size_t workspace_bytes,
                               void* stream);

/* ------------------------------------------------------------------------------------------
 * Negative sampling on the GPU (the step before the row lookups).
 * The reference draws them on host threads: per query `k` entity ids that are not answers of the
 * query, uniformly or through an alias table of degree-proportional weights
 * (naive_sampler.cpp:28-50, alias_method.cpp:33-99), or one shared list per batch with a mask of
 * the entries that are answers (sampler.cpp:90-99, naive_sampler.cpp:33-38).  Its generator is
 * seeded from the clock (utils.cpp:33-39); here the draws are a pure function of (seed, offset,
 * position): Philox 4x32-10 keyed by `seed`, counter `offset + position`.
 *
 * smore_alias_build: HOST routine (host pointers, n entries each): the alias tables of `weights`
 * by the reference's procedure, so that the tables are identical to the reference's.
 * smore_sample_negatives: negatives[b, j] for b < n_queries, j < k.  prob_small / choice_small /
 * choice_large: device copies of the alias tables, or all NULL for uniform draws.  answer_ptr
 * [n_queries + 1] / answer_ids: per query its answers in ascending order (CSR, device), or both NULL;
 * a draw that is an answer is repeated (at most 64 times).  Advance `offset` by n_queries * k per
 * call to continue the stream.
 * smore_negative_mask: is_negative[b, j] = 0.0 if negatives[j] is an answer of query b, else 1.0.
 * ------------------------------------------------------------------------------------------ */
SMORE_API int smore_alias_build(const double* weights, size_t n, double* prob_small, int64_t* choice_small,
                      int64_t* choice_large);
SMORE_API int smore_sample_negatives(uint64_t seed, uint64_t offset, size_t n_entities, const double* prob_small,
                           const int64_t* choice_small, const int64_t* choice_large,
                           const int64_t* answer_ptr, const int64_t* answer_ids, size_t n_queries, size_t k,
                           int64_t* negatives, void* stream);
SMORE_API int smore_negative_mask(const int64_t* negatives, size_t k, const int64_t* answer_ptr,
                        const int64_t* answer_ids, size_t n_queries, float* is_negative, void* stream);

/* ------------------------------------------------------------------------------------------
 * Dot-product scoring of B queries against ONE shared set of K candidate rows on the tensor
 * cores (tcgen05 / TMEM through CUTLASS sm100 templates).  DistMult and ComplEx scores are inner
 * products (dist_kernel.h:187-204, 324-349); with shared candidates the op and both gradients are
 * dense GEMMs — what complex.py:186 does with torch.mm:
 *     dst[B, K]     = query[B, W] . cand[K, W]^T
 *     g_query[B, W] = gout[B, K]  . cand[K, W]
 *     g_cand[K, W]  = gout[B, K]^T . query[B, W]
 * W = dim for DistMult; 2*dim for ComplEx with the query given as [re | im], like the rows.
 * B, K and W must be multiples of 4 (16-byte TMA strides), else SMORE_ERR_BAD_SHAPE and the
 * caller falls back to smore_dist_forward / _backward (SIMT, exact fp32 order).
 * precision: SMORE_DOT_TF32 — products of 10-bit-mantissa inputs, fp32 accumulation (error about
 * 1e-3 of sum |terms|); SMORE_DOT_FP32 — each operand split into three bf16 terms, nine MMAs per
 * product, fp32-level accuracy at a third of the rate.
 * workspace: device scratch of smore_dot_workspace_bytes(...) bytes.  smore_dot_available() is 0
 * when the library was built without a CUTLASS header tree.
 * ------------------------------------------------------------------------------------------ */
#define SMORE_DOT_TF32 0
#define SMORE_DOT_FP32 1
SMORE_API int smore_dot_available(void);
/* 1 when the optional companion library libsmore_b200_2sm.so (the same products on tiles shared by
 * two SMs, tcgen05 cta_group::2) sits next to this library and was loaded; 0: one-SM tiles only. */
SMORE_API int smore_dot_two_sm(void);
SMORE_API size_t smore_dot_workspace_bytes(size_t B, size_t K, size_t W, int precision);
SMORE_API int smore_dot_forward_shared(const float* cand, const float* query, float* dst, size_t B, size_t K,
                             size_t W, int precision, void* workspace, size_t workspace_bytes,
                             void* stream);
SMORE_API int smore_dot_backward_shared(const float* gout, const float* cand, const float* query, float* g_cand,
                              float* g_query, size_t B, size_t K, size_t W, int precision,
                              void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * Row-sharded table over the GPUs of one box (one process per GPU).
 * Replaces the reference's sharing of the table through CPU shared memory with pinned PCIe
 * staging (embed_rw.py:53-134, extlib_cuda.cpp:82-144, kg_reasoning.py:144-147): rows
 * [g*S, (g+1)*S) of the table and of its Adam state live in the memory of GPU g; requesters and
 * owners read each other's memory with plain loads over NVLink.  None of these calls waits on
 * another rank; the caller orders the phases of a step (stream-ordered collectives).
 * ------------------------------------------------------------------------------------------ */

/* Peer-visible memory is the caller's business: the pointers given to these entry points must
 * be dereferenceable from the calling GPU (same-process peer access, or blocks mapped into every
 * process by a symmetric-memory allocator; a CUDA IPC mapping works but is slow for random rows). */

/* staging[u, :] = shard_ptrs[id / rows_per_shard][id % rows_per_shard, :] for id = uniq[u],
 * u < *n_unique: each distinct row of the step crosses NVLink once and lands in local memory,
 * where the distance kernels then read it (by slot).  shard_ptrs: device array of the ranks'
 * shard base pointers (peer-mapped). */
SMORE_API int smore_fetch_rows(const float* const* shard_ptrs, size_t rows_per_shard, const int64_t* uniq,
                     const int32_t* n_unique, size_t capacity, size_t width, float* staging,
                     void* stream);

/* Prefetching: rows may be pulled for the NEXT step while the current step is still running
 * (other stream), which hides the NVLink transfer behind the distance kernels.  Rows whose owner
 * updates them afterwards would be stale, so owners publish the rows they updated in a step as a
 * bitmap over their shard (smore_shard_mark_dirty: clears the bitmap, then sets one bit per row of
 * uniq[0 .. *n_unique)), and the requester re-pulls exactly the marked rows after the step's last
 * barrier (smore_refresh_rows; dirty_ptrs = device array of the n_ranks bitmaps, peer-mapped;
 * bitmap_scratch = n_ranks * ceil(rows_per_shard / 32) words of local memory that receive a copy
 * of all bitmaps first).  The result equals fetching everything after the barrier.
 * smore_fetch_rows_background is smore_fetch_rows on at most max_ctas thread blocks, so that the
 * kernels of the current step, launched afterwards on another stream, find room on every SM
 * instead of queueing behind the copy (one block per SM keeps NVLink busy).  For rows of up to
 * 20 KB it moves every row with two bulk asynchronous copies (peer memory -> shared memory ->
 * local staging block; untiled, no multicast) issued by 64-thread blocks, so that the copy takes
 * next to no registers, issue slots or load/store bandwidth from those kernels. */
SMORE_API int smore_fetch_rows_background(const float* const* shard_ptrs, size_t rows_per_shard,
                                const int64_t* uniq, const int32_t* n_unique, size_t capacity,
                                size_t width, float* staging, size_t max_ctas, void* stream);

SMORE_API int smore_refresh_rows(const float* const* shard_ptrs, const uint32_t* const* dirty_ptrs,
                       size_t n_ranks, size_t rows_per_shard, const int64_t* uniq,
                       const int32_t* n_unique, size_t capacity, size_t width, float* staging,
                       uint32_t* bitmap_scratch, void* stream);
SMORE_API int smore_shard_mark_dirty(const int64_t* uniq, const int32_t* n_unique, size_t capacity,
                           size_t shard_rows, uint32_t* dirty, void* stream);

/* Owner side of the gradient return.  Every rank publishes up to n_plans (<= 4) sorted lists of
 * distinct global row ids per step with a gradient row per id; list (g, p) has room for
 * plan_caps[p] ids (host array, same on all ranks), its current length is the int32 that
 * nuniq_ptrs[g*n_plans+p] points to (0 = unused this step).  Lists are numbered l = g*n_plans + p.
 *
 * smore_shard_owner_plan prepares an owner's update from them.  The lists are sorted and the owner's
 * rows are the id range [base, base + shard_rows), so what it needs of each list is one contiguous
 * run, found by binary search; the runs are copied as local row ids into `ids` (run after run, in
 * list order: the position of an id there encodes its list and index), then de-duplicated as
 * smore_unique_rows does: uniq / slot / counts / n_unique over the owner's distinct local rows, and
 * src[u] = one position in `ids` that holds row uniq[u].  `runs` receives the run table
 * (SMORE_SHARD_RUNS_INTS int32 of device memory) that smore_shard_reduce_update_rows reads.
 * `dirty`, if not NULL, is this rank's updated-rows bitmap: cleared, then one bit set per distinct
 * row (smore_shard_mark_dirty).  capacity: room in ids / uniq / slot / counts / src, at least
 * n_ranks * sum(plan_caps) (everything could fall into one shard); only the part in use is touched.
 * workspace: smore_shard_owner_plan_workspace_bytes(shard_rows) bytes, 256-byte aligned. */
#define SMORE_SHARD_RUNS_INTS 80
SMORE_API size_t smore_shard_owner_plan_workspace_bytes(size_t shard_rows);
SMORE_API int smore_shard_owner_plan(const int64_t* const* uniq_ptrs, const int32_t* const* nuniq_ptrs,
                           size_t n_ranks, size_t n_plans, const int32_t* plan_caps, int64_t base,
                           size_t shard_rows, size_t capacity, int64_t* ids, int32_t* runs, int64_t* uniq,
                           int32_t* slot, int32_t* counts, int32_t* src, int32_t* n_unique,
                           uint32_t* dirty, void* workspace, size_t workspace_bytes, void* stream);

/* For each distinct local row u < *n_unique: pull its gradient rows from the lists that contain
 * it (grad_ptrs[l] + j*width, peer memory; n_lists = n_ranks * n_plans), add them in list order,
 * and apply the Adam update of smore_sparse_update_rows to table / m / v of this shard - transfer,
 * reduction and update in one kernel, one pass.  Rows of 144 bytes to about 12 KB take the ring
 * form: each warp keeps several bulk asynchronous copies (peer memory -> shared memory; untiled, no
 * multicast) in flight ahead of the row it is updating; waits are bounded and report through bit 1
 * of smore_async_status. */
SMORE_API int smore_shard_reduce_update_rows(float* table, float* m, float* v, const int64_t* uniq,
                                   const int32_t* counts, const int32_t* src, const int32_t* n_unique,
                                   size_t capacity, const float* const* grad_ptrs, const int64_t* ids,
                                   const int32_t* runs, size_t n_lists, size_t width, double lr,
                                   double beta1, double beta2, double eps, int64_t step, int squeeze,
                                   void* stream);

/* The same with the step-dependent scalars read from device memory (see smore_adam_step_scalars),
 * for hosts that replay a captured CUDA graph step after step. */
SMORE_API int smore_shard_reduce_update_rows_dev(float* table, float* m, float* v, const int64_t* uniq,
                                       const int32_t* counts, const int32_t* src, const int32_t* n_unique,
                                       size_t capacity, const float* const* grad_ptrs, const int64_t* ids,
                                       const int32_t* runs, size_t n_lists, size_t width, double lr,
                                       double beta1, double beta2, double eps, const float* step_scalars,
                                       int squeeze, void* stream);

/* ---- Owner-side scoring on a row-sharded table --------------------------------------------------
 * The candidate-scoring ops of a training step read B*K table rows per rank (ext_ops.py:15-22 on
 * the rows that kg_reasoning.py:299-304 looks up).  Pulling those rows to the rank that holds the
 * queries, and pushing their gradients back, costs a row (1.6 KB at dim 400) per pair and
 * direction over NVLink.  Here the queries travel instead: each rank publishes its candidate ids,
 * its queries and, in the backward pass, the upstream gradients of its scores in peer-visible
 * memory; the OWNER of the rows scores every rank's pairs that fall into its range against its own
 * shard, returns 4 or 8 bytes per pair, and in the backward pass applies the row gradients where
 * the rows live (Adam folded in, as smore_rows_backward_fused_adam) and leaves a partial query
 * gradient per rank.  No kernel waits for another rank: the caller orders the phases with
 * stream-ordered barriers (publish -> select/score -> read results; publish upstream gradients ->
 * differentiate/update -> sum the partial query gradients).
 *
 * Rank r's descriptor is int32[8] {n_queries, K, branches, 0...}: its ids are [n_queries, K] int64
 * global row ids, its queries [n_queries, branches, dim] per operand (branches = 2: a union query,
 * both branches scored against the same candidates), its results / upstream gradients [n_queries,
 * branches, K] per output.  Every rank runs the same scoring op in a step: the owner's calls name
 * the (n_queries, rows_per_query = K, branches) they were launched for, and a rank whose descriptor
 * says otherwise is left out (bit 3 of smore_async_status).  All `*_ptrs` arguments are device arrays with one (peer) pointer per rank.
 * max_queries / pairs_capacity are what every rank's buffers were sized for; a descriptor beyond
 * them, or more selected pairs than `capacity`, drops the work concerned and sets bit 3 of
 * smore_async_status.
 *
 * smore_owner_select_pairs: for every (rank, query) the pairs whose id lies in [base, base +
 *   shard_rows) become one segment of the compact arrays: rows[] (local row ids), positions[]
 *   (query * branches * K + k on the requester: branch 0), in increasing k; segments[(rank * max_queries + query) * 2 +
 *   {0, 1}] = {first compact position, count}; n_selected[0] = pairs selected (int32[2]).
 * smore_owner_gather_queries: first_all / second_all[(rank * max_queries + query), dim] <- the
 *   ranks' queries (second_* may be NULL for one-operand distances); first_rank: the rank whose
 *   queries are copied first (pass the caller's own rank: the owners then read different peers at
 *   any moment).
 * smore_rows_forward_ragged / smore_rows_backward_fused_adam_ragged: the row-stream kernels with
 *   query q = segment q scoring rows[segments[2q] .. + segments[2q+1]); results (out0, out1) and
 *   upstream gradients (gout0, gout1) are indexed by compact position - or, with `positions`,
 *   result / upstream gradient of compact position c lives at positions[c] in the arrays of the
 *   rank that owns the segment (rank = q / segments_per_rank; out*_ptrs / gout*_ptrs: one base
 *   pointer per rank, peer memory; branch u of a pair sits u * branch_stride further) and the local
 *   arrays may be NULL.  Queries and query gradients of rank r start at r * segments_per_rank * dim
 *   floats, query q of that rank at q * branches * dim inside them.  Backward: slot / slot_count / g_rows
 *   / uniq / m / v and the Adam arguments as in smore_rows_backward_fused_adam, over the owner's
 *   distinct rows.  Rows of 1 KB to about 4 KB, dim a multiple of 4 above 256 (SMORE_ERR_BAD_SHAPE
 *   otherwise, nothing enqueued).  dist_id may be SMORE_DIST_BOX_BOTH.
 * smore_owner_plan: smore_shard_owner_plan with the first *n_selected entries of `ids` already
 *   holding the selected pairs' local row ids (pair_capacity = room reserved for them; capacity
 *   >= pair_capacity + n_ranks * sum(plan_caps)): the lists' runs are appended behind them and the
 *   whole array is de-duplicated, so that slot / counts cover both kinds of contribution.
 * smore_owner_add_list_rows: g_rows[slot[p]] (+)= the gradient row of list position p, for the
 *   compact positions of the lists' runs (store if counts == 1, atomic add otherwise); `expect` =
 *   about how many there are (sizes the grid).
 * smore_owner_sum_query_grads: out[q, :] = sum over owners o of part_ptrs[o][(my_rank *
 *   max_queries + q), :], in owner order (the requester's query gradient). */
SMORE_API int smore_owner_select_pairs(const int64_t* const* pair_id_ptrs, const int32_t* const* desc_ptrs,
                             size_t n_ranks, size_t max_queries, size_t pairs_capacity, size_t n_queries,
                             size_t rows_per_query, size_t branches, int64_t base, size_t shard_rows,
                             size_t capacity, int64_t* rows, int32_t* positions, int32_t* segments,
                             int32_t* n_selected, void* stream);
SMORE_API int smore_owner_gather_queries(const float* const* first_ptrs, const float* const* second_ptrs,
                               const int32_t* const* desc_ptrs, size_t n_ranks, size_t max_queries,
                               size_t pairs_capacity, size_t n_queries, size_t rows_per_query, size_t branches,
                               size_t dim, size_t first_rank, float* first_all, float* second_all,
                               void* stream);
SMORE_API int smore_rows_forward_ragged(int dist_id, const float* table, const int64_t* rows, size_t n_table_rows,
                              const float* first, const float* second, const int32_t* segments,
                              size_t n_segments, size_t dim, float* out0, float* out1, const int32_t* positions,
                              size_t segments_per_rank, float* const* out0_ptrs, float* const* out1_ptrs,
                              size_t branches, size_t branch_stride, void* stream);
SMORE_API int smore_rows_backward_fused_adam_ragged(int dist_id, const float* gout0, const float* gout1, float* table,
                                          const int64_t* rows, size_t n_table_rows, const float* first,
                                          const float* second, const int32_t* segments, size_t n_segments,
                                          const int32_t* slot, const int32_t* slot_count, float* g_rows,
                                          float* g_first, float* g_second, size_t dim, float* m, float* v,
                                          int64_t* uniq, double lr, double beta1, double beta2, double eps,
                                          int64_t step, const float* step_scalars, const int32_t* positions,
                                          size_t segments_per_rank, const float* const* gout0_ptrs,
                                          const float* const* gout1_ptrs, size_t branches, size_t branch_stride,
                                          void* stream);
SMORE_API int smore_owner_plan(const int64_t* const* uniq_ptrs, const int32_t* const* nuniq_ptrs, size_t n_ranks,
                     size_t n_plans, const int32_t* plan_caps, int64_t base, size_t shard_rows, size_t capacity,
                     int64_t* ids, int32_t* runs, int64_t* uniq, int32_t* slot, int32_t* counts,
                     int32_t* n_unique, uint32_t* dirty, void* workspace, size_t workspace_bytes,
                     const int32_t* n_selected, size_t pair_capacity, void* stream);
SMORE_API int smore_owner_add_list_rows(const float* const* grad_ptrs, const int32_t* runs, size_t n_lists,
                              const int32_t* slot, const int32_t* counts, float* g_rows, size_t width,
                              size_t expect, void* stream);
SMORE_API int smore_owner_sum_query_grads(const float* const* part_ptrs, size_t n_ranks, size_t my_rank,
                                size_t max_queries, size_t n_queries, size_t dim, float* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SMORE_B200_H_ */
