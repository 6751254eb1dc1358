/*
 * gsb200 -- C ABI of the B200 (sm_100a) sampling kernels.
 *
 * This is the boundary a host layer binds to (ctypes, cgo, JNI, a torch
 * extension ...): plain pointers and sizes, no framework types.  Every pointer
 * named "device" must point into the memory of the CUDA device that is current
 * on the calling thread; `cuda_stream` is a cudaStream_t passed as void*.
 * Functions enqueue work on that stream and return without synchronising
 * unless their comment says otherwise.  There is no CPU fallback: a call on a
 * machine without a usable device returns GSB_ERR_CUDA.
 *
 * Each entry point names the gSampler interface it replaces (path:line in the
 * gSampler source tree).  Ids crossing this ABI are int64 except the graph's
 * `indices` array, which may be int32 or int64 (`indices_dtype`).
 *
 * Sizes that are only known on the device (number of sampled edges, number of
 * unique nodes) are returned in device memory; entry points that consume such
 * a size accept it as a device pointer so that layers chain without a host
 * round trip.  Outputs are written into caller-allocated buffers whose
 * capacity the caller states; exceeding a capacity raises GSB_ERRBIT_CAPACITY
 * in the device error word instead of writing out of bounds.
 */
#ifndef GSB200_H_
#define GSB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define GSB_API __attribute__((visibility("default")))
#else
#define GSB_API
#endif

/* return codes */
enum {
  GSB_OK = 0,
  GSB_ERR_INVALID = 1,     /* bad argument (null pointer, negative size, bad enum) */
  GSB_ERR_UNSUPPORTED = 2, /* valid request outside the implemented range (see message) */
  GSB_ERR_WORKSPACE = 3,   /* workspace smaller than *_workspace_bytes() */
  GSB_ERR_CUDA = 4,        /* a CUDA runtime call failed; see gsb_last_cuda_error() */
  GSB_ERR_SCRATCH_LIMIT = 5 /* request larger than the fixed scratch of a *_noalloc entry point */
};

/* indices_dtype */
enum { GSB_I32 = 0, GSB_I64 = 1 };

/* bits of the device error word (`d_err`, an int in device memory that the
 * caller zeroes once and may poll after synchronising) */
enum {
  GSB_ERRBIT_LOOKBACK_TIMEOUT = 1,
  GSB_ERRBIT_TABLE_FULL = 2,
  GSB_ERRBIT_KEY_MISSING = 4,
  GSB_ERRBIT_CAPACITY = 8,
  GSB_ERRBIT_BAD_INPUT = 16
};

GSB_API int gsb_abi_version(void);
GSB_API const char* gsb_status_string(int status);
/* cudaGetErrorString of the last failing runtime call made by this library on
 * the calling thread ("" if none). */
GSB_API const char* gsb_last_cuda_error(void);

/* Launch accounting (no counterpart in the reference, whose only timers are
 * host time.time() loops, python/gs/jit/module.py:268-278).
 * gsb_kernel_launches: kernels launched by this library since it was loaded.
 * gsb_timing_enable(1): from now on every launch is bracketed by CUDA events on
 * its stream; (0) stops and drops what was collected.
 * gsb_timing_collect: synchronises the device and returns the number of
 * (kernel name, tag) groups seen since timing was enabled, with their summed
 * duration and launch count; the tag is the layer index inside
 * gsb_graphsage_sample and 0 elsewhere.  Returns -1 on error. */
GSB_API uint64_t gsb_kernel_launches(void);
GSB_API int gsb_timing_enable(int on);
GSB_API int gsb_timing_collect(int max_entries, const char** names, int* tags, double* total_ms,
                               int64_t* launches);

/* ------------------------------------------------------------------ sampling
 * Per-column fanout sampling, optionally fused with column slicing.
 * Replaces Graph::FusedSlicingSampling / BatchFusedSlicingSampling
 * (src/graph.cc:383-454, src/batch_graph.cc:190-212 ->
 * src/cuda/fusion/slice_sampling.cu:99-177) when `seeds` is given, and
 * Graph::Sampling on CSC (src/graph.cc:182-244 -> src/cuda/sampling.cu:103-172)
 * when `seeds` is NULL (column i of the operand is column slot i).
 *
 *  indptr[num_cols+1] int64, indices[nnz] (int32|int64), device.  A seed outside
 *  [0, num_cols), or a column whose offsets decrease, sets GSB_ERRBIT_BAD_INPUT
 *  and counts as an empty column; `indptr` is not read for it.
 *  seeds[S_max] int64 device or NULL.  d_S: optional device int64 holding the
 *  live number of column slots (<= S_max); NULL means S_max.
 *  K fanout (1..8192).  replace: 0 = min(deg,K) distinct edges per column,
 *  1 = K draws (0 for an empty column).
 *  (seed, stream) select the random stream; column slot i always consumes
 *  draws (seed, stream, i, 0..K-1), independent of launch geometry.
 *  Outputs (device): sub_indptr[S_max+1]; out_rows / out_cols / out_sel with
 *  capacity E_cap elements (out_cols may be NULL): row id, local column slot,
 *  edge position in `indices`.  d_num_edges (optional) receives the edge count.
 *  Column degrees must be < 2^32.
 */
GSB_API size_t gsb_sample_cols_workspace_bytes(int64_t S_max, int64_t K);
GSB_API int gsb_sample_cols(const int64_t* indptr, const void* indices, int indices_dtype,
                            int64_t num_cols, const int64_t* seeds, int64_t S_max,
                            const int64_t* d_S, int64_t K,
                            int replace, uint64_t seed, uint32_t stream, int64_t* sub_indptr,
                            int64_t* out_rows, int64_t* out_cols, int64_t* out_sel, int64_t E_cap,
                            int64_t* d_num_edges, void* workspace, size_t workspace_bytes,
                            int* d_err, void* cuda_stream);

/* gsb_sample_cols without a workspace and without any allocation.  It has no
 * counterpart in the reference (whose operators allocate through torch on every
 * call).  It exists for callers that are not allowed to allocate device memory:
 * code embedded in an application that owns the memory budget and passes in
 * only input and output buffers, or latency-sensitive threads that must not
 * touch the allocator because cudaMalloc / cudaFree synchronise the device.
 * The kernel's scratch (tile ticket + prefix status words) is a fixed array
 * inside the library, 512 KB + 264 B per GPU that loads it, so the call accepts
 * at most gsb_sample_cols_noalloc_max_columns(K) column slots (65 536 tiles:
 * 16 777 216 slots for K <= 32) and returns GSB_ERR_SCRATCH_LIMIT beyond that.
 * The first call on each device looks up the array's device address; make that
 * first call before starting any stream capture.  On EVERY call the device that
 * owns `cuda_stream` and the buffers must be the calling thread's current
 * device: the array is chosen by cudaGetDevice().  All calls on a device share the one array: it still holds the
 * previous call's words when a call starts (the used part is zeroed on the
 * stream before the launch), and two calls that overlap on the GPU -- different
 * streams, or a second host thread -- race on it.  Same arguments and results
 * as gsb_sample_cols otherwise; no cudaMalloc/cudaFree or allocating library
 * routine is called while launch timing (gsb_timing_enable) is off. */
GSB_API int64_t gsb_sample_cols_noalloc_max_columns(int64_t K);
GSB_API int gsb_sample_cols_noalloc(const int64_t* indptr, const void* indices, int indices_dtype,
                                    int64_t num_cols, const int64_t* seeds, int64_t S_max,
                                    const int64_t* d_S,
                                    int64_t K, int replace, uint64_t seed, uint32_t stream,
                                    int64_t* sub_indptr, int64_t* out_rows, int64_t* out_cols,
                                    int64_t* out_sel, int64_t E_cap, int64_t* d_num_edges,
                                    int* d_err, void* cuda_stream);

/* Weighted per-column sampling (A-Res keys, without replacement; CDF search
 * with replacement).  Replaces Graph::SamplingProbs (src/graph.cc:246-308 ->
 * src/cuda/sampling_probs.cu:190-281).  probs[nnz] float32 device, aligned
 * with `indices`.  Same outputs as gsb_sample_cols.  K <= 1024. */
GSB_API size_t gsb_sample_cols_probs_workspace_bytes(int64_t S_max, int64_t K);
GSB_API int gsb_sample_cols_probs(const int64_t* indptr, const void* indices, int indices_dtype,
                                  int64_t num_cols, const float* probs, const int64_t* seeds,
                                  int64_t S_max,
                                  const int64_t* d_S, int64_t K, int replace, uint64_t seed,
                                  uint32_t stream, int64_t* sub_indptr, int64_t* out_rows,
                                  int64_t* out_cols, int64_t* out_sel, int64_t E_cap,
                                  int64_t* d_num_edges, void* workspace, size_t workspace_bytes,
                                  int* d_err, void* cuda_stream);

/* ------------------------------------------------------------------ slicing
 * Column slicing A[:, seeds].  Replaces Graph::Slicing axis=1 on CSC and
 * Graph::BatchColSlicing (src/graph.cc:90-179, src/batch_graph.cc:13-104 ->
 * src/cuda/slicing.cu:121-181, src/cuda/batch/slicing.cu:40-120).
 * Two calls because the edge count sizes the outputs:
 *   count: sub_indptr[S+1] = exclusive scan of the seeds' degrees (a seed outside
 *          [0, num_cols) sets GSB_ERRBIT_BAD_INPUT and counts as an empty column).
 *   fill : out_rows/out_cols/out_sel[E] with E = sub_indptr[S] (host value).
 * col_bptr[B+1] + encoding_size > 0 add b*encoding_size to the row ids of
 * minibatch b (the reference's `encoding` mode); pass NULL/0 otherwise. */
GSB_API size_t gsb_slice_cols_workspace_bytes(int64_t S);
GSB_API int gsb_slice_cols_count(const int64_t* indptr, int64_t num_cols, const int64_t* seeds,
                                 int64_t S, int64_t* sub_indptr, void* workspace,
                                 size_t workspace_bytes, int* d_err, void* cuda_stream);
GSB_API int gsb_slice_cols_fill(const int64_t* indptr, const void* indices, int indices_dtype,
                                const int64_t* seeds, int64_t S, const int64_t* sub_indptr,
                                int64_t E, int64_t* out_rows, int64_t* out_cols, int64_t* out_sel,
                                const int64_t* col_bptr, int64_t B, int64_t encoding_size,
                                void* cuda_stream);

/* ------------------------------------------------------------------ unique / relabel
 * Per-minibatch first-occurrence unique + relabel.  Replaces
 * Graph::BatchGraphRelabel / BatchGetValidNodes (src/batch_graph.cc:214-284 ->
 * src/cuda/batch/batch_relabel.cu:376-499) and, with B = 1, Graph::GraphRelabel
 * / GetValidNodes (src/graph.cc:577-608 -> src/cuda/unique_reindex.cu:80-199).
 *
 * Minibatch b owns seeds[seeds_ptr[b]..seeds_ptr[b+1]) and edges
 * [edge_ptr[b]..edge_ptr[b+1]).  Its node list is the first-occurrence unique
 * of [seeds_b..., coo_row_b...]; `unique` is the concatenation of the lists,
 * unique_ptr[B+1] their offsets.  out_row[e] / out_col[e] are the positions of
 * coo_row[e] and of seeds[coo_col[e]] inside the minibatch's list (coo_col
 * holds LOCAL column slots, i.e. indices into `seeds`).  out_row/out_col may
 * both be NULL (all_nodes only).  S_max/E_max bound seeds_ptr[B]/edge_ptr[B],
 * which are read on the device.  `unique` has capacity U_cap.
 * id_bound > 0 states the exclusive upper bound of the ids; an id outside
 * [0, id_bound) -- or outside [0, 2^32-1) when id_bound is 0 -- sets
 * GSB_ERRBIT_BAD_INPUT and is relabelled to -1.
 * Limits: node ids < 2^32-1, S_max+E_max < 2^31.
 */
GSB_API size_t gsb_batch_relabel_workspace_bytes(int64_t S_max, int64_t E_max, int64_t B);
GSB_API int gsb_batch_relabel(const int64_t* seeds, const int64_t* seeds_ptr, int64_t B,
                              int64_t S_max, const int64_t* coo_row, const int64_t* coo_col,
                              const int64_t* edge_ptr, int64_t E_max, int64_t id_bound,
                              int64_t* unique, int64_t U_cap, int64_t* unique_ptr,
                              int64_t* out_row, int64_t* out_col, void* workspace,
                              size_t workspace_bytes, int* d_err, void* cuda_stream);

/* out[i] = src[idx[i]] for i < n (int64).  Used for edge_ptr =
 * sub_indptr[seeds_ptr] (src/batch_graph.cc:203). */
GSB_API int gsb_gather_i64(const int64_t* src, const int64_t* idx, int64_t n, int64_t* out,
                           void* cuda_stream);

/* Row gather for node / edge data: row i of `out` = row idx[i] of `src`, rows
 * of row_bytes bytes, contiguous.  `src` is device memory or page-locked host
 * memory (read in place); `out` is device memory.  An index outside
 * [0, src_rows) sets GSB_ERRBIT_BAD_INPUT and leaves its output row untouched.
 * Replaces IndexSelectCPUFromGPU (src/cuda/index_select_uvm.cu:8-49) and the
 * feature / edge-data gathers the callers issue right after sampling
 * (python/gs/matrix_api/matrix.py:19-23; examples/graphsage/graphsage_e2e.py:111-118). */
GSB_API int gsb_gather_rows(const void* src, int64_t row_bytes, int64_t src_rows,
                            const int64_t* idx, int64_t n, void* out, int* d_err,
                            void* cuda_stream);

/* ------------------------------------------------------------------ format conversion
 * CSC -> COO column expansion: out[e] = column owning edge e.  Replaces
 * CSC2COOCUDA (src/cuda/format_transform.cu:23-46). */
GSB_API int gsb_expand_indptr(const int64_t* indptr, int64_t nseg, int64_t nnz, int64_t* out,
                              void* cuda_stream);
/* Sorted COO -> CSC offsets: indptr[k] = #keys < k, k in [0,nkeys].  Replaces the
 * col_sorted branch of COO2CSCCUDA (src/cuda/format_transform.cu:121-142). */
GSB_API int gsb_indptr_from_sorted(const int64_t* keys, int64_t nnz, int64_t nkeys,
                                   int64_t* indptr, void* cuda_stream);
/* Unsorted COO -> CSC / CSR: entries grouped by key (in [0, nkeys)), the entries of a key in
 * their original order.  indptr[nkeys+1] = offsets of the groups, out_vals[nnz] = the values in
 * grouped order, out_pos[nnz] = the position each came from (the edge-id permutation).  A
 * counting sort: histogram, scan, scatter, per-segment sort by original position.  nnz < 2^31,
 * values in [0, 2^32); a key outside [0, nkeys) or a value outside that range sets
 * GSB_ERRBIT_BAD_INPUT.  Replaces the unsorted branches of COO2CSCCUDA / COO2CSRCUDA
 * (src/cuda/format_transform.cu:66-86, 108-120: a device-wide radix sort of (key, position)). */
/* Compaction of an id axis (Graph::Compact): the sorted distinct ids among ids[n] (all below
 * `bound`, the graph's number of rows or columns) and the map id -> position among them.
 * gsb_compact_rank builds the rank table in the workspace (one presence bit per possible id and
 * a running sum per 32-bit word: 3/8 of a byte per possible id) and
 * writes the number of distinct ids to d_count (device); gsb_compact_apply then writes the sorted
 * distinct ids (unique[count], may be NULL) and / or maps an id array of the same id set
 * (out[i] = position of ids[i]; -1 for an id that is not below bound).  Replaces
 * TensorCompactCUDA (src/cuda/compact.cu:10-30: a library sort + unique). */
GSB_API size_t gsb_compact_workspace_bytes(int64_t bound);
GSB_API int gsb_compact_rank(const void* ids, int ids_dtype, int64_t n, int64_t bound, void* workspace,
                             size_t workspace_bytes, int64_t* d_count, int* d_err, void* cuda_stream);
GSB_API int gsb_compact_apply(const void* workspace, int64_t bound, int64_t* unique, const void* ids,
                              int ids_dtype, int64_t n, int64_t* out, void* cuda_stream);
/* Position lookup: out[j] = the smallest i with data[i] == keys[j], or -1 when there is none
 * (an open-addressing table in the workspace; the key -1 stands for "empty" and cannot be looked
 * up: in `data` it sets GSB_ERRBIT_BAD_INPUT, in `keys` it gives -1).  Replaces
 * IndexHashMapInsertCUDA + IndexHashMapSearchCUDA (src/cuda/index_search.cu:101-157), whose
 * table keeps whichever of several equal entries wrote last. */
GSB_API size_t gsb_index_search_workspace_bytes(int64_t n);
GSB_API int gsb_index_search(const int64_t* data, int64_t n, const int64_t* keys, int64_t m, int64_t* out,
                             void* workspace, size_t workspace_bytes, int* d_err, void* cuda_stream);
GSB_API size_t gsb_group_by_key_workspace_bytes(int64_t nnz, int64_t nkeys);
GSB_API int gsb_group_by_key(const int64_t* keys, const int64_t* vals, int64_t nnz, int64_t nkeys,
                             int64_t* indptr, int64_t* out_vals, int64_t* out_pos, void* workspace,
                             size_t workspace_bytes, int* d_err, void* cuda_stream);

/* ------------------------------------------------------------------ per-segment sort
 * Sorts the ids of every segment of a CSC / CSR ascending, in place (node2vec's membership
 * search needs sorted columns).  Replaces SortIndicesCUDA (src/cuda/sort_indices.cu:11-37, one
 * CUB segmented radix sort) and SortIndicesCPU (src/cpu/sort_indices.cc:27-48), reached from
 * Graph::SortCSCIndices (src/graph.cc:610-629).  nnz bounds indptr[nseg]; the workspace holds two
 * work lists and a scratch copy used by segments above 4096 entries only. */
GSB_API size_t gsb_sort_segments_workspace_bytes(int64_t nseg, int64_t nnz, int indices_dtype);
GSB_API int gsb_sort_segments(const int64_t* indptr, void* indices, int indices_dtype, int64_t nseg,
                              int64_t nnz, void* workspace, size_t workspace_bytes, int* d_err,
                              void* cuda_stream);

/* ------------------------------------------------------------------ slicing across
 * Keep the entries of a CSC (CSR) whose row (column) id is in `ids[R]`, each
 * renamed to its position in `ids` (the smallest one for a repeated id), the
 * entry order inside every segment preserved.  Replaces OnIndicesSlicingCUDA
 * (src/cuda/slicing.cu:184-308), reached from Graph::Slicing axis=0 on CSC
 * (src/graph.cc:116-119) and Graph::BatchRowSlicing (src/batch_graph.cc:144-157).
 * Both passes walk the entries, not the segments (cost independent of the
 * degree distribution); nnz_max bounds indptr[nseg], which is read on the device.
 * count: out_indptr[nseg+1]; builds the membership map in the workspace.
 * fill : out_ids / out_seg (nullable) / out_sel [E], E = out_indptr[nseg]
 *        (host value); must be given the workspace of the matching count call.
 * id_bound = exclusive upper bound of the ids stored in `indices`. */
GSB_API size_t gsb_slice_across_workspace_bytes(int64_t nnz_max, int64_t id_bound);
GSB_API int gsb_slice_across_count(const int64_t* indptr, const void* indices, int indices_dtype,
                                   int64_t nseg, int64_t nnz_max, const int64_t* ids, int64_t R,
                                   int64_t id_bound, int64_t* out_indptr, void* workspace,
                                   size_t workspace_bytes, int* d_err, void* cuda_stream);
GSB_API int gsb_slice_across_fill(const int64_t* indptr, const void* indices, int indices_dtype,
                                  int64_t nseg, int64_t nnz_max, int64_t id_bound, int64_t* out_ids,
                                  int64_t* out_seg, int64_t* out_sel, void* workspace,
                                  size_t workspace_bytes, int* d_err, void* cuda_stream);
/* Column AND row selection per minibatch (induced sub-matrices): minibatch b
 * keeps, of the columns cols[col_ptr[b]..col_ptr[b+1]), the entries whose row
 * id occurs in rows[row_ptr[b]..row_ptr[b+1]).  out_ids = position of the row
 * id in `rows` (counted from the start of the whole array; the smallest for a
 * repeated id), out_seg = column slot, out_sel = position of the entry in the
 * operand.  Same count / fill protocol as above (S = col_ptr[B], R =
 * row_ptr[B]).  Replaces BatchCSCColRowSlicingCUDA and CSCColRowSlicingCUDA
 * (src/cuda/fusion/column_row_slicing.cu:154-362), reached from
 * Graph::BatchColRowSlcing (src/batch_graph.cc:107-141). */
GSB_API size_t gsb_slice_cols_rows_workspace_bytes(int64_t S, int64_t R, int64_t B);
GSB_API int gsb_slice_cols_rows_count(const int64_t* indptr, const void* indices,
                                      int indices_dtype, int64_t num_cols, const int64_t* cols,
                                      const int64_t* col_ptr, int64_t S, const int64_t* rows,
                                      const int64_t* row_ptr, int64_t R, int64_t B,
                                      int64_t* out_indptr, void* workspace, size_t workspace_bytes,
                                      int* d_err, void* cuda_stream);
GSB_API int gsb_slice_cols_rows_fill(const int64_t* indptr, const void* indices, int indices_dtype,
                                     int64_t num_cols, const int64_t* cols, const int64_t* col_ptr,
                                     int64_t S, const int64_t* row_ptr, int64_t R, int64_t B,
                                     const int64_t* out_indptr, int64_t* out_ids, int64_t* out_seg,
                                     int64_t* out_sel, const void* workspace, void* cuda_stream);
/* The same filter on a COO: keep edge e iff key[e] is in `ids`; out_key = the
 * position in `ids`, out_other = other[e], out_sel = e, in edge order; the
 * count goes to *d_count (device).  Outputs need capacity nnz.  Replaces
 * COORowSlicingCUDA (src/cuda/slicing.cu:310-377). */
GSB_API size_t gsb_coo_filter_workspace_bytes(int64_t nnz, int64_t id_bound);
GSB_API int gsb_coo_filter(const int64_t* key, const int64_t* other, int64_t nnz,
                           const int64_t* ids, int64_t R, int64_t id_bound, int64_t* out_key,
                           int64_t* out_other, int64_t* out_sel, int64_t* d_count, void* workspace,
                           size_t workspace_bytes, int* d_err, void* cuda_stream);

/* ------------------------------------------------------------------ SpMM / SDDMM (fp32)
 * op: 0 add, 1 sub, 2 mul, 3 div, 4 copy_lhs, 5 copy_rhs, 6 square_rhs, 7 rhs/lhs.
 * reduce: 0 sum, 1 max, 2 min.  Feature rows are contiguous ([n, len]); *_off
 * are optional broadcast offset tables of out_len entries (NULL = identity, a
 * length-1 operand broadcasts).
 * gsb_spmm_segmented: out[seg, :] (+)= reduce over the entries i of segment
 *   seg of op(u[indices[i], :], e[eid(i), :]), eid = e_ids[i] or i.  sum adds
 *   into `out` (caller zero-fills); max/min overwrite, empty segments give 0.
 *   Replaces SpMMCSC and the fused CSC reductions (src/cuda/spmm.cu:107-148,
 *   253-348; src/cuda/fusion/fused_csc_e_square_sum.cu:21-131;
 *   src/cuda/fusion/fused_csc_e_div_u_sum.cu:15-124).
 * gsb_spmm_coo_sum: sum reduction on an unsorted COO with atomics; u_target 0:
 *   features on rows, sums on columns; 2: the reverse.  Replaces SpMMCOO
 *   (src/cuda/spmm.cu:23-56,170-210) and the fused COO sums.
 * gsb_sddmm_coo: out[eid, :] = op(lhs[sel], rhs[sel]), target 0 = row id,
 *   1 = edge id, 2 = column id.  Replaces SDDMMCOO / SDDMMCSC
 *   (src/cuda/sddmm.cu:23-61,120-297). */
GSB_API int gsb_spmm_segmented(const int64_t* indptr, const void* indices, int indices_dtype,
                               const int64_t* e_ids, int64_t nseg, int op, int reduce,
                               const float* u, int64_t u_len, const float* e, int64_t e_len,
                               const int64_t* u_off, const int64_t* e_off, float* out,
                               int64_t out_len, int64_t* arg_u, int64_t* arg_e, void* cuda_stream);
GSB_API int gsb_spmm_coo_sum(const int64_t* row, const int64_t* col, const int64_t* e_ids,
                             int64_t nnz, int op, int u_target, const float* u, int64_t u_len,
                             const float* e, int64_t e_len, const int64_t* u_off,
                             const int64_t* e_off, float* out, int64_t out_len, void* cuda_stream);
GSB_API int gsb_sddmm_coo(const int64_t* row, const int64_t* col, const int64_t* e_ids,
                          int64_t nnz, int op, const float* lhs, int64_t lhs_len, int lhs_target,
                          const float* rhs, int64_t rhs_len, int rhs_target, const int64_t* lhs_off,
                          const int64_t* rhs_off, float* out, int64_t out_len, void* cuda_stream);
/* The `dot` edge map: out[eid, f] = sum over k < reduce of lhs[sel, off_l(f) * reduce + k] *
 * rhs[sel, off_r(f) * reduce + k]; features are [n, len] with len a multiple of `reduce`, the
 * offset tables (NULL = identity, or 0 for an operand of one group) index groups of `reduce`
 * values.  Replaces the binary::Dot instantiation of SDDMMCOO (src/cuda/functor.h:119-138,
 * src/cuda/sddmm.cu:23-61,186). */
GSB_API int gsb_sddmm_coo_dot(const int64_t* row, const int64_t* col, const int64_t* e_ids,
                              int64_t nnz, const float* lhs, int64_t lhs_len, int lhs_target,
                              const float* rhs, int64_t rhs_len, int rhs_target,
                              const int64_t* lhs_off, const int64_t* rhs_off, int64_t reduce,
                              float* out, int64_t out_len, void* cuda_stream);

/* Two u-op-v edge maps over one COO in one pass: out1[eid, :] = op(lhs1[row, :], rhs1[col, :]) and
 * out2[eid, :] = op(lhs2[row, :], rhs2[col, :]); both pairs share shapes and broadcast tables.
 * Replaces FUSED_COO_U_OP_V / FUSED_CSC_U_OP_V (src/cuda/fusion/fused_coo_u_op_v.cu:21-137,
 * src/cuda/fusion/fused_csc_u_op_v.cu:21-150), reached from Graph::FusedUOPV (src/graph.cc:341-356). */
GSB_API int gsb_u_op_v_pair(const int64_t* row, const int64_t* col, const int64_t* e_ids,
                            int64_t nnz, int op, const float* lhs1, const float* rhs1, float* out1,
                            const float* lhs2, const float* rhs2, float* out2, int64_t lhs_len,
                            int64_t rhs_len, const int64_t* lhs_off, const int64_t* rhs_off,
                            int64_t out_len, void* cuda_stream);

/* ------------------------------------------------------------------ collective sampling
 * gsb_list_sample: for every segment [range[b], range[b+1]) choose min(K, len)
 * candidates without replacement -- uniformly (probs NULL) or with weights
 * probs[R] (A-Res keys; weight <= 0 is chosen last) -- and write their
 * positions to out_idx (weighted: ascending; uniform: reservoir slot order, as
 * the reference's ListSampling); out_range[B+1] = offsets of the picks.  range[0]
 * must be 0 (anything else sets GSB_ERRBIT_BAD_INPUT).  R
 * bounds range[B]; out_idx holds min(R, B * K) entries.  For a uniform choice
 * from ONE list (probs NULL, B == 1) range may be NULL: the list is [0, R),
 * min(K, R) picks are written and out_range is not touched (may be NULL);
 * the uniform choice needs no workspace.  Replaces ListSampling / ListSamplingProbs /
 * BatchListSamplingProbs without replacement (src/cuda/list_sampling.cu:20-73,
 * src/cuda/list_sampling_probs.cu:11-89, src/cuda/batch/list_sampling_probs.cu:29-107),
 * which return the same set in descending-key order.
 * gsb_list_sample_replace: K independent draws from [0, n), uniform or by
 * inverse CDF (the reference's replace=true branches). */
GSB_API size_t gsb_list_sample_workspace_bytes(int64_t R, int64_t B);
GSB_API int gsb_list_sample(const float* probs, const int64_t* range, int64_t B, int64_t R,
                            int64_t K, uint64_t seed, uint32_t stream, int64_t* out_idx,
                            int64_t* out_range, void* workspace, size_t workspace_bytes,
                            int* d_err, void* cuda_stream);
GSB_API int gsb_list_sample_replace(const float* probs, int64_t n, int64_t K, uint64_t seed,
                                    uint32_t stream, int64_t* out_idx, void* workspace,
                                    size_t workspace_bytes, void* cuda_stream);

/* ------------------------------------------------------------------ random walks
 * N walkers, walk_length steps over the in-neighbour lists; out is step-major,
 * out[s * N + w], s in [0, walk_length]; -1 from the first dead end on.  Walker
 * w consumes the draws (seed, stream, w, 0..) in order.  Replaces
 * FusedRandomWalkCUDA (src/cuda/fusion/random_walk.cu:10-70) and
 * FusedNode2VecCUDA (src/cuda/fusion/node2vec.cu:67-162; needs sorted
 * columns).  indptr32 (optional, may be NULL): the same offsets as 32-bit
 * unsigned values, usable when the graph has fewer than 2^32 entries -- every
 * walker gathers two offsets at every step, and the half-size array stays in
 * L2 where the 64-bit one does not; when given, `indptr` is not read.
 * Unlike the reference, a draw equal to 1.0 is clamped to the last
 * neighbour and a "previous node" outside [0, num_nodes) counts as unconnected
 * instead of reading out of bounds. */
GSB_API int gsb_random_walk(const int64_t* indptr, const uint32_t* indptr32, const void* indices,
                            int indices_dtype, int64_t num_nodes, const int64_t* seeds, int64_t N,
                            int64_t walk_length, uint64_t seed, uint32_t stream, int64_t* out,
                            int* d_err, void* cuda_stream);
GSB_API int gsb_node2vec(const int64_t* indptr, const uint32_t* indptr32, const void* indices,
                         int indices_dtype, int64_t num_nodes, const int64_t* seeds, int64_t N,
                         int64_t walk_length,
                         double p, double q, uint64_t seed, uint32_t stream, int64_t* out,
                         int* d_err, void* cuda_stream);

/* ------------------------------------------------------------------ whole sampler
 * L-layer GraphSAGE super-batch sampler: per layer fused slice+sample then
 * per-minibatch unique/relabel, the next layer's seeds being this layer's
 * node lists -- the operator sequence of examples/graphsage/graphsage_e2e.py:37-44
 * after gs.jit.compile's fusion passes (python/gs/jit/optimize.py:124-179,
 * 280-325).  No host synchronisation between layers.
 *
 * The caller provides, per layer l, the buffers of gsb_layer_buffers with the
 * stated capacities; S_cap[0] >= S0.  S_cap[l+1] >= S_cap[l] + E_cap[l] and
 * E_cap[l] >= S_cap[l] * fanout[l] can never overflow; smaller capacities
 * (e.g. measured on a warm-up step) are allowed, an overflow then raises
 * GSB_ERRBIT_CAPACITY and the affected layers come back empty.
 * After the call (and a stream sync) each layer's counts are in d_counts[3*l
 * .. 3*l+2] = {S_l, E_l, U_l}.  S0 is an upper bound of the seed count; the
 * live count is seeds_ptr[B], read on the device, so the same launch sequence
 * (e.g. a recorded CUDA graph) serves shorter super-batches too.
 * Layer l draws from the random stream (seed, stream_base + l): a caller that wants different
 * draws from one call to the next advances stream_base by num_layers per call (the reference
 * seeds every call with the same constant, src/cuda/fusion/slice_sampling.cu:154).
 * num_cols = columns of the graph (every layer's seeds are checked against it:
 * on a graph with more rows than columns a sampled row id may not be a valid
 * column); id_bound = exclusive bound of the row ids, for the relabel stage.
 */
typedef struct {
  int64_t S_cap, E_cap;   /* capacities in elements: seeds / edges of this layer      */
  int64_t* sub_indptr;    /* [S_cap+1]                                                */
  int64_t* rows;          /* [E_cap] sampled row ids (global)                         */
  int64_t* cols;          /* [E_cap] local column slot                                */
  int64_t* sel;           /* [E_cap] edge position in the graph                       */
  int64_t* edge_ptr;      /* [B+1]                                                    */
  int64_t* unique;        /* [S_cap+E_cap] node lists; seeds of the next layer        */
  int64_t* unique_ptr;    /* [B+1]                                                    */
  int64_t* block_row;     /* [E_cap] relabelled rows                                  */
  int64_t* block_col;     /* [E_cap] relabelled cols                                  */
} gsb_layer_buffers;

GSB_API size_t gsb_graphsage_workspace_bytes(int64_t B, int num_layers,
                                             const gsb_layer_buffers* layers,
                                             const int64_t* fanouts);
GSB_API int gsb_graphsage_sample(const int64_t* indptr, const void* indices, int indices_dtype,
                                 int64_t num_cols, int64_t id_bound, const int64_t* seeds,
                                 const int64_t* seeds_ptr,
                                 int64_t B, int64_t S0, int num_layers, const int64_t* fanouts,
                                 uint64_t seed, uint32_t stream_base, const gsb_layer_buffers* layers,
                                 int64_t* d_counts, void* workspace, size_t workspace_bytes,
                                 int* d_err, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* GSB200_H_ */
