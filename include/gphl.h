/*
 * gphl.h - C ABI of the B200 (sm_100a) sparse message-passing kernel library.
 *
 * Every entry point takes plain device pointers and sizes and a CUDA stream (passed as
 * void*, NULL = the legacy default stream), launches asynchronously on that stream and
 * returns GPHL_OK or a negative error code; gphl_last_error() gives the message of the
 * calling thread's last failure.  Nothing here allocates or synchronises unless its comment
 * says so.  The TorchScript operator library (libgraphiler.so) and the ctypes binding are
 * thin callers of these functions.
 *
 * The reference binds this path through the TorchScript operator registry rather than a C
 * interface; each entry point names the registered operator / kernel it stands behind.
 *
 * Graph arrays follow the reference's DGLGraph layout (include/dglgraph.h:54-74):
 * `pointer` (n_rows+1) int32, `node_idx` / `edge_idx` (nnz) int32 grouped by row; edge-level
 * tensors are indexed by edge id.  With the in_* arrays the rows are destinations (CSC,
 * reduce side); with the out_* arrays they are sources (CSR).
 *
 * Floating point: fp32 in/out ("f32") or bf16 storage with fp32 arithmetic ("bf16").  All
 * reductions accumulate exactly to the last rounding, in a fixed order: column pairs alternate between
 * one double per column (fp64 pipe) and a compensated two-sum fp32 pair (fp32 pipe), products of two
 * fp32 values are formed exactly (fused multiply-add in double, or the fp32 product plus its error
 * term).  Results are deterministic and independent of how rows are split or sharded.
 */
#ifndef GPHL_H_
#define GPHL_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GPHL_OK 0
#define GPHL_ERR_INVALID_ARGUMENT (-1) /* null pointer, negative size, unsupported shape   */
#define GPHL_ERR_CUDA (-2)             /* a CUDA runtime call or launch failed             */
#define GPHL_MAX_PEERS 16              /* receivers of one multi-receiver launch           */
#define GPHL_ERR_UNSUPPORTED (-3)      /* shape outside what the kernels cover             */
#define GPHL_ERR_TOO_LARGE (-4)        /* exceeds a stated fixed capacity                   */

/* Message of the calling thread's last failed call ("" if none). */
const char *gphl_last_error(void);
/* Library version, (major << 16) | minor. */
int gphl_version(void);
/* Number of kernel launches issued by this process through the library (monotone). */
int64_t gphl_launch_count(void);

/* ---- row-split plan ------------------------------------------------------------------
 * Rows longer than `chunk` entries (hub nodes of power-law graphs) are cut into pieces of
 * `chunk` entries that different warps process; the pieces of one row are then combined in
 * ascending order.  The plan depends only on the pointer array and `chunk`, never on the
 * GPU count.  gphl_plan_create copies the pointer array to the host once (it synchronises
 * `stream`), allocates the plan's device arrays and its scratch for `max_feat` fp32
 * columns per piece; gphl_plan_destroy frees them.  Replaces the reference's one thread
 * (or one warp) per row with a serial neighbour loop (spmm.cu:192-280, spmm.cuh:30-71). */
typedef struct gphl_plan gphl_plan;
#define GPHL_DEFAULT_CHUNK 512
int gphl_plan_create(const int32_t *pointer, int64_t n_rows, int32_t chunk, int64_t max_feat,
                     void *stream, gphl_plan **out_plan);
void gphl_plan_destroy(gphl_plan *plan);
int64_t gphl_plan_num_items(const gphl_plan *plan);      /* work items (rows + extra pieces)   */
int64_t gphl_plan_num_split_rows(const gphl_plan *plan); /* rows that were cut                 */
int64_t gphl_plan_scratch_bytes(const gphl_plan *plan);
int64_t gphl_plan_num_pieces(const gphl_plan *plan);     /* pieces of cut rows = scratch slots */
/* A plan created with max_feat = 0 owns no scratch.  A caller with its own allocator (the TorchScript shims use
 * PyTorch's caching allocator, so that no operator call reaches cudaMalloc) binds a 16-byte aligned buffer of
 * 2 * num_pieces * round_up(max_feat, 8) floats before calls whose feature width is at most max_feat.  The plan
 * does not own a bound buffer.  Not to be called while another thread uses the plan. */
int gphl_plan_bind_scratch(gphl_plan *plan, void *scratch, int64_t max_feat);

/* ---- validation of graph arrays (no counterpart in the reference, which checks nothing: src/dglgraph.cpp:5-24) ------
 * The kernels trust their index arrays.  These check them once, where a graph enters the library: the pointer array
 * is non-decreasing, starts at 0 and ends at n_entries; every idx value lies in [0, idx_limit) and every eidx value
 * (optional) in [0, eidx_limit).  One pass over the arrays on `stream`, which is synchronised; returns GPHL_OK or
 * GPHL_ERR_INVALID_ARGUMENT with gphl_last_error() naming the violation. */
int gphl_validate_csr(const int32_t *pointer, int64_t n_rows, int64_t n_entries, const int32_t *idx, int64_t idx_limit,
                      const int32_t *eidx, int64_t eidx_limit, void *stream);
int gphl_validate_index_i64(const int64_t *index, int64_t n, int64_t limit, void *stream);

/* ---- SpMM: y[v,:] = sum_{i in seg(v)} x[idx[i],:] ------------------------------------
 * copy_u_sum when idx = in_node_indices (my_ops::SpMMSrc, spmm.cu:375-389) and copy_e_sum
 * when idx = in_edge_indices (my_ops::SpMMEdge, spmm.cu:359-373); both go to cuSPARSE in
 * the reference (spmm.cu:57-104).  x is (n_src_rows, feat) row-major, y (n_rows, feat).
 * `plan` may be NULL (one warp per row, no splitting). */
int gphl_spmm_gather_sum_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx,
                             int64_t n_rows, int64_t feat, const float *x, float *y, void *stream);
int gphl_spmm_gather_sum_bf16(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx,
                              int64_t n_rows, int64_t feat, const void *x, void *y, void *stream);

/* The same sum with options.  dst_scale (n_rows floats, may be NULL) multiplies each finished row
 * and GPHL_EPILOGUE_RELU clamps it at zero, so that a GCN layer's `relu(norm * sum)`
 * (examples/GCN/GCN.py:21-27) needs no further pass over the output.  GPHL_ACCUM_FAST replaces the
 * compensated accumulation by plain fp32 adds (the arithmetic of the reference's kernels): about a
 * third of the instructions, but individual sums may then miss rtol 1e-5 / atol 1e-6. */
#define GPHL_ACCUM_FAST 1
#define GPHL_EPILOGUE_RELU 2
int gphl_spmm_gather_sum_ex_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx,
                                int64_t n_rows, int64_t feat, const float *x, const float *dst_scale,
                                int32_t flags, float *y, void *stream);
int gphl_spmm_gather_sum_ex_bf16(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx,
                                 int64_t n_rows, int64_t feat, const void *x, const float *dst_scale,
                                 int32_t flags, void *y, void *stream);

/* ---- SpMM: y[v,h,:] = sum_i x[node_idx[i],h,:] * w[edge_idx[i],h] ---------------------
 * my_ops::gspmm_src_mul_e_sum (CSC arrays, spmm.cu:286-320) and my_ops::gspmm_dst_mul_e_sum
 * (CSR arrays, spmm.cu:322-356); kernels u_mul_e_sum_kernel(_neat) (spmm.cu:192-280), which
 * cover one head and 64 columns only.  x (n, heads*dim), w (n_edges, heads), y (n_rows,
 * heads*dim).  edge_idx may be NULL when edge ids equal row-grouped positions. */
int gphl_spmm_u_mul_e_sum_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx,
                              const int32_t *edge_idx, int64_t n_rows, int64_t heads, int64_t dim,
                              const float *x, const float *w, float *y, void *stream);

/* ---- general g-SpMM --------------------------------------------------------------------
 * SpMMCsrKernel with its functors and broadcast offsets (spmm.cuh:30-123, functor.cuh:18-213, bcast.h:21-35,
 * bcast.cc:20-77), which no registered operator of the reference reaches:
 *   out[v,j] = reduce_{i in row v} op(u[node_idx[i], u_off[j]], e[edge_idx[i], e_off[j]])
 * op: add, sub, mul, div, copy_lhs (u only), copy_rhs (e only), evaluated in fp32 as written; reduce: sum (terms
 * accumulated in double, rounded once), max, min (bit-exact; ties keep the first position; an empty row yields
 * -inf / +inf and argument 0, as the reference's kernel does).  arg_u / arg_e (n_rows x out_len int32, optional):
 * the neighbour id / edge id behind every max or min.  u_off / e_off: one int64 column offset per output column, or
 * both NULL when u and e already have out_len columns.  edge_idx NULL: edge id == position. */
#define GPHL_OP_ADD 0
#define GPHL_OP_SUB 1
#define GPHL_OP_MUL 2
#define GPHL_OP_DIV 3
#define GPHL_OP_COPY_LHS 4
#define GPHL_OP_COPY_RHS 5
#define GPHL_REDUCE_SUM 0
#define GPHL_REDUCE_MAX 1
#define GPHL_REDUCE_MIN 2
int gphl_gspmm_f32(int32_t op, int32_t reduce, const int32_t *pointer, const int32_t *node_idx, const int32_t *edge_idx,
                   int64_t n_rows, int64_t out_len, const float *u, int64_t u_len, const float *e, int64_t e_len,
                   const int64_t *u_off, const int64_t *e_off, float *out, int32_t *arg_u, int32_t *arg_e, void *stream);

/* ---- SDDMM: z[e,:] = l[src[e],:] + r[dst[e],:] ----------------------------------------
 * my_ops::gsddmm_u_add_v_mul_alpha (sddmm.cu:118-134; kernel SDDMMCooKernel,
 * sddmm.cuh:34-71; `alpha` is ignored there and has no counterpart here).  COO arrays in
 * edge-id order, int64 as the reference stores them, or an int32 copy. */
int gphl_sddmm_u_add_v_f32_i64(const int64_t *src, const int64_t *dst, int64_t n_edges, int64_t feat,
                               const float *l, const float *r, float *z, void *stream);
int gphl_sddmm_u_add_v_f32_i32(const int32_t *src, const int32_t *dst, int64_t n_edges, int64_t feat,
                               const float *l, const float *r, float *z, void *stream);

/* ---- SDDMM: z[e,h] = sum_d l[src[e],h,d] * r[dst[e],h,d] ------------------------------
 * u_dot_v: functor binary::Dot (functor.cuh:103-116) with SDDMMCooTreeReduceKernel
 * (sddmm.cuh:80-120).  The reference registers no operator for it. */
int gphl_sddmm_u_dot_v_f32_i64(const int64_t *src, const int64_t *dst, int64_t n_edges, int64_t heads,
                               int64_t dim, const float *l, const float *r, float *z, void *stream);
int gphl_sddmm_u_dot_v_f32_i32(const int32_t *src, const int32_t *dst, int64_t n_edges, int64_t heads,
                               int64_t dim, const float *l, const float *r, float *z, void *stream);
/* The same dot products walked in destination-row order over the CSC arrays (the reference's SDDMM has a CSR
 * variant beside the COO one, sddmm.cuh:150-199 SDDMMCsrKernel): for every position i of row v,
 * z[eid[i],h] = sum_d l[idx[i],h,d] * r[v,h,d]; r[v] is read once per row, not once per edge.  `eidx` NULL means
 * edge id == position.  `plan` (optional) is the row-split plan of `pointer`.  Heads of 4, 8, ..., 128 columns, rows
 * of at most 512 columns, 16-byte aligned; other shapes return GPHL_ERR_UNSUPPORTED (use the COO form). */
int gphl_sddmm_u_dot_v_csc_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *idx, const int32_t *eidx,
                               int64_t n_rows, int64_t heads, int64_t dim, const float *l, const float *r, float *z,
                               void *stream);

/* ---- segment softmax: per row v and head h, softmax over x[edge_idx[seg(v)],h] ---------
 * my_ops::SegmentSoftmax (segment_softmax.cu:3-24; kernel softmax_v,
 * segment_softmax_kernel.cu:4-49, one head only; the multi-head kernel there is an empty
 * stub).  x, y (n_edges, heads) indexed by edge id; y is written at every edge id that
 * appears in edge_idx.  `stats` is caller scratch of 2*n_rows*heads floats (row maxima and
 * reciprocal sums).  edge_idx may be NULL when edge ids equal positions. */
int gphl_segment_softmax_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *edge_idx,
                             int64_t n_rows, int64_t heads, const float *x, float *y, float *stats,
                             void *stream);

/* Segment softmax that allocates nothing and needs no scratch argument.  No counterpart in the
 * reference.  It is meant for callers that cannot obtain device memory at call time - a process
 * that hands the whole GPU to its own pool at start-up and bans cudaMalloc afterwards, or a plugin
 * whose host framework owns the allocator - and gives the same result as gphl_segment_softmax_f32
 * with plan = NULL (one warp per row, no row splitting).  The row statistics are kept in an 8 MiB
 * array inside the library image (held on every GPU that loads the library until exit), which
 * bounds the problem size: n_rows * heads <= GPHL_SOFTMAX_NOALLOC_MAX_ROW_HEADS and heads below that number, otherwise
 * GPHL_ERR_TOO_LARGE is returned and nothing is launched.  The first call on each device looks up
 * the array's address (cudaGetSymbolAddress) with that device current; make that first call
 * before any stream capture begins.  It calls no cudaMalloc / cudaFree or allocating library
 * routine.  All calls on one device share the array: calls whose kernels may overlap on the GPU
 * (different streams, different host threads) race on it and must be serialised by the caller.
 * No clearing is needed between calls: every entry that is read was written by the same call. */
#define GPHL_SOFTMAX_NOALLOC_MAX_ROW_HEADS (1 << 20)
int gphl_segment_softmax_noalloc_f32(const int32_t *pointer, const int32_t *edge_idx, int64_t n_rows,
                                     int64_t heads, const float *x, float *y, void *stream);

/* ---- fused attention: SDDMM u_add_v -> leaky-relu -> edge softmax -> u_mul_e_sum --------
 * out[v,h,:] = sum_i softmax_i(lrelu(el[u_i,h] + er[v,h])) * z[u_i,h,:].  The reference
 * runs this as gsddmm_u_add_v_mul_alpha, aten::leaky_relu_, SegmentSoftmax and
 * gspmm_src_mul_e_sum with three (E,H) round trips through memory; here no edge-level
 * tensor is materialised unless `alpha_out` (n_edges, heads; indexed by edge id through
 * edge_idx, or by position when edge_idx is NULL) is non-NULL.  `stats`: 2*n_rows*heads
 * floats of caller scratch. */
int gphl_gat_fused_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx,
                       const int32_t *edge_idx, int64_t n_rows, int64_t heads, int64_t dim,
                       const float *el, const float *er, const float *z, float slope, float *out,
                       float *alpha_out, float *stats, void *stream);
int gphl_gat_fused_bf16(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx,
                        int64_t n_rows, int64_t heads, int64_t dim, const float *el, const float *er,
                        const void *z, float slope, void *out, float *stats, void *stream);
/* The same with `flags` (GPHL_ACCUM_FAST: plain fp32 accumulation of the weighted rows). */
int gphl_gat_fused_ex_f32(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx,
                          const int32_t *edge_idx, int64_t n_rows, int64_t heads, int64_t dim,
                          const float *el, const float *er, const float *z, float slope, int32_t flags,
                          float *out, float *alpha_out, float *stats, void *stream);
int gphl_gat_fused_ex_bf16(const gphl_plan *plan, const int32_t *pointer, const int32_t *node_idx,
                           int64_t n_rows, int64_t heads, int64_t dim, const float *el, const float *er,
                           const void *z, float slope, int32_t flags, void *out, float *stats,
                           void *stream);

/* Per-node attention scores of the GAT layer: el[n,h] = sum_d z[n,h,d] * attn_src[h,d] and er
 * likewise with attn_dst (the reference computes them as mm(z, attn_weight) on the two halves of
 * its attention vector, examples/GAT/GAT.py:25-31 after the optimizer's split pass,
 * src/optimizer/split.cpp:9-33).  z (n_nodes, heads*dim), attn_* (heads, dim), el / er (n_nodes,
 * heads).  One pass over z. */
int gphl_gat_head_scores_f32(const float *z, const float *attn_src, const float *attn_dst, int64_t n_nodes,
                             int64_t heads, int64_t dim, float *el, float *er, void *stream);

/* ---- broadcasts: y[i,:] = x[idx[i],:] (row gather of row_bytes bytes) -------------------
 * my_ops::BroadcastSrcNode / DstNode / NodeType / EdgeType (broadcast.cu:58-100, ATen
 * advanced indexing there); the composed SrcNodeType / DstNodeType forms pass idx2 so that
 * y[i] = x[idx[idx2[i]]] without materialising the intermediate. */
int gphl_gather_rows_i64(const int64_t *idx, const int64_t *idx2, int64_t n_out, int64_t row_bytes,
                         const void *x, void *y, void *stream);
int gphl_gather_rows_i32(const int32_t *idx, const int32_t *idx2, int64_t n_out, int64_t row_bytes,
                         const void *x, void *y, void *stream);
/* The sending side of a sparse row exchange, one launch for all receivers: receiver p gets rows
 * x[idx[src_start[p] + k]], k in [0, count[p]), at rows dst_start[p] + k of its buffer dst[p].  A buffer may be
 * another GPU's memory mapped into this process: the kernel reads local memory and writes with plain stores (no
 * TMA, no multicast), and deals the rows so that concurrent stores go to different receivers.  The four arrays are
 * host arrays of n_peers <= GPHL_MAX_PEERS entries; rows are multiples of 16 bytes.  No counterpart in the reference
 * (single GPU). */
int gphl_scatter_rows_peers_i64(const int64_t *idx, int32_t n_peers, const int64_t *src_start, const int64_t *count,
                                void *const *dst, const int64_t *dst_start, int64_t row_bytes, const void *x, void *stream);

/* ---- typed linear: y[p_t:p_{t+1},:] = x[p_t:p_{t+1},:] @ w[t] ---------------------------
 * my_ops::SegmentMMNode / SegmentMMEdge (segment_mm.cu:4-33: a device-to-host copy of the
 * pointer, one at::mm per type, one concatenation).  x (m, k), w (n_types, k, n), y (m, n),
 * all row-major fp32; type_pointer (n_types+1) int32 on the device and never read on the
 * host.  gather_idx (m) may be non-NULL to take row i of the product from x[gather_idx[i]]
 * (fuses the BroadcastSrcNode that precedes SegmentMMEdge in the reference's RGCN/HGT
 * graphs). */
int gphl_segment_mm_f32(const float *x, const float *w, const int32_t *type_pointer, int64_t n_types,
                        int64_t m, int64_t k, int64_t n, const int64_t *gather_idx, float *y,
                        void *stream);

/* The same product on the tensor cores (tcgen05.mma, accumulators in tensor memory), with fp32-level
 * accuracy: operands are split into three bf16 terms and six products are accumulated in fp32.
 * Optional epilogue: y[i,:] *= row_scale[i] (m floats, may be NULL), then max(., 0) if relu != 0 -
 * with n_types = 1 and type_pointer = {0, m} this is a dense layer `relu(scale * (x @ w))`.
 * Needs k % 4 == 0 and 16-byte aligned x, y, workspace (else GPHL_ERR_UNSUPPORTED: use
 * gphl_segment_mm_f32).  `workspace`: gphl_segment_mm_tc_workspace_bytes(n_types, k, n) bytes of
 * caller scratch for the split, transposed weights (rewritten by every call). */
int64_t gphl_segment_mm_tc_workspace_bytes(int64_t n_types, int64_t k, int64_t n);
int gphl_segment_mm_tc_f32(const float *x, const float *w, const int32_t *type_pointer, int64_t n_types,
                           int64_t m, int64_t k, int64_t n, const int64_t *gather_idx,
                           const float *row_scale, int32_t relu, void *workspace, float *y, void *stream);
/* The same in two steps, for weights that are constants of a layer: prepare_weights splits and transposes w into
 * `workspace` once; prepared_f32 multiplies with a workspace prepared earlier (for the same n_types, k, n) and
 * launches the tensor-core kernel only.  The kernel receives the weight slabs by TMA (cp.async.bulk.tensor, 128-byte
 * swizzle) from a tensor map over `workspace`, which must lie in the launching GPU's own memory. */
int gphl_segment_mm_tc_prepare_weights(const float *w, int64_t n_types, int64_t k, int64_t n, void *workspace, void *stream);
int gphl_segment_mm_tc_prepared_f32(const float *x, const void *workspace, const int32_t *type_pointer, int64_t n_types,
                                    int64_t m, int64_t k, int64_t n, const int64_t *gather_idx, const float *row_scale,
                                    int32_t relu, float *y, void *stream);
/* The prepared typed linear with the sending side of a sparse row exchange fused into its epilogue (no counterpart in
 * the single-GPU reference): output row i is stored, besides y (which may be NULL), at row (e & 0xffffffffff) of
 * receiver (e >> 40)'s buffer peer_base[e >> 40] for every entry e = fan_entry[f], f in [fan_ptr[i], fan_ptr[i+1]).
 * fan_ptr (m + 1 int32) and fan_entry (int64) are device arrays; peer_base is a host array of n_peers <=
 * GPHL_MAX_PEERS device pointers, each a (rows, n) float matrix that may live in another GPU's memory mapped into this
 * process.  The kernel reads local memory only and writes with plain stores (no TMA store, no multicast). */
int gphl_segment_mm_tc_fanout_f32(const float *x, const void *workspace, const int32_t *type_pointer, int64_t n_types,
                                  int64_t m, int64_t k, int64_t n, const float *row_scale, int32_t relu, float *y,
                                  int32_t n_peers, void *const *peer_base, const int32_t *fan_ptr, const int64_t *fan_entry,
                                  void *stream);
/* Barrier waits that ran out inside tensor-core kernels since the library was loaded (0 in a
 * healthy process; each kernel wait is bounded and a block that gives up frees its tensor memory
 * and returns).  Synchronises the device. */
int gphl_tc_wait_timeouts(int *count);
/* Exercises that give-up path without any fault: launches one warp that waits, for at most `polls`
 * polls (<= 2^20), on a barrier nothing completes; it must return and raise the counter above by one. */
int gphl_debug_wait_selftest(int32_t polls, void *stream);
int gphl_debug_reset_wait_timeouts(void); /* sets the counter back to 0 (synchronises) */

#ifdef __cplusplus
}
#endif
#endif /* GPHL_H_ */
