/* dgnn_b200 -- C ABI of the B200 (sm_100a) fused GNN-layer kernels.
 *
 * Drop-in boundary for the six torch extension modules of dgSPARSE/dgNN
 * (fused_gatconv, fused_gmmconv, fused_edgeconv, mhsddmm, mhtranspose,
 * format_conversion).  Each entry point below names the reference binding it
 * replaces (path within the dgNN project : line).
 *
 * Conventions
 *  - every pointer is a DEVICE pointer on the current CUDA device; inputs are
 *    borrowed, outputs and workspaces are caller-allocated; the library never
 *    allocates or frees device memory and keeps no state between calls;
 *  - floating data is fp32, row-major, contiguous; node / edge ids are int32;
 *    index-pointer arrays (row_ptr, col_ptr) are int32 or int64, chosen by
 *    `idx_bits` (32 or 64); permutations are int32 (nnz < 2^31);
 *  - CSR rows are destination nodes, columns are source nodes;
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream); calls
 *    only enqueue work and do not synchronise;
 *  - return value: 0 = ok, < 0 = argument error (dgnn_status), > 0 = cudaError_t
 *    reported by the launch.  dgnn_status_string() explains either.
 *  - a NULL or too small workspace where one is required gives
 *    DGNN_ERR_WORKSPACE; sizes come from the *_workspace_bytes() queries.
 */
#ifndef DGNN_B200_H
#define DGNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum dgnn_status {
  DGNN_OK = 0,
  DGNN_ERR_NULL = -1,        /* required pointer is NULL */
  DGNN_ERR_SHAPE = -2,       /* negative or inconsistent size */
  DGNN_ERR_IDX_BITS = -3,    /* idx_bits is not 32 or 64 */
  DGNN_ERR_ALIGN = -4,       /* pointer not aligned for vector access */
  DGNN_ERR_OVERFLOW = -5,    /* size does not fit the index type */
  DGNN_ERR_WORKSPACE = -6,   /* workspace missing or too small */
  DGNN_ERR_VALUE = -7,       /* scalar argument out of range */
  DGNN_ERR_STATIC_LIMIT = -8 /* size beyond the fixed scratch of an allocation-free entry point */
} dgnn_status;

int dgnn_version(void);
const char* dgnn_status_string(int status);
/* Guard mode: validation of the index arrays a caller hands over, for use in front of the operators while a
 * program is being brought up (the reference checks nothing: its asserts are compiled out, a bad index is an
 * out-of-bounds access, dgNN/src/fused_gatconv/fused_gatconv.cpp:15-29).  report is a device int[3] that the
 * caller sets to {0, INT_MAX, 0} beforehand: [0] = kind of the first defect noted (0 none; 1 ptr[0] != 0;
 * 2 ptr decreases; 3 ptr[n] != nnz; 4 index outside [0, limit)), [1] = smallest position with a defect, [2] = the
 * value found there.  Nothing but the checked arrays is read.  The Python wrappers run these checks on every
 * call when DGNN_BOUNDS_CHECK=1 is set and raise before any operator kernel is launched. */
int dgnn_check_ptr(int64_t n, int64_t nnz, const void* ptr, int idx_bits, int32_t* report, void* stream);
int dgnn_check_index(int64_t n, const int32_t* idx, int64_t limit, int32_t* report, void* stream);
/* edges per chunk used when rows longer than this are split across warps */
int64_t dgnn_seg_chunk(void);

/* ---- GAT -----------------------------------------------------------------
 * dgnn_gat_forward replaces fused_gatconv.gat_forward and .gat_inference
 * (dgNN/src/fused_gatconv/fused_gatconv.cpp:11-32, 38-60; kernels
 * fused_gatconv_kernel.cu:24-118, 391-478).
 *   e = LeakyReLU(attn_row[r,h] + attn_col[c,h]); alpha = softmax over row r;
 *   out[r,h,:] = sum_e keep_e * alpha_e / (1 - attn_drop) * in_feat[c_e,h,:]
 *   keep_e = edge_mask[e,h] > attn_drop  (edge_mask NULL: every edge kept;
 *   required non-NULL when attn_drop > 0).
 * edge_max / edge_sum [n_rows,h] receive the row maximum and sum of exp saved
 * for the backward pass; pass both NULL for inference.  An empty row gives
 * out = 0, edge_max = -1e38, edge_sum = 0.  attn_col / in_feat are indexed by
 * column id, so they may hold more rows than n_rows (row-block sharding).
 */
size_t dgnn_gat_forward_workspace_bytes(int64_t n_rows, int64_t nnz, int h, int f);
int dgnn_gat_forward(int64_t n_rows, int64_t nnz, int h, int f,
                     const void* row_ptr, int idx_bits, const int32_t* col_ind,
                     const float* attn_row, const float* attn_col, const float* in_feat,
                     float negative_slope, float attn_drop, const float* edge_mask,
                     float* out, float* edge_max, float* edge_sum,
                     void* workspace, size_t workspace_bytes, void* stream);

/* Staged forward for sharded graphs whose source features arrive block by block: the
 * columns are split into blocks, each call sweeps the edges of one block (row_ptr /
 * col_ind of that sub-matrix, attn_col / in_feat of that block) and the per-row softmax
 * state (max, sum, accumulator; dgnn_gat_forward_state_bytes) is carried in `state`.
 * first != 0 starts from an empty state, last != 0 normalises and writes out / edge_max /
 * edge_sum (they may be NULL otherwise).  first = last = 1 is dgnn_gat_forward.  `bias`
 * (NULL or [h*f]) is added to the normalised output by the last call: the bias add of the
 * layer (dgNN/layers/gatconv_layer.py:86-87) as a kernel epilogue.
 * out_neg [n_rows,h,f] and a_neg [n_rows,h] (both NULL or both given; float4 layout only, see
 * dgnn_gat_fast_shape) receive the share of the result that comes from edges whose score lies on the
 * negative side of the LeakyReLU: out_neg = sum_{e: leaky_e < 0} keep_e alpha_e/(1-p) in_feat[c_e],
 * a_neg = sum_{e: leaky_e < 0} alpha_e.  dgnn_gat_rowstat_full turns them into grad_attn_row, which
 * the reference obtains from a per-edge array (fused_backward_kernel, fused_gatconv_kernel.cu:931-957).
 * stage_mask (NULL, or one byte per row; at most 8 stages) makes the stages sparse: bit p of stage_mask[r] says
 * that row r has edges in stage `stage` = p.  A row then starts from an empty state in its first such stage, is
 * normalised and written out in its last one, and is not touched -- no state read or written -- in any other
 * stage; rows without edges in any stage are written by stage 0.  The output pointers must then be the same
 * valid buffers in every stage.  Without a mask every row takes part in every stage (first / last mark the ends).
 * Shapes whose heads hold two or more float4 vectors per lane (e.g. 8 heads x 32) gather in_feat with 256-bit loads
 * when it is 32-byte aligned and with 128-bit loads in another lane layout otherwise; the carried state differs
 * between the two, so every stage of one sweep must pass an in_feat of the same alignment class (any row of a
 * 32-byte aligned tensor is: rows are multiples of 32 bytes there).
 * The staged form has no counterpart in the reference, which is single-GPU. */
int dgnn_gat_fast_shape(int h, int f);   /* 1 when (h, f) uses the float4 layout: f = 4*2^k, h*f <= 1024 */
size_t dgnn_gat_forward_state_bytes(int64_t n_rows, int h, int f);
int dgnn_gat_forward_staged(int64_t n_rows, int64_t nnz, int h, int f,
                            const void* row_ptr, int idx_bits, const int32_t* col_ind,
                            const float* attn_row, const float* attn_col, const float* in_feat,
                            float negative_slope, float attn_drop, const float* edge_mask,
                            const float* bias, float* out, float* edge_max, float* edge_sum,
                            float* out_neg, float* a_neg,
                            float* state, int first, int last,
                            const uint8_t* stage_mask, int stage, const uint32_t* hot_cols,
                            void* workspace, size_t workspace_bytes, void* stream);

/* Row statistics for the backward pass: pack[r,h] = (attn_row, edge_max,
 * 1/edge_sum, S) with S[r,h] = <grad_out[r,h,:], out[r,h,:]>, which equals the
 * reference's per-row sum of alpha*g (fused_gatconv_kernel.cu:903-929) without
 * an edge pass.  pack is [n_rows,h,4] fp32, 16-byte aligned. */
int dgnn_gat_rowstat(int64_t n_rows, int h, int f,
                     const float* attn_row, const float* edge_max, const float* edge_sum,
                     const float* out, const float* grad_out, float* pack, void* stream);

/* Row statistics when `out` carries the fused bias: S uses out - bias, and grad_bias [h*f] =
 * sum_r grad_out[r,:] is produced on the way (fixed-order reduction).  Float4 layout only
 * (f = 4*2^k, h*f <= 1024; DGNN_ERR_SHAPE otherwise). */
size_t dgnn_gat_rowstat_bias_workspace_bytes(int h, int f);
int dgnn_gat_rowstat_bias(int64_t n_rows, int h, int f,
                          const float* attn_row, const float* edge_max, const float* edge_sum,
                          const float* out, const float* grad_out, const float* bias,
                          float* pack, float* grad_bias,
                          void* workspace, size_t workspace_bytes, void* stream);

/* Everything the backward needs from the destination rows in one pass over grad_out, out (and out_neg):
 * pack as above (S uses out - bias when bias is given, and grad_bias [h*f] = sum_r grad_out[r,:] is
 * produced in a fixed order); with out_neg / a_neg (from dgnn_gat_forward_staged)
 *   grad_attn_row[r,h] = (1 - slope) * (S[r,h] * a_neg[r,h] - <grad_out[r,h,:], out_neg[r,h,:]>),
 * equal to the reference's sum over the row's edges of d_e (fused_gatconv_kernel.cu:931-957) without
 * the per-edge array, its scattered write and its row reduction; grad_copy (NULL or [n_rows,h,f])
 * receives a copy of grad_out (on the sharded path: the buffer that other ranks read).  bias/grad_bias,
 * out_neg/a_neg/grad_attn_row are each all NULL or all given.  send_ptr [n_rows+1] / send_pos (NULL, or both
 * given with send_grad [send rows,h,f] and send_pack [send rows,h,4]) fan row r's grad_out and pack out to the
 * send-buffer rows send_pos[send_ptr[r] .. send_ptr[r+1]) -- one per peer and chunk of the sharded layer that
 * fetches the row -- so that no separate packing pass is needed.  Float4 layout only.  The workspace
 * (dgnn_gat_rowstat_bias_workspace_bytes) is needed only with a bias. */
int dgnn_gat_rowstat_full(int64_t n_rows, int h, int f,
                          const float* attn_row, const float* edge_max, const float* edge_sum,
                          const float* out, const float* grad_out, const float* bias,
                          const float* out_neg, const float* a_neg, float negative_slope,
                          float* pack, float* grad_attn_row, float* grad_bias, float* grad_copy,
                          const int32_t* send_ptr, const int32_t* send_pos, float* send_grad, float* send_pack,
                          void* workspace, size_t workspace_bytes, void* stream);

/* Column pass of the backward over the CSC form of an [n_rows x n_cols] block:
 *   grad_feat[c,h,:]   = sum_{e in col c} keep*alpha/(1-p) * grad_out[row_e,h,:]
 *   g_e                = keep/(1-p) * <grad_out[row_e,h,:], in_feat[c,h,:]>
 *   d_e                = alpha_e * (g_e - S_row) * (slope if leaky<0 else 1)
 *   grad_attn_col[c,h] = sum_{e in col c} d_e
 *   grad_attn_row[r,h] = sum_{e in row r} d_e      (via grad_edge, CSR order)
 * replaces mhspmm_backward_kernel + mhsddmm + fused_backward_kernel
 * (fused_gatconv_kernel.cu:712-763, 814-890, 892-968); no float atomics.
 * in_feat / attn_col / grad_feat / grad_attn_col have n_cols rows; pack and
 * grad_out have n_rows rows; permute[j] is the CSR position of CSC entry j and
 * row_ptr is the CSR index pointer of the same block.
 * grad_attn_row may be NULL (the caller takes it from dgnn_gat_rowstat_full): the per-edge array is
 * then neither written nor reduced, row_ptr and permute may be NULL, an edge_mask is indexed by CSC
 * position, and the smaller workspace of dgnn_gat_backward_cols_workspace_bytes(.., 0) suffices. */
size_t dgnn_gat_backward_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t nnz, int h, int f);
size_t dgnn_gat_backward_cols_workspace_bytes(int64_t nnz, int h, int f, int with_grad_attn_row);
int dgnn_gat_backward_cols(int64_t n_rows, int64_t n_cols, int64_t nnz, int h, int f,
                           const void* row_ptr, const void* col_ptr, int idx_bits,
                           const int32_t* row_ind, const int32_t* permute,
                           const float* pack, const float* edge_mask,
                           const float* in_feat, const float* attn_col, const float* grad_out,
                           float negative_slope, float attn_drop,
                           float* grad_feat, float* grad_attn_row, float* grad_attn_col,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Staged column pass: the destination rows are split into blocks, each call sweeps the
 * edges of one row block (its CSC / CSR arrays, pack and grad_out of that block) and the
 * per-column accumulators (dgnn_gat_backward_state_bytes) are carried in `state`;
 * grad_feat / grad_attn_col are written by the last call, grad_attn_row (of the block's
 * rows, unless NULL) by every call.  first = last = 1 is dgnn_gat_backward_cols.  stage_mask / stage: as for
 * dgnn_gat_forward_staged, one byte per column.  hot_rows: as hot_cols there, one bit per destination row (from
 * dgnn_hot_rows on the CSR row pointer): the grad_out / pack rows that stay in the L2.  As in the forward, the lane
 * layout (and with it the carried state) depends on whether in_feat and grad_out are 32-byte aligned: every stage of
 * one sweep must pass tensors of the same alignment class. */
size_t dgnn_gat_backward_state_bytes(int64_t n_cols, int h, int f);
int dgnn_gat_backward_cols_staged(int64_t n_rows, int64_t n_cols, int64_t nnz, int h, int f,
                                  const void* row_ptr, const void* col_ptr, int idx_bits,
                                  const int32_t* row_ind, const int32_t* permute,
                                  const float* pack, const float* edge_mask,
                                  const float* in_feat, const float* attn_col, const float* grad_out,
                                  float negative_slope, float attn_drop,
                                  float* grad_feat, float* grad_attn_row, float* grad_attn_col,
                                  float* state, int first, int last,
                                  const uint8_t* stage_mask, int stage, const uint32_t* hot_rows,
                                  void* workspace, size_t workspace_bytes, void* stream);

/* Whole backward on a square graph: replaces fused_gatconv.gat_backward
 * (fused_gatconv.cpp:104-166).  `out` is the forward result (the reference
 * recomputes the row sums from edges instead). */
int dgnn_gat_backward(int64_t n, int64_t nnz, int h, int f,
                      const void* row_ptr, const void* col_ptr, int idx_bits,
                      const int32_t* row_ind, const int32_t* permute,
                      const float* edge_max, const float* edge_sum, const float* edge_mask,
                      const float* in_feat, const float* out,
                      const float* attn_row, const float* attn_col, const float* grad_out,
                      float negative_slope, float attn_drop,
                      float* grad_feat, float* grad_attn_row, float* grad_attn_col,
                      void* workspace, size_t workspace_bytes, void* stream);

/* Attention logits of the GAT layer around the operator (the reference computes them with
 * tensor ops, dgNN/layers/gatconv_layer.py:74-75): attn_row[n,h] = <feat[n,h,:], attn_l[h,:]>,
 * attn_col[n,h] = <feat[n,h,:], attn_r[h,:]> in one pass.  The backward adds
 * grad_row (x) attn_l + grad_col (x) attn_r into grad_feat IN PLACE and writes the parameter
 * gradients grad_l, grad_r [h,f] (fixed-order reduction).  Only shapes with f = 4*2^k and
 * h*f <= 1024 are supported (DGNN_ERR_SHAPE otherwise: the caller uses tensor ops instead). */
int dgnn_gat_logits_forward(int64_t n, int h, int f, const float* feat,
                            const float* attn_l, const float* attn_r,
                            float* attn_row, float* attn_col, void* stream);
/* The same with a fan-out (see dgnn_gat_rowstat_full): feat[r] and attn_col[r] are also written to the
 * send-buffer rows send_pos[send_ptr[r] .. send_ptr[r+1]) of send_feat [send rows,h,f] / send_attn_col [send rows,h]. */
int dgnn_gat_logits_forward_fan(int64_t n, int h, int f, const float* feat,
                                const float* attn_l, const float* attn_r,
                                float* attn_row, float* attn_col,
                                const int32_t* send_ptr, const int32_t* send_pos,
                                float* send_feat, float* send_attn_col, void* stream);
size_t dgnn_gat_logits_backward_workspace_bytes(int h, int f);
int dgnn_gat_logits_backward(int64_t n, int h, int f, const float* feat,
                             const float* attn_l, const float* attn_r,
                             const float* grad_row, const float* grad_col,
                             float* grad_feat, float* grad_l, float* grad_r,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Dense node projection in front of the operator: out[m,n] = x[m,k] * W, fp32 in and out, W given
 * as [k,n] (w_kn = 1: `torch.matmul(feat, self.W)`, dgNN/layers/gatconv_layer.py:71) or as an
 * nn.Linear weight [n,k] (w_kn = 0).  Runs on the tcgen05 tensor cores with every operand split into
 * two tf32 parts and three products accumulated in fp32 (relative error ~2^-21, the level of an fp32
 * FMA chain).  Supported: n a multiple of 128, k a multiple of 4 and at most 128, m below 2^31
 * (dgnn_project_supported; DGNN_ERR_SHAPE otherwise, the caller then uses a library GEMM).  x and out
 * dense and 16-byte aligned.  Every wait inside the kernel is bounded; dgnn_project_status returns 0
 * unless one ran out. */
int dgnn_project_supported(int64_t m, int n, int k);
size_t dgnn_project_workspace_bytes(int n);
int dgnn_project_forward(int64_t m, int n, int k, const float* x, const float* w, int w_kn, float* out,
                         void* workspace, size_t workspace_bytes, void* stream);
/* Weight gradient of the projection, grad_w = x^T * grad_out (k x n, written [k,n] with w_kn = 1 or
 * [n,k] with w_kn = 0), same shapes, accuracy and tensor-core path as dgnn_project_forward; the
 * reduction over the m rows is split over the CTAs and the partials are added in a fixed order, so
 * the result is reproducible.  In the reference this product is autograd's backward of
 * `torch.matmul(feat, self.W)` (dgNN/layers/gatconv_layer.py:71). */
size_t dgnn_project_wgrad_workspace_bytes(int n);
int dgnn_project_wgrad(int64_t m, int n, int k, const float* x, const float* grad_out, float* grad_w, int w_kn,
                       void* workspace, size_t workspace_bytes, void* stream);
int dgnn_project_status(const void* workspace, void* stream, int* status_out);
/* The second word of a projection workspace is set like the first but never cleared by the calls: a caller
 * that keeps one workspace for many calls (and zeroed its first 8 bytes once) learns here whether any call
 * since then gave up in a wait; clear != 0 zeroes the word after reading.  Synchronises the stream. */
int dgnn_project_sticky_status(void* workspace, void* stream, int* status_out, int clear);
/* Test knobs of the projection kernels (process-wide): wait_limit_cycles > 0 replaces the ~2 s limit of every
 * bounded wait (0 restores it); skip_first_arrive != 0 makes the producer warps withhold the announcement of
 * their first stage, so that the consumer's wait runs out.  A test uses both to run the give-up path (all
 * roles leave, tensor memory is freed, the status words are set, the call returns) without hanging the GPU. */
int dgnn_project_set_test_knobs(int64_t wait_limit_cycles, int skip_first_arrive);

/* Uniform floats in (0,1] from a counter-based Philox4x32-10 stream; stands in
 * for the cuRAND fill of edge_mask (fused_gatconv_kernel.cu:333-341). */
int dgnn_uniform_fill(uint64_t seed, uint64_t offset, int64_t n, float* out, void* stream);

/* The same stream addressed by edge: out[i*h + j] = element edge_id[i]*h + j of the stream of
 * dgnn_uniform_fill(seed, offset).  With edge_id[i] = position of the edge in the CSR of the whole
 * graph, every rank of a sharded layer draws the mask value of an edge that the single-GPU layer
 * draws, in whatever order its own graph pieces hold the edges (forward: destination owner, CSR
 * order; backward: source owner, CSC order).  No counterpart in the reference, which is single-GPU. */
int dgnn_uniform_fill_edges(uint64_t seed, uint64_t offset, int64_t nnz, int h,
                            const int32_t* edge_id, float* out, void* stream);

/* ---- halo exchange of the row-block sharded layer (no counterpart in the reference) ----------
 * dst_a[i,:] = src_a[rank_i][idx_i,:] (and the same for tensor b when row_bytes_b > 0) for
 * i < n_rows, where codes[i] = (rank_i << dgnn_halo_rank_shift()) | idx_i names a row of the block
 * that rank_i owns.  src_a / src_b are HOST arrays of n_ranks device pointers to the owners'
 * buffers ([src_rows, row_bytes] each): this GPU's own memory or peer mappings of other GPUs'
 * memory (read with plain loads over NVLink; no TMA, no multicast).  Row sizes are multiples of 16
 * bytes, all pointers 16-byte aligned, n_ranks <= dgnn_halo_max_ranks(), src_rows <= 2^shift.  A code
 * that names a rank or row out of range is skipped (never dereferenced) and *status (device int,
 * may be NULL) becomes 1.  max_ctas > 0 bounds the grid so that the fetch can run beside other
 * kernels. */
int dgnn_halo_max_ranks(void);
int dgnn_halo_rank_shift(void);
int dgnn_halo_pull(int64_t n_rows, const int32_t* codes, int n_ranks, int64_t src_rows,
                   const void* const* src_a, void* dst_a, int row_bytes_a,
                   const void* const* src_b, void* dst_b, int row_bytes_b,
                   int max_ctas, int32_t* status, void* stream);

/* ---- multi-head SDDMM / transpose -----------------------------------------
 * out[e,h] = <a[row_e,h,:], b[col_e,h,:]>; replaces mhsddmm.mhsddmm
 * (dgNN/src/sddmm/mhsddmm.cc:11-28, mhsddmm_kernel.cu:5-99). */
size_t dgnn_mhsddmm_workspace_bytes(void);
int dgnn_mhsddmm(int64_t n_rows, int64_t nnz, int h, int f,
                 const void* row_ptr, int idx_bits, const int32_t* col_ind,
                 const float* a, const float* b, float* out,
                 void* workspace, size_t workspace_bytes, void* stream);
/* Single-head SDDMM over an edge list in any order: out[e] = <d1[row_ind[e],:], d2[col_ind[e],:]>,
 * d1 [m,k], d2 [n,k]; stands where sddmm.coo_sddmm stands (dgNN/src/sddmm/sddmm.cpp:12-27, a module
 * the reference does not build).  sddmm.csr_sddmm (sddmm.cpp:29-44) is dgnn_mhsddmm with h = 1. */
int dgnn_coo_sddmm(int64_t nnz, int k, const int32_t* row_ind, const int32_t* col_ind,
                   const float* d1, const float* d2, float* out, void* stream);
/* out[i,:] = in[permute[i],:] for [nnz,h] fp32; replaces mhtranspose.mhtranspose
 * (dgNN/src/csr2csc/mhtranspose.cc:10-18, mhtranspose_kernel.cu:6-47). */
int dgnn_mhtranspose(int64_t nnz, int h, const int32_t* permute,
                     const float* in, float* out, void* stream);

/* ---- MoNet / GMM ----------------------------------------------------------
 * w[e,k] = exp(-0.5 sum_d ((pseudo[e,d]-mu[k,d]) inv_sigma[k,d])^2);
 * out[r,k,:] = sum_{e in row r} w[e,k] node_feat[col_e,k,:]; replaces
 * fused_gmmconv.gmmconv (fused_gmmconv.cpp:37-47, fused_gmmconv_kernel.cu:24-55). */
size_t dgnn_gmm_forward_workspace_bytes(int64_t n_rows, int64_t nnz, int kernels, int f);
int dgnn_gmm_forward(int64_t n_rows, int64_t nnz, int kernels, int dim, int f,
                     const void* row_ptr, int idx_bits, const int32_t* col_ind,
                     const float* node_feat, const float* pseudo,
                     const float* mu, const float* inv_sigma, float* out,
                     void* workspace, size_t workspace_bytes, void* stream);
/* replaces fused_gmmconv.Gaussian (fused_gmmconv.cpp:29-35, kernel :11-22) */
int dgnn_gaussian(int64_t nnz, int kernels, int dim, const float* pseudo,
                  const float* mu, const float* inv_sigma, float* gauss, void* stream);
/* Gradients of the Gaussian weights w.r.t. pseudo [nnz,dim], mu and inv_sigma
 * [kernels,dim] given grad_gauss [nnz,kernels]; stands where
 * fused_gmmconv.GaussianBp stands (fused_gmmconv.cpp:49-57), computing the
 * derivative of the forward formula (the reference kernel :57-87 does not).
 * Deterministic two-stage reduction through the workspace. */
size_t dgnn_gaussian_bp_workspace_bytes(int64_t nnz, int kernels, int dim);
int dgnn_gaussian_bp(int64_t nnz, int kernels, int dim, const float* pseudo,
                     const float* mu, const float* inv_sigma, const float* grad_gauss,
                     float* pseudo_out, float* mu_out, float* sigma_out,
                     void* workspace, size_t workspace_bytes, void* stream);

/* ---- EdgeConv -------------------------------------------------------------
 * out[i,f] = max_j (h_dst[i,f] + h_src[src_ind[i*k+j],f]); max_idx[i,f] = that
 * source id (smallest j on ties); replaces fused_edgeconv.edgeconv_forward
 * (fused_edgeconv.cpp:11-27, fused_edgeconv_kernel.cu:7-74).  max_idx is int32
 * (the reference stores the id in a float tensor). */
int dgnn_edgeconv_forward(int64_t m, int f, int k, const int32_t* src_ind,
                          const float* h_src, const float* h_dst,
                          float* out, int32_t* max_idx, void* stream);
/* grad_src = 0; grad_src[max_idx[i,f],f] += grad_out[i,f]; replaces
 * fused_edgeconv.edgeconv_backward (fused_edgeconv.cpp:32-45, kernel :76-100);
 * the zero fill is ordered before the scatter. */
int dgnn_edgeconv_backward(int64_t m, int f, const int32_t* max_idx,
                           const float* grad_out, float* grad_src, void* stream);
/* The same gradient with a fixed summation order (bit-reproducible; the scatter-add above is not): col_ptr [m+1]
 * / row_ind = the CSC form of the neighbour graph (dgnn_csr2csc of row_ptr = 0, k, 2k, ... and src_ind), int32.
 * grad_src[s, j] = sum over the destinations i of s's in-edges, ascending, with max_idx[i, j] == s, of
 * grad_out[i, j]; a destination that lists s twice counts once.  No counterpart in the reference, whose backward
 * races (fused_edgeconv_kernel.cu:76-100). */
int dgnn_edgeconv_backward_ordered(int64_t m, int f, const int32_t* col_ptr, const int32_t* row_ind,
                                   const int32_t* max_idx, const float* grad_out, float* grad_src, void* stream);

/* ---- format conversion ----------------------------------------------------
 * Stable counting sort of CSR entries by column: col_ptr [n_cols+1] (width
 * idx_bits), row_ind [nnz], permute [nnz] = CSR position of each CSC entry;
 * entries of a column keep CSR order.  Replaces format_conversion.csr2csc
 * (dgNN/src/convert/convert.cpp:16-28, convert_kernel.cu:6-42: cuSPARSE
 * csr2cscEx2 with the position carried as an fp32 value). */
size_t dgnn_csr2csc_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t nnz);
int dgnn_csr2csc(int64_t n_rows, int64_t n_cols, int64_t nnz,
                 const void* row_ptr, int idx_bits, const int32_t* col_ind,
                 void* col_ptr, int32_t* row_ind, int32_t* permute,
                 void* workspace, size_t workspace_bytes, void* stream);
/* Same conversion as dgnn_csr2csc for callers that cannot hand over a workspace
 * because they are not allowed to allocate device memory at that point: code
 * that runs after a host application has claimed the whole GPU for its own pool,
 * plug-ins that are given buffers for inputs and outputs only, and services that
 * forbid allocation after start-up so that memory use stays fixed.  It has no
 * counterpart in the reference.  The scratch is a 32 MiB array inside the library
 * image (every GPU that loads the library holds it until the process exits), so
 * sizes are limited: nnz <= dgnn_csr2csc_static_max_nnz() (2^20) and n_cols <=
 * dgnn_csr2csc_static_max_cols() (2^20); anything larger returns
 * DGNN_ERR_STATIC_LIMIT.  The call neither allocates nor frees.  The first call
 * on each device looks up the array's device address (cudaGetSymbolAddress) with
 * that device current; make that first call before any stream capture begins.
 * With CUDA's default lazy module loading the array itself is only set up on a
 * device when this library's code is first used there, so that first call can
 * still take the 32 MiB from the device: make one warm-up call per device at
 * start-up, before the host application claims the memory (or run with
 * CUDA_MODULE_LOADING=EAGER).  The address is remembered per device ordinal for
 * the life of the process: do not call cudaDeviceReset between calls.
 * All calls on a device share the one array: calls that may overlap on the GPU
 * (different streams, different threads) race and must be serialised by the caller. */
int64_t dgnn_csr2csc_static_max_nnz(void);
int64_t dgnn_csr2csc_static_max_cols(void);
int dgnn_csr2csc_static(int64_t n_rows, int64_t n_cols, int64_t nnz,
                        const void* row_ptr, int idx_bits, const int32_t* col_ind,
                        void* col_ptr, int32_t* row_ind, int32_t* permute, void* stream);
/* ---- graph preparation on the device (the step in front of the operators) ---------------------
 * dgnn_coo_sort orders an edge list by (destination, source), duplicates kept: two stable radix sorts of
 * (key, value) pairs with the passes of dgnn_csr2csc -- by source with the destination riding along, then by
 * destination.  Followed by dgnn_coo2csr and dgnn_csr2csc it yields every array the operators take from an
 * edge list in any order; it stands where the scipy recipe of the reference's training scripts stands
 * (dgNN/script/train/train_gatconv.py:78-94: csr_matrix(...), tocsc()).  Node ids are int32 below n_nodes. */
size_t dgnn_coo_sort_workspace_bytes(int64_t nnz, int64_t n_nodes);
int dgnn_coo_sort(int64_t nnz, int64_t n_nodes, const int32_t* dst, const int32_t* src,
                  int32_t* dst_sorted, int32_t* src_sorted,
                  void* workspace, size_t workspace_bytes, void* stream);
/* k nearest neighbours inside every cloud of points [n_clouds, n_points, dim] (squared Euclidean distance,
 * the point itself included, ascending distance, ties to the smaller index): src_ind[(c*n_points + i)*k + j] =
 * c*n_points + (j-th neighbour of point i of cloud c), the regular graph dgnn_edgeconv_forward takes.  Stands
 * where DGL's KNNGraph stands in the reference's point-cloud script (dgNN/script/train/train_edgeconv.py:49).
 * Distances are accumulated with separately rounded multiplies and adds, so the result is reproducible bit for
 * bit.  k <= dgnn_knn_max_k() (32) and k <= n_points. */
int dgnn_knn_max_k(void);
int dgnn_knn_graph(int64_t n_clouds, int64_t n_points, int dim, int k, const float* points,
                   int32_t* src_ind, void* stream);

/* Rows of a gathered tensor that should stay in the L2 (no counterpart in the reference, whose kernels load every
 * row alike, dgNN/src/fused_gatconv/fused_gatconv_kernel.cu:68-100).  indptr [n+1] gives every row's reference count
 * -- the CSC column pointer for the forward gather of in_feat by source, the CSR row pointer for the backward
 * gather of grad_out by destination.  hot_bits [ceil(n/32)] gets bit r & 31 of word r >> 5 set for the rows whose
 * count is at least T, T >= 1 being the smallest threshold that marks at most max_hot rows (rows without
 * references are never marked; counts of 4095 and more fall into one class).  Pass the result as hot_cols /
 * hot_rows to the staged GAT sweeps. */
size_t dgnn_hot_rows_workspace_bytes(void);
/* Sets aside `bytes` of the L2 (clamped to the device's maximum) for lines loaded with the evict_last priority:
 * cudaLimitPersistingL2CacheSize of the calling process's context on the current device; nothing outlasts the
 * process.  Returns the size in force afterwards, or minus a CUDA error code. */
int64_t dgnn_l2_set_aside(int64_t bytes);
int dgnn_hot_rows(int64_t n, const void* indptr, int idx_bits, int64_t max_hot, uint32_t* hot_bits,
                  void* workspace, size_t workspace_bytes, void* stream);
/* row_ptr[i] = number of entries with row id < i, for sorted COO row ids;
 * replaces format_conversion.coo2csr (convert.cpp:32-35, convert_kernel.cu:44-59) */
int dgnn_coo2csr(int64_t nnz, int64_t m, const int32_t* row_ind,
                 void* row_ptr, int idx_bits, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DGNN_B200_H */
