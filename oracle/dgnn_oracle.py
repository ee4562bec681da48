"""CPU restatement of the dgNN fused GNN-layer operators (TEST INFRASTRUCTURE ONLY).

This module is the checker for the CUDA library: only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it.  The product
path (``dgnn_b200``) never imports it and has no CPU fallback.

Every function restates, in plain PyTorch index arithmetic on the CPU, what one
reference CUDA kernel computes.  The reference has no CPU implementation and no
stored golden vectors, so the restatement is pinned in two ways:

* ``tests/golden/*.npz`` hold outputs of the reference's own CUDA kernels
  (rebuilt for sm_100a by ``oracle/build_ref.py``) run on a B200 on seeded
  inputs by ``tests/golden/make_golden.py``; ``tests/test_oracle_golden.py``
  checks this module against them on the CPU.
* on a GPU box the live reference build is compared with this module directly
  (``tests/test_ref_live.py``).

All functions work in the dtype of their floating inputs (fp32 for parity,
fp64 for self-checks).  CSR rows are destination nodes, columns are source
nodes; ``row_ptr`` may be int32 or int64, ``col_ind`` is int32/int64.
"""
from __future__ import annotations

import numpy as np
import torch

NEG_INIT = -1e38  # initial value of the running row maximum (fused_gatconv_kernel.cu:45)


# ----------------------------------------------------------------------------
# helpers
# ----------------------------------------------------------------------------
def edge_rows(row_ptr: torch.Tensor) -> torch.Tensor:
    """Row id of every CSR position (the reference finds it by binary search,
    util/computeUtil.h:38-54)."""
    rp = row_ptr.long()
    n = rp.numel() - 1
    return torch.repeat_interleave(torch.arange(n, dtype=torch.long), rp[1:] - rp[:-1])


def leaky_relu(x: torch.Tensor, slope: float) -> torch.Tensor:
    """Macro at fused_gatconv_kernel.cu:13: x > 0 ? x : x * slope."""
    return torch.where(x > 0, x, x * slope)


# ----------------------------------------------------------------------------
# GAT  (dgNN/src/fused_gatconv/fused_gatconv_kernel.cu)
# ----------------------------------------------------------------------------
def gat_edge_softmax(attn_row, attn_col, row_ptr, col_ind, slope):
    """Edge score, LeakyReLU, row max, row sum of exp and the normalised
    attention of every edge (passes 1 and 2 of fused_forward_kernel,
    fused_gatconv_kernel.cu:47-83).  Returns (leaky [E,H], edge_max [N,H],
    edge_sum [N,H], alpha [E,H])."""
    rows = edge_rows(row_ptr)
    cols = col_ind.long()
    n, h = attn_row.shape
    leaky = leaky_relu(attn_row[rows] + attn_col[cols], slope)
    edge_max = torch.full((n, h), NEG_INIT, dtype=attn_row.dtype)
    if rows.numel():
        edge_max = edge_max.scatter_reduce(0, rows[:, None].expand(-1, h), leaky, "amax", include_self=True)
    p = torch.exp(leaky - edge_max[rows])
    edge_sum = torch.zeros((n, h), dtype=attn_row.dtype).index_add_(0, rows, p)
    alpha = p / edge_sum[rows]
    return leaky, edge_max, edge_sum, alpha


def gat_forward(attn_row, attn_col, row_ptr, col_ind, slope, in_feat, attn_drop=0.0, edge_mask=None):
    """fused_forward_kernel (fused_gatconv_kernel.cu:24-118):
    out[r,h,:] = sum_e keep_e * alpha_e / (1 - p) * in_feat[col_e,h,:],
    keep_e = edge_mask[e,h] > attn_drop.  Returns (out, edge_max, edge_sum).
    An empty row gives out = 0, edge_max = -1e38, edge_sum = 0."""
    rows = edge_rows(row_ptr)
    cols = col_ind.long()
    n, h = attn_row.shape
    f = in_feat.shape[2]
    _, edge_max, edge_sum, alpha = gat_edge_softmax(attn_row, attn_col, row_ptr, col_ind, slope)
    w = alpha
    if edge_mask is not None:
        w = w * (edge_mask > attn_drop).to(w.dtype)
    w = w / (1.0 - attn_drop)
    out = torch.zeros((n, h, f), dtype=in_feat.dtype)
    out.index_add_(0, rows, w[:, :, None] * in_feat[cols])
    return out, edge_max, edge_sum


def gat_forward_negative_side(attn_row, attn_col, row_ptr, col_ind, slope, in_feat, attn_drop=0.0, edge_mask=None):
    """The share of gat_forward's result carried by edges whose LeakyReLU output is negative (the edges
    whose gradient fused_backward_kernel scales by the slope, fused_gatconv_kernel.cu:953-954):
      out_neg[r,h,:] = sum_{e: leaky_e < 0} keep_e alpha_e / (1 - p) in_feat[col_e,h,:]
      a_neg[r,h]     = sum_{e: leaky_e < 0} alpha_e.
    With S = <grad_out, out> the row gradient of gat_backward equals
      grad_attn_row = (1 - slope) * (S * a_neg - <grad_out, out_neg>),
    which is how the CUDA library obtains it (checked against gat_backward in the tests)."""
    rows = edge_rows(row_ptr)
    cols = col_ind.long()
    n, h = attn_row.shape
    leaky, _, _, alpha = gat_edge_softmax(attn_row, attn_col, row_ptr, col_ind, slope)
    neg = (leaky < 0).to(alpha.dtype)
    w = alpha * neg
    a_neg = torch.zeros((n, h), dtype=alpha.dtype).index_add_(0, rows, w)
    if edge_mask is not None:
        w = w * (edge_mask > attn_drop).to(w.dtype)
    w = w / (1.0 - attn_drop)
    out_neg = torch.zeros((n, h, in_feat.shape[2]), dtype=in_feat.dtype).index_add_(0, rows, w[:, :, None] * in_feat[cols])
    return out_neg, a_neg


def gat_backward(slope, attn_drop, row_ptr, col_ind, edge_max, edge_sum, edge_mask,
                 in_feat, attn_row, attn_col, grad_out, s_row=None):
    """mhspmm_backward_kernel + mhsddmm + fused_backward_kernel
    (fused_gatconv_kernel.cu:712-763, 814-890, 892-968).
    Returns (grad_feat [N,H,F], grad_attn_row [N,H], grad_attn_col [N,H]).
    The CSC arrays of the reference signature only reorder the same sums, so the
    restatement works from CSR alone.  The matrix may be a column block of a
    larger graph ([n_rows x n_cols], in_feat / attn_col with n_cols rows); the
    per-row sums S then have to come from the whole rows and are passed as
    `s_row` [n_rows,H]."""
    rows = edge_rows(row_ptr)
    cols = col_ind.long()
    n, h = attn_row.shape
    leaky = leaky_relu(attn_row[rows] + attn_col[cols], slope)
    alpha = torch.exp(leaky - edge_max[rows]) / edge_sum[rows]
    keep = torch.ones_like(alpha) if edge_mask is None else (edge_mask > attn_drop).to(alpha.dtype)
    scale = keep / (1.0 - attn_drop)
    # grad_feat[c] = sum_{e: col=c} keep * alpha / (1-p) * grad_out[row_e]      (:712-763)
    grad_feat = torch.zeros_like(in_feat)
    grad_feat.index_add_(0, cols, (alpha * scale)[:, :, None] * grad_out[rows])
    # g_e = <grad_out[row_e], in_feat[col_e]>                                      (:814-890)
    g = (grad_out[rows] * in_feat[cols]).sum(-1) * scale
    # S_r = sum_e alpha_e g_e ; d_e = alpha_e (g_e - S_r) * (slope if leaky<0)     (:892-968)
    if s_row is None:
        s_row = torch.zeros((n, h), dtype=alpha.dtype).index_add_(0, rows, alpha * g)
    d = alpha * (g - s_row[rows])
    d = torch.where(leaky < 0, d * slope, d)
    grad_attn_row = torch.zeros((n, h), dtype=alpha.dtype).index_add_(0, rows, d)
    grad_attn_col = torch.zeros((attn_col.shape[0], h), dtype=alpha.dtype).index_add_(0, cols, d)
    return grad_feat, grad_attn_row, grad_attn_col


def gat_forward_differentiable(attn_row, attn_col, row_ptr, col_ind, slope, in_feat):
    """Same forward built only from differentiable torch ops (no saved
    statistics), used to check gat_backward against autograd."""
    rows = edge_rows(row_ptr)
    cols = col_ind.long()
    n, h = attn_row.shape
    s = attn_row[rows] + attn_col[cols]
    leaky = torch.where(s > 0, s, s * slope)
    m = torch.full((n, h), NEG_INIT, dtype=s.dtype).scatter_reduce(
        0, rows[:, None].expand(-1, h), leaky.detach(), "amax", include_self=True)
    p = torch.exp(leaky - m[rows])
    z = torch.zeros((n, h), dtype=s.dtype).index_add(0, rows, p)
    alpha = p / z[rows]
    out = torch.zeros((n, h, in_feat.shape[2]), dtype=in_feat.dtype)
    return out.index_add(0, rows, alpha[:, :, None] * in_feat[cols])


# ----------------------------------------------------------------------------
# multi-head SDDMM / transpose  (sddmm/mhsddmm_kernel.cu, csr2csc/mhtranspose_kernel.cu)
# ----------------------------------------------------------------------------
def mhsddmm(row_ptr, col_ind, grad, feature):
    """out[e,h] = <grad[row_e,h,:], feature[col_e,h,:]>  (mhsddmm_kernel.cu:5-81)."""
    rows = edge_rows(row_ptr)
    return (grad[rows] * feature[col_ind.long()]).sum(-1)


def mhtranspose(permute, attention):
    """out[i,:] = attention[permute[i],:]  (mhtranspose_kernel.cu:6-26); a bit copy."""
    return attention[permute.long()].clone()


# ----------------------------------------------------------------------------
# MoNet / GMM  (fused_gmmconv/fused_gmmconv_kernel.cu)
# ----------------------------------------------------------------------------
def gaussian(pseudo, mu, inv_sigma):
    """w[e,k] = exp(-0.5 * sum_d ((pseudo[e,d]-mu[k,d]) * inv_sigma[k,d])^2)
    (kernel `gaussian`, fused_gmmconv_kernel.cu:11-22)."""
    t = (pseudo[:, None, :] - mu[None, :, :]) * inv_sigma[None, :, :]
    return torch.exp(-0.5 * (t * t).sum(-1))


def gmm_forward(row_ptr, col_ind, node_feat, pseudo, mu, inv_sigma):
    """out[r,k,:] = sum_{e in row r} w[e,k] * node_feat[col_e,k,:]
    (kernel `fuseGmm`, fused_gmmconv_kernel.cu:24-55); pseudo is indexed by the
    position of the edge in (row_ptr, col_ind)."""
    rows = edge_rows(row_ptr)
    w = gaussian(pseudo, mu, inv_sigma)
    out = torch.zeros((row_ptr.numel() - 1,) + tuple(node_feat.shape[1:]), dtype=node_feat.dtype)
    return out.index_add_(0, rows, w[:, :, None] * node_feat[col_ind.long()])


def gaussian_backward(pseudo, mu, inv_sigma, grad_gauss):
    """Gradients of w = gaussian(pseudo, mu, inv_sigma) given dL/dw = grad_gauss [E,K].
    The reference kernel `gaussian_bp` (fused_gmmconv_kernel.cu:57-87) does not
    compute these (it adds into uninitialised outputs, its warp reductions act
    on by-value copies, and it adds one dimension-summed scalar to every
    dimension), so this follows the derivative of the forward formula:
      dw/dmu[k,d]     =  w t_d s_d          dw/dpseudo[e,d] = -w t_d s_d
      dw/dsigma[k,d]  = -w t_d (p_d - mu_d)   with t_d = (p_d - mu_d) s_d.
    Returns (pseudo_out [E,dim], mu_out [K,dim], sigma_out [K,dim])."""
    diff = pseudo[:, None, :] - mu[None, :, :]           # [E,K,D]
    t = diff * inv_sigma[None, :, :]
    w = torch.exp(-0.5 * (t * t).sum(-1))                # [E,K]
    gw = (grad_gauss * w)[:, :, None]                    # [E,K,1]
    dmu = (gw * t * inv_sigma[None]).sum(0)
    dsig = (-gw * t * diff).sum(0)
    dps = (-gw * t * inv_sigma[None]).sum(1)
    return dps, dmu, dsig


# ----------------------------------------------------------------------------
# EdgeConv  (fused_edgeconv/fused_edgeconv_kernel.cu)
# ----------------------------------------------------------------------------
def edgeconv_forward(k, src_ind, h_src, h_dst):
    """out[i,f] = max_j (h_dst[i,f] + h_src[src_ind[i*k+j], f]); max_idx[i,f] is the
    source id that attains it (edgeconv_forward_kernel, fused_edgeconv_kernel.cu:7-49).
    On exact ties the reference's butterfly is order dependent; the smallest j is
    taken here.  Returns (out [M,F], max_idx [M,F] int64)."""
    m, f = h_src.shape
    src = src_ind.long().view(m, k)
    cand = h_dst[:, None, :] + h_src[src]                 # [M,k,F]
    out = cand.max(dim=1).values
    first = (cand == out[:, None, :]).to(torch.int8).argmax(dim=1)   # smallest j on ties
    max_idx = torch.gather(src, 1, first)
    return out, max_idx


def edgeconv_backward(grad_out, max_idx):
    """grad_src[max_idx[i,f], f] += grad_out[i,f] on a zero tensor (the intent of
    edgeconv_backward_kernel, fused_edgeconv_kernel.cu:76-86; the reference
    zeroes inside the scattering kernel and so races)."""
    grad_src = torch.zeros_like(grad_out)
    return grad_src.scatter_add_(0, max_idx.long(), grad_out)


# ----------------------------------------------------------------------------
# format conversion  (convert/convert_kernel.cu: cuSPARSE csr2cscEx2 / Xcoo2csr)
# ----------------------------------------------------------------------------
def csr2csc(row_ptr, col_ind, n_cols=None):
    """Stable counting sort of the CSR entries by column: col_ptr [n_cols+1],
    row_ind [E] (row of each entry), permute [E] (its CSR position).  Within a
    column the entries keep their CSR order.  The reference calls
    cusparseCsr2cscEx2 (convert_kernel.cu:13-21) with the position carried as an
    fp32 value; its callers use scipy's tocsc() (script/train/train_gatconv.py:78-94),
    which this matches.  Returns int64 numpy-backed tensors."""
    rp = row_ptr.long().numpy()
    ci = col_ind.long().numpy()
    n_rows = rp.shape[0] - 1
    n_cols = n_rows if n_cols is None else n_cols
    rows = np.repeat(np.arange(n_rows, dtype=np.int64), rp[1:] - rp[:-1])
    perm = np.argsort(ci, kind="stable")
    col_ptr = np.zeros(n_cols + 1, dtype=np.int64)
    np.cumsum(np.bincount(ci, minlength=n_cols), out=col_ptr[1:])
    return torch.from_numpy(col_ptr), torch.from_numpy(rows[perm]), torch.from_numpy(perm.astype(np.int64))


def coo2csr(row_ind, m):
    """row_ptr[i] = number of entries whose row id is < i, for sorted COO row ids
    (cusparseXcoo2csr, convert_kernel.cu:44-49)."""
    ri = row_ind.long().numpy()
    return torch.from_numpy(np.searchsorted(ri, np.arange(m + 1), side="left").astype(np.int64))


def coo_sort(dst, src):
    """Edge list ordered by (dst, src), duplicates kept: what scipy's csr_matrix((data, (row, col))) followed by
    sort_indices() gives the reference's scripts (script/train/train_gatconv.py:78-82)."""
    d, s_ = dst.long().numpy(), src.long().numpy()
    order = np.lexsort((s_, d))
    return torch.from_numpy(d[order]), torch.from_numpy(s_[order])


def knn_graph(points, k):
    """k nearest neighbours inside every cloud of points [B,P,D] (the graph the reference builds with DGL's
    KNNGraph, script/train/train_edgeconv.py:49): squared distances accumulated dimension by dimension in fp32
    with separately rounded multiply and add, the point itself included, ascending distance, ties to the smaller
    index.  Returns src_ind [B*P*k] int64 with global ids cloud*P + neighbour."""
    x = points.detach().cpu().numpy().astype(np.float32)
    b, p, dim = x.shape
    out = np.empty((b, p, k), dtype=np.int64)
    for c in range(b):
        d2 = np.zeros((p, p), dtype=np.float32)
        for dd in range(dim):
            diff = (x[c, :, None, dd] - x[c, None, :, dd]).astype(np.float32)
            d2 = (d2 + (diff * diff).astype(np.float32)).astype(np.float32)
        out[c] = np.argsort(d2, axis=1, kind="stable")[:, :k] + c * p
    return torch.from_numpy(out.reshape(-1))


# ----------------------------------------------------------------------------
# whole layers (dgNN/layers/*.py) -- used for the CPU baseline timing
# ----------------------------------------------------------------------------
def gat_layer_forward(row_ptr, col_ind, feat, W, attn_l, attn_r, slope, heads, out_feats):
    """GATConv.forward without dropout/bias/residual (layers/gatconv_layer.py:69-80),
    differentiable (autograd supplies the backward of the CPU baseline)."""
    h = torch.matmul(feat, W).view(-1, heads, out_feats)
    attn_row = (attn_l * h).sum(-1)
    attn_col = (attn_r * h).sum(-1)
    return gat_forward_differentiable(attn_row, attn_col, row_ptr, col_ind, slope, h)


def gat_fused_step_cpu(attn_row, attn_col, row_ptr, col_ind, slope, in_feat, grad_out, chunk_rows=None):
    """One forward+backward of the fused GAT operator on the CPU, processed in
    destination-row chunks so that the [E,H,F] message tensor stays bounded.
    Returns (out, grad_feat, grad_attn_row, grad_attn_col)."""
    n = row_ptr.numel() - 1
    rp = row_ptr.long()
    chunk_rows = n if chunk_rows is None else chunk_rows
    out = torch.empty_like(in_feat)
    grad_feat = torch.zeros_like(in_feat)
    g_row = torch.empty_like(attn_row)
    g_col = torch.zeros_like(attn_col)
    for r0 in range(0, n, chunk_rows):
        r1 = min(n, r0 + chunk_rows)
        lo, hi = int(rp[r0]), int(rp[r1])
        sub_ptr = rp[r0:r1 + 1] - lo
        sub_col = col_ind[lo:hi]
        # local rows r0..r1 see global columns: evaluate with a row-sliced attn_row
        o, emax, esum = _gat_forward_rows(attn_row[r0:r1], attn_col, sub_ptr, sub_col, slope, in_feat)
        out[r0:r1] = o
        gf, gr, gc = _gat_backward_rows(slope, sub_ptr, sub_col, emax, esum, in_feat,
                                        attn_row[r0:r1], attn_col, grad_out[r0:r1])
        grad_feat += gf
        g_row[r0:r1] = gr
        g_col += gc
    return out, grad_feat, g_row, g_col


def _gat_forward_rows(attn_row_blk, attn_col, sub_ptr, sub_col, slope, in_feat):
    rows = edge_rows(sub_ptr)
    cols = sub_col.long()
    nb, h = attn_row_blk.shape
    leaky = leaky_relu(attn_row_blk[rows] + attn_col[cols], slope)
    emax = torch.full((nb, h), NEG_INIT, dtype=leaky.dtype)
    if rows.numel():
        emax = emax.scatter_reduce(0, rows[:, None].expand(-1, h), leaky, "amax", include_self=True)
    p = torch.exp(leaky - emax[rows])
    esum = torch.zeros((nb, h), dtype=p.dtype).index_add_(0, rows, p)
    alpha = p / esum[rows]
    out = torch.zeros((nb,) + tuple(in_feat.shape[1:]), dtype=in_feat.dtype)
    out.index_add_(0, rows, alpha[:, :, None] * in_feat[cols])
    return out, emax, esum


def _gat_backward_rows(slope, sub_ptr, sub_col, emax, esum, in_feat, attn_row_blk, attn_col, grad_blk,
                       grad_feat_acc=None, grad_col_acc=None):
    """Backward of one destination-row chunk; when the accumulators are given the
    source-side gradients are added into them in place (no full-size temporaries)."""
    rows = edge_rows(sub_ptr)
    cols = sub_col.long()
    nb, h = attn_row_blk.shape
    leaky = leaky_relu(attn_row_blk[rows] + attn_col[cols], slope)
    alpha = torch.exp(leaky - emax[rows]) / esum[rows]
    gf = torch.zeros_like(in_feat) if grad_feat_acc is None else grad_feat_acc
    gf.index_add_(0, cols, alpha[:, :, None] * grad_blk[rows])
    g = (grad_blk[rows] * in_feat[cols]).sum(-1)
    s_row = torch.zeros((nb, h), dtype=g.dtype).index_add_(0, rows, alpha * g)
    d = alpha * (g - s_row[rows])
    d = torch.where(leaky < 0, d * slope, d)
    gr = torch.zeros((nb, h), dtype=g.dtype).index_add_(0, rows, d)
    gc = torch.zeros_like(attn_col) if grad_col_acc is None else grad_col_acc
    gc.index_add_(0, cols, d)
    return gf, gr, gc
