"""Stand-in for the reference extension module `fused_gatconv`
(dgNN/src/fused_gatconv/fused_gatconv.cpp:168-174): gat_forward, gat_forward_tb,
gat_backward, gat_inference with the same arguments and return lists."""
import torch

from .. import kernels


def _draw_seed() -> int:
    # the reference seeds cuRAND from the wall clock (fused_gatconv_kernel.cu:331);
    # here the seed comes from torch's CPU generator so torch.manual_seed reproduces it
    return int(torch.randint(0, 2**62, (1,), dtype=torch.int64).item())


def make_edge_mask(nnz, h, attn_drop, device):
    """Uniform (0,1] randoms [nnz,h]; an edge is kept where mask > attn_drop.  With
    attn_drop == 0 every edge is kept, so a stride-0 view of a single 1.0 is
    returned instead of nnz*h floats."""
    if attn_drop > 0.0:
        return kernels.uniform_fill((nnz, h), _draw_seed(), 0, device)
    return torch.ones(1, dtype=torch.float32, device=device).expand(nnz, h)


def gat_forward(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat, attn_drop):
    """-> [out_feat, edge_max, edge_sum, edge_mask]  (fused_gatconv.cpp:11-32)"""
    mask = make_edge_mask(col_ind.numel(), in_feat.shape[1], float(attn_drop), in_feat.device)
    out, emax, esum = kernels.gat_forward(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat,
                                          float(attn_drop), mask if attn_drop > 0.0 else None)
    return [out, emax, esum, mask]


def gat_forward_tb(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat, tile_scheduler):
    """-> [out_feat, edge_max, edge_sum]  (fused_gatconv.cpp:68-95).  The regular
    forward already splits long rows on the device, so the tile list is not needed
    and is ignored."""
    out, emax, esum = kernels.gat_forward(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat)
    return [out, emax, esum]


def gat_inference(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat):
    """-> out_feat  (fused_gatconv.cpp:38-60)"""
    return kernels.gat_forward(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat, save_stats=False)[0]


def gat_backward(negative_slope, attn_drop, row_ptr, col_ind, col_ptr, row_ind, permute, edge_max, edge_sum,
                 edge_mask, in_feat, attn_row, attn_col, grad, out_feat=None):
    """-> [grad_feat, grad_attn_row, grad_attn_col]  (fused_gatconv.cpp:104-166).
    The kernels need the forward output for the per-row term <grad, out>; the
    reference signature does not carry it, so it is recomputed when `out_feat`
    is not given (dgNN.operators passes it and skips the recomputation)."""
    attn_drop = float(attn_drop)
    mask = edge_mask if attn_drop > 0.0 else None
    if out_feat is None:
        out_feat = kernels.gat_forward(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat, attn_drop,
                                       mask, save_stats=False)[0]
    gf, gr, gc = kernels.gat_backward(negative_slope, attn_drop, row_ptr, col_ptr, row_ind, permute, edge_max,
                                      edge_sum, mask, in_feat, out_feat, attn_row, attn_col, grad)
    return [gf, gr, gc]
