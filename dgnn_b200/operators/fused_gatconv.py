"""GATConvFuse / GATConvFuse_inference / FusedGATFunction
(dgNN/operators/fused_gatconv.py:6-34 of the reference): same arguments, same
outputs, same gradient tuple."""
import torch

from .. import kernels
from ..ext import fused_gatconv as fused_gat


def GATConvFuse(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind, permute, negative_slope, in_feat, attn_drop):
    return FusedGATFunction.apply(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind, permute, negative_slope,
                                  in_feat, attn_drop)


def GATConvFuse_inference(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat):
    return fused_gat.gat_inference(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat)


class FusedGATFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind, permute, negative_slope, in_feat,
                attn_drop):
        out_feat, edge_max, edge_sum, edge_mask = fused_gat.gat_forward(
            attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat, attn_drop)
        # the forward output is saved too: the backward's per-row term is <grad_out, out>
        ctx.save_for_backward(row_ptr, col_ind, col_ptr, row_ind, permute, edge_max, edge_sum, edge_mask, in_feat,
                              attn_row, attn_col, out_feat)
        ctx.negative_slope = negative_slope
        ctx.attn_drop = attn_drop
        return out_feat

    @staticmethod
    def backward(ctx, grad_out):
        (row_ptr, col_ind, col_ptr, row_ind, permute, edge_max, edge_sum, edge_mask, in_feat, attn_row, attn_col,
         out_feat) = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        grad_feat, grad_attn_row, grad_attn_col = fused_gat.gat_backward(
            ctx.negative_slope, ctx.attn_drop, row_ptr, col_ind, col_ptr, row_ind, permute, edge_max, edge_sum,
            edge_mask, in_feat, attn_row, attn_col, grad_out, out_feat)
        return grad_attn_row, grad_attn_col, None, None, None, None, None, None, grad_feat, None


def GATLayerFuse(h, attn_l, attn_r, row_ptr, col_ind, col_ptr, row_ind, permute, negative_slope, attn_drop):
    """Attention logits + fused aggregation as one autograd node: the same result as
    GATConvFuse((attn_l*h).sum(-1), (attn_r*h).sum(-1), ..., h, attn_drop) (the
    composition in layers/gatconv_layer.py:74-80 of the reference) with the logits
    and their gradients computed by streaming kernels, and the three gradient
    contributions to h summed in place."""
    return FusedGATLayerFunction.apply(h, attn_l, attn_r, row_ptr, col_ind, col_ptr, row_ind, permute,
                                       negative_slope, attn_drop)


class FusedGATLayerFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, attn_l, attn_r, row_ptr, col_ind, col_ptr, row_ind, permute, negative_slope, attn_drop):
        h = h.contiguous()
        attn_row, attn_col = kernels.gat_logits_forward(h, attn_l, attn_r)
        out_feat, edge_max, edge_sum, edge_mask = fused_gat.gat_forward(
            attn_row, attn_col, row_ptr, col_ind, negative_slope, h, attn_drop)
        ctx.save_for_backward(row_ptr, col_ind, col_ptr, row_ind, permute, edge_max, edge_sum, edge_mask, h,
                              attn_row, attn_col, out_feat, attn_l, attn_r)
        ctx.negative_slope = negative_slope
        ctx.attn_drop = attn_drop
        return out_feat

    @staticmethod
    def backward(ctx, grad_out):
        (row_ptr, col_ind, col_ptr, row_ind, permute, edge_max, edge_sum, edge_mask, h, attn_row, attn_col,
         out_feat, attn_l, attn_r) = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        grad_h, grad_attn_row, grad_attn_col = fused_gat.gat_backward(
            ctx.negative_slope, ctx.attn_drop, row_ptr, col_ind, col_ptr, row_ind, permute, edge_max, edge_sum,
            edge_mask, h, attn_row, attn_col, grad_out, out_feat)
        grad_l, grad_r = kernels.gat_logits_backward(h, attn_l, attn_r, grad_attn_row, grad_attn_col, grad_h)
        return grad_h, grad_l.view_as(attn_l), grad_r.view_as(attn_r), None, None, None, None, None, None, None
