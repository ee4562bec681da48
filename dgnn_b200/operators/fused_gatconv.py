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


def _hot_sources(col_ptr, feat):
    """Source rows the forward keeps in the L2: the most referenced columns (a feature row and its logits)."""
    return kernels.l2_hot(col_ptr, 4 * feat.shape[1] * (feat.shape[2] + 1))


def _hot_destinations(row_ptr, grad_out):
    """Destination rows the backward keeps in the L2: the longest rows (a grad_out row and its statistics)."""
    return kernels.l2_hot(row_ptr, 4 * grad_out.shape[1] * (grad_out.shape[2] + 4))


class FusedGATFunction(torch.autograd.Function):
    """On the float4 layout (kernels.gat_fast_shape) the forward also keeps the share of the result that
    comes from edges on the negative side of the LeakyReLU; the backward then gets grad_attn_row from the
    destination rows alone (kernels.gat_rowstat_full) and the column pass writes no per-edge array.  Other
    shapes go through the extension-module calls of the reference signature."""

    @staticmethod
    def forward(ctx, attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind, permute, negative_slope, in_feat,
                attn_drop):
        attn_drop = float(attn_drop)
        ctx.negative_slope = negative_slope
        ctx.attn_drop = attn_drop
        ctx.neg = in_feat.is_cuda and in_feat.dim() == 3 and kernels.gat_fast_shape(in_feat.shape[1], in_feat.shape[2])
        if ctx.neg:
            edge_mask = fused_gat.make_edge_mask(col_ind.numel(), in_feat.shape[1], attn_drop, in_feat.device)
            out_feat, edge_max, edge_sum, out_neg, a_neg = kernels.gat_forward(
                attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat, attn_drop,
                edge_mask if attn_drop > 0.0 else None, neg=True, hot=_hot_sources(col_ptr, in_feat))
            ctx.save_for_backward(col_ptr, row_ind, permute, edge_max, edge_sum, edge_mask, in_feat, attn_row,
                                  attn_col, out_feat, out_neg, a_neg, row_ptr)
            return out_feat
        out_feat, edge_max, edge_sum, edge_mask = fused_gat.gat_forward(
            attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat, attn_drop)
        # the forward output is saved too: the backward's per-row term is <grad_out, out>
        ctx.save_for_backward(row_ptr, col_ind, col_ptr, row_ind, permute, edge_max, edge_sum, edge_mask, in_feat,
                              attn_row, attn_col, out_feat)
        return out_feat

    @staticmethod
    def backward(ctx, grad_out):
        grad_out = grad_out.contiguous()
        if ctx.neg:
            (col_ptr, row_ind, permute, edge_max, edge_sum, edge_mask, in_feat, attn_row, attn_col, out_feat,
             out_neg, a_neg, row_ptr) = ctx.saved_tensors
            pack, grad_attn_row, _ = kernels.gat_rowstat_full(attn_row, edge_max, edge_sum, out_feat, grad_out,
                                                              ctx.negative_slope, out_neg=out_neg, a_neg=a_neg)
            masked = ctx.attn_drop > 0.0
            grad_feat, _, grad_attn_col = kernels.gat_backward_cols(
                None, col_ptr, row_ind, permute if masked else None, pack, edge_mask if masked else None, in_feat,
                attn_col, grad_out, ctx.negative_slope, ctx.attn_drop, row_grad=False,
                hot=_hot_destinations(row_ptr, grad_out))
            return grad_attn_row, grad_attn_col, None, None, None, None, None, None, grad_feat, None
        (row_ptr, col_ind, col_ptr, row_ind, permute, edge_max, edge_sum, edge_mask, in_feat, attn_row, attn_col,
         out_feat) = ctx.saved_tensors
        grad_feat, grad_attn_row, grad_attn_col = fused_gat.gat_backward(
            ctx.negative_slope, ctx.attn_drop, row_ptr, col_ind, col_ptr, row_ind, permute, edge_max, edge_sum,
            edge_mask, in_feat, attn_row, attn_col, grad_out, out_feat)
        return grad_attn_row, grad_attn_col, None, None, None, None, None, None, grad_feat, None


def GATLayerFuse(h, attn_l, attn_r, row_ptr, col_ind, col_ptr, row_ind, permute, negative_slope, attn_drop,
                 bias=None):
    """Attention logits + fused aggregation (+ bias) as one autograd node: the same result as
    GATConvFuse((attn_l*h).sum(-1), (attn_r*h).sum(-1), ..., h, attn_drop) + bias (the
    composition in layers/gatconv_layer.py:74-87 of the reference) with the logits and their
    gradients computed by streaming kernels, the bias added in the aggregation kernel's
    epilogue, its gradient reduced inside the row-statistics pass, and the three gradient
    contributions to h summed in place."""
    return FusedGATLayerFunction.apply(h, attn_l, attn_r, row_ptr, col_ind, col_ptr, row_ind, permute,
                                       negative_slope, attn_drop, bias)


class FusedGATLayerFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, attn_l, attn_r, row_ptr, col_ind, col_ptr, row_ind, permute, negative_slope, attn_drop, bias):
        h = h.contiguous()
        attn_row, attn_col = kernels.gat_logits_forward(h, attn_l, attn_r)
        attn_drop = float(attn_drop)
        edge_mask = fused_gat.make_edge_mask(col_ind.numel(), h.shape[1], attn_drop, h.device)
        out_feat, edge_max, edge_sum, out_neg, a_neg = kernels.gat_forward(
            attn_row, attn_col, row_ptr, col_ind, negative_slope, h, attn_drop,
            edge_mask if attn_drop > 0.0 else None, True, bias, neg=True, hot=_hot_sources(col_ptr, h))
        saved = [col_ptr, row_ind, permute, edge_max, edge_sum, edge_mask, h, attn_row, attn_col, out_feat,
                 out_neg, a_neg, attn_l, attn_r, row_ptr]
        if bias is not None:
            saved.append(bias)
        ctx.save_for_backward(*saved)
        ctx.has_bias = bias is not None
        ctx.negative_slope = negative_slope
        ctx.attn_drop = attn_drop
        return out_feat

    @staticmethod
    def backward(ctx, grad_out):
        (col_ptr, row_ind, permute, edge_max, edge_sum, edge_mask, h, attn_row, attn_col, out_feat,
         out_neg, a_neg, attn_l, attn_r, row_ptr) = ctx.saved_tensors[:15]
        grad_out = grad_out.contiguous()
        masked = ctx.attn_drop > 0.0
        bias = ctx.saved_tensors[15] if ctx.has_bias else None
        # pack, grad_attn_row and the bias gradient all come out of one pass over the destination rows
        pack, grad_attn_row, grad_bias = kernels.gat_rowstat_full(attn_row, edge_max, edge_sum, out_feat, grad_out,
                                                                  ctx.negative_slope, bias=bias, out_neg=out_neg,
                                                                  a_neg=a_neg)
        if grad_bias is not None:
            grad_bias = grad_bias.view_as(bias)
        grad_h, _, grad_attn_col = kernels.gat_backward_cols(
            None, col_ptr, row_ind, permute if masked else None, pack, edge_mask if masked else None, h, attn_col,
            grad_out, ctx.negative_slope, ctx.attn_drop, row_grad=False, hot=_hot_destinations(row_ptr, grad_out))
        grad_l, grad_r = kernels.gat_logits_backward(h, attn_l, attn_r, grad_attn_row, grad_attn_col, grad_h)
        return (grad_h, grad_l.view_as(attn_l), grad_r.view_as(attn_r), None, None, None, None, None, None, None,
                grad_bias)
