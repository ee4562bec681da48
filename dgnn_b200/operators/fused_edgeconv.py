"""EdgeConvFuse / FusedEdgeConvFunction (dgNN/operators/fused_edgeconv.py:8-22 of the reference)."""
import torch

from .. import kernels


def EdgeConvFuse(k, src_ind, h_src, h_dst):
    return FusedEdgeConvFunction.apply(k, src_ind, h_src, h_dst)


class FusedEdgeConvFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, k, src_ind, h_src, h_dst):
        out_feat, max_idx = kernels.edgeconv_forward(k, src_ind, h_src, h_dst)  # max_idx stays int32
        ctx.save_for_backward(max_idx, src_ind)
        ctx.k = int(k)
        return out_feat

    @staticmethod
    def backward(ctx, grad_out):
        max_idx, src_ind = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        if torch.are_deterministic_algorithms_enabled():
            # torch.use_deterministic_algorithms(True): the gather over the transposed graph instead of the scatter-add
            grad_src = kernels.edgeconv_backward_ordered(ctx.k, src_ind, grad_out, max_idx)
        else:
            grad_src = kernels.edgeconv_backward(grad_out, max_idx)
        return None, None, grad_src, grad_out
