"""Dense node projection h = feat @ W in front of the fused GAT operator
(`torch.matmul(feat, self.W)`, dgNN/layers/gatconv_layer.py:71 of the reference).

The forward and the weight gradient run on the tcgen05 tensor cores
(dgnn_project_forward / dgnn_project_wgrad: operands split into two tf32 parts,
three products, fp32 accumulation -- fp32 accuracy) for the shapes those kernels
handle; other shapes, and the gradient with respect to the input features, are
plain library GEMMs through torch."""
import torch

from .. import kernels


class ProjectFunction(torch.autograd.Function):
    """`out` comes first: when it is a view, autograd treats the first input of a function that marks an
    input dirty as the tensor written in place (the convention of the built-in in-place operators) and routes
    the other inputs' gradients by position."""

    @staticmethod
    def forward(ctx, out, feat, weight):
        ctx.save_for_backward(feat, weight)
        res = kernels.project_forward(feat, weight, w_kn=True, out=out)
        if out is not None:
            ctx.mark_dirty(out)          # the caller's buffer is the result
        return res

    @staticmethod
    def backward(ctx, grad_out):
        feat, weight = ctx.saved_tensors
        grad_feat = grad_out @ weight.t() if ctx.needs_input_grad[1] else None
        grad_weight = None
        if ctx.needs_input_grad[2]:
            grad_weight = kernels.project_wgrad(feat, grad_out.contiguous(), w_kn=True)
        return None, grad_feat, grad_weight


def project(feat, weight, out=None):
    """feat [M,K] @ weight [K,N] -> [M,N].  `out` (a contiguous float32 [M,N] tensor without autograd history,
    e.g. a detached view of a persistent buffer) receives the result when given."""
    if (feat.is_cuda and feat.dtype == torch.float32 and weight.dtype == torch.float32 and feat.dim() == 2
            and feat.is_contiguous() and weight.is_contiguous()
            and kernels.project_supported(feat.shape[0], weight.shape[1], feat.shape[1])):
        return ProjectFunction.apply(out, feat, weight)
    res = torch.matmul(feat, weight)
    if out is None:
        return res
    return _CopyInto.apply(out, res)


class _CopyInto(torch.autograd.Function):
    """out <- src with the gradient passed through (library-GEMM path of project(out=...))."""

    @staticmethod
    def forward(ctx, out, src):
        out.copy_(src)
        ctx.mark_dirty(out)
        return out

    @staticmethod
    def backward(ctx, grad):
        return None, grad
