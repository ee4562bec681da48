"""GmmConvFuse / GmmFuseFunction (dgNN/operators/fused_gmmconv.py:9-27 of the reference)."""
import torch

from ..ext import fused_gmmconv as gmm
from ..ext import mhsddmm, mhtranspose


def GmmConvFuse(rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma):
    return GmmFuseFunction.apply(rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma)


class GmmFuseFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma):
        out = gmm.gmmconv(rowptr, colind, node_feat, pseudo, mu, sigma)  # [N, K, F]
        ctx.save_for_backward(rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma)
        return out

    @staticmethod
    def backward(ctx, grad_out):  # [N, K, F]
        rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        gaussian_grad = mhsddmm.mhsddmm(rowptr, colind, grad_out, node_feat)          # dL/dw [E,K]
        pseudo_tran = mhtranspose.mhtranspose(permute, pseudo)                       # pseudo in CSC order
        node_feat_grad = gmm.gmmconv(colptr, rowind, grad_out, pseudo_tran, mu, sigma)  # transposed aggregation
        pseudo_out, mu_out, sigma_out = gmm.GaussianBp(pseudo, mu, sigma, gaussian_grad)
        return None, None, None, None, None, node_feat_grad, pseudo_out, mu_out, sigma_out
