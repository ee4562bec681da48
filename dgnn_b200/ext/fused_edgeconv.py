"""Stand-in for the reference extension module `fused_edgeconv`
(dgNN/src/fused_edgeconv/fused_edgeconv.cpp:47-51)."""
from .. import kernels


def edgeconv_forward(k, src_ind, h_src, h_dst):
    """-> [out_feat, max_idx]; max_idx is a float tensor of source ids as in the
    reference (fused_edgeconv_kernel.cu:58-59)."""
    out, idx = kernels.edgeconv_forward(k, src_ind, h_src, h_dst)
    return [out, idx.float()]


def edgeconv_backward(grad_out, max_idx):
    """-> grad_src; max_idx int32 (the reference caller converts with .int())."""
    return kernels.edgeconv_backward(grad_out, max_idx)
