"""Stand-in for the reference extension module `fused_gmmconv`
(dgNN/src/fused_gmmconv/fused_gmmconv.cpp:59-64): gmmconv, Gaussian, GaussianBp."""
from .. import kernels


def gmmconv(rowptr, colind, node_feat, pseudo, mu, sigma):
    """-> out [N,K,F]  (fused_gmmconv.cpp:37-47); `sigma` is the inverse std."""
    return kernels.gmm_forward(rowptr, colind, node_feat, pseudo, mu, sigma)


def Gaussian(pseudo, mu, sigma):
    """-> w [E,K]  (fused_gmmconv.cpp:29-35)"""
    return kernels.gaussian(pseudo, mu, sigma)


def GaussianBp(pseudo, mu, sigma, grad_out):
    """-> [pseudo_out, mu_out, sigma_out]  (fused_gmmconv.cpp:49-57)"""
    return list(kernels.gaussian_bp(pseudo, mu, sigma, grad_out))
