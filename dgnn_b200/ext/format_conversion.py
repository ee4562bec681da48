"""Stand-in for the reference extension module `format_conversion`
(dgNN/src/convert/convert.cpp:37-41)."""
import torch

from .. import kernels


def csr2csc(rowptr, colind, csr_data):
    """-> [colptr, rowind, cscval]  (convert.cpp:16-28).  cscval[j] = csr_data[p]
    where p is the CSR position of CSC entry j.  Use csr2csc_permute() for the
    exact int32 positions: the reference carries them through this fp32 value
    array, which is exact only below 2^24 entries."""
    colptr, rowind, permute = kernels.csr2csc(rowptr, colind)
    return [colptr, rowind, csr_data[permute.long()]]


def csr2csc_permute(rowptr, colind, n_cols=None):
    """-> (colptr, rowind, permute int32): the three arrays the fused operators take."""
    return kernels.csr2csc(rowptr, colind, n_cols)


def coo2csr(cooRowInd, m):
    """-> rowptr [m+1] int32  (convert.cpp:32-35)"""
    return kernels.coo2csr(cooRowInd, m, torch.int32)
