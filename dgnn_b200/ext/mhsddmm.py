"""Stand-in for the reference extension module `mhsddmm` (dgNN/src/sddmm/mhsddmm.cc:30-33)."""
from .. import kernels


def mhsddmm(rowptr, colind, grad, feature):
    """-> out [E,H] = <grad[row_e,h,:], feature[col_e,h,:]>  (mhsddmm.cc:11-28)"""
    return kernels.mhsddmm(rowptr, colind, grad, feature)
