"""Stand-in for the reference's single-head `sddmm` extension module
(dgNN/src/sddmm/sddmm.cpp:46-50; the reference's setup.py does not build it)."""
from .. import kernels


def coo_sddmm(rowind, colind, D1, D2):
    """-> out [nnz], out[e] = <D1[rowind[e]], D2[colind[e]]>  (sddmm.cpp:12-27)"""
    return kernels.coo_sddmm(rowind, colind, D1, D2)


def csr_sddmm(rowptr, colind, D1, D2):
    """-> out [nnz] in CSR order, out[e] = <D1[row_e], D2[colind[e]]>  (sddmm.cpp:29-44)"""
    return kernels.mhsddmm(rowptr, colind, D1.unsqueeze(1), D2.unsqueeze(1)).view(-1)
