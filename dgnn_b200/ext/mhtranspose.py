"""Stand-in for the reference extension module `mhtranspose` (dgNN/src/csr2csc/mhtranspose.cc:20-23)."""
from .. import kernels


def mhtranspose(permute, attention):
    """-> out [E,H], out[i,:] = attention[permute[i],:]  (mhtranspose.cc:10-18)"""
    return kernels.mhtranspose(permute, attention)
