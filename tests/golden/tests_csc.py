"""scipy CSC of a CSR graph as int32 tensors (the reference's data preparation,
script/train/train_gatconv.py:78-94)."""
import numpy as np
import scipy.sparse as sp
import torch


def scipy_csc_int32(row_ptr, col_ind):
    rp = row_ptr.cpu().numpy().astype(np.int64)
    ci = col_ind.cpu().numpy().astype(np.int64)
    n = rp.shape[0] - 1
    csr = sp.csr_matrix((np.arange(ci.shape[0], dtype=np.int64), ci, rp), shape=(n, n))
    csr.has_canonical_format = True
    csc = csr.tocsc()
    return (torch.from_numpy(csc.indptr.astype(np.int32)), torch.from_numpy(csc.indices.astype(np.int32)),
            torch.from_numpy(csc.data.astype(np.int32)))
