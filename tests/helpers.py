"""Shared helpers of the test-suite."""
import numpy as np
import torch

RTOL, ATOL = 1e-4, 1e-5   # fp32 tolerance of the reference's own functional scripts


def assert_close(a, b, what, rtol=RTOL, atol=ATOL):
    a = a.detach().cpu().double()
    b = b.detach().cpu().double()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    if a.numel() == 0:
        return
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    assert not bool(bad.any()), (f"{what}: {int(bad.sum())}/{a.numel()} elements differ; max abs err "
                                 f"{float(err.max()):.3e}, worst ratio {float((err / tol).max()):.2f}")


def assert_equal(a, b, what):
    a = a.detach().cpu()
    b = b.detach().cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    assert torch.equal(a.long() if not a.is_floating_point() else a, b.long() if not b.is_floating_point() else b), \
        f"{what}: not bit-equal"


def gat_inputs(row_ptr, n, h, f, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    attn_row = torch.randn(n, h, generator=g) * scale
    attn_col = torch.randn(n, h, generator=g) * scale
    in_feat = torch.randn(n, h, f, generator=g)
    grad_out = torch.randn(n, h, f, generator=g)
    return attn_row, attn_col, in_feat, grad_out


def scipy_csc(row_ptr, col_ind, n_cols=None):
    """col_ptr, row_ind, permute exactly as the reference's data preparation builds
    them (script/train/train_gatconv.py:78-94): scipy CSR with data = CSR position,
    then tocsc()."""
    import scipy.sparse as sp
    rp = row_ptr.cpu().numpy().astype(np.int64)
    ci = col_ind.cpu().numpy().astype(np.int64)
    n_rows = rp.shape[0] - 1
    n_cols = n_rows if n_cols is None else n_cols
    data = np.arange(ci.shape[0], dtype=np.int64)
    csr = sp.csr_matrix((data, ci, rp), shape=(n_rows, n_cols))
    csr.has_canonical_format = True   # keep duplicates: never sum them
    csc = csr.tocsc()
    return (torch.from_numpy(csc.indptr.astype(np.int64)), torch.from_numpy(csc.indices.astype(np.int64)),
            torch.from_numpy(csc.data.astype(np.int64)))
