"""The allocation-free CSR -> CSC entry point (dgnn_csr2csc_static).

Some callers may not allocate device memory when they need the conversion: a
host application has already claimed the GPU's memory for its own pool, or a
plug-in interface hands over input and output buffers and nothing else, or a
service rules out allocation after start-up.  For them the library keeps the
conversion's scratch in a fixed 32 MiB array of its own.  This test calls that
entry point through the C ABI twice in a row, on two different graphs, and
requires bit-equal results with the regular entry point (which takes a
caller-supplied workspace); it also checks that sizes beyond the fixed array
are refused.  The file sorts last so that a run stopping at the first failure
has already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from dgnn_b200 import _C, kernels, synth

pytestmark = pytest.mark.gpu


def _static_csr2csc(rp, ci, n_cols, outputs=None):
    """Call dgnn_csr2csc_static with caller-owned inputs and outputs only."""
    lib = _C.lib()
    dev = ci.device
    bits = 64 if rp.dtype == torch.int64 else 32
    n_rows, nnz = rp.numel() - 1, ci.numel()
    if outputs is None:
        outputs = (torch.empty(n_cols + 1, dtype=rp.dtype, device=dev), torch.empty(nnz, dtype=torch.int32, device=dev),
                   torch.empty(nnz, dtype=torch.int32, device=dev))
    col_ptr, row_ind, permute = outputs
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    rc = lib.dgnn_csr2csc_static(n_rows, n_cols, nnz, p(rp), bits, p(ci), p(col_ptr), p(row_ind), p(permute), stream)
    return rc, col_ptr, row_ind, permute


def test_static_scratch_matches_workspace_entry_point_twice(cuda):
    graphs = [
        synth.random_graph(5000, 20, seed=31, long_rows=[(7, 4000)], ptr_dtype=np.int64),   # ~100 k entries, 2 radix passes
        synth.random_graph(300, 6, seed=32, ptr_dtype=np.int32),                            # small: leaves stale scratch behind
        synth.random_graph(70000, 9, seed=33, ptr_dtype=np.int32),                          # ~630 k entries, 3 radix passes
    ]
    for rp, ci in graphs:                      # back-to-back calls share the one scratch array
        rp, ci = rp.to(cuda), ci.to(cuda)
        n = rp.numel() - 1
        rc, cp, ri, pm = _static_csr2csc(rp, ci, n)
        assert rc == 0, _C.lib().dgnn_status_string(rc)
        ecp, eri, epm = kernels.csr2csc(rp, ci)
        torch.cuda.synchronize()
        assert torch.equal(cp, ecp) and torch.equal(ri, eri) and torch.equal(pm, epm)
    # a further call takes no device memory: the free memory of the device is the same before and after
    outputs = (torch.empty_like(cp), torch.empty_like(ri), torch.empty_like(pm))   # the caller's buffers exist beforehand
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(cuda)
    rc, cp2, ri2, pm2 = _static_csr2csc(rp, ci, n, outputs)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(cuda)
    assert rc == 0 and free_after == free_before
    assert torch.equal(cp2, ecp) and torch.equal(ri2, eri) and torch.equal(pm2, epm)


def test_static_scratch_at_its_size_limit(cuda):
    """nnz = n_cols = 2^20, the largest case the fixed array serves (three radix passes, ~28 of the 32 MiB)."""
    lib = _C.lib()
    nnz = n_cols = int(lib.dgnn_csr2csc_static_max_nnz())
    g = torch.Generator().manual_seed(5)
    n_rows = 4096
    rows = torch.sort(torch.randint(0, n_rows, (nnz,), generator=g)).values
    rp = torch.zeros(n_rows + 1, dtype=torch.int64)
    rp[1:] = torch.cumsum(torch.bincount(rows, minlength=n_rows), 0)
    ci = torch.randint(0, n_cols, (nnz,), generator=g, dtype=torch.int32)
    rp, ci = rp.to(cuda), ci.to(cuda)
    rc, cp, ri, pm = _static_csr2csc(rp, ci, n_cols)
    assert rc == 0, lib.dgnn_status_string(rc)
    ecp, eri, epm = kernels.csr2csc(rp, ci, n_cols)
    torch.cuda.synchronize()
    assert torch.equal(cp, ecp) and torch.equal(ri, eri) and torch.equal(pm, epm)


def test_static_scratch_rejects_sizes_beyond_its_limit(cuda):
    lib = _C.lib()
    max_nnz, max_cols = lib.dgnn_csr2csc_static_max_nnz(), lib.dgnn_csr2csc_static_max_cols()
    assert max_nnz == 1 << 20 and max_cols == 1 << 20
    null = ctypes.c_void_p(None)
    assert lib.dgnn_csr2csc_static(10, 10, max_nnz + 1, null, 32, null, null, null, null, null) == -8
    assert lib.dgnn_csr2csc_static(10, max_cols + 1, 5, null, 32, null, null, null, null, null) == -8
    assert b"fixed scratch" in lib.dgnn_status_string(-8)
