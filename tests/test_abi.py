"""The C-ABI library loads without a GPU, exports every symbol the header
declares, and rejects bad arguments before touching the device."""
import ctypes
import os
import re

import pytest

from dgnn_b200 import _C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "dgnn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dgnn_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = _C.lib()
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _C.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_C.SIGNATURES) == declared


def test_version_and_status_strings():
    lib = _C.lib()
    assert lib.dgnn_version() >= 100
    assert lib.dgnn_seg_chunk() >= 32
    assert lib.dgnn_status_string(0) == b"ok"
    for code in range(-8, 0):
        assert lib.dgnn_status_string(code) not in (b"ok", b"unknown dgnn status")


def test_argument_errors_return_before_any_launch():
    lib = _C.lib()
    null = ctypes.c_void_p(None)
    # negative size
    assert lib.dgnn_gat_forward(-1, 0, 1, 4, null, 32, null, null, null, null, 0.2, 0.0, null, null, null, null,
                                null, 0, null) == -2
    # bad index width
    assert lib.dgnn_gat_forward(4, 0, 1, 4, null, 16, null, null, null, null, 0.2, 0.0, null, null, null, null,
                                null, 0, null) == -3
    # dropout probability out of range
    assert lib.dgnn_gat_forward(4, 0, 1, 4, null, 32, null, null, null, null, 0.2, 1.5, null, null, null, null,
                                null, 0, null) == -7
    # NULL pointers
    assert lib.dgnn_gat_forward(4, 0, 1, 4, null, 32, null, null, null, null, 0.2, 0.0, null, null, null, null,
                                null, 0, null) == -1
    assert lib.dgnn_mhtranspose(5, 2, null, null, null, null) == -1
    assert lib.dgnn_csr2csc(3, 3, 0, null, 32, null, null, null, null, null, 0, null) == -1
    assert lib.dgnn_edgeconv_forward(3, 0, 2, null, null, null, null, null, null) == -2
    # 32-bit index pointers cannot address 2^31 edges
    assert lib.dgnn_mhsddmm(4, 2**31, 1, 4, null, 32, null, null, null, null, null, 0, null) == -5


def test_workspace_queries():
    lib = _C.lib()
    seg = lib.dgnn_seg_chunk()
    assert lib.dgnn_gat_forward_workspace_bytes(10, seg, 8, 32) == 256          # no row can be long: just the row counter
    big = lib.dgnn_gat_forward_workspace_bytes(10, 100 * seg, 8, 32)
    assert big >= 2 * 100 * (8 * 32 + 16) * 4
    assert lib.dgnn_csr2csc_workspace_bytes(1000, 1000, 50000) > 0
    assert lib.dgnn_gat_backward_workspace_bytes(1000, 1000, 50000, 8, 32) >= 50000 * 8 * 4


def test_cpu_tensors_are_rejected():
    import torch
    from dgnn_b200 import kernels
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        kernels.mhtranspose(torch.zeros(3, dtype=torch.int32), torch.zeros(3, 2))


def test_wgrad_workspace_covers_one_cta_per_column_group():
    """dgnn_project_wgrad launches (CTAs per group) x groups CTAs, never fewer than one per 128-column group, and
    every CTA writes a 128 x 128 fp32 partial: the workspace query must cover groups > SM count as well (the SM
    count is read from the device, 148 when there is none)."""
    from dgnn_b200 import _C
    lib = _C.lib()
    small = lib.dgnn_project_wgrad_workspace_bytes(256)
    for groups in (1, 2, 148, 149, 400):
        got = lib.dgnn_project_wgrad_workspace_bytes(128 * groups)
        assert got >= 256 + groups * 128 * 128 * 4
        assert got >= small
