"""Tensor-level wrappers over the C ABI: validate, allocate outputs, launch.

Each function enqueues kernels on the current stream of the inputs' device and
returns torch tensors; nothing synchronises.
"""
from __future__ import annotations

import os

import torch

from . import _C
from ._C import _cuda_f32, _cuda_i32, _cuda_ptr, _p, _same_bits, _stream, _workspace, check, device_guard, lib


# ------------------------------------------------------------- guard mode
def guard_enabled() -> bool:
    """DGNN_BOUNDS_CHECK=1: every wrapper validates the index arrays it is given (index pointers start at 0, do not
    decrease and end at the entry count; ids lie inside the tensors they index) and raises before an operator kernel
    is launched.  Each check synchronises: a switch for bringing a program up, not for production runs."""
    import os
    return os.environ.get("DGNN_BOUNDS_CHECK", "0") not in ("", "0")


_GUARD_KINDS = {1: "the index pointer does not start at 0", 2: "the index pointer decreases",
                3: "the index pointer does not end at the number of entries", 4: "an id lies outside the tensor it indexes"}


def guard_check(what, ptr=None, nnz=None, index=None, limit=None):
    """Validate an index pointer (`ptr` [n+1] against `nnz` entries) and / or an id array (`index` in [0, limit))."""
    t = ptr if ptr is not None else index
    dev = t.device
    with device_guard(dev):
        report = torch.tensor([0, 2**31 - 1, 0], dtype=torch.int32, device=dev)
        if ptr is not None:
            bits = 64 if ptr.dtype == torch.int64 else 32
            check(lib().dgnn_check_ptr(ptr.numel() - 1, int(nnz), _p(ptr), bits, _p(report), _stream(dev)), "check_ptr")
        if index is not None and index.numel():
            check(lib().dgnn_check_index(index.numel(), _p(index), int(limit), _p(report), _stream(dev)), "check_index")
        kind, pos, val = report.tolist()
    if kind:
        raise RuntimeError(f"dgnn_b200 guard: {what}: {_GUARD_KINDS.get(kind, kind)} (first at position {pos}, value {val}"
                           + (f", limit {int(limit)}" if kind == 4 else "") + ")")


def _dims3(t, name):
    if t.dim() != 3:
        raise RuntimeError(f"dgnn_b200: {name} must be [N,H,F], got shape {tuple(t.shape)}")
    return t.shape


# ------------------------------------------------------------------- GAT
def gat_fast_shape(h, f) -> bool:
    """True when (h, f) runs on the float4 layout (f = 4*2^k, h*f <= 1024): the shapes that have the
    staged sweeps, the bias epilogue and the negative-side outputs."""
    return bool(lib().dgnn_gat_fast_shape(int(h), int(f)))


def _hot_arg(hot, n):
    """Validate a hot-row bit set for a gather out of a tensor of n rows."""
    if hot is None:
        return None
    if not (hot.is_cuda and hot.dtype == torch.int32 and hot.is_contiguous() and hot.numel() >= (n + 31) // 32):
        raise RuntimeError("dgnn_b200: a hot-row set is a contiguous int32 CUDA tensor of ceil(n/32) words (hot_rows)")
    return hot


def hot_rows(indptr, max_hot):
    """Bit set [ceil(n/32)] int32 of the rows whose segment of `indptr` [n+1] is among the longest: at most
    max_hot rows, chosen by a length threshold (dgnn_hot_rows)."""
    indptr, bits = _cuda_ptr(indptr, "indptr")
    n = indptr.numel() - 1
    dev = indptr.device
    with device_guard(dev):
        out = torch.empty(((n + 31) // 32,), dtype=torch.int32, device=dev)
        ws = torch.empty((lib().dgnn_hot_rows_workspace_bytes(),), dtype=torch.uint8, device=dev)
        check(lib().dgnn_hot_rows(n, _p(indptr), bits, int(max_hot), _p(out), _p(ws), ws.numel(), _stream(dev)),
              "hot_rows")
    return out


def l2_set_aside(nbytes, device=None):
    """Set aside part of the L2 of `device` for the hot rows (dgnn_l2_set_aside); returns the bytes in force."""
    with device_guard(torch.device("cuda", torch.cuda.current_device()) if device is None else device):
        got = lib().dgnn_l2_set_aside(int(nbytes))
    if got < 0:
        raise RuntimeError(f"dgnn_b200: l2_set_aside: CUDA error {-got}")
    return got


def l2_hot_budget_bytes():
    """Bytes of often-referenced rows the sweeps try to keep in the L2 (DGNN_L2_HOT_MB; 0 = off, the default:
    on a B200 the hint cuts the DRAM reads of the sweeps by a quarter at R-MAT 2.4 M / 120 M but not their time,
    which the delivery of rows from the L2 to the SMs bounds)."""
    return int(float(os.environ.get("DGNN_L2_HOT_MB", "0")) * 2**20)


def l2_hot(indptr, row_bytes):
    """The hot-row set of a gather of rows of `row_bytes` bytes addressed through `indptr`, or None when the whole
    tensor is small enough for the L2's own replacement (twice the budget) or the budget is 0."""
    n = indptr.numel() - 1
    budget = l2_hot_budget_bytes()
    if budget <= 0 or n * row_bytes <= 2 * budget:
        return None
    return hot_rows(indptr, budget // row_bytes)


def gat_forward(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat, attn_drop=0.0,
                edge_mask=None, save_stats=True, bias=None, neg=False, hot=None):
    """Fused GAT forward.  Returns (out, edge_max, edge_sum); the statistics are
    None when save_stats is False (inference).  `bias` [H*F] is added to the output
    inside the kernel when given.  With neg=True (float4 layout only) two more tensors
    follow: out_neg [N,H,F] and a_neg [N,H], the share of the result that comes from
    edges on the negative side of the LeakyReLU (gat_rowstat_full turns them into
    grad_attn_row).  `hot` (from l2_hot / hot_rows on the CSC column pointer) marks the
    source rows that are kept in the L2."""
    attn_row = _cuda_f32(attn_row, "attn_row")
    attn_col = _cuda_f32(attn_col, "attn_col")
    in_feat = _cuda_f32(in_feat, "in_feat")
    col_ind = _cuda_i32(col_ind, "col_ind")
    row_ptr, bits = _cuda_ptr(row_ptr, "row_ptr")
    _, h, f = _dims3(in_feat, "in_feat")
    n_rows = row_ptr.numel() - 1
    nnz = col_ind.numel()
    if attn_row.shape != (n_rows, h):
        raise RuntimeError(f"dgnn_b200: attn_row must be [{n_rows},{h}], got {tuple(attn_row.shape)}")
    if attn_col.dim() != 2 or attn_col.shape[1] != h or attn_col.shape[0] != in_feat.shape[0]:
        raise RuntimeError("dgnn_b200: attn_col must be [n_src,H] with n_src = in_feat.shape[0]")
    if guard_enabled():
        guard_check("gat_forward", row_ptr, nnz, col_ind, in_feat.shape[0])
    if attn_drop > 0.0:
        if edge_mask is None:
            raise RuntimeError("dgnn_b200: attn_drop > 0 needs an edge_mask")
        edge_mask = _cuda_f32(edge_mask, "edge_mask")
        if edge_mask.shape != (nnz, h):
            raise RuntimeError(f"dgnn_b200: edge_mask must be [{nnz},{h}]")
    else:
        edge_mask = None
    dev = in_feat.device
    with device_guard(dev):
        out = torch.empty((n_rows, h, f), dtype=torch.float32, device=dev)
        edge_max = torch.empty((n_rows, h), dtype=torch.float32, device=dev) if save_stats else None
        edge_sum = torch.empty((n_rows, h), dtype=torch.float32, device=dev) if save_stats else None
        ws_bytes = lib().dgnn_gat_forward_workspace_bytes(n_rows, nnz, h, f)
        ws = _workspace(ws_bytes, dev)
        out_neg = a_neg = None
        if neg:
            out_neg = torch.empty((n_rows, h, f), dtype=torch.float32, device=dev)
            a_neg = torch.empty((n_rows, h), dtype=torch.float32, device=dev)
        hot = _hot_arg(hot, in_feat.shape[0])
        if bias is None and not neg and hot is None:
            check(lib().dgnn_gat_forward(n_rows, nnz, h, f, _p(row_ptr), bits, _p(col_ind), _p(attn_row),
                                         _p(attn_col), _p(in_feat), float(negative_slope), float(attn_drop),
                                         _p(edge_mask), _p(out), _p(edge_max), _p(edge_sum), _p(ws), ws.numel(),
                                         _stream(dev)), "gat_forward")
        else:
            if bias is not None:
                bias = _cuda_f32(bias, "bias").reshape(h * f)
            check(lib().dgnn_gat_forward_staged(n_rows, nnz, h, f, _p(row_ptr), bits, _p(col_ind), _p(attn_row),
                                                _p(attn_col), _p(in_feat), float(negative_slope), float(attn_drop),
                                                _p(edge_mask), _p(bias), _p(out), _p(edge_max), _p(edge_sum),
                                                _p(out_neg), _p(a_neg), None,
                                                1, 1, None, 0, _p(hot), _p(ws), ws.numel(), _stream(dev)),
                  "gat_forward(bias/neg)")
    if neg:
        return out, edge_max, edge_sum, out_neg, a_neg
    return out, edge_max, edge_sum


def _fan_args(fan, n_rows):
    """(send_ptr, send_pos, send_a, send_b) of a fan-out, or four Nones.  fan = dict(ptr [n_rows+1] int32, pos int32,
    a = send buffer of the wide tensor, b = send buffer of the narrow one)."""
    if fan is None:
        return None, None, None, None
    ptr, pos = _cuda_i32(fan["ptr"], "fan ptr"), _cuda_i32(fan["pos"], "fan pos")
    if ptr.numel() != n_rows + 1:
        raise RuntimeError("dgnn_b200: the fan-out pointer must have one entry per row plus one")
    for t in (fan["a"], fan["b"]):
        if not (t.is_cuda and t.is_contiguous() and t.dtype == torch.float32):
            raise RuntimeError("dgnn_b200: send buffers must be contiguous float32 CUDA tensors")
    return ptr, pos, fan["a"], fan["b"]


def gat_rowstat_full(attn_row, edge_max, edge_sum, out, grad_out, negative_slope, bias=None, out_neg=None,
                     a_neg=None, pack=None, grad_copy=None, fan=None):
    """One pass over the destination rows for the backward: returns (pack [N,H,4], grad_attn_row [N,H]
    or None, grad_bias [H*F] or None).  grad_attn_row needs out_neg / a_neg of gat_forward(neg=True);
    grad_bias needs the bias that the forward added to `out`.  `pack` and `grad_copy` (a copy of
    grad_out) are written into the given tensors when passed; `fan` (see _fan_args) additionally writes every
    row's grad_out and pack to its places in the send buffers that other ranks read."""
    out = _cuda_f32(out, "out")
    grad_out = _cuda_f32(grad_out, "grad_out")
    n, h, f = _dims3(out, "out")
    dev = out.device
    with device_guard(dev):
        if pack is None:
            pack = torch.empty((n, h, 4), dtype=torch.float32, device=dev)
        elif not (pack.is_cuda and pack.is_contiguous() and pack.dtype == torch.float32 and pack.shape == (n, h, 4)):
            raise RuntimeError("dgnn_b200: pack must be a contiguous float32 CUDA tensor [N,H,4]")
        if grad_copy is not None and not (grad_copy.is_cuda and grad_copy.is_contiguous()
                                          and grad_copy.dtype == torch.float32 and grad_copy.shape == grad_out.shape):
            raise RuntimeError("dgnn_b200: grad_copy must be a contiguous float32 CUDA tensor shaped like grad_out")
        grad_row = grad_bias = None
        ws = None
        if bias is not None:
            bias = _cuda_f32(bias, "bias").reshape(h * f)
            grad_bias = torch.empty(h * f, dtype=torch.float32, device=dev)
            ws = _workspace(lib().dgnn_gat_rowstat_bias_workspace_bytes(h, f), dev)
        if out_neg is not None:
            out_neg = _cuda_f32(out_neg, "out_neg")
            a_neg = _cuda_f32(a_neg, "a_neg")
            grad_row = torch.empty((n, h), dtype=torch.float32, device=dev)
        f_ptr, f_pos, f_a, f_b = _fan_args(fan, n)
        check(lib().dgnn_gat_rowstat_full(n, h, f, _p(_cuda_f32(attn_row, "attn_row")), _p(_cuda_f32(edge_max, "edge_max")),
                                          _p(_cuda_f32(edge_sum, "edge_sum")), _p(out), _p(grad_out), _p(bias),
                                          _p(out_neg), _p(a_neg), float(negative_slope), _p(pack), _p(grad_row),
                                          _p(grad_bias), _p(grad_copy), _p(f_ptr), _p(f_pos), _p(f_a), _p(f_b),
                                          _p(ws), ws.numel() if ws is not None else 0,
                                          _stream(dev)), "gat_rowstat_full")
    return pack, grad_row, grad_bias


def gat_rowstat_bias(attn_row, edge_max, edge_sum, out, grad_out, bias):
    """Row statistics when `out` includes the fused bias; returns (pack [N,H,4], grad_bias [H*F])."""
    out = _cuda_f32(out, "out")
    grad_out = _cuda_f32(grad_out, "grad_out")
    n, h, f = _dims3(out, "out")
    bias = _cuda_f32(bias, "bias").reshape(h * f)
    dev = out.device
    with device_guard(dev):
        pack = torch.empty((n, h, 4), dtype=torch.float32, device=dev)
        grad_bias = torch.empty(h * f, dtype=torch.float32, device=dev)
        ws = _workspace(lib().dgnn_gat_rowstat_bias_workspace_bytes(h, f), dev)
        check(lib().dgnn_gat_rowstat_bias(n, h, f, _p(_cuda_f32(attn_row, "attn_row")), _p(_cuda_f32(edge_max, "edge_max")),
                                          _p(_cuda_f32(edge_sum, "edge_sum")), _p(out), _p(grad_out), _p(bias), _p(pack),
                                          _p(grad_bias), _p(ws), ws.numel(), _stream(dev)), "gat_rowstat_bias")
    return pack, grad_bias


def gat_rowstat(attn_row, edge_max, edge_sum, out, grad_out):
    """pack[r,h] = (attn_row, edge_max, 1/edge_sum, <grad_out[r,h], out[r,h]>) as [N,H,4]."""
    out = _cuda_f32(out, "out")
    grad_out = _cuda_f32(grad_out, "grad_out")
    n, h, f = _dims3(out, "out")
    dev = out.device
    with device_guard(dev):
        pack = torch.empty((n, h, 4), dtype=torch.float32, device=dev)
        check(lib().dgnn_gat_rowstat(n, h, f, _p(_cuda_f32(attn_row, "attn_row")), _p(_cuda_f32(edge_max, "edge_max")),
                                     _p(_cuda_f32(edge_sum, "edge_sum")), _p(out), _p(grad_out), _p(pack),
                                     _stream(dev)), "gat_rowstat")
    return pack


def gat_backward_cols(row_ptr, col_ptr, row_ind, permute, pack, edge_mask, in_feat, attn_col, grad_out,
                      negative_slope, attn_drop=0.0, row_grad=True, hot=None):
    """Column pass of the backward on an [n_rows x n_cols] block (see the header).  `hot` (from l2_hot / hot_rows
    on the CSR row pointer) marks the destination rows whose grad_out / pack rows are kept in the L2.
    Returns (grad_feat [n_cols,H,F], grad_attn_row [n_rows,H], grad_attn_col [n_cols,H]).
    With row_grad=False grad_attn_row is None (it comes from gat_rowstat_full), the per-edge array is
    skipped, row_ptr / permute may be None and an edge_mask is indexed by CSC position."""
    in_feat = _cuda_f32(in_feat, "in_feat")
    attn_col = _cuda_f32(attn_col, "attn_col")
    grad_out = _cuda_f32(grad_out, "grad_out")
    pack = _cuda_f32(pack, "pack")
    row_ind = _cuda_i32(row_ind, "row_ind")
    col_ptr, bits = _cuda_ptr(col_ptr, "col_ptr")
    if row_grad:
        permute = _cuda_i32(permute, "permute")
        row_ptr, rbits = _cuda_ptr(row_ptr, "row_ptr")
        if rbits != bits:
            row_ptr = _same_bits(bits, row_ptr, "row_ptr")
    else:
        permute = _cuda_i32(permute, "permute") if permute is not None else None
        row_ptr = None
    n_cols, h, f = _dims3(in_feat, "in_feat")
    n_rows = grad_out.shape[0]
    nnz = row_ind.numel()
    if row_grad and row_ptr.numel() - 1 != n_rows:
        raise RuntimeError("dgnn_b200: row_ptr length must be grad_out.shape[0] + 1")
    if col_ptr.numel() - 1 != n_cols:
        raise RuntimeError("dgnn_b200: col_ptr length must be in_feat.shape[0] + 1")
    if grad_out.shape != (n_rows, h, f) or pack.shape != (n_rows, h, 4):
        raise RuntimeError("dgnn_b200: grad_out / pack must have one row per CSR row")
    if guard_enabled():
        guard_check("gat_backward_cols (CSC)", col_ptr, nnz, row_ind, n_rows)
        if permute is not None:
            guard_check("gat_backward_cols (permute)", index=permute, limit=nnz)
        if row_ptr is not None:
            guard_check("gat_backward_cols (CSR)", row_ptr, nnz)
    if attn_drop > 0.0:
        edge_mask = _cuda_f32(edge_mask, "edge_mask")
    else:
        edge_mask = None
    dev = in_feat.device
    with device_guard(dev):
        grad_feat = torch.empty((n_cols, h, f), dtype=torch.float32, device=dev)
        grad_attn_row = torch.empty((n_rows, h), dtype=torch.float32, device=dev) if row_grad else None
        grad_attn_col = torch.empty((n_cols, h), dtype=torch.float32, device=dev)
        ws = _workspace(lib().dgnn_gat_backward_cols_workspace_bytes(nnz, h, f, int(row_grad)), dev)
        hot = _hot_arg(hot, n_rows)
        check(lib().dgnn_gat_backward_cols_staged(n_rows, n_cols, nnz, h, f, _p(row_ptr), _p(col_ptr), bits,
                                                  _p(row_ind), _p(permute), _p(pack), _p(edge_mask), _p(in_feat),
                                                  _p(attn_col), _p(grad_out), float(negative_slope), float(attn_drop),
                                                  _p(grad_feat), _p(grad_attn_row), _p(grad_attn_col), None, 1, 1,
                                                  None, 0, _p(hot), _p(ws), ws.numel(), _stream(dev)),
              "gat_backward_cols")
    return grad_feat, grad_attn_row, grad_attn_col


def gat_backward(negative_slope, attn_drop, row_ptr, col_ptr, row_ind, permute, edge_max, edge_sum, edge_mask,
                 in_feat, out, attn_row, attn_col, grad_out):
    """Whole backward on a square graph.  Returns (grad_feat, grad_attn_row, grad_attn_col)."""
    in_feat = _cuda_f32(in_feat, "in_feat")
    out = _cuda_f32(out, "out")
    grad_out = _cuda_f32(grad_out, "grad_out")
    attn_row = _cuda_f32(attn_row, "attn_row")
    attn_col = _cuda_f32(attn_col, "attn_col")
    edge_max = _cuda_f32(edge_max, "edge_max")
    edge_sum = _cuda_f32(edge_sum, "edge_sum")
    row_ind = _cuda_i32(row_ind, "row_ind")
    permute = _cuda_i32(permute, "permute")
    row_ptr, bits = _cuda_ptr(row_ptr, "row_ptr")
    col_ptr, cbits = _cuda_ptr(col_ptr, "col_ptr")
    if cbits != bits:
        col_ptr = _same_bits(bits, col_ptr, "col_ptr")
    n, h, f = _dims3(in_feat, "in_feat")
    nnz = row_ind.numel()
    if row_ptr.numel() - 1 != n or col_ptr.numel() - 1 != n:
        raise RuntimeError("dgnn_b200: gat_backward needs a square graph (row_ptr, col_ptr of length N+1)")
    if grad_out.shape != (n, h, f) or out.shape != (n, h, f):
        raise RuntimeError("dgnn_b200: grad_out / out must be [N,H,F]")
    if guard_enabled():
        guard_check("gat_backward (CSC)", col_ptr, nnz, row_ind, n)
        guard_check("gat_backward (CSR, permute)", row_ptr, nnz, permute, nnz)
    if attn_drop > 0.0:
        edge_mask = _cuda_f32(edge_mask, "edge_mask")
    else:
        edge_mask = None
    dev = in_feat.device
    with device_guard(dev):
        grad_feat = torch.empty((n, h, f), dtype=torch.float32, device=dev)
        grad_attn_row = torch.empty((n, h), dtype=torch.float32, device=dev)
        grad_attn_col = torch.empty((n, h), dtype=torch.float32, device=dev)
        ws = _workspace(lib().dgnn_gat_backward_workspace_bytes(n, n, nnz, h, f), dev)
        check(lib().dgnn_gat_backward(n, nnz, h, f, _p(row_ptr), _p(col_ptr), bits, _p(row_ind), _p(permute),
                                      _p(edge_max), _p(edge_sum), _p(edge_mask), _p(in_feat), _p(out),
                                      _p(attn_row), _p(attn_col), _p(grad_out), float(negative_slope),
                                      float(attn_drop), _p(grad_feat), _p(grad_attn_row), _p(grad_attn_col),
                                      _p(ws), ws.numel(), _stream(dev)), "gat_backward")
    return grad_feat, grad_attn_row, grad_attn_col


def logits_supported(h, f):
    """Shapes the fused attention-logit kernels handle (f = 4 * 2^k, h*f <= 1024)."""
    f4 = f // 4
    return f % 4 == 0 and f4 > 0 and (f4 & (f4 - 1)) == 0 and h * f <= 1024


def gat_logits_forward(feat, attn_l, attn_r, out_row=None, out_col=None, fan=None):
    """attn_row, attn_col [N,H] from feat [N,H,F] and the attention vectors [.., H, F]; written into
    out_row / out_col when given (contiguous float32 [N,H] on the same device).  `fan` (see _fan_args) also
    writes every row of feat and attn_col to its places in the send buffers that other ranks read."""
    feat = _cuda_f32(feat, "feat")
    n, h, f = _dims3(feat, "feat")
    attn_l = _cuda_f32(attn_l, "attn_l").reshape(h, f)
    attn_r = _cuda_f32(attn_r, "attn_r").reshape(h, f)
    dev = feat.device
    for t, name in ((out_row, "out_row"), (out_col, "out_col")):
        if t is not None and not (t.is_cuda and t.is_contiguous() and t.dtype == torch.float32 and t.shape == (n, h)):
            raise RuntimeError(f"dgnn_b200: {name} must be a contiguous float32 CUDA tensor [{n},{h}]")
    with device_guard(dev):
        attn_row = torch.empty((n, h), dtype=torch.float32, device=dev) if out_row is None else out_row
        attn_col = torch.empty((n, h), dtype=torch.float32, device=dev) if out_col is None else out_col
        f_ptr, f_pos, f_a, f_b = _fan_args(fan, n)
        check(lib().dgnn_gat_logits_forward_fan(n, h, f, _p(feat), _p(attn_l), _p(attn_r), _p(attn_row), _p(attn_col),
                                                _p(f_ptr), _p(f_pos), _p(f_a), _p(f_b), _stream(dev)), "gat_logits_forward")
    return attn_row, attn_col


def gat_logits_backward(feat, attn_l, attn_r, grad_row, grad_col, grad_feat):
    """grad_feat += grad_row (x) attn_l + grad_col (x) attn_r (in place); returns (grad_l, grad_r) [H,F]."""
    feat = _cuda_f32(feat, "feat")
    n, h, f = _dims3(feat, "feat")
    attn_l = _cuda_f32(attn_l, "attn_l").reshape(h, f)
    attn_r = _cuda_f32(attn_r, "attn_r").reshape(h, f)
    grad_row = _cuda_f32(grad_row, "grad_row")
    grad_col = _cuda_f32(grad_col, "grad_col")
    if not (grad_feat.is_cuda and grad_feat.is_contiguous() and grad_feat.dtype == torch.float32
            and grad_feat.shape == feat.shape):
        raise RuntimeError("dgnn_b200: grad_feat must be a contiguous float32 CUDA tensor shaped like feat")
    dev = feat.device
    with device_guard(dev):
        grad_l = torch.empty((h, f), dtype=torch.float32, device=dev)
        grad_r = torch.empty((h, f), dtype=torch.float32, device=dev)
        ws = _workspace(lib().dgnn_gat_logits_backward_workspace_bytes(h, f), dev)
        check(lib().dgnn_gat_logits_backward(n, h, f, _p(feat), _p(attn_l), _p(attn_r), _p(grad_row), _p(grad_col),
                                             _p(grad_feat), _p(grad_l), _p(grad_r), _p(ws), ws.numel(), _stream(dev)),
              "gat_logits_backward")
    return grad_l, grad_r


def uniform_fill(shape, seed, offset, device):
    """Uniform (0,1] floats from the library's Philox stream."""
    dev = torch.device(device)
    with device_guard(dev):
        out = torch.empty(shape, dtype=torch.float32, device=dev)
        check(lib().dgnn_uniform_fill(int(seed) & (2**64 - 1), int(offset), out.numel(), _p(out), _stream(dev)),
              "uniform_fill")
    return out


def uniform_fill_edges(edge_id, h, seed, offset=0):
    """[len(edge_id), h] floats: row i holds elements edge_id[i]*h .. +h of the stream of
    uniform_fill(seed, offset), i.e. the values that uniform_fill((nnz, h), seed, offset) puts in row edge_id[i]."""
    edge_id = _cuda_i32(edge_id, "edge_id")
    dev = edge_id.device
    with device_guard(dev):
        out = torch.empty((edge_id.numel(), int(h)), dtype=torch.float32, device=dev)
        check(lib().dgnn_uniform_fill_edges(int(seed) & (2**64 - 1), int(offset), edge_id.numel(), int(h), _p(edge_id),
                                            _p(out), _stream(dev)), "uniform_fill_edges")
    return out


def halo_pull(codes, src_a, dst_a, src_b=None, dst_b=None, max_ctas=0, status=None):
    """dst_a[i] = src_a[rank_i][idx_i] for every code (rank_i << dgnn_halo_rank_shift | idx_i); src_a is the list
    of the owners' buffers (tensors on this device or peer mappings), all [src_rows, ...] of one row size.
    A second tensor pair with the same row list can ride along.  Enqueued on the current stream."""
    import ctypes
    codes = _cuda_i32(codes, "codes")
    n = codes.numel()
    dev = dst_a.device

    def table(srcs, dst, name):
        rows = srcs[0].shape[0]
        row_bytes = (dst.numel() // max(n, 1)) * 4
        for t in srcs:
            if not (t.is_cuda and t.is_contiguous() and t.dtype == torch.float32 and t.shape[0] == rows
                    and t.shape[1:] == dst.shape[1:]):
                raise RuntimeError(f"dgnn_b200: halo_pull {name}: owners' buffers must be contiguous float32 [rows, ...] "
                                   "with the row shape of the destination")
        if not (dst.is_cuda and dst.is_contiguous() and dst.dtype == torch.float32 and dst.shape[0] == n):
            raise RuntimeError(f"dgnn_b200: halo_pull {name}: destination must be contiguous float32 [len(codes), ...]")
        arr = (ctypes.c_void_p * len(srcs))(*[t.data_ptr() for t in srcs])
        return arr, rows, row_bytes

    if n == 0:
        return
    arr_a, rows, rb_a = table(src_a, dst_a, "a")
    arr_b, rb_b = None, 0
    if src_b is not None:
        if len(src_b) != len(src_a):
            raise RuntimeError("dgnn_b200: halo_pull: both tensors need one buffer per rank")
        arr_b, rows_b, rb_b = table(src_b, dst_b, "b")
        if rows_b != rows:
            raise RuntimeError("dgnn_b200: halo_pull: both tensors must have the same number of rows per owner")
    with device_guard(dev):
        check(lib().dgnn_halo_pull(n, _p(codes), len(src_a), rows, arr_a, _p(dst_a), rb_a, arr_b,
                                   _p(dst_b) if dst_b is not None else None, rb_b, int(max_ctas),
                                   _p(status), _stream(dev)), "halo_pull")


# ------------------------------------------------------- dense projection
# One workspace per (device, stream), kept for the life of the process: calls on a stream are ordered, so they can
# share it, and its second word collects the status of every call (dgnn_project_sticky_status), which
# project_check() reads at a point where the caller synchronises anyway.
_PROJECT_WS = {}
_PROJECT_RETIRED = []


def _project_ws(nbytes, dev):
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), torch.cuda.current_stream(dev).cuda_stream)
    ws = _PROJECT_WS.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _PROJECT_RETIRED.append((key, ws))          # its status word stays readable
        ws = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=dev)
        ws[:8].zero_()
        _PROJECT_WS[key] = ws
    return ws


def project_check(device=None):
    """Raise if any tensor-core projection call on `device` (default: every device) gave up in one of its bounded
    waits since the last check; its result was then invalid.  Synchronises the streams that ran projections."""
    import ctypes
    bad = []
    for key, ws in list(_PROJECT_WS.items()) + list(_PROJECT_RETIRED):
        if device is not None and torch.device(device).index not in (None, key[0]):
            continue
        st = ctypes.c_int(0)
        with torch.cuda.device(key[0]):
            check(lib().dgnn_project_sticky_status(_p(ws), ctypes.c_void_p(key[1]), ctypes.byref(st), 1), "project_sticky_status")
        if st.value != 0:
            bad.append((key[0], st.value))
    if bad:
        raise RuntimeError("dgnn_b200: a projection kernel gave up in a bounded wait (device, wait id): "
                           f"{bad}; results of the projections since the last check are invalid")


def project_supported(m, n, k) -> bool:
    """Shapes the tensor-core projection handles (n % 128 == 0, k % 4 == 0, k <= 128)."""
    return bool(lib().dgnn_project_supported(int(m), int(n), int(k)))


def project_forward(x, w, w_kn=False, check_status=False, out=None):
    """out[M,N] = x[M,K] @ W in fp32 accuracy on the tcgen05 tensor cores (3 x tf32 split); w is an
    nn.Linear weight [N,K], or [K,N] with w_kn=True.  check_status=True synchronises and raises if a
    wait inside the kernel ran out.  `out` (contiguous float32 [M,N]) receives the result when given."""
    x = _cuda_f32(x, "x")
    w = _cuda_f32(w, "w")
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[0 if w_kn else 1]:
        raise RuntimeError("dgnn_b200: project_forward expects x [M,K] and w [N,K] (or [K,N] with w_kn)")
    m, k = x.shape
    n = w.shape[1 if w_kn else 0]
    dev = x.device
    if out is not None and not (out.is_cuda and out.is_contiguous() and out.dtype == torch.float32
                                and out.shape == (m, n) and out.data_ptr() % 16 == 0):
        raise RuntimeError(f"dgnn_b200: project_forward: out must be a contiguous, 16-byte aligned float32 CUDA tensor [{m},{n}]")
    with device_guard(dev):
        if out is None:
            out = torch.empty((m, n), dtype=torch.float32, device=dev)
        nbytes = lib().dgnn_project_workspace_bytes(n)
        ws = _project_ws(nbytes, dev)
        check(lib().dgnn_project_forward(m, n, k, _p(x), _p(w), int(bool(w_kn)), _p(out), _p(ws), nbytes, _stream(dev)),
              "project_forward")
        if check_status:
            import ctypes
            st = ctypes.c_int(0)
            check(lib().dgnn_project_status(_p(ws), _stream(dev), ctypes.byref(st)), "project_status")
            if st.value != 0:
                raise RuntimeError(f"dgnn_b200: project_forward gave up in wait {st.value}; the result is invalid")
    return out


def project_wgrad(x, grad_out, w_kn=False, check_status=False):
    """grad_w = x[M,K]^T @ grad_out[M,N] on the tensor cores (3 x tf32 split), returned [N,K] or, with
    w_kn=True, [K,N]."""
    x = _cuda_f32(x, "x")
    grad_out = _cuda_f32(grad_out, "grad_out")
    if x.dim() != 2 or grad_out.dim() != 2 or x.shape[0] != grad_out.shape[0]:
        raise RuntimeError("dgnn_b200: project_wgrad expects x [M,K] and grad_out [M,N]")
    m, k = x.shape
    n = grad_out.shape[1]
    dev = x.device
    with device_guard(dev):
        grad_w = torch.empty((k, n) if w_kn else (n, k), dtype=torch.float32, device=dev)
        nbytes = lib().dgnn_project_wgrad_workspace_bytes(n)
        ws = _project_ws(nbytes, dev)
        check(lib().dgnn_project_wgrad(m, n, k, _p(x), _p(grad_out), _p(grad_w), int(bool(w_kn)), _p(ws), nbytes,
                                       _stream(dev)), "project_wgrad")
        if check_status:
            import ctypes
            st = ctypes.c_int(0)
            check(lib().dgnn_project_status(_p(ws), _stream(dev), ctypes.byref(st)), "project_status")
            if st.value != 0:
                raise RuntimeError(f"dgnn_b200: project_wgrad gave up in wait {st.value}; the result is invalid")
    return grad_w


# ------------------------------------------------------- SDDMM / transpose
def mhsddmm(row_ptr, col_ind, a, b):
    """out[e,h] = <a[row_e,h,:], b[col_e,h,:]>, [E,H]."""
    a = _cuda_f32(a, "grad")
    b = _cuda_f32(b, "feature")
    col_ind = _cuda_i32(col_ind, "colind")
    row_ptr, bits = _cuda_ptr(row_ptr, "rowptr")
    _, h, f = _dims3(b, "feature")
    n_rows = row_ptr.numel() - 1
    if a.shape[0] != n_rows or a.shape[1:] != b.shape[1:]:
        raise RuntimeError("dgnn_b200: mhsddmm operands must be [V,H,F] with V = len(rowptr) - 1 rows in `grad`")
    nnz = col_ind.numel()
    dev = b.device
    if guard_enabled():
        guard_check("mhsddmm", row_ptr, nnz, col_ind, b.shape[0])
    with device_guard(dev):
        out = torch.empty((nnz, h), dtype=torch.float32, device=dev)
        ws = _workspace(lib().dgnn_mhsddmm_workspace_bytes(), dev)
        check(lib().dgnn_mhsddmm(n_rows, nnz, h, f, _p(row_ptr), bits, _p(col_ind), _p(a), _p(b), _p(out),
                                 _p(ws), ws.numel(), _stream(dev)), "mhsddmm")
    return out


def coo_sddmm(row_ind, col_ind, d1, d2):
    """out[e] = <d1[row_ind[e]], d2[col_ind[e]]> for a COO edge list in any order."""
    row_ind = _cuda_i32(row_ind, "rowind")
    col_ind = _cuda_i32(col_ind, "colind")
    d1 = _cuda_f32(d1, "D1")
    d2 = _cuda_f32(d2, "D2")
    if d1.dim() != 2 or d2.dim() != 2 or d1.shape[1] != d2.shape[1] or row_ind.numel() != col_ind.numel():
        raise RuntimeError("dgnn_b200: coo_sddmm needs D1 [m,k], D2 [n,k] and two index arrays of equal length")
    nnz, k = row_ind.numel(), d1.shape[1]
    dev = d1.device
    if guard_enabled():
        guard_check("coo_sddmm (rows)", index=row_ind, limit=d1.shape[0])
        guard_check("coo_sddmm (columns)", index=col_ind, limit=d2.shape[0])
    with device_guard(dev):
        out = torch.empty(nnz, dtype=torch.float32, device=dev)
        check(lib().dgnn_coo_sddmm(nnz, k, _p(row_ind), _p(col_ind), _p(d1), _p(d2), _p(out), _stream(dev)), "coo_sddmm")
    return out


def mhtranspose(permute, attention):
    """out[i,:] = attention[permute[i],:]."""
    permute = _cuda_i32(permute, "permute")
    attention = _cuda_f32(attention, "attention")
    if attention.dim() != 2:
        raise RuntimeError("dgnn_b200: mhtranspose input must be [E,H]")
    nnz, h = permute.numel(), attention.shape[1]
    dev = attention.device
    if guard_enabled():
        guard_check("mhtranspose", index=permute, limit=attention.shape[0])
    with device_guard(dev):
        out = torch.empty((nnz, h), dtype=torch.float32, device=dev)
        check(lib().dgnn_mhtranspose(nnz, h, _p(permute), _p(attention), _p(out), _stream(dev)), "mhtranspose")
    return out


# --------------------------------------------------------------------- GMM
def gmm_forward(row_ptr, col_ind, node_feat, pseudo, mu, inv_sigma):
    node_feat = _cuda_f32(node_feat, "node_feat")
    pseudo = _cuda_f32(pseudo, "pseudo")
    mu = _cuda_f32(mu, "mu")
    inv_sigma = _cuda_f32(inv_sigma, "sigma")
    col_ind = _cuda_i32(col_ind, "colind")
    row_ptr, bits = _cuda_ptr(row_ptr, "rowptr")
    _, k, f = _dims3(node_feat, "node_feat")
    n_rows, nnz = row_ptr.numel() - 1, col_ind.numel()
    dim = mu.shape[1]
    if mu.shape != (k, dim) or inv_sigma.shape != (k, dim) or pseudo.shape != (nnz, dim):
        raise RuntimeError("dgnn_b200: gmmconv needs mu, sigma [K,dim] and pseudo [E,dim]")
    if guard_enabled():
        guard_check("gmm_forward", row_ptr, nnz, col_ind, node_feat.shape[0])
    dev = node_feat.device
    with device_guard(dev):
        out = torch.empty((n_rows, k, f), dtype=torch.float32, device=dev)
        ws = _workspace(lib().dgnn_gmm_forward_workspace_bytes(n_rows, nnz, k, f), dev)
        check(lib().dgnn_gmm_forward(n_rows, nnz, k, dim, f, _p(row_ptr), bits, _p(col_ind), _p(node_feat),
                                     _p(pseudo), _p(mu), _p(inv_sigma), _p(out), _p(ws), ws.numel(),
                                     _stream(dev)), "gmm_forward")
    return out


def gaussian(pseudo, mu, inv_sigma):
    pseudo = _cuda_f32(pseudo, "pseudo")
    mu = _cuda_f32(mu, "mu")
    inv_sigma = _cuda_f32(inv_sigma, "sigma")
    nnz, dim = pseudo.shape
    k = mu.shape[0]
    dev = pseudo.device
    with device_guard(dev):
        out = torch.empty((nnz, k), dtype=torch.float32, device=dev)
        check(lib().dgnn_gaussian(nnz, k, dim, _p(pseudo), _p(mu), _p(inv_sigma), _p(out), _stream(dev)), "gaussian")
    return out


def gaussian_bp(pseudo, mu, inv_sigma, grad_gauss):
    pseudo = _cuda_f32(pseudo, "pseudo")
    mu = _cuda_f32(mu, "mu")
    inv_sigma = _cuda_f32(inv_sigma, "sigma")
    grad_gauss = _cuda_f32(grad_gauss, "grad_gauss")
    nnz, dim = pseudo.shape
    k = mu.shape[0]
    if grad_gauss.shape != (nnz, k):
        raise RuntimeError("dgnn_b200: GaussianBp needs grad [E,K]")
    dev = pseudo.device
    with device_guard(dev):
        pseudo_out = torch.empty((nnz, dim), dtype=torch.float32, device=dev)
        mu_out = torch.empty((k, dim), dtype=torch.float32, device=dev)
        sigma_out = torch.empty((k, dim), dtype=torch.float32, device=dev)
        ws = _workspace(lib().dgnn_gaussian_bp_workspace_bytes(nnz, k, dim), dev)
        check(lib().dgnn_gaussian_bp(nnz, k, dim, _p(pseudo), _p(mu), _p(inv_sigma), _p(grad_gauss), _p(pseudo_out),
                                     _p(mu_out), _p(sigma_out), _p(ws), ws.numel(), _stream(dev)), "gaussian_bp")
    return pseudo_out, mu_out, sigma_out


# ---------------------------------------------------------------- EdgeConv
def edgeconv_forward(k, src_ind, h_src, h_dst):
    """Returns (out [M,F] fp32, max_idx [M,F] int32)."""
    h_src = _cuda_f32(h_src, "h_src")
    h_dst = _cuda_f32(h_dst, "h_dst")
    src_ind = _cuda_i32(src_ind, "src_ind")
    m, f = h_src.shape
    if h_dst.shape != (m, f) or src_ind.numel() != m * int(k):
        raise RuntimeError("dgnn_b200: edgeconv needs h_src, h_dst [M,F] and src_ind [M*k]")
    if guard_enabled():
        guard_check("edgeconv_forward", index=src_ind, limit=m)
    dev = h_src.device
    with device_guard(dev):
        out = torch.empty((m, f), dtype=torch.float32, device=dev)
        max_idx = torch.empty((m, f), dtype=torch.int32, device=dev)
        check(lib().dgnn_edgeconv_forward(m, f, int(k), _p(src_ind), _p(h_src), _p(h_dst), _p(out), _p(max_idx),
                                          _stream(dev)), "edgeconv_forward")
    return out, max_idx


def edgeconv_backward(grad_out, max_idx):
    grad_out = _cuda_f32(grad_out, "grad_out")
    max_idx = _cuda_i32(max_idx, "max_idx")
    m, f = grad_out.shape
    dev = grad_out.device
    if guard_enabled():
        guard_check("edgeconv_backward", index=max_idx.reshape(-1), limit=m)
    with device_guard(dev):
        grad_src = torch.empty((m, f), dtype=torch.float32, device=dev)
        check(lib().dgnn_edgeconv_backward(m, f, _p(max_idx), _p(grad_out), _p(grad_src), _stream(dev)),
              "edgeconv_backward")
    return grad_src


def edgeconv_backward_ordered(k, src_ind, grad_out, max_idx):
    """edgeconv_backward with a fixed summation order (bit-reproducible): the in-edges of every source point come
    from the CSC form of the regular neighbour graph (k entries per destination), built here by csr2csc."""
    grad_out = _cuda_f32(grad_out, "grad_out")
    max_idx = _cuda_i32(max_idx, "max_idx")
    src_ind = _cuda_i32(src_ind, "src_ind")
    m, f = grad_out.shape
    if src_ind.numel() != m * int(k):
        raise RuntimeError("dgnn_b200: src_ind must hold k entries per destination point")
    dev = grad_out.device
    with device_guard(dev):
        row_ptr = torch.arange(0, m * int(k) + 1, max(int(k), 1), dtype=torch.int32, device=dev)[: m + 1] if k > 0 \
            else torch.zeros(m + 1, dtype=torch.int32, device=dev)
        col_ptr, row_ind, _ = csr2csc(row_ptr, src_ind, n_cols=m)
        grad_src = torch.empty((m, f), dtype=torch.float32, device=dev)
        check(lib().dgnn_edgeconv_backward_ordered(m, f, _p(col_ptr), _p(row_ind), _p(max_idx), _p(grad_out),
                                                   _p(grad_src), _stream(dev)), "edgeconv_backward_ordered")
    return grad_src


# -------------------------------------------------------------- conversion
def csr2csc(row_ptr, col_ind, n_cols=None):
    """Returns (col_ptr [same width as row_ptr], row_ind int32, permute int32)."""
    col_ind = _cuda_i32(col_ind, "colind")
    row_ptr, bits = _cuda_ptr(row_ptr, "rowptr")
    n_rows, nnz = row_ptr.numel() - 1, col_ind.numel()
    n_cols = n_rows if n_cols is None else int(n_cols)
    dev = col_ind.device
    if guard_enabled():
        guard_check("csr2csc", row_ptr, nnz, col_ind, n_cols)
    with device_guard(dev):
        col_ptr = torch.empty(n_cols + 1, dtype=row_ptr.dtype, device=dev)
        row_ind = torch.empty(nnz, dtype=torch.int32, device=dev)
        permute = torch.empty(nnz, dtype=torch.int32, device=dev)
        ws = _workspace(lib().dgnn_csr2csc_workspace_bytes(n_rows, n_cols, nnz), dev)
        check(lib().dgnn_csr2csc(n_rows, n_cols, nnz, _p(row_ptr), bits, _p(col_ind), _p(col_ptr), _p(row_ind),
                                 _p(permute), _p(ws), ws.numel(), _stream(dev)), "csr2csc")
    return col_ptr, row_ind, permute


def coo2csr(row_ind, m, dtype=torch.int32):
    row_ind = _cuda_i32(row_ind, "cooRowInd")
    dev = row_ind.device
    bits = 32 if dtype == torch.int32 else 64
    with device_guard(dev):
        row_ptr = torch.empty(int(m) + 1, dtype=dtype, device=dev)
        check(lib().dgnn_coo2csr(row_ind.numel(), int(m), _p(row_ind), _p(row_ptr), bits, _stream(dev)), "coo2csr")
    return row_ptr


def coo_sort(dst, src, n_nodes):
    """Edge list (int32 ids, any order, duplicates kept) sorted by (dst, src): returns (dst_sorted, src_sorted)."""
    dst = _cuda_i32(dst, "dst")
    src = _cuda_i32(src, "src")
    if dst.numel() != src.numel():
        raise RuntimeError("dgnn_b200: coo_sort needs one source per destination")
    nnz = dst.numel()
    dev = dst.device
    if guard_enabled():
        guard_check("coo_sort (destinations)", index=dst, limit=n_nodes)
        guard_check("coo_sort (sources)", index=src, limit=n_nodes)
    with device_guard(dev):
        d_out = torch.empty(nnz, dtype=torch.int32, device=dev)
        s_out = torch.empty(nnz, dtype=torch.int32, device=dev)
        ws = _workspace(lib().dgnn_coo_sort_workspace_bytes(nnz, int(n_nodes)), dev)
        check(lib().dgnn_coo_sort(nnz, int(n_nodes), _p(dst), _p(src), _p(d_out), _p(s_out), _p(ws), ws.numel(),
                                  _stream(dev)), "coo_sort")
    return d_out, s_out


def knn_graph(points, k):
    """points [B,P,D] -> src_ind [B*P*k] int32 with global ids (cloud*P + neighbour), the point itself first."""
    points = _cuda_f32(points, "points")
    if points.dim() != 3:
        raise RuntimeError("dgnn_b200: knn_graph needs points [B,P,D]")
    b, p, d = points.shape
    dev = points.device
    with device_guard(dev):
        out = torch.empty(b * p * int(k), dtype=torch.int32, device=dev)
        check(lib().dgnn_knn_graph(b, p, d, int(k), _p(points), _p(out), _stream(dev)), "knn_graph")
    return out


# ------------------------------------------------ staged (block-by-block) GAT
def gat_forward_state(n_rows, h, f, device):
    """Per-row softmax state carried between the calls of a staged forward."""
    nbytes = lib().dgnn_gat_forward_state_bytes(int(n_rows), int(h), int(f))
    return torch.empty(max(nbytes // 4, 4), dtype=torch.float32, device=device)


def gat_backward_state(n_cols, h, f, device):
    nbytes = lib().dgnn_gat_backward_state_bytes(int(n_cols), int(h), int(f))
    return torch.empty(max(nbytes // 4, 4), dtype=torch.float32, device=device)


def gat_forward_staged(attn_row, attn_col_blk, row_ptr, col_ind, negative_slope, feat_blk, state, first, last, bias=None,
                       attn_drop=0.0, edge_mask=None, neg=False, save_stats=True, stage_mask=None, stage=0, outs=None,
                       hot=None):
    """One stage of the forward over the edges whose source lies in one column block.
    Returns (out, edge_max, edge_sum[, out_neg, a_neg]) from the last stage, None before.  `bias` [H*F] is
    added to the output when a row is written out; `edge_mask` [nnz,H] (with attn_drop > 0) follows the
    order of this stage's col_ind; neg=True must be passed to every stage of a sweep that wants the
    negative-side outputs (the carried state holds their accumulators).
    stage_mask [n_rows] uint8 (bit p = the row has edges in stage p) makes the stages sparse: a row is only
    touched in its own stages and written out in its last one, so the outputs must exist from the first stage
    on: the tuple is returned by every stage and has to be passed back in as `outs`."""
    attn_row = _cuda_f32(attn_row, "attn_row")
    attn_col_blk = _cuda_f32(attn_col_blk, "attn_col")
    feat_blk = _cuda_f32(feat_blk, "in_feat")
    col_ind = _cuda_i32(col_ind, "col_ind")
    row_ptr, bits = _cuda_ptr(row_ptr, "row_ptr")
    _, h, f = _dims3(feat_blk, "in_feat")
    n_rows, nnz = row_ptr.numel() - 1, col_ind.numel()
    if guard_enabled():
        guard_check("gat_forward_staged", row_ptr, nnz, col_ind, min(feat_blk.shape[0], attn_col_blk.shape[0]))
    if attn_drop > 0.0:
        edge_mask = _cuda_f32(edge_mask, "edge_mask")
        if edge_mask.shape != (nnz, h):
            raise RuntimeError(f"dgnn_b200: edge_mask must be [{nnz},{h}]")
    else:
        edge_mask = None
    if stage_mask is not None and not (stage_mask.is_cuda and stage_mask.dtype == torch.uint8 and stage_mask.numel() == n_rows
                                       and stage_mask.is_contiguous()):
        raise RuntimeError("dgnn_b200: stage_mask must be a contiguous uint8 CUDA tensor with one entry per row")
    dev = feat_blk.device
    with device_guard(dev):
        out = emax = esum = out_neg = a_neg = None
        if outs is not None:
            out, emax, esum, out_neg, a_neg = (tuple(outs) + (None, None))[:5]
        elif last or stage_mask is not None:
            out = torch.empty((n_rows, h, f), dtype=torch.float32, device=dev)
            if save_stats:
                emax = torch.empty((n_rows, h), dtype=torch.float32, device=dev)
                esum = torch.empty((n_rows, h), dtype=torch.float32, device=dev)
            if neg:
                out_neg = torch.empty((n_rows, h, f), dtype=torch.float32, device=dev)
                a_neg = torch.empty((n_rows, h), dtype=torch.float32, device=dev)
        if neg and out_neg is None:   # every stage gets the pointers: they select the kernel variant whose state carries the accumulators
            out_neg = torch.empty((1, h, f), dtype=torch.float32, device=dev)
            a_neg = torch.empty((1, h), dtype=torch.float32, device=dev)
        ws = _workspace(lib().dgnn_gat_forward_workspace_bytes(n_rows, nnz, h, f), dev)
        if bias is not None:
            bias = _cuda_f32(bias, "bias").reshape(h * f)
        check(lib().dgnn_gat_forward_staged(n_rows, nnz, h, f, _p(row_ptr), bits, _p(col_ind), _p(attn_row),
                                            _p(attn_col_blk), _p(feat_blk), float(negative_slope), float(attn_drop),
                                            _p(edge_mask), _p(bias) if bias is not None else None,
                                            _p(out), _p(emax), _p(esum), _p(out_neg), _p(a_neg), _p(state),
                                            int(bool(first)), int(bool(last)), _p(stage_mask), int(stage),
                                            _p(_hot_arg(hot, feat_blk.shape[0])),
                                            _p(ws), ws.numel(), _stream(dev)), "gat_forward_staged")
    if not last and stage_mask is None:
        return None
    return (out, emax, esum, out_neg, a_neg) if neg else (out, emax, esum)


def gat_backward_cols_staged(row_ptr, col_ptr, row_ind, permute, pack_blk, in_feat, attn_col, grad_blk,
                             negative_slope, state, first, last, attn_drop=0.0, edge_mask=None, row_grad=True,
                             stage_mask=None, stage=0, outs=None, hot=None):
    """One stage of the backward column pass over the edges whose destination lies in one
    row block.  Returns (grad_attn_row of the block's rows or None, grad_feat or None, grad_attn_col or None).
    With row_grad=False (grad_attn_row comes from gat_rowstat_full) row_ptr and permute may be None and an
    `edge_mask` [nnz,H] follows the order of this stage's row_ind.  stage_mask [n_cols] uint8 / stage / outs =
    (grad_feat, grad_attn_col): sparse stages as in gat_forward_staged (every stage returns the outputs)."""
    in_feat = _cuda_f32(in_feat, "in_feat")
    attn_col = _cuda_f32(attn_col, "attn_col")
    grad_blk = _cuda_f32(grad_blk, "grad_out")
    pack_blk = _cuda_f32(pack_blk, "pack")
    row_ind = _cuda_i32(row_ind, "row_ind")
    col_ptr, bits = _cuda_ptr(col_ptr, "col_ptr")
    if row_grad:
        permute = _cuda_i32(permute, "permute")
        row_ptr, rbits = _cuda_ptr(row_ptr, "row_ptr")
        if rbits != bits:
            row_ptr = _same_bits(bits, row_ptr, "row_ptr")
    else:
        permute = _cuda_i32(permute, "permute") if permute is not None else None
        row_ptr = None
    n_cols, h, f = _dims3(in_feat, "in_feat")
    n_rows, nnz = grad_blk.shape[0], row_ind.numel()
    if (grad_blk.shape != (n_rows, h, f) or pack_blk.shape != (n_rows, h, 4) or col_ptr.numel() - 1 != n_cols
            or (row_grad and row_ptr.numel() - 1 != n_rows)):
        raise RuntimeError("dgnn_b200: staged backward: block shapes do not match the sub-matrix")
    if guard_enabled():
        guard_check("gat_backward_cols_staged (CSC)", col_ptr, nnz, row_ind, n_rows)
        if permute is not None:
            guard_check("gat_backward_cols_staged (permute)", index=permute, limit=nnz)
    if attn_drop > 0.0:
        edge_mask = _cuda_f32(edge_mask, "edge_mask")
        if edge_mask.shape != (nnz, h):
            raise RuntimeError(f"dgnn_b200: edge_mask must be [{nnz},{h}]")
    else:
        edge_mask = None
    dev = in_feat.device
    with device_guard(dev):
        grad_feat = grad_col = None
        if outs is not None:
            grad_feat, grad_col = outs
        elif last or stage_mask is not None:
            grad_feat = torch.empty((n_cols, h, f), dtype=torch.float32, device=dev)
            grad_col = torch.empty((n_cols, h), dtype=torch.float32, device=dev)
        grad_row = torch.empty((n_rows, h), dtype=torch.float32, device=dev) if row_grad else None
        ws = _workspace(lib().dgnn_gat_backward_cols_workspace_bytes(nnz, h, f, int(row_grad)), dev)
        check(lib().dgnn_gat_backward_cols_staged(n_rows, n_cols, nnz, h, f, _p(row_ptr), _p(col_ptr), bits,
                                                  _p(row_ind), _p(permute), _p(pack_blk), _p(edge_mask), _p(in_feat),
                                                  _p(attn_col), _p(grad_blk), float(negative_slope), float(attn_drop),
                                                  _p(grad_feat), _p(grad_row), _p(grad_col), _p(state),
                                                  int(bool(first)), int(bool(last)), _p(stage_mask), int(stage),
                                                  _p(_hot_arg(hot, n_rows)), _p(ws), ws.numel(), _stream(dev)),
              "gat_backward_cols_staged")
    return grad_row, grad_feat, grad_col
