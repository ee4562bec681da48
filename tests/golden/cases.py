"""Seeded inputs on which the reference's own CUDA kernels are run (on a GPU box)
to produce golden vectors.  Sizes and shapes are restricted to what those
kernels handle without reading or writing out of bounds (checked by reading
them): feature widths that are multiples of 32 for the GAT and GMM kernels
(fused_gatconv_kernel.cu:87,111 and fused_gmmconv_kernel.cu:49 index a full
32-lane slab), a single Gaussian kernel for fuseGmm (its 32-float shared array
is shared by all kernels' warps, fused_gmmconv_kernel.cu:45), an edge count that
is a multiple of 32 for `gaussian` (no bounds guard, :13-21), and pseudo /
node_feat buffers padded past their logical end (fuseGmm reads up to 31 edges
past the row end, :40)."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from dgnn_b200 import synth  # noqa: E402


def graph(seed, n=300, avg=6, long_rows=((3, 70), (200, 33))):
    return synth.random_graph(n, avg, seed, long_rows=list(long_rows))


def gat_case(seed, h, f):
    rp, ci = graph(seed)
    n = rp.numel() - 1
    g = torch.Generator().manual_seed(100 + seed)
    return dict(row_ptr=rp, col_ind=ci, attn_row=torch.randn(n, h, generator=g), attn_col=torch.randn(n, h, generator=g),
                in_feat=torch.randn(n, h, f, generator=g), grad_out=torch.randn(n, h, f, generator=g), slope=0.2)


def sddmm_case(seed, h, f):
    rp, ci = graph(seed)
    n = rp.numel() - 1
    g = torch.Generator().manual_seed(200 + seed)
    return dict(row_ptr=rp, col_ind=ci, a=torch.randn(n, h, f, generator=g), b=torch.randn(n, h, f, generator=g))


def transpose_case(seed, h, nnz=4099):
    g = torch.Generator().manual_seed(300 + seed)
    return dict(permute=torch.randperm(nnz, generator=g).int(), x=torch.randn(nnz, h, generator=g))


def gmm_case(seed, f=32, dim=2):
    rp, ci = graph(seed)
    n, nnz = rp.numel() - 1, ci.numel()
    g = torch.Generator().manual_seed(400 + seed)
    return dict(row_ptr=rp, col_ind=ci, node_feat=torch.randn(n, 1, f, generator=g),
                pseudo=torch.rand(nnz, dim, generator=g), mu=torch.rand(1, dim, generator=g),
                inv_sigma=torch.rand(1, dim, generator=g) + 0.5)


def gaussian_case(seed, k=3, dim=2, nnz=2048):
    g = torch.Generator().manual_seed(500 + seed)
    return dict(pseudo=torch.rand(nnz, dim, generator=g), mu=torch.rand(k, dim, generator=g),
                inv_sigma=torch.rand(k, dim, generator=g) + 0.5)


def edgeconv_case(seed, m=256, k=20, f=64):
    g = torch.Generator().manual_seed(600 + seed)
    return dict(k=k, src_ind=torch.randint(0, m, (m * k,), generator=g, dtype=torch.int32),
                h_src=torch.randn(m, f, generator=g), h_dst=torch.randn(m, f, generator=g))


CASES = {
    "gat_h4_f32": lambda: gat_case(1, 4, 32),
    "gat_h1_f64": lambda: gat_case(2, 1, 64),
    "gat_h8_f32": lambda: gat_case(3, 8, 32),
    "sddmm_h3_f16": lambda: sddmm_case(1, 3, 16),
    "sddmm_h4_f64": lambda: sddmm_case(2, 4, 64),
    "transpose_h2": lambda: transpose_case(1, 2),
    "transpose_h4": lambda: transpose_case(2, 4),
    "gmm_k1_f32": lambda: gmm_case(1),
    "gaussian_k3": lambda: gaussian_case(1),
    "edgeconv_k20_f64": lambda: edgeconv_case(1),
    "convert": lambda: dict(zip(("row_ptr", "col_ind"), graph(7))),
}


def padded(t, extra_rows=64):
    """Copy `t` into the head of a larger zero buffer and return the logical view."""
    big = torch.zeros((t.shape[0] + extra_rows,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    big[: t.shape[0]] = t
    return big[: t.shape[0]]


def run_reference(name, case, ref, dev):
    """Run the reference extension modules `ref` (dict name -> module) on one case; returns a dict of outputs."""
    from tests_csc import scipy_csc_int32
    d = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    if name.startswith("gat"):
        cp, ri, pm = [t.to(dev) for t in scipy_csc_int32(case["row_ptr"], case["col_ind"])]
        out, emax, esum, mask = ref["fused_gatconv"].gat_forward(d["attn_row"], d["attn_col"], d["row_ptr"], d["col_ind"],
                                                                d["slope"], d["in_feat"], 0.0)
        gf, gr, gc = ref["fused_gatconv"].gat_backward(d["slope"], 0.0, d["row_ptr"], d["col_ind"], cp, ri, pm, emax, esum,
                                                       mask, d["in_feat"], d["attn_row"], d["attn_col"], d["grad_out"])
        inf = ref["fused_gatconv"].gat_inference(d["attn_row"], d["attn_col"], d["row_ptr"], d["col_ind"], d["slope"], d["in_feat"])
        return dict(out=out, edge_max=emax, edge_sum=esum, grad_feat=gf, grad_attn_row=gr, grad_attn_col=gc, out_inference=inf)
    if name.startswith("sddmm"):
        return dict(out=ref["mhsddmm"].mhsddmm(d["row_ptr"], d["col_ind"], d["a"], d["b"]))
    if name.startswith("transpose"):
        return dict(out=ref["mhtranspose"].mhtranspose(d["permute"], d["x"]))
    if name.startswith("gmm"):
        return dict(out=ref["fused_gmmconv"].gmmconv(d["row_ptr"], d["col_ind"], padded(d["node_feat"]), padded(d["pseudo"]),
                                                     d["mu"], d["inv_sigma"]))
    if name.startswith("gaussian"):
        return dict(out=ref["fused_gmmconv"].Gaussian(d["pseudo"], d["mu"], d["inv_sigma"]))
    if name.startswith("edgeconv"):
        out, idx = ref["fused_edgeconv"].edgeconv_forward(d["k"], d["src_ind"], d["h_src"], d["h_dst"])
        return dict(out=out, max_idx=idx)
    if name == "convert":
        nnz = d["col_ind"].numel()
        vals = torch.arange(nnz, dtype=torch.float32, device=dev)
        colptr, rowind, cscval = ref["format_conversion"].csr2csc(d["row_ptr"], d["col_ind"], vals)
        rows = torch.repeat_interleave(torch.arange(d["row_ptr"].numel() - 1, device=dev),
                                       (d["row_ptr"][1:] - d["row_ptr"][:-1]).long()).int()
        rowptr = ref["format_conversion"].coo2csr(rows, d["row_ptr"].numel() - 1)
        return dict(col_ptr=colptr, row_ind=rowind, csc_val=cscval, coo2csr=rowptr)
    raise KeyError(name)
