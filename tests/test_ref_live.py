"""On a GPU box: the reference's own kernels (oracle/_ref, built for sm_100a)
against the oracle and against the new kernels on the golden cases, the stored
fixtures against a fresh run, and a side-by-side timing at a medium size."""
import json
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "oracle"))

import build_ref  # noqa: E402
import cases  # noqa: E402
from dgnn_b200 import kernels, synth  # noqa: E402
from helpers import scipy_csc  # noqa: E402
from test_oracle_golden import compare, oracle_outputs  # noqa: E402

pytestmark = pytest.mark.gpu

# timing records of the side-by-side tests are printed; they are also written as JSON when this names a folder
RESULTS_DIR = os.environ.get("DGNN_RESULTS_DIR", "")


def _record(file_name, rec, indent=None):
    if not RESULTS_DIR:
        return
    os.makedirs(RESULTS_DIR, exist_ok=True)
    with open(os.path.join(RESULTS_DIR, file_name), "w") as fh:
        json.dump(rec, fh, indent=indent)


@pytest.fixture(scope="module")
def ref(cuda):
    mods = build_ref.load()
    if mods is None:
        pytest.skip("oracle/_ref not built (python oracle/build_ref.py)")
    return mods


def ours_outputs(name, case, dev):
    d = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    if name.startswith("gat"):
        cp, ri, pm = [t.int().to(dev) for t in scipy_csc(case["row_ptr"], case["col_ind"])]
        out, emax, esum = kernels.gat_forward(d["attn_row"], d["attn_col"], d["row_ptr"], d["col_ind"], d["slope"], d["in_feat"])
        gf, gr, gc = kernels.gat_backward(d["slope"], 0.0, d["row_ptr"], cp, ri, pm, emax, esum, None, d["in_feat"], out,
                                          d["attn_row"], d["attn_col"], d["grad_out"])
        inf = kernels.gat_forward(d["attn_row"], d["attn_col"], d["row_ptr"], d["col_ind"], d["slope"], d["in_feat"],
                                  save_stats=False)[0]
        return dict(out=out, edge_max=emax, edge_sum=esum, grad_feat=gf, grad_attn_row=gr, grad_attn_col=gc, out_inference=inf)
    if name.startswith("sddmm"):
        return dict(out=kernels.mhsddmm(d["row_ptr"], d["col_ind"], d["a"], d["b"]))
    if name.startswith("transpose"):
        return dict(out=kernels.mhtranspose(d["permute"], d["x"]))
    if name.startswith("gmm"):
        return dict(out=kernels.gmm_forward(d["row_ptr"], d["col_ind"], d["node_feat"], d["pseudo"], d["mu"], d["inv_sigma"]))
    if name.startswith("gaussian"):
        return dict(out=kernels.gaussian(d["pseudo"], d["mu"], d["inv_sigma"]))
    if name.startswith("edgeconv"):
        out, idx = kernels.edgeconv_forward(d["k"], d["src_ind"], d["h_src"], d["h_dst"])
        return dict(out=out, max_idx=idx)
    if name == "convert":
        cp, ri, pm = kernels.csr2csc(d["row_ptr"], d["col_ind"])
        rows = torch.repeat_interleave(torch.arange(d["row_ptr"].numel() - 1, device=dev),
                                       (d["row_ptr"][1:] - d["row_ptr"][:-1]).long()).int()
        return dict(col_ptr=cp, row_ind=ri, csc_val=pm, coo2csr=kernels.coo2csr(rows, d["row_ptr"].numel() - 1))
    raise KeyError(name)


@pytest.mark.parametrize("name", list(cases.CASES))
def test_reference_vs_oracle_vs_ours(cuda, ref, name):
    case = cases.CASES[name]()
    r = {k: v.detach().cpu() for k, v in cases.run_reference(name, case, ref, cuda).items()}
    torch.cuda.synchronize()
    compare(name, oracle_outputs(name, case), r, "oracle")
    compare(name, {k: v.detach().cpu() for k, v in ours_outputs(name, case, cuda).items()}, r, "dgnn_b200")
    fixture = os.path.join(HERE, "golden", name + ".npz")
    if os.path.exists(fixture):   # the committed vectors are what the reference still produces
        z = np.load(fixture)
        stored = {k[4:]: torch.from_numpy(z[k]) for k in z.files if k.startswith("ref_")}
        compare(name, r, stored, "fresh reference run")


def _time(fn, iters=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def test_side_by_side_timing(cuda, ref):
    """Fused GAT forward+backward, reference kernels vs these kernels, on an R-MAT graph
    (300 k nodes, 12 M edges, 8 heads x 32) -- results agree and the times are recorded."""
    n, e, h, f = 300_000, 12_000_000, 8, 32
    rp, ci = synth.rmat_graph(n, e, seed=4, device=cuda, ptr_dtype=torch.int32)
    cp, ri, pm = kernels.csr2csc(rp, ci)
    g = torch.Generator(device=cuda).manual_seed(0)
    ar, ac = torch.randn(n, h, device=cuda, generator=g), torch.randn(n, h, device=cuda, generator=g)
    x, go = torch.randn(n, h, f, device=cuda, generator=g), torch.randn(n, h, f, device=cuda, generator=g)
    fg = ref["fused_gatconv"]

    def ref_step():
        out, emax, esum, mask = fg.gat_forward(ar, ac, rp, ci, 0.2, x, 0.0)
        return (out,) + tuple(fg.gat_backward(0.2, 0.0, rp, ci, cp, ri, pm, emax, esum, mask, x, ar, ac, go))

    def our_step():
        out, emax, esum = kernels.gat_forward(ar, ac, rp, ci, 0.2, x)
        return (out,) + kernels.gat_backward(0.2, 0.0, rp, cp, ri, pm, emax, esum, None, x, out, ar, ac, go)

    a, b = ref_step(), our_step()
    for u, v, name in zip(a, b, ("out", "grad_feat", "grad_attn_row", "grad_attn_col")):
        err = (u - v).abs()
        tol = 1e-5 + 1e-4 * u.abs()
        frac_bad = float((err > 4 * tol).float().mean())
        assert frac_bad < 1e-5, f"{name}: {frac_bad:.2e} of the elements differ from the reference kernels"
    t_ref, t_our = _time(ref_step), _time(our_step)
    rec = dict(workload="rmat n=300k e=12M h=8 f=32 fused GAT fwd+bwd", ref_ms=t_ref, ours_ms=t_our, speedup=t_ref / t_our)
    print("SIDE_BY_SIDE", json.dumps(rec))
    _record("side_by_side.json", rec)
    assert t_our < t_ref * 1.5


def test_side_by_side_full_size(cuda, ref):
    """The benchmark's own graph (R-MAT, 2.4 M nodes, 120 M edges, 8 heads x 32) through the reference's kernels,
    once.  Every index expression of fused_forward_kernel, mhspmm_backward_kernel, mhsddmm and
    fused_backward_kernel (fused_gatconv_kernel.cu:24-118, 712-763, 814-890, 892-968) is an int: the largest ones,
    edge * heads = 9.6e8 and node * heads * features = 6.1e8, stay below 2^31, and 120 M is a multiple of 16, so
    mhsddmm has no tail blocks.  The reference needs int32 row pointers; results are compared on the way."""
    n, e, h, f = 2_400_000, 120_000_000, 8, 32
    free, _ = torch.cuda.mem_get_info(cuda)
    if free < 60e9:
        pytest.skip("needs about 60 GB of free device memory")
    rp, ci = synth.rmat_graph(n, e, seed=4, device=cuda, ptr_dtype=torch.int32)
    cp, ri, pm = kernels.csr2csc(rp, ci)
    g = torch.Generator(device=cuda).manual_seed(0)
    ar, ac = torch.randn(n, h, device=cuda, generator=g), torch.randn(n, h, device=cuda, generator=g)
    x, go = torch.randn(n, h, f, device=cuda, generator=g), torch.randn(n, h, f, device=cuda, generator=g)
    fg = ref["fused_gatconv"]

    def ref_step():
        out, emax, esum, mask = fg.gat_forward(ar, ac, rp, ci, 0.2, x, 0.0)
        return (out,) + tuple(fg.gat_backward(0.2, 0.0, rp, ci, cp, ri, pm, emax, esum, mask, x, ar, ac, go))

    def our_step():
        out, emax, esum, out_neg, a_neg = kernels.gat_forward(ar, ac, rp, ci, 0.2, x, neg=True)
        pack, gr, _ = kernels.gat_rowstat_full(ar, emax, esum, out, go, 0.2, out_neg=out_neg, a_neg=a_neg)
        gf, _, gc = kernels.gat_backward_cols(None, cp, ri, None, pack, None, x, ac, go, 0.2, row_grad=False)
        return out, gf, gr, gc

    a, b = ref_step(), our_step()
    for u, v, name in zip(a, b, ("out", "grad_feat", "grad_attn_row", "grad_attn_col")):
        # rows and columns of up to 290 k edges: the band is relative to each entry plus a part in 10^5 of the largest
        tol = 1e-5 + 1e-4 * u.abs() + 1e-5 * float(u.abs().max())
        frac_bad = float(((u - v).abs() > 4 * tol).float().mean())
        assert frac_bad < 1e-5, f"{name}: {frac_bad:.2e} of the elements differ from the reference kernels"
    del a, b
    t_ref, t_our = _time(ref_step, 3, 1), _time(our_step, 5, 2)
    rec = dict(workload="rmat n=2.4M e=120M h=8 f=32 fused GAT fwd+bwd (int32 row_ptr)", ref_ms=t_ref, ours_ms=t_our,
               speedup=t_ref / t_our)
    print("SIDE_BY_SIDE_FULL", json.dumps(rec))
    _record("side_by_side_full.json", rec)
    assert t_our < t_ref


def test_side_by_side_other_ops(cuda, ref):
    """Every other operator against the reference's kernel on the same GPU, at sizes and shapes the
    reference kernels handle (int32, widths that are multiples of 32, one Gaussian kernel): results agree
    and both times are recorded in side_by_side_ops.json in the results folder."""
    rec = {}
    n, e, h, f = 300_000, 12_000_000, 8, 32
    rp, ci = synth.rmat_graph(n, e, seed=4, device=cuda, ptr_dtype=torch.int32)
    g = torch.Generator(device=cuda).manual_seed(1)

    # multi-head SDDMM
    a, b = torch.randn(n, h, f, device=cuda, generator=g), torch.randn(n, h, f, device=cuda, generator=g)
    r_out, o_out = ref["mhsddmm"].mhsddmm(rp, ci, a, b), kernels.mhsddmm(rp, ci, a, b)
    assert float(((r_out - o_out).abs() / (1e-4 + 1e-4 * r_out.abs())).max()) < 2.0
    rec["mhsddmm 300k/12M 8x32"] = (_time(lambda: ref["mhsddmm"].mhsddmm(rp, ci, a, b)), _time(lambda: kernels.mhsddmm(rp, ci, a, b)))
    del a, b, r_out, o_out

    # CSR -> CSC (the reference carries the position as an fp32 value: exact below 2^24 entries)
    vals = torch.arange(e, dtype=torch.float32, device=cuda)
    colptr, rowind, cscval = ref["format_conversion"].csr2csc(rp, ci, vals)
    cp, ri, pm = kernels.csr2csc(rp, ci)
    assert torch.equal(colptr, cp) and torch.equal(rowind, ri) and torch.equal(cscval.int(), pm)
    rec["csr2csc 300k/12M"] = (_time(lambda: ref["format_conversion"].csr2csc(rp, ci, vals)), _time(lambda: kernels.csr2csc(rp, ci)))

    # multi-head transpose
    x = torch.randn(e, h, device=cuda, generator=g)
    assert torch.equal(ref["mhtranspose"].mhtranspose(pm, x), kernels.mhtranspose(pm, x))
    rec["mhtranspose 12M x 8"] = (_time(lambda: ref["mhtranspose"].mhtranspose(pm, x)), _time(lambda: kernels.mhtranspose(pm, x)))
    del x, vals, colptr, rowind, cscval

    # MoNet aggregation, one Gaussian kernel, 32 channels (buffers padded: the reference reads past the row end)
    feat = cases.padded(torch.randn(n, 1, 32, device=cuda, generator=g))
    pseudo = cases.padded(torch.rand(e, 2, device=cuda, generator=g))
    mu, sig = torch.rand(1, 2, device=cuda, generator=g), torch.rand(1, 2, device=cuda, generator=g) + 0.5
    r_out, o_out = ref["fused_gmmconv"].gmmconv(rp, ci, feat, pseudo, mu, sig), kernels.gmm_forward(rp, ci, feat, pseudo, mu, sig)
    assert float(((r_out - o_out).abs() / (1e-3 + 1e-3 * r_out.abs())).max()) < 2.0
    rec["gmmconv 300k/12M 1x32"] = (_time(lambda: ref["fused_gmmconv"].gmmconv(rp, ci, feat, pseudo, mu, sig)),
                                    _time(lambda: kernels.gmm_forward(rp, ci, feat, pseudo, mu, sig)))
    del feat, pseudo, rp, ci, cp, ri, pm

    # EdgeConv forward at the point-cloud configuration (32 x 2048 points, k = 20, 64 channels)
    pts = synth.unit_sphere_clouds(32, 2048, seed=3, device=cuda)
    src = synth.knn_src_ind(pts, 20)
    m = 32 * 2048
    hs, hd = torch.randn(m, 64, device=cuda, generator=g), torch.randn(m, 64, device=cuda, generator=g)
    r_out, r_idx = ref["fused_edgeconv"].edgeconv_forward(20, src, hs, hd)
    o_out, o_idx = kernels.edgeconv_forward(20, src, hs, hd)
    assert torch.equal(r_out, o_out) and torch.equal(r_idx.int(), o_idx)
    rec["edgeconv_forward 65536 x 20 x 64"] = (_time(lambda: ref["fused_edgeconv"].edgeconv_forward(20, src, hs, hd), 30),
                                                _time(lambda: kernels.edgeconv_forward(20, src, hs, hd), 30))

    out = {k: {"ref_ms": round(v[0], 4), "ours_ms": round(v[1], 4), "speedup": round(v[0] / v[1], 2)} for k, v in rec.items()}
    print("SIDE_BY_SIDE_OPS", json.dumps(out))
    _record("side_by_side_ops.json", out, indent=1)


def test_side_by_side_small_graph(cuda, ref):
    """The citation-graph size the reference publishes its numbers on (2708 nodes, ~13 k edges, 4 x 64):
    fused GAT forward+backward, reference kernels vs these kernels (operator calls only)."""
    rp, ci = synth.powerlaw_graph()
    n, h, f = rp.numel() - 1, 4, 64
    rp, ci = rp.to(cuda), ci.to(cuda)
    cp, ri, pm = kernels.csr2csc(rp, ci)
    g = torch.Generator(device=cuda).manual_seed(0)
    ar, ac = torch.randn(n, h, device=cuda, generator=g), torch.randn(n, h, device=cuda, generator=g)
    x, go = torch.randn(n, h, f, device=cuda, generator=g), torch.randn(n, h, f, device=cuda, generator=g)
    fg = ref["fused_gatconv"]

    def ref_step():
        out, emax, esum, mask = fg.gat_forward(ar, ac, rp, ci, 0.2, x, 0.0)
        return (out,) + tuple(fg.gat_backward(0.2, 0.0, rp, ci, cp, ri, pm, emax, esum, mask, x, ar, ac, go))

    def our_step():
        out, emax, esum = kernels.gat_forward(ar, ac, rp, ci, 0.2, x)
        return (out,) + kernels.gat_backward(0.2, 0.0, rp, cp, ri, pm, emax, esum, None, x, out, ar, ac, go)

    # the reference's backward adds with float atomics, so its own result moves from run to run where terms
    # cancel: the band is relative to each entry plus a part in 10^5 of the tensor's largest entry
    for u, v, name in zip(ref_step(), our_step(), ("out", "grad_feat", "grad_attn_row", "grad_attn_col")):
        tol = 2e-5 + 1e-4 * u.abs() + 1e-5 * float(u.abs().max())
        assert float(((u - v).abs() / tol).max()) < 2.0, name
    t_ref, t_our = _time(ref_step, 50, 5), _time(our_step, 50, 5)
    rec = dict(workload="2708 nodes / 13264 edges, 4 x 64, fused GAT fwd+bwd", ref_ms=t_ref, ours_ms=t_our, speedup=t_ref / t_our)
    print("SIDE_BY_SIDE_SMALL", json.dumps(rec))
    _record("side_by_side_small.json", rec)


def _fp64_truth(case):
    d = {k: (v.double() if isinstance(v, torch.Tensor) and v.is_floating_point() else v) for k, v in case.items()}
    from oracle import dgnn_oracle as orc
    out, emax, esum = orc.gat_forward(d["attn_row"], d["attn_col"], d["row_ptr"], d["col_ind"], d["slope"], d["in_feat"])
    gf, gr, gc = orc.gat_backward(d["slope"], 0.0, d["row_ptr"], d["col_ind"], emax, esum, None, d["in_feat"],
                                  d["attn_row"], d["attn_col"], d["grad_out"])
    return dict(out=out, grad_feat=gf, grad_attn_row=gr, grad_attn_col=gc)


def _long_row_case():
    """Rows of 500 to 3000 edges (sums of thousands of terms), widths the reference kernels handle."""
    rp, ci = synth.random_graph(400, 12, 5, long_rows=[(3, 3000), (9, 1100), (250, 500)])
    n = rp.numel() - 1
    g = torch.Generator().manual_seed(77)
    return dict(row_ptr=rp, col_ind=ci, attn_row=torch.randn(n, 8, generator=g), attn_col=torch.randn(n, 8, generator=g),
                in_feat=torch.randn(n, 8, 32, generator=g), grad_out=torch.randn(n, 8, 32, generator=g), slope=0.2)


@pytest.mark.parametrize("name", ["gat_h4_f32", "gat_h1_f64", "gat_h8_f32", "long_rows"])
def test_error_against_fp64_is_no_larger_than_the_reference_kernels(cuda, ref, name):
    """Where a test of this suite allows more than 1e-5 absolute (the attention gradients: sums of hundreds to
    thousands of products of O(1) terms), the band is justified here: measured against the oracle evaluated in
    fp64, every output of these kernels is either inside the contract's own band (1e-5 absolute + 1e-4 relative)
    or no further from the truth than twice the reference's own fp32 kernels on the same inputs -- for both ways
    this library computes the row gradient (per-edge array, and negative-side forward outputs)."""
    case = _long_row_case() if name == "long_rows" else cases.CASES[name]()
    truth = _fp64_truth(case)
    r = {k: v.detach().cpu().double() for k, v in cases.run_reference("gat", case, ref, cuda).items()}
    o = {k: v.detach().cpu().double() for k, v in ours_outputs("gat", case, cuda).items()}
    d = {k: (v.to(cuda) if isinstance(v, torch.Tensor) else v) for k, v in case.items()}
    cp, ri, pm = [t.int().to(cuda) for t in scipy_csc(case["row_ptr"], case["col_ind"])]
    out, emax, esum, out_neg, a_neg = kernels.gat_forward(d["attn_row"], d["attn_col"], d["row_ptr"], d["col_ind"], d["slope"],
                                                          d["in_feat"], neg=True)
    pack, gr2, _ = kernels.gat_rowstat_full(d["attn_row"], emax, esum, out, d["grad_out"], d["slope"], out_neg=out_neg, a_neg=a_neg)
    o["grad_attn_row_from_negative_side"] = gr2.detach().cpu().double()
    report = {}
    for key in ("out", "grad_feat", "grad_attn_row", "grad_attn_col", "grad_attn_row_from_negative_side"):
        t = truth[key.replace("_from_negative_side", "")]
        e_ours = float((o[key] - t).abs().max())
        e_ref = float((r[key.replace("_from_negative_side", "")] - t).abs().max())
        in_contract = bool(((o[key] - t).abs() <= 1e-5 + 1e-4 * t.abs()).all())
        report[key] = dict(ours=e_ours, reference=e_ref, inside_contract_band=in_contract)
        assert in_contract or e_ours <= 2.0 * e_ref, (name, key, e_ours, e_ref)
    print("ERROR_VS_FP64", name, json.dumps(report))
    _record(f"error_vs_fp64_{name}.json", report, indent=1)
