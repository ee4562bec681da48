"""CPU checks of the oracle itself: analytic backward formulas against autograd
in fp64, conversions against scipy, degenerate graphs."""
import numpy as np
import pytest
import torch

from dgnn_b200 import synth
from helpers import assert_close, assert_equal, gat_inputs, scipy_csc
from oracle import dgnn_oracle as orc


def _graph(n=60, avg=5, seed=0, long_rows=((3, 70), (17, 33))):
    return synth.random_graph(n, avg, seed, long_rows=long_rows)


@pytest.mark.parametrize("h,f", [(1, 4), (3, 5), (4, 8)])
def test_gat_backward_matches_autograd_fp64(h, f):
    row_ptr, col_ind = _graph()
    n = row_ptr.numel() - 1
    ar, ac, x, g = [t.double() for t in gat_inputs(row_ptr, n, h, f, seed=5)]
    ar.requires_grad_(); ac.requires_grad_(); x.requires_grad_()
    out = orc.gat_forward_differentiable(ar, ac, row_ptr, col_ind, 0.2, x)
    out.backward(g)
    o2, emax, esum = orc.gat_forward(ar.detach(), ac.detach(), row_ptr, col_ind, 0.2, x.detach())
    assert_close(o2, out, "forward vs differentiable forward", 1e-12, 1e-12)
    gf, gr, gc = orc.gat_backward(0.2, 0.0, row_ptr, col_ind, emax, esum, None, x.detach(), ar.detach(),
                                  ac.detach(), g)
    assert_close(gf, x.grad, "grad_feat", 1e-10, 1e-12)
    assert_close(gr, ar.grad, "grad_attn_row", 1e-10, 1e-12)
    assert_close(gc, ac.grad, "grad_attn_col", 1e-10, 1e-12)


def test_gat_rowsum_identity():
    """S_r = sum_e alpha_e g_e equals <grad_out[r], out[r]> (the identity the CUDA backward uses),
    also under dropout."""
    row_ptr, col_ind = _graph()
    n, h, f = row_ptr.numel() - 1, 4, 8
    ar, ac, x, g = [t.double() for t in gat_inputs(row_ptr, n, h, f, seed=7)]
    mask = torch.rand(col_ind.numel(), h, dtype=torch.double, generator=torch.Generator().manual_seed(1))
    p = 0.3
    out, emax, esum = orc.gat_forward(ar, ac, row_ptr, col_ind, 0.2, x, p, mask)
    rows = orc.edge_rows(row_ptr)
    _, _, _, alpha = orc.gat_edge_softmax(ar, ac, row_ptr, col_ind, 0.2)
    ge = (g[rows] * x[col_ind.long()]).sum(-1) * (mask > p) / (1 - p)
    s_edges = torch.zeros(n, h, dtype=torch.double).index_add_(0, rows, alpha * ge)
    assert_close((g * out).sum(-1), s_edges, "row sum identity", 1e-10, 1e-12)


def test_gat_empty_rows_and_stats():
    row_ptr = torch.tensor([0, 0, 2, 2, 3], dtype=torch.int32)
    col_ind = torch.tensor([0, 3, 1], dtype=torch.int32)
    ar, ac, x, _ = gat_inputs(row_ptr, 4, 2, 4, seed=1)
    out, emax, esum = orc.gat_forward(ar, ac, row_ptr, col_ind, 0.2, x)
    assert torch.all(out[0] == 0) and torch.all(out[2] == 0)
    assert torch.all(emax[0] == torch.tensor(-1e38)) and torch.all(esum[0] == 0)
    # a single-edge row copies the source row
    assert_close(out[3], x[1], "degree-1 row")


def test_csr2csc_matches_scipy_with_duplicates():
    row_ptr, col_ind = synth.random_graph(200, 6, seed=3, long_rows=[(5, 300)])
    cp, ri, pm = orc.csr2csc(row_ptr, col_ind)
    scp, sri, spm = scipy_csc(row_ptr, col_ind)
    assert_equal(cp, scp, "col_ptr"); assert_equal(ri, sri, "row_ind"); assert_equal(pm, spm, "permute")
    # permute is a permutation and respects CSR order inside every column
    assert torch.equal(torch.sort(pm).values, torch.arange(col_ind.numel()))
    for c in range(0, 200, 17):
        seg = pm[cp[c]:cp[c + 1]]
        assert torch.all(seg[1:] > seg[:-1])


def test_coo2csr():
    rows = torch.tensor([0, 0, 2, 2, 2, 5], dtype=torch.int32)
    assert orc.coo2csr(rows, 7).tolist() == [0, 2, 2, 5, 5, 5, 6, 6]
    assert orc.coo2csr(torch.zeros(0, dtype=torch.int32), 3).tolist() == [0, 0, 0, 0]


def test_sddmm_and_transpose():
    row_ptr, col_ind = _graph()
    n = row_ptr.numel() - 1
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(n, 3, 5, generator=g), torch.randn(n, 3, 5, generator=g)
    out = orc.mhsddmm(row_ptr, col_ind, a, b)
    rows = orc.edge_rows(row_ptr)
    e = 11
    assert_close(out[e], (a[rows[e]] * b[col_ind[e].long()]).sum(-1), "one edge")
    perm = torch.randperm(col_ind.numel(), generator=g)
    assert torch.equal(orc.mhtranspose(perm, out), out[perm])


def test_gmm_forward_backward_autograd_fp64():
    row_ptr, col_ind = _graph()
    n, k, dim, f = row_ptr.numel() - 1, 3, 2, 4
    g = torch.Generator().manual_seed(2)
    feat = torch.randn(n, k, f, generator=g, dtype=torch.double, requires_grad=True)
    pseudo = torch.rand(col_ind.numel(), dim, generator=g, dtype=torch.double, requires_grad=True)
    mu = torch.rand(k, dim, generator=g, dtype=torch.double, requires_grad=True)
    sig = (torch.rand(k, dim, generator=g, dtype=torch.double) + 0.5).requires_grad_()
    go = torch.randn(n, k, f, generator=g, dtype=torch.double)
    out = orc.gmm_forward(row_ptr, col_ind, feat, pseudo, mu, sig)
    out.backward(go)
    # the operator's backward recipe (operators/fused_gmmconv.py:20-27 of the reference) with the intended Gaussian gradient
    cp, ri, pm = orc.csr2csc(row_ptr, col_ind)
    gg = orc.mhsddmm(row_ptr, col_ind, go, feat.detach())
    feat_grad = orc.gmm_forward(cp, ri, go, orc.mhtranspose(pm, pseudo.detach()), mu.detach(), sig.detach())
    dps, dmu, dsig = orc.gaussian_backward(pseudo.detach(), mu.detach(), sig.detach(), gg)
    assert_close(feat_grad, feat.grad, "node_feat grad", 1e-10, 1e-12)
    assert_close(dps, pseudo.grad, "pseudo grad", 1e-10, 1e-12)
    assert_close(dmu, mu.grad, "mu grad", 1e-10, 1e-12)
    assert_close(dsig, sig.grad, "sigma grad", 1e-10, 1e-12)


def test_edgeconv_forward_backward():
    g = torch.Generator().manual_seed(4)
    m, k, f = 50, 7, 6
    src = torch.randint(0, m, (m * k,), generator=g, dtype=torch.int32)
    hs = torch.randn(m, f, generator=g, dtype=torch.double, requires_grad=True)
    hd = torch.randn(m, f, generator=g, dtype=torch.double, requires_grad=True)
    out, idx = orc.edgeconv_forward(k, src, hs, hd)
    ref = (hd[:, None, :] + hs[src.long().view(m, k)]).max(dim=1).values
    assert_close(out, ref, "edgeconv out", 0, 0)
    go = torch.randn(m, f, generator=g, dtype=torch.double)
    ref.backward(go)
    assert_close(orc.edgeconv_backward(go, idx), hs.grad, "grad_src", 1e-12, 1e-12)
    assert_close(go, hd.grad, "grad_dst", 0, 0)
    # ties: the smallest j wins
    hs2 = torch.zeros(3, 2); hd2 = torch.zeros(3, 2)
    _, idx2 = orc.edgeconv_forward(2, torch.tensor([2, 1, 0, 2, 1, 0], dtype=torch.int32), hs2, hd2)
    assert idx2[:, 0].tolist() == [2, 0, 1]


def test_chunked_cpu_step_equals_unchunked():
    row_ptr, col_ind = _graph(n=90)
    n, h, f = 90, 2, 4
    ar, ac, x, g = gat_inputs(row_ptr, n, h, f, seed=9)
    full = orc.gat_fused_step_cpu(ar, ac, row_ptr, col_ind, 0.2, x, g)
    part = orc.gat_fused_step_cpu(ar, ac, row_ptr, col_ind, 0.2, x, g, chunk_rows=13)
    for a, b, name in zip(full, part, ("out", "grad_feat", "grad_row", "grad_col")):
        assert_close(a, b, name)


def test_knn_and_coo_sort_oracles():
    """kNN against a float64 brute force on points without near-ties; the edge sort against python's sorted()."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 50, 4, generator=g)
    got = orc.knn_graph(x, 6).view(3, 50, 6)
    d = torch.cdist(x.double(), x.double())
    ref = d.argsort(dim=2, stable=True)[:, :, :6] + (torch.arange(3) * 50)[:, None, None]
    assert torch.equal(got, ref)
    dst = torch.randint(0, 20, (300,), generator=g)
    src = torch.randint(0, 20, (300,), generator=g)
    d_s, s_s = orc.coo_sort(dst, src)
    assert list(zip(d_s.tolist(), s_s.tolist())) == sorted(zip(dst.tolist(), src.tolist()))
