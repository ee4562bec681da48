"""Size-independent properties at the full benchmark size (2.4 M nodes, 120 M edges,
8 heads x 32, int64 row_ptr), where the CPU oracle is too slow: conversion invariants,
softmax normalisation, linearity, and the checksum that links the two attention
gradients.  A 16 M-edge prefix of the same graph is also compared with the oracle."""
import pytest
import torch

from dgnn_b200 import kernels, synth
from helpers import assert_close, assert_equal
from oracle import dgnn_oracle as orc

pytestmark = pytest.mark.gpu

N, E, H, F = 2_400_000, 120_000_000, 8, 32


@pytest.fixture(scope="module")
def big(cuda):
    free, _ = torch.cuda.mem_get_info()
    if free < 60 * 2**30:
        pytest.skip("needs about 60 GB of free device memory")
    rp, ci = synth.rmat_graph(N, E, seed=4, device=cuda, ptr_dtype=torch.int64)
    cp, ri, pm = kernels.csr2csc(rp, ci)
    return rp, ci, cp, ri, pm


def test_csr2csc_invariants_full_size(big):
    rp, ci, cp, ri, pm = big
    # col_ptr is the prefix sum of the column histogram
    counts = torch.bincount(ci.long(), minlength=N)
    ref_ptr = torch.zeros(N + 1, dtype=torch.int64, device=ci.device)
    torch.cumsum(counts, 0, out=ref_ptr[1:])
    assert torch.equal(cp, ref_ptr)
    del counts, ref_ptr
    # permute is a permutation of 0..E-1
    seen = torch.zeros(E, dtype=torch.bool, device=ci.device)
    seen[pm.long()] = True
    assert bool(seen.all())
    del seen
    # entry j of the CSC is CSR entry permute[j]: same column, and row_ind is that entry's row
    cols_of_csc = torch.repeat_interleave(torch.arange(N, device=ci.device, dtype=torch.int32), (cp[1:] - cp[:-1]))
    assert torch.equal(ci[pm.long()], cols_of_csc)
    del cols_of_csc
    rows_of_perm = (torch.searchsorted(rp, pm.long(), right=True) - 1).int()
    assert torch.equal(rows_of_perm, ri)
    del rows_of_perm
    # stability: inside a column the CSR positions increase
    inc = pm[1:] > pm[:-1]
    boundary = torch.zeros(E - 1, dtype=torch.bool, device=ci.device)
    b = cp[1:-1]
    b = b[(b > 0) & (b < E)] - 1
    boundary[b] = True
    assert bool((inc | boundary).all())


def test_gat_properties_full_size(big):
    rp, ci, cp, ri, pm = big
    dev = ci.device
    g = torch.Generator(device=dev).manual_seed(7)
    ar, ac = torch.randn(N, H, device=dev, generator=g), torch.randn(N, H, device=dev, generator=g)
    x, go = torch.randn(N, H, F, device=dev, generator=g), torch.randn(N, H, F, device=dev, generator=g)
    deg = rp[1:] - rp[:-1]
    nonempty = deg > 0
    # softmax weights of a row sum to one: constant features come back unchanged
    ones = torch.ones(N, H, F, device=dev)
    out1, emax, esum = kernels.gat_forward(ar, ac, rp, ci, 0.2, ones)
    assert float((out1[nonempty] - 1).abs().max()) < 1e-5
    assert float(out1[~nonempty].abs().max()) == 0.0
    assert bool((esum[nonempty] >= 1 - 1e-6).all()) and bool((esum[nonempty] <= deg[nonempty, None] * (1 + 1e-5)).all())
    del ones, out1
    # linearity in the features
    out, emax2, esum2 = kernels.gat_forward(ar, ac, rp, ci, 0.2, x)
    assert torch.equal(emax, emax2) and torch.equal(esum, esum2)
    out3 = kernels.gat_forward(ar, ac, rp, ci, 0.2, x * 3.0, save_stats=False)[0]
    assert_close(out3, out * 3.0, "linearity", rtol=1e-5, atol=1e-5)
    del out3
    # both attention gradients are sums of the same per-edge terms: equal totals per head
    gf, gr, gc = kernels.gat_backward(0.2, 0.0, rp, cp, ri, pm, emax, esum, None, x, out, ar, ac, go)
    tot_r, tot_c = gr.double().sum(0), gc.double().sum(0)
    scale = gr.double().abs().sum(0)
    assert bool(((tot_r - tot_c).abs() <= 1e-5 * scale).all()), (tot_r, tot_c)
    # without the leaky slope the row gradient vanishes (sum_e alpha_e (g_e - S) = 0)
    out_s, em_s, es_s = kernels.gat_forward(ar, ac, rp, ci, 1.0, x)
    _, gr1, _ = kernels.gat_backward(1.0, 0.0, rp, cp, ri, pm, em_s, es_s, None, x, out_s, ar, ac, go)
    assert float(gr1.abs().max()) < 5e-3 * float(gr.abs().max())
    # grad_feat is linear in grad_out
    gf2, _, _ = kernels.gat_backward(0.2, 0.0, rp, cp, ri, pm, emax, esum, None, x, out, ar, ac, go * 2.0)
    assert_close(gf2, gf * 2.0, "grad_feat linearity", rtol=1e-5, atol=1e-5)


def test_prefix_of_the_big_graph_against_oracle(big):
    """The first rows of the 120 M-edge graph holding about 1.5 M edges, with the global source features."""
    rp, ci, *_ = big
    dev = ci.device
    r1 = int(torch.searchsorted(rp, torch.tensor([1_500_000], device=dev))[0])
    e1 = int(rp[r1])
    sub_ptr, sub_col = rp[: r1 + 1].clone(), ci[:e1].clone()
    g = torch.Generator(device=dev).manual_seed(9)
    n_src = 400_000   # columns folded into a smaller source range so that the CPU side stays small
    sub_col = (sub_col % n_src).int()
    ar = torch.randn(r1, H, device=dev, generator=g)
    ac, x = torch.randn(n_src, H, device=dev, generator=g), torch.randn(n_src, H, F, device=dev, generator=g)
    out, emax, esum = kernels.gat_forward(ar, ac, sub_ptr, sub_col, 0.2, x)
    o_ref, m_ref, z_ref = orc._gat_forward_rows(ar.cpu(), ac.cpu(), sub_ptr.cpu(), sub_col.cpu(), 0.2, x.cpu())
    assert_close(out, o_ref, "out (rows with up to ~290 k edges)", atol=2e-5)
    assert_equal(emax, m_ref, "edge_max")
    assert_close(esum, z_ref, "edge_sum")
