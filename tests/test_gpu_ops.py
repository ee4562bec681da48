"""GPU parity of SDDMM, transpose, GMM, EdgeConv and the conversions against the oracle."""
import numpy as np
import pytest
import torch

from dgnn_b200 import kernels, synth
from dgnn_b200.ext import format_conversion, fused_edgeconv
from dgnn_b200.operators import EdgeConvFuse, GmmConvFuse
from helpers import assert_close, assert_equal, scipy_csc
from oracle import dgnn_oracle as orc

pytestmark = pytest.mark.gpu
SEG = 1024


def _graph(kind, ptr64=False):
    dt = np.int64 if ptr64 else np.int32
    if kind == "tiny":
        return synth.random_graph(40, 3, 1, long_rows=[(0, 1), (5, 33), (9, 65)], ptr_dtype=dt)
    if kind == "medium":
        return synth.random_graph(700, 9, 2, long_rows=[(3, 100), (400, 257)], ptr_dtype=dt)
    return synth.random_graph(900, 6, 3, long_rows=[(7, SEG + 1), (8, 3 * SEG + 17), (500, 2 * SEG)], ptr_dtype=dt)


@pytest.mark.parametrize("h,f", [(1, 64), (3, 16), (4, 64), (8, 32), (16, 64), (2, 256), (3, 5), (1, 1), (2, 33)])
@pytest.mark.parametrize("kind", ["tiny", "medium", "long"])
def test_mhsddmm(cuda, kind, h, f):
    rp, ci = _graph(kind)
    n = rp.numel() - 1
    g = torch.Generator().manual_seed(3)
    a, b = torch.randn(n, h, f, generator=g), torch.randn(n, h, f, generator=g)
    out = kernels.mhsddmm(rp.to(cuda), ci.to(cuda), a.to(cuda), b.to(cuda))
    assert_close(out, orc.mhsddmm(rp, ci, a, b), "mhsddmm")


@pytest.mark.parametrize("h", [1, 2, 3, 4, 8, 16])
def test_mhtranspose_bit_exact(cuda, h):
    g = torch.Generator().manual_seed(5)
    nnz = 10007
    perm = torch.randperm(nnz, generator=g).int()
    x = torch.randn(nnz, h, generator=g)
    assert_equal(kernels.mhtranspose(perm.to(cuda), x.to(cuda)), orc.mhtranspose(perm, x), "mhtranspose")
    assert kernels.mhtranspose(perm[:0].to(cuda), x[:0].to(cuda)).shape == (0, h)


@pytest.mark.parametrize("kind,ptr64", [("tiny", False), ("medium", False), ("long", False), ("long", True)])
def test_csr2csc_bit_exact(cuda, kind, ptr64):
    rp, ci = _graph(kind, ptr64)
    cp, ri, pm = kernels.csr2csc(rp.to(cuda), ci.to(cuda))
    scp, sri, spm = scipy_csc(rp, ci)
    assert cp.dtype == rp.dtype
    assert_equal(cp, scp, "col_ptr"); assert_equal(ri, sri, "row_ind"); assert_equal(pm, spm, "permute")
    ocp, ori, opm = orc.csr2csc(rp, ci)
    assert_equal(cp, ocp, "col_ptr vs oracle"); assert_equal(ri, ori, "row_ind vs oracle"); assert_equal(pm, opm, "permute vs oracle")


@pytest.mark.parametrize("n,nnz", [(1, 5), (300, 5000), (70000, 300000), (2**17 + 3, 1 << 20)])
def test_csr2csc_sizes_and_passes(cuda, n, nnz):
    """1, 2 and 3 radix passes (n_cols <= 2^8, 2^16, 2^24), several tiles, duplicates."""
    g = torch.Generator().manual_seed(n)
    dst = torch.randint(0, n, (nnz,), generator=g)
    src = torch.randint(0, n, (nnz,), generator=g)
    src[: nnz // 8] = src[0]                       # a hub column
    rp, ci = synth.csr_from_edges(dst.numpy(), src.numpy(), n)
    cp, ri, pm = kernels.csr2csc(rp.to(cuda), ci.to(cuda))
    ocp, ori, opm = orc.csr2csc(rp, ci)
    assert_equal(cp, ocp, "col_ptr"); assert_equal(ri, ori, "row_ind"); assert_equal(pm, opm, "permute")


def test_csr2csc_rectangular_and_empty(cuda):
    rp = torch.tensor([0, 2, 2, 5], dtype=torch.int32)
    ci = torch.tensor([6, 1, 0, 6, 6], dtype=torch.int32)
    cp, ri, pm = kernels.csr2csc(rp.to(cuda), ci.to(cuda), n_cols=7)
    ocp, ori, opm = orc.csr2csc(rp, ci, 7)
    assert_equal(cp, ocp, "col_ptr"); assert_equal(ri, ori, "row_ind"); assert_equal(pm, opm, "permute")
    cp, ri, pm = kernels.csr2csc(torch.zeros(4, dtype=torch.int32, device=cuda), torch.zeros(0, dtype=torch.int32, device=cuda))
    assert cp.tolist() == [0, 0, 0, 0] and ri.numel() == 0


def test_format_conversion_module(cuda):
    rp, ci = _graph("medium")
    vals = torch.arange(ci.numel(), dtype=torch.float32)
    colptr, rowind, cscval = format_conversion.csr2csc(rp.to(cuda), ci.to(cuda), vals.to(cuda))
    scp, sri, spm = scipy_csc(rp, ci)
    assert_equal(colptr, scp, "colptr"); assert_equal(rowind, sri, "rowind"); assert_equal(cscval.long(), spm, "values = positions")
    rows = orc.edge_rows(rp).int()
    assert_equal(format_conversion.coo2csr(rows.to(cuda), rp.numel() - 1), rp, "coo2csr")
    assert_equal(kernels.coo2csr(rows.to(cuda), rp.numel() - 1, torch.int64), rp, "coo2csr int64")
    assert kernels.coo2csr(rows[:0].to(cuda), 3).tolist() == [0, 0, 0, 0]


@pytest.mark.parametrize("k,f,dim", [(3, 16, 2), (1, 64, 1), (2, 5, 3), (4, 32, 2)])
@pytest.mark.parametrize("kind", ["tiny", "medium", "long"])
def test_gmm_forward_backward(cuda, kind, k, f, dim):
    rp, ci = _graph(kind)
    n, nnz = rp.numel() - 1, ci.numel()
    g = torch.Generator().manual_seed(8)
    feat = torch.randn(n, k, f, generator=g)
    pseudo = torch.rand(nnz, dim, generator=g)
    mu = torch.rand(k, dim, generator=g)
    sig = torch.rand(k, dim, generator=g) + 0.5
    go = torch.randn(n, k, f, generator=g)
    # oracle: autograd through the CPU forward (fp64 for the reference gradients)
    f64 = [t.double().requires_grad_() for t in (feat, pseudo, mu, sig)]
    ref = orc.gmm_forward(rp, ci, *f64)
    ref.backward(go.double())
    cp, ri, pm = scipy_csc(rp, ci)
    dev = [t.to(cuda).requires_grad_() for t in (feat, pseudo, mu, sig)]
    out = GmmConvFuse(rp.to(cuda), ci.to(cuda), cp.int().to(cuda), ri.int().to(cuda), pm.int().to(cuda), *dev)
    out.backward(go.to(cuda))
    # rows of thousands of edges sum in a different order than the fp64 reference: scale atol with the row length
    assert_close(out, ref.float(), "gmm out", rtol=1e-4, atol=1e-5 if kind != "long" else 5e-4)
    assert_close(kernels.gaussian(dev[1].detach(), dev[2].detach(), dev[3].detach()),
                 orc.gaussian(pseudo, mu, sig), "gaussian")
    scale = max(1.0, float(f64[2].grad.abs().max()))
    assert_close(dev[0].grad, f64[0].grad.float(), "node_feat grad")
    assert_close(dev[1].grad, f64[1].grad.float(), "pseudo grad", atol=1e-4)
    assert_close(dev[2].grad, f64[2].grad.float(), "mu grad", rtol=1e-4, atol=1e-4 * scale)
    assert_close(dev[3].grad, f64[3].grad.float(), "sigma grad", rtol=1e-4, atol=1e-4 * scale)


@pytest.mark.parametrize("m,k,f", [(500, 20, 64), (300, 7, 128), (100, 40, 3), (64, 1, 6), (33, 5, 256)])
def test_edgeconv(cuda, m, k, f):
    g = torch.Generator().manual_seed(m)
    src = torch.randint(0, m, (m * k,), generator=g, dtype=torch.int32)
    hs, hd, go = (torch.randn(m, f, generator=g) for _ in range(3))
    o_ref, i_ref = orc.edgeconv_forward(k, src, hs, hd)
    out, idx = kernels.edgeconv_forward(k, src.to(cuda), hs.to(cuda), hd.to(cuda))
    assert_equal(out, o_ref, "edgeconv out (a max of identical sums: bit-exact)")
    assert_equal(idx, i_ref, "max_idx")
    out_f, idx_f = fused_edgeconv.edgeconv_forward(k, src.to(cuda), hs.to(cuda), hd.to(cuda))
    assert idx_f.dtype == torch.float32 and torch.equal(idx_f.int(), idx)
    assert_close(kernels.edgeconv_backward(go.to(cuda), idx), orc.edgeconv_backward(go, i_ref), "grad_src")
    # autograd surface
    a = hs.to(cuda).requires_grad_(); b = hd.to(cuda).requires_grad_()
    EdgeConvFuse(k, src.to(cuda), a, b).backward(go.to(cuda))
    assert_close(a.grad, orc.edgeconv_backward(go, i_ref), "h_src grad"); assert_equal(b.grad, go, "h_dst grad")


@pytest.mark.parametrize("m,k,f", [(300, 20, 64), (1000, 5, 12), (64, 1, 4), (2048, 20, 128)])
def test_edgeconv_backward_ordered_is_reproducible(cuda, m, k, f):
    """The gather over the transposed neighbour graph: same gradient as the scatter-add, one fixed summation order
    (ascending destination, which is also the order of the CPU oracle: bit-equal to it), repeated neighbours in a
    list counted once, and chosen by the operator under torch.use_deterministic_algorithms(True)."""
    g = torch.Generator().manual_seed(m + k)
    src = torch.randint(0, max(m // 8, 1), (m * k,), generator=g, dtype=torch.int32)   # few sources: many ties and repeats
    hs, hd, go = (torch.randn(m, f, generator=g) for _ in range(3))
    hs[: m // 16] = 0.5                                                              # equal sums: the first neighbour wins
    _, i_ref = orc.edgeconv_forward(k, src, hs, hd)
    want = orc.edgeconv_backward(go, i_ref)
    _, idx = kernels.edgeconv_forward(k, src.to(cuda), hs.to(cuda), hd.to(cuda))
    got = kernels.edgeconv_backward_ordered(k, src.to(cuda), go.to(cuda), idx)
    assert_close(got, want, "ordered grad_src")
    assert_close(kernels.edgeconv_backward(go.to(cuda), idx), want, "scatter-add grad_src")
    for _ in range(3):
        assert_equal(kernels.edgeconv_backward_ordered(k, src.to(cuda), go.to(cuda), idx), got, "repeat of the ordered backward")
    seq = torch.zeros(m, f)
    flat = i_ref.long()
    for i in range(m):                                   # sequential fp32 adds in ascending destination order
        seq[flat[i], torch.arange(f)] += go[i]
    assert_equal(got, seq, "ordered grad_src against sequential fp32 adds")
    a = hs.to(cuda).requires_grad_(); b = hd.to(cuda).requires_grad_()
    torch.use_deterministic_algorithms(True)
    try:
        EdgeConvFuse(k, src.to(cuda), a, b).backward(go.to(cuda))
    finally:
        torch.use_deterministic_algorithms(False)
    assert_equal(a.grad, got, "h_src grad under deterministic algorithms")


def test_edgeconv_ties_pick_first_neighbour(cuda):
    hs = torch.zeros(4, 8); hd = torch.zeros(4, 8)
    src = torch.tensor([3, 1, 2, 0, 1, 1, 2, 3], dtype=torch.int32)
    _, idx = kernels.edgeconv_forward(2, src.to(cuda), hs.to(cuda), hd.to(cuda))
    assert idx[:, 0].tolist() == [3, 2, 1, 2]


def test_c3_config_edgeconv_stack(cuda):
    """Config 3 at reduced batch: kNN k=20 on unit-sphere clouds, widths 3-64-64-128, through the layer API."""
    from dgnn_b200.layers import EdgeConv
    x = synth.unit_sphere_clouds(4, 512, seed=3)
    src = synth.knn_src_ind(x, 20)
    feat = x.reshape(-1, 3)
    torch.manual_seed(3)
    layers = [EdgeConv(3, 64), EdgeConv(64, 64), EdgeConv(64, 128)]
    h_ref = feat
    for l in layers:   # CPU reference of the same stack
        hs = l.theta(h_ref); hd = l.phi(h_ref) - hs
        h_ref = orc.edgeconv_forward(20, src, hs, hd)[0]
    h = feat.to(cuda)
    for l in layers:
        h = l.to(cuda)(20, src.to(cuda), h)
    assert_close(h, h_ref, "3-layer EdgeConv stack", rtol=1e-4, atol=1e-4)


def test_uniform_fill_statistics(cuda):
    u = kernels.uniform_fill((1 << 20,), seed=7, offset=0, device=cuda)
    assert float(u.min()) > 0.0 and float(u.max()) <= 1.0
    assert abs(float(u.mean()) - 0.5) < 2e-3 and abs(float(u.var()) - 1 / 12) < 2e-3
    assert torch.equal(u, kernels.uniform_fill((1 << 20,), seed=7, offset=0, device=cuda))
    assert not torch.equal(u, kernels.uniform_fill((1 << 20,), seed=8, offset=0, device=cuda))


def test_c2_config_gmm_layer(cuda):
    """Config 2: the 2708-node graph, pseudo = (deg_src^-1/2, deg_dst^-1/2), 3 kernels, 1433 -> 16, through the layer API."""
    from dgnn_b200.layers import GMMConv
    rp, ci = synth.powerlaw_graph()
    n, nnz = rp.numel() - 1, ci.numel()
    pseudo = synth.monet_pseudo(rp, ci)
    g = torch.Generator().manual_seed(2)
    feat = (torch.rand(n, 1433, generator=g) < 0.013).float()
    torch.manual_seed(2)
    layer = GMMConv(1433, 16, 2, 3)
    with torch.no_grad():
        layer.mu.copy_(torch.rand(3, 2, generator=g))
    cot = torch.randn(n, 16, generator=g)
    # CPU oracle of the layer, autograd backward in fp64
    fc_w, mu, sig = [p.detach().double().clone().requires_grad_() for p in (layer.fc.weight, layer.mu, layer.inv_sigma)]
    node_feat = (feat.double() @ fc_w.t()).view(-1, 3, 16)
    ref = orc.gmm_forward(rp, ci, node_feat, pseudo.double(), mu, sig).sum(1)
    (ref * cot.double()).sum().backward()
    cp, ri, pm = scipy_csc(rp, ci)
    layer = layer.to(cuda)
    out = layer(rp.to(cuda), ci.to(cuda), cp.int().to(cuda), ri.int().to(cuda), pm.int().to(cuda), feat.to(cuda), pseudo.to(cuda))
    (out * cot.to(cuda)).sum().backward()
    assert_close(out, ref.float(), "GMM layer out", rtol=1e-3, atol=1e-5)      # tolerance of the reference's own GMM script
    for got, want, name in ((layer.fc.weight.grad, fc_w.grad, "d fc"), (layer.mu.grad, mu.grad, "d mu"),
                            (layer.inv_sigma.grad, sig.grad, "d inv_sigma")):
        scale = max(1.0, float(want.abs().max()))
        assert_close(got, want.float(), name, rtol=1e-3, atol=1e-4 * scale)


def test_single_head_sddmm_module(cuda):
    """sddmm.coo_sddmm / sddmm.csr_sddmm (the reference's unbuilt single-head module)."""
    from dgnn_b200.ext import sddmm
    rp, ci = _graph("medium")
    n = rp.numel() - 1
    g = torch.Generator().manual_seed(4)
    for k in (64, 30, 7):
        d1, d2 = torch.randn(n, k, generator=g), torch.randn(n, k, generator=g)
        rows = orc.edge_rows(rp)
        ref = (d1[rows] * d2[ci.long()]).sum(-1)
        out = sddmm.csr_sddmm(rp.to(cuda), ci.to(cuda), d1.to(cuda), d2.to(cuda))
        assert_close(out, ref, f"csr_sddmm k={k}")
        perm = torch.randperm(ci.numel(), generator=g)          # COO edges in a scrambled order
        out = sddmm.coo_sddmm(rows[perm].int().to(cuda), ci[perm].to(cuda), d1.to(cuda), d2.to(cuda))
        assert_close(out, ref[perm], f"coo_sddmm k={k}")


def test_build_graph_and_knn_on_device(cuda):
    from dgnn_b200 import graph
    g = torch.Generator().manual_seed(6)
    n, e = 500, 6000
    src, dst = torch.randint(0, n, (e,), generator=g), torch.randint(0, n, (e,), generator=g)
    gr = graph.build_graph(src.to(cuda), dst.to(cuda), n)
    rp, ci = synth.csr_from_edges(dst.numpy(), src.numpy(), n)
    cp, ri, pm = scipy_csc(rp, ci)
    assert_equal(gr.row_ptr, rp, "row_ptr"); assert_equal(gr.col_ind, ci, "col_ind")
    assert_equal(gr.col_ptr, cp, "col_ptr"); assert_equal(gr.row_ind, ri, "row_ind"); assert_equal(gr.permute, pm, "permute")
    gl = graph.build_graph(src.to(cuda), dst.to(cuda), n, add_self_loops=True)
    deg = (gl.row_ptr[1:] - gl.row_ptr[:-1])
    assert int(deg.min()) >= 1


@pytest.mark.parametrize("n,e", [(1, 5), (300, 1), (70_000, 400_000), (5_000_000, 3_000_000)])
def test_coo_sort_bit_exact(cuda, n, e):
    """1, 3 (17-bit ids) and 3 (23-bit ids) radix passes per key; duplicates and empty rows included."""
    g = torch.Generator().manual_seed(n + e)
    src = torch.randint(0, n, (e,), generator=g, dtype=torch.int32)
    dst = torch.randint(0, n, (e,), generator=g, dtype=torch.int32)
    d_ref, s_ref = orc.coo_sort(dst, src)
    d_out, s_out = kernels.coo_sort(dst.to(cuda), src.to(cuda), n)
    assert_equal(d_out, d_ref, "sorted destinations")
    assert_equal(s_out, s_ref, "sorted sources")


@pytest.mark.parametrize("b,p,dim,k", [(5, 128, 3, 8), (2, 300, 3, 20), (3, 77, 64, 20), (1, 40, 5, 32), (2, 2048, 3, 20)])
def test_knn_graph_bit_exact(cuda, b, p, dim, k):
    g = torch.Generator().manual_seed(b * p + k)
    x = torch.randn(b, p, dim, generator=g)
    x[0, 3] = x[0, 1]                                   # an exact duplicate: ties go to the smaller index
    from dgnn_b200 import graph
    got = graph.knn_graph(x.to(cuda), k)
    assert_equal(got, orc.knn_graph(x, k), "kNN src_ind")
    first = got.view(b, p, k)[:, :, 0].cpu()
    self_ids = (torch.arange(b)[:, None] * p + torch.arange(p)[None, :])
    assert bool((first == self_ids)[0, [0, 1, 2, 4]].all()) and int(first[0, 3]) == 1    # itself first, except the duplicate


def test_knn_feeds_edgeconv_like_the_brute_force_graph(cuda):
    """On clouds without near-ties the kernel's graph equals the cdist + topk graph of the test harness."""
    x = synth.unit_sphere_clouds(4, 256, seed=1, device=cuda)
    from dgnn_b200 import graph
    a = graph.knn_graph(x, 8).view(4, 256, 8).sort(dim=2).values
    b_ = synth.knn_src_ind(x, 8).view(4, 256, 8).sort(dim=2).values
    assert float((a == b_).float().mean()) > 0.999


def test_guard_mode_validates_index_arrays(cuda, monkeypatch):
    """DGNN_BOUNDS_CHECK=1: valid inputs pass through every wrapper, an id outside the tensor it indexes or a broken
    index pointer raises before any operator kernel is launched (nothing is read out of bounds)."""
    monkeypatch.setenv("DGNN_BOUNDS_CHECK", "1")
    assert kernels.guard_enabled()
    rp, ci = synth.random_graph(200, 5, seed=8)
    n, h, f = rp.numel() - 1, 4, 8
    g = torch.Generator().manual_seed(0)
    ar, ac = torch.randn(n, h, generator=g).to(cuda), torch.randn(n, h, generator=g).to(cuda)
    x, go = torch.randn(n, h, f, generator=g).to(cuda), torch.randn(n, h, f, generator=g).to(cuda)
    rp_d, ci_d = rp.to(cuda), ci.to(cuda)
    cp, ri, pm = kernels.csr2csc(rp_d, ci_d)
    out, emax, esum = kernels.gat_forward(ar, ac, rp_d, ci_d, 0.2, x)
    kernels.gat_backward(0.2, 0.0, rp_d, cp, ri, pm, emax, esum, None, x, out, ar, ac, go)
    kernels.mhsddmm(rp_d, ci_d, x, x)
    kernels.mhtranspose(pm, torch.randn(ci.numel(), h, device=cuda))
    bad_col = ci_d.clone()
    bad_col[17] = n                                            # one past the last source node
    with pytest.raises(RuntimeError, match=r"guard: gat_forward: an id lies outside .*position 17, value 200"):
        kernels.gat_forward(ar, ac, rp_d, bad_col, 0.2, x)
    with pytest.raises(RuntimeError, match="guard: csr2csc"):
        kernels.csr2csc(rp_d, bad_col)
    bad_ptr = rp_d.clone()
    bad_ptr[5] = bad_ptr[6] + 3                                # decreases between rows 5 and 6
    with pytest.raises(RuntimeError, match="guard: mhsddmm: the index pointer decreases"):
        kernels.mhsddmm(bad_ptr, ci_d, x, x)
    short_ptr = rp_d.clone()
    short_ptr[-1] -= 1
    with pytest.raises(RuntimeError, match="guard: gat_forward: the index pointer"):
        kernels.gat_forward(ar, ac, short_ptr, ci_d, 0.2, x)
    with pytest.raises(RuntimeError, match="guard: edgeconv_forward"):
        kernels.edgeconv_forward(2, torch.tensor([0, 1, 2, 3, -1, 0], dtype=torch.int32, device=cuda),
                                 torch.zeros(3, 4, device=cuda), torch.zeros(3, 4, device=cuda))
    monkeypatch.setenv("DGNN_BOUNDS_CHECK", "0")
    assert not kernels.guard_enabled()


def _hot_rows_expected(ptr, max_hot):
    """numpy restatement of dgnn_hot_rows: counts clamp at 4095, threshold = smallest t >= 1 that marks <= max_hot rows."""
    import numpy as np
    d = np.minimum(np.diff(ptr.numpy().astype(np.int64)), 4095)
    thr = 4096
    for t in range(1, 4096):
        if int((d >= t).sum()) <= max_hot:
            thr = t
            break
    hot = np.diff(ptr.numpy().astype(np.int64)) >= thr
    words = np.zeros((len(hot) + 31) // 32 * 32, dtype=bool)
    words[:len(hot)] = hot
    packed = (words.reshape(-1, 32).astype(np.uint64) << np.arange(32, dtype=np.uint64)).sum(axis=1).astype(np.uint32)
    return torch.from_numpy(packed.view(np.int32).copy()), thr


@pytest.mark.parametrize("ptr64", [False, True])
@pytest.mark.parametrize("n,avg,max_hot", [(1, 3, 1), (33, 2, 0), (1000, 6, 50), (70_001, 9, 3000), (5000, 4, 10**9)])
def test_hot_rows_bit_exact(cuda, n, avg, max_hot, ptr64):
    rp, ci = synth.random_graph(n, avg, seed=n + max_hot, long_rows=((n // 2, 6000),) if n >= 1000 else ())
    if ptr64:
        rp = rp.long()
    want, thr = _hot_rows_expected(rp, max_hot)
    got = kernels.hot_rows(rp.to(cuda), max_hot)
    assert_equal(got, want, f"hot-row words (threshold {thr})")
    n_hot = sum(bin(int(w) & 0xffffffff).count("1") for w in got.cpu().tolist())
    assert n_hot <= max(max_hot, 0) or thr == 4096


def test_hot_rows_change_no_result(cuda, monkeypatch):
    """Cache hints only: the sweeps with a hot-row set give the same bits as without, on the same-head layout
    (8 heads x 32) and on a layout that ignores the set (4 x 8); the operator path picks a set up from
    DGNN_L2_HOT_MB once the gathered tensor is larger than twice the budget."""
    rp, ci = synth.random_graph(3000, 12, seed=5, long_rows=((7, 2500), (1500, 1100)))
    n = rp.numel() - 1
    rp_d, ci_d = rp.to(cuda), ci.to(cuda)
    cp, ri, pm = kernels.csr2csc(rp_d, ci_d)
    for h, f in ((8, 32), (4, 8)):
        g = torch.Generator().manual_seed(h)
        ar, ac = torch.randn(n, h, generator=g).to(cuda), torch.randn(n, h, generator=g).to(cuda)
        x, go = torch.randn(n, h, f, generator=g).to(cuda), torch.randn(n, h, f, generator=g).to(cuda)
        hot_c, hot_r = kernels.hot_rows(cp, 200), kernels.hot_rows(rp_d, 200)
        assert int(hot_c.ne(0).sum()) > 0 and int(hot_r.ne(0).sum()) > 0
        base = kernels.gat_forward(ar, ac, rp_d, ci_d, 0.2, x, neg=True)
        hinted = kernels.gat_forward(ar, ac, rp_d, ci_d, 0.2, x, neg=True, hot=hot_c)
        for a, b, name in zip(base, hinted, ("out", "edge_max", "edge_sum", "out_neg", "a_neg")):
            assert_equal(b, a, f"forward {name} with hot rows ({h}x{f})")
        pack, _, _ = kernels.gat_rowstat_full(ar, base[1], base[2], base[0], go, 0.2, out_neg=base[3], a_neg=base[4])
        b0 = kernels.gat_backward_cols(None, cp, ri, None, pack, None, x, ac, go, 0.2, row_grad=False)
        b1 = kernels.gat_backward_cols(None, cp, ri, None, pack, None, x, ac, go, 0.2, row_grad=False, hot=hot_r)
        assert_equal(b1[0], b0[0], f"grad_feat with hot rows ({h}x{f})")
        assert_equal(b1[2], b0[2], f"grad_attn_col with hot rows ({h}x{f})")
    with pytest.raises(RuntimeError, match="hot-row set"):
        kernels.gat_forward(ar, ac, rp_d, ci_d, 0.2, x, neg=True, hot=hot_c[:3])
    # operator path: budget 0.25 MB against a 3.1 MB feature tensor -> a set is used; results unchanged
    from dgnn_b200.operators import GATConvFuse
    h, f = 8, 32
    g = torch.Generator().manual_seed(3)
    ar, ac = torch.randn(n, h, generator=g).to(cuda), torch.randn(n, h, generator=g).to(cuda)
    x = torch.randn(n, h, f, generator=g).to(cuda)
    outs = []
    for mb in ("0", "0.25"):
        monkeypatch.setenv("DGNN_L2_HOT_MB", mb)
        assert (kernels.l2_hot(cp, 4 * h * (f + 1)) is None) == (mb == "0")
        xr = x.clone().requires_grad_(True)
        y = GATConvFuse(ar, ac, rp_d, ci_d, cp, ri, pm, 0.2, xr, 0.0)
        y.square().sum().backward()
        outs.append((y.detach(), xr.grad))
    assert_equal(outs[1][0], outs[0][0], "operator output with hot rows")
    assert_equal(outs[1][1], outs[0][1], "operator grad_feat with hot rows")
