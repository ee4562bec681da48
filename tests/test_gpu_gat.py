"""GPU parity of the fused GAT kernels against the CPU oracle (through the C ABI)."""
import pytest
import torch

from dgnn_b200 import kernels, synth
from dgnn_b200.ext import fused_gatconv
from dgnn_b200.operators import GATConvFuse, GATConvFuse_inference
from helpers import assert_close, assert_equal, gat_inputs, scipy_csc
from oracle import dgnn_oracle as orc

pytestmark = pytest.mark.gpu

SEG = 1024  # long-row split threshold of the library (dgnn_seg_chunk)


def _case(n, avg, seed, long_rows=(), ptr64=False):
    import numpy as np
    rp, ci = synth.random_graph(n, avg, seed, long_rows=long_rows, ptr_dtype=np.int64 if ptr64 else np.int32)
    return rp, ci


GRAPHS = {
    "tiny": dict(n=40, avg=3, seed=1, long_rows=[(0, 1), (5, 33), (9, 65)]),
    "medium": dict(n=700, avg=9, seed=2, long_rows=[(3, 100), (400, 257)]),
    "long_rows": dict(n=900, avg=6, seed=3, long_rows=[(7, SEG + 1), (8, 3 * SEG + 17), (500, 2 * SEG), (899, SEG + 300)]),
}
SHAPES = [(1, 4), (1, 64), (3, 16), (4, 64), (8, 32), (2, 256), (16, 64), (3, 5), (2, 12), (1, 1), (4, 33)]


def _fwd_bwd_check(cuda, rp, ci, h, f, seed, slope=0.2, p=0.0):
    n = rp.numel() - 1
    ar, ac, x, g = gat_inputs(rp, n, h, f, seed)
    mask = None
    if p > 0:
        mask = torch.rand(ci.numel(), h, generator=torch.Generator().manual_seed(seed + 1))
    o_ref, m_ref, z_ref = orc.gat_forward(ar, ac, rp, ci, slope, x, p, mask)
    gf_ref, gr_ref, gc_ref = orc.gat_backward(slope, p, rp, ci, m_ref, z_ref, mask, x, ar, ac, g)
    d = lambda t: None if t is None else t.to(cuda)
    out, emax, esum = kernels.gat_forward(d(ar), d(ac), d(rp), d(ci), slope, d(x), p, d(mask))
    assert_close(out, o_ref, "out")
    assert_equal(emax, m_ref, "edge_max")          # a max is exact
    assert_close(esum, z_ref, "edge_sum")
    cp, ri, pm = scipy_csc(rp, ci)
    gf, gr, gc = kernels.gat_backward(slope, p, d(rp), d(cp.to(rp.dtype)), d(ri.int()), d(pm.int()), emax, esum,
                                      d(mask), d(x), out, d(ar), d(ac), d(g))
    assert_close(gf, gf_ref, "grad_feat")
    assert_close(gr, gr_ref, "grad_attn_row", atol=2e-5)
    assert_close(gc, gc_ref, "grad_attn_col", atol=2e-5)
    # inference path: same output, no statistics
    out2, a, b = kernels.gat_forward(d(ar), d(ac), d(rp), d(ci), slope, d(x), p, d(mask), save_stats=False)
    assert a is None and b is None
    assert_equal(out2, out, "inference out")
    if not kernels.gat_fast_shape(h, f):
        return
    # negative-side outputs and the row gradient derived from them (no per-edge array, no permutation)
    on_ref, an_ref = orc.gat_forward_negative_side(ar, ac, rp, ci, slope, x, p, mask)
    out3, emax3, esum3, out_neg, a_neg = kernels.gat_forward(d(ar), d(ac), d(rp), d(ci), slope, d(x), p, d(mask), neg=True)
    assert_equal(out3, out, "out with negative-side outputs")
    assert_equal(emax3, emax, "edge_max with negative-side outputs")
    assert_equal(esum3, esum, "edge_sum with negative-side outputs")
    assert_close(out_neg, on_ref, "out_neg")
    assert_close(a_neg, an_ref, "a_neg")
    pack, gr2, _ = kernels.gat_rowstat_full(d(ar), emax, esum, out, d(g), slope, out_neg=out_neg, a_neg=a_neg)
    gf2, none_row, gc2 = kernels.gat_backward_cols(None, d(cp.to(rp.dtype)), d(ri.int()), d(pm.int()) if p > 0 else None,
                                                   pack, d(mask), d(x), d(ac), d(g), slope, p, row_grad=False)
    assert none_row is None
    assert_equal(gf2, gf, "grad_feat without the per-edge array")
    assert_equal(gc2, gc, "grad_attn_col without the per-edge array")
    assert_close(gr2, gr_ref, "grad_attn_row from the negative-side outputs", atol=2e-5)


@pytest.mark.parametrize("h,f", SHAPES)
@pytest.mark.parametrize("graph", ["tiny", "medium"])
def test_gat_parity_shapes(cuda, graph, h, f):
    rp, ci = _case(**GRAPHS[graph])
    _fwd_bwd_check(cuda, rp, ci, h, f, seed=11)


@pytest.mark.parametrize("h,f", [(8, 32), (4, 64), (1, 16), (3, 7), (16, 64)])
@pytest.mark.parametrize("ptr64", [False, True])
def test_gat_parity_long_rows(cuda, h, f, ptr64):
    rp, ci = _case(ptr64=ptr64, **GRAPHS["long_rows"])
    _fwd_bwd_check(cuda, rp, ci, h, f, seed=12)


@pytest.mark.parametrize("h,f", [(4, 64), (3, 5)])
@pytest.mark.parametrize("graph", ["medium", "long_rows"])
def test_gat_parity_dropout_mask(cuda, graph, h, f):
    rp, ci = _case(**GRAPHS[graph])
    _fwd_bwd_check(cuda, rp, ci, h, f, seed=13, p=0.4)


def test_gat_degenerate_graphs(cuda):
    # no edges at all, and a graph whose rows are all empty but one
    for rp, ci in [(torch.zeros(6, dtype=torch.int32), torch.zeros(0, dtype=torch.int32)),
                   (torch.tensor([0, 0, 0, 3, 3], dtype=torch.int32), torch.tensor([1, 1, 3], dtype=torch.int32))]:
        _fwd_bwd_check(cuda, rp, ci, 2, 8, seed=3)


def test_gat_negative_and_extreme_scores(cuda):
    rp, ci = _case(**GRAPHS["medium"])
    n = rp.numel() - 1
    ar, ac, x, g = gat_inputs(rp, n, 4, 16, 21, scale=30.0)   # softmax saturates: exp arguments down to -100s
    o_ref, m_ref, z_ref = orc.gat_forward(ar, ac, rp, ci, 0.2, x)
    out, emax, esum = kernels.gat_forward(ar.to(cuda), ac.to(cuda), rp.to(cuda), ci.to(cuda), 0.2, x.to(cuda))
    assert_close(out, o_ref, "out"); assert_equal(emax, m_ref, "edge_max"); assert_close(esum, z_ref, "edge_sum")


def test_c1_config_layer_parity(cuda):
    """Config 1: 2708 nodes, 10556 directed edges + self-loops, 1433 -> 4 heads x 64, through the layer API."""
    from dgnn_b200.layers import GATConv
    rp, ci = synth.powerlaw_graph()
    n, nnz = rp.numel() - 1, ci.numel()
    assert n == 2708 and nnz == 10556 + 2708
    g = torch.Generator().manual_seed(1)
    feat = (torch.rand(n, 1433, generator=g) < 0.013).float()
    layer = GATConv(1433, 64, 4)
    with torch.no_grad():
        layer.W.copy_(synth.xavier_uniform((1433, 256), 1433, 256, g))
        layer.attn_l.copy_(synth.xavier_uniform((1, 4, 64), 64, 64, g))
        layer.attn_r.copy_(synth.xavier_uniform((1, 4, 64), 64, 64, g))
    cot = torch.randn(n, 4, 64, generator=g)
    # CPU oracle of the whole layer, autograd backward
    W, al, ar_ = [p.detach().clone().requires_grad_() for p in (layer.W, layer.attn_l, layer.attn_r)]
    ref = orc.gat_layer_forward(rp, ci, feat, W, al, ar_, 0.2, 4, 64)
    (ref * cot).sum().backward()
    cp, ri, pm = scipy_csc(rp, ci)
    layer = layer.to(cuda).train()
    out = layer(rp.to(cuda), ci.to(cuda), cp.int().to(cuda), ri.int().to(cuda), pm.int().to(cuda), feat.to(cuda))
    (out * cot.to(cuda)).sum().backward()
    assert_close(out, ref, "layer out")
    assert_close(layer.W.grad, W.grad, "dW", atol=5e-5)
    assert_close(layer.attn_l.grad, al.grad, "d attn_l", atol=5e-5)
    assert_close(layer.attn_r.grad, ar_.grad, "d attn_r", atol=5e-5)
    layer.eval()
    with torch.no_grad():
        out_eval = layer(rp.to(cuda), ci.to(cuda), cp.int().to(cuda), ri.int().to(cuda), pm.int().to(cuda), feat.to(cuda))
    assert_close(out_eval, ref, "eval out")


def test_ext_module_surface(cuda):
    """fused_gatconv.* keeps the reference's argument lists and return lists."""
    rp, ci = _case(**GRAPHS["medium"])
    n, h, f = rp.numel() - 1, 4, 32
    ar, ac, x, g = [t.to(cuda) for t in gat_inputs(rp, n, h, f, 2)]
    cp, ri, pm = [t.int().to(cuda) for t in scipy_csc(rp, ci)]
    rp, ci = rp.to(cuda), ci.to(cuda)
    out, emax, esum, mask = fused_gatconv.gat_forward(ar, ac, rp, ci, 0.2, x, 0.0)
    assert mask.shape == (ci.numel(), h)
    gf, gr, gc = fused_gatconv.gat_backward(0.2, 0.0, rp, ci, cp, ri, pm, emax, esum, mask, x, ar, ac, g)  # no out_feat given
    gf2, gr2, gc2 = fused_gatconv.gat_backward(0.2, 0.0, rp, ci, cp, ri, pm, emax, esum, mask, x, ar, ac, g, out)
    assert_equal(gf, gf2, "grad_feat"); assert_equal(gr, gr2, "grad_row"); assert_equal(gc, gc2, "grad_col")
    assert_equal(fused_gatconv.gat_inference(ar, ac, rp, ci, 0.2, x), out, "inference")
    tb = fused_gatconv.gat_forward_tb(ar, ac, rp, ci, 0.2, x, None)
    assert len(tb) == 3 and torch.equal(tb[0], out)
    # dropout through the operator: statistical check of the keep rate and scaling
    torch.manual_seed(0)
    out_d, _, _, mask_d = fused_gatconv.gat_forward(ar, ac, rp, ci, 0.2, x, 0.5)
    keep = (mask_d > 0.5).float().mean().item()
    assert 0.45 < keep < 0.55
    o_ref, _, _ = orc.gat_forward(ar.cpu(), ac.cpu(), rp.cpu(), ci.cpu(), 0.2, x.cpu(), 0.5, mask_d.cpu())
    assert_close(out_d, o_ref, "dropout forward with the drawn mask")


def test_deterministic_repeat(cuda):
    rp, ci = _case(**GRAPHS["long_rows"])
    n, h, f = rp.numel() - 1, 8, 32
    ar, ac, x, g = [t.to(cuda) for t in gat_inputs(rp, n, h, f, 4)]
    cp, ri, pm = [t.int().to(cuda) for t in scipy_csc(rp, ci)]
    rp, ci = rp.to(cuda), ci.to(cuda)
    runs = []
    for _ in range(2):
        out, emax, esum = kernels.gat_forward(ar, ac, rp, ci, 0.2, x)
        runs.append((out,) + kernels.gat_backward(0.2, 0.0, rp, cp, ri, pm, emax, esum, None, x, out, ar, ac, g))
    for a, b in zip(*runs):
        assert torch.equal(a, b)   # no float atomics anywhere: bit-identical


@pytest.mark.parametrize("h,f", [(8, 32), (4, 64), (1, 16), (3, 16), (16, 64), (2, 4)])
def test_logits_kernels_match_tensor_ops(cuda, h, f):
    g = torch.Generator().manual_seed(h * 100 + f)
    n = 3001
    x = torch.randn(n, h, f, generator=g)
    al, ar = torch.randn(1, h, f, generator=g), torch.randn(1, h, f, generator=g)
    g_row, g_col = torch.randn(n, h, generator=g), torch.randn(n, h, generator=g)
    g_feat = torch.randn(n, h, f, generator=g)
    xd, ald, ard = x.double(), al.double(), ar.double()
    a_row, a_col = kernels.gat_logits_forward(x.to(cuda), al.to(cuda), ar.to(cuda))
    assert_close(a_row, (xd * ald).sum(-1).float(), "attn_row")
    assert_close(a_col, (xd * ard).sum(-1).float(), "attn_col")
    gf = g_feat.clone().to(cuda)
    gl, gr = kernels.gat_logits_backward(x.to(cuda), al.to(cuda), ar.to(cuda), g_row.to(cuda), g_col.to(cuda), gf)
    ref_feat = g_feat.double() + g_row.double()[:, :, None] * ald + g_col.double()[:, :, None] * ard
    assert_close(gf, ref_feat.float(), "grad_feat accumulated in place")
    assert_close(gl, (g_row.double()[:, :, None] * xd).sum(0).float(), "grad attn_l", atol=1e-3)
    assert_close(gr, (g_col.double()[:, :, None] * xd).sum(0).float(), "grad attn_r", atol=1e-3)


@pytest.mark.parametrize("residual", [True, False])
def test_layer_fused_path_equals_composed_path(cuda, residual):
    """GATConv's single-node training path (GATLayerFuse) against the reference composition
    (tensor-op logits + GATConvFuse), outputs and every parameter gradient."""
    from dgnn_b200.layers import GATConv
    from dgnn_b200.operators import GATConvFuse
    rp, ci = _case(**GRAPHS["long_rows"])
    n = rp.numel() - 1
    cp, ri, pm = [t.int().to(cuda) for t in scipy_csc(rp, ci)]
    rp, ci = rp.to(cuda), ci.to(cuda)
    torch.manual_seed(0)
    # residual: in_feats == heads*out_feats gives the identity branch; without it the bias goes into the kernel epilogue
    layer = GATConv(256, 32, 8, residual=residual).to(cuda).train()
    with torch.no_grad():
        layer.bias.uniform_(-1.0, 1.0)
    feat = torch.randn(n, 256, device=cuda)
    cot = torch.randn(n, 8, 32, device=cuda)
    out = layer(rp, ci, cp, ri, pm, feat)
    out.backward(cot)
    got = {k: p.grad.clone() for k, p in layer.named_parameters()}
    layer.zero_grad()
    h = torch.matmul(feat, layer.W).view(-1, 8, 32)
    ref = GATConvFuse((h * layer.attn_l).sum(-1), (h * layer.attn_r).sum(-1), rp, ci, cp, ri, pm, 0.2, h, 0.0)
    if residual:
        ref = ref + layer.res_fc(h).view(-1, 8, 32)
    ref = ref + layer.bias.view(-1, 8, 32)
    ref.backward(cot)
    assert_close(out, ref, "layer output")
    for k, p in layer.named_parameters():
        scale = max(1.0, float(p.grad.abs().max()))
        assert_close(got[k], p.grad, f"grad {k}", atol=1e-4 * scale)


@pytest.mark.parametrize("h,f", [(8, 32), (8, 64), (16, 64)])
def test_rows_that_are_only_16_byte_aligned(cuda, h, f):
    """The same-head layout gathers with 256-bit loads and needs 32-byte aligned rows; tensors that start 16 bytes
    into an allocation take the other lane layout (128-bit accesses) and give the same results."""
    rp, ci = synth.random_graph(1500, 9, seed=3, long_rows=((5, 2100),))
    n = rp.numel() - 1
    rp_d, ci_d = rp.to(cuda), ci.to(cuda)
    cp, ri, pm = kernels.csr2csc(rp_d, ci_d)
    g = torch.Generator().manual_seed(h + f)
    ar, ac = torch.randn(n, h, generator=g).to(cuda), torch.randn(n, h, generator=g).to(cuda)
    x, go = torch.randn(n, h, f, generator=g).to(cuda), torch.randn(n, h, f, generator=g).to(cuda)

    def shifted(t):                                        # a copy that starts 16 bytes into its allocation
        buf = torch.empty(t.numel() + 4, dtype=t.dtype, device=t.device)
        v = buf[4:].view(t.shape)
        v.copy_(t)
        assert v.data_ptr() % 32 == 16
        return v

    base = kernels.gat_forward(ar, ac, rp_d, ci_d, 0.2, x, neg=True)
    off = kernels.gat_forward(ar, ac, rp_d, ci_d, 0.2, shifted(x), neg=True)
    for a, b, name in zip(base, off, ("out", "edge_max", "edge_sum", "out_neg", "a_neg")):
        assert_close(b, a, f"forward {name}, in_feat 16-byte aligned", rtol=1e-5, atol=1e-6)
    pack, _, _ = kernels.gat_rowstat_full(ar, base[1], base[2], base[0], go, 0.2, out_neg=base[3], a_neg=base[4])
    b0 = kernels.gat_backward_cols(None, cp, ri, None, pack, None, x, ac, go, 0.2, row_grad=False)
    b1 = kernels.gat_backward_cols(None, cp, ri, None, pack, None, shifted(x), ac, shifted(go), 0.2, row_grad=False)
    assert_close(b1[0], b0[0], "grad_feat, 16-byte aligned inputs", rtol=1e-4, atol=1e-5)
    assert_close(b1[2], b0[2], "grad_attn_col, 16-byte aligned inputs", rtol=1e-4, atol=2e-5)
