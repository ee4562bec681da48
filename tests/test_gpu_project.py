"""Tensor-core node projection (dgnn_project_forward) against an fp64 matmul, through the C ABI."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _check(m, k, n, seed):
    from dgnn_b200 import kernels
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(m, k, device=dev, generator=g) * 3.0
    w = (torch.rand(n, k, device=dev, generator=g) - 0.5) * 0.7
    out = kernels.project_forward(x, w, check_status=True)
    ref = x.double() @ w.double().t()
    bound = x.abs().double() @ w.abs().double().t()      # sum of |x||w| per output
    err = (out.double() - ref).abs()
    # 3 x tf32: ~2^-21 per product plus fp32 accumulation over k <= 128 terms
    assert bool((err <= 4e-6 * bound + 1e-30).all()), float((err / (bound + 1e-30)).max())
    return out


@pytest.mark.parametrize("m", [1, 127, 128, 129, 1000, 40000])
def test_project_rows(m):
    _check(m, 100, 256, seed=m)


@pytest.mark.parametrize("k", [4, 8, 32, 36, 64, 100, 128])
def test_project_inner(k):
    _check(777, k, 256, seed=k)


@pytest.mark.parametrize("n", [128, 256, 512])
def test_project_columns(n):
    _check(3001, 100, n, seed=n)


def test_project_matches_fp32_matmul_level():
    """The split product is as close to the exact result as the fp32 library GEMM is."""
    from dgnn_b200 import kernels
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(9)
    x = torch.randn(20000, 100, device=dev, generator=g)
    w = torch.randn(256, 100, device=dev, generator=g)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        lib32 = x @ w.t()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    ref = x.double() @ w.double().t()
    out = kernels.project_forward(x, w, check_status=True)
    e_mine = float((out.double() - ref).abs().max())
    e_lib = float((lib32.double() - ref).abs().max())
    assert e_mine <= 4.0 * e_lib + 1e-6, (e_mine, e_lib)


def test_project_rejects_unsupported_shapes():
    from dgnn_b200 import kernels
    assert not kernels.project_supported(10, 100, 100)   # n not a multiple of 128
    assert not kernels.project_supported(10, 256, 130)   # k too large
    assert not kernels.project_supported(10, 256, 6)     # k not a multiple of 4
    assert kernels.project_supported(10, 256, 100)
    with pytest.raises(RuntimeError):
        kernels.project_forward(torch.zeros(4, 6, device="cuda"), torch.zeros(256, 6, device="cuda"))


def test_project_weight_as_k_by_n():
    """W stored [K,N] as the GAT layer keeps it."""
    from dgnn_b200 import kernels
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(21)
    x = torch.randn(5000, 100, device=dev, generator=g)
    w = torch.randn(100, 256, device=dev, generator=g)
    out = kernels.project_forward(x, w, w_kn=True, check_status=True)
    ref = x.double() @ w.double()
    bound = x.abs().double() @ w.abs().double()
    assert bool(((out.double() - ref).abs() <= 4e-6 * bound).all())


def _check_wgrad(m, k, n, seed, w_kn):
    from dgnn_b200 import kernels
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(m, k, device=dev, generator=g)
    go = torch.randn(m, n, device=dev, generator=g) * 0.5
    gw = kernels.project_wgrad(x, go, w_kn=w_kn, check_status=True)
    ref = x.double().t() @ go.double()                      # [K,N]
    bound = x.abs().double().t() @ go.abs().double()
    if not w_kn:
        ref, bound = ref.t(), bound.t()
    err = (gw.double() - ref).abs()
    # split products ~2^-21 each, fp32 accumulation over m terms in the tensor core and across partials
    assert bool((err <= 2e-5 * bound + 1e-30).all()), float((err / (bound + 1e-30)).max())


@pytest.mark.parametrize("m", [1, 31, 32, 33, 1000, 4736, 100000])
def test_project_wgrad_rows(m):
    _check_wgrad(m, 100, 256, seed=m, w_kn=True)


@pytest.mark.parametrize("k,n", [(4, 128), (32, 128), (36, 256), (128, 256), (100, 512)])
def test_project_wgrad_shapes(k, n):
    _check_wgrad(5000, k, n, seed=k + n, w_kn=False)


def test_projection_function_gradients():
    """The autograd node of the layer's projection against torch.matmul in fp64."""
    from dgnn_b200.operators.projection import project
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(3000, 100, device=dev, generator=g, requires_grad=True)
    w = torch.randn(100, 256, device=dev, generator=g, requires_grad=True)
    cot = torch.randn(3000, 256, device=dev, generator=g)
    out = project(x, w)
    out.backward(cot)
    xd, wd = x.detach().double().requires_grad_(), w.detach().double().requires_grad_()
    (xd @ wd).backward(cot.double())
    assert torch.allclose(out.double(), xd @ wd, rtol=1e-5, atol=1e-4)
    assert torch.allclose(w.grad.double(), wd.grad, rtol=1e-4, atol=1e-3)
    assert torch.allclose(x.grad.double(), xd.grad, rtol=1e-4, atol=1e-3)


def test_wgrad_accuracy_does_not_degrade_with_rows():
    """The weight gradient sums over all rows; the tensor core's accumulator truncates, so the kernel drains it
    every 1024 rows.  At 1.2 M rows the result must stay at the level of the fp32 library GEMM (it was 40 x worse
    with one accumulation chain per CTA)."""
    from dgnn_b200 import kernels
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1)
    m = 1_200_000
    x = torch.randn(m, 100, device=dev, generator=g)
    go = torch.randn(m, 256, device=dev, generator=g)
    ref = x.double().t() @ go.double()
    got = kernels.project_wgrad(x, go, w_kn=True, check_status=True)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        lib32 = x.t() @ go
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    e_mine = float((got.double() - ref).abs().max() / ref.abs().max())
    e_lib = float((lib32.double() - ref).abs().max() / ref.abs().max())
    assert e_mine <= max(4.0 * e_lib, 1e-5), (e_mine, e_lib)
    kernels.project_check()


@pytest.mark.parametrize("which", ["forward", "wgrad"])
def test_a_wait_that_runs_out_sets_the_status_and_returns(which):
    """The producer warps withhold their first announcement and the wait limit is a millisecond: the consumer's
    wait runs out (and with it the waits of the roles behind it), every role leaves its loop, tensor memory is
    freed, the call returns and the status names the highest-numbered wait that gave up.  Nothing hangs and the
    next call works."""
    from dgnn_b200 import _C, kernels
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(2)
    x = torch.randn(4096, 100, device=dev, generator=g)
    w = torch.randn(100, 256, device=dev, generator=g)
    go = torch.randn(4096, 256, device=dev, generator=g)
    kernels.project_check()                                   # clean slate
    assert _C.lib().dgnn_project_set_test_knobs(2_000_000, 1) == 0
    try:
        with pytest.raises(RuntimeError, match="gave up in wait [1-9]"):
            if which == "forward":
                kernels.project_forward(x, w, w_kn=True, check_status=True)
            else:
                kernels.project_wgrad(x, go, w_kn=True, check_status=True)
        torch.cuda.synchronize()
    finally:
        assert _C.lib().dgnn_project_set_test_knobs(0, 0) == 0
    with pytest.raises(RuntimeError, match="gave up in a bounded wait"):
        kernels.project_check()                               # the sticky word remembers it ...
    kernels.project_check()                                   # ... once
    out = kernels.project_forward(x, w, w_kn=True, check_status=True)
    assert torch.allclose(out, x @ w, rtol=1e-4, atol=1e-4)
    kernels.project_check()
