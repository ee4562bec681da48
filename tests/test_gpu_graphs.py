"""A whole GATConv training step (projection, logits, fused aggregation, backward) captured in a CUDA
graph and replayed: on small graphs the step is launch-bound, and every entry point of the library is
stream-ordered (workspaces come from torch's allocator, counters are reset with asynchronous memsets),
so the capture needs nothing special."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("in_feats,heads,width", [(100, 4, 64), (64, 8, 32), (33, 2, 16)])
def test_layer_step_replays_from_a_cuda_graph(in_feats, heads, width):
    from dgnn_b200 import kernels, synth
    from dgnn_b200.layers import GATConv
    dev = torch.device("cuda")
    rp, ci = synth.powerlaw_graph()
    n = rp.numel() - 1
    rp, ci = rp.to(dev), ci.to(dev)
    cp, ri, pm = kernels.csr2csc(rp, ci)
    torch.manual_seed(3)
    layer = GATConv(in_feats, width, heads).to(dev).train()
    gen = torch.Generator(device=dev).manual_seed(11)
    x_static = torch.randn(n, in_feats, device=dev, generator=gen)
    cot = torch.randn(n, heads, width, device=dev, generator=gen)

    def step(x):
        out = layer(rp, ci, cp, ri, pm, x)
        (out * cot).sum().backward()
        return out

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            layer.zero_grad(set_to_none=True)
            step(x_static)
    torch.cuda.current_stream().wait_stream(side)

    layer.zero_grad(set_to_none=True)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_static = step(x_static)
    grads_static = [p.grad for p in layer.parameters()]

    for trial in range(2):
        x_new = torch.randn(n, in_feats, device=dev, generator=gen)
        x_static.copy_(x_new)
        graph.replay()
        got_out = out_static.clone()
        got_grads = [g.clone() for g in grads_static]
        layer.zero_grad(set_to_none=True)
        ref_out = step(x_new)
        ref_grads = [p.grad for p in layer.parameters()]
        assert torch.equal(got_out, ref_out), trial
        for a, b in zip(got_grads, ref_grads):
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-6), trial
        layer.zero_grad(set_to_none=True)
