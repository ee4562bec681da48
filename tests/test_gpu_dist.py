"""The sharded GAT layer on GPUs.

One GPU: all ranks emulated in one process (LocalTransport) -- the real kernels, the real halo fetch kernel
reading the owners' buffers, the staged sweeps -- against the single-GPU operator.
Two or more GPUs: one process per GPU over NCCL with the halo rows fetched from symmetric memory, the
ShardedGATConv module against the single-GPU GATConv module.  The host logic is covered on the CPU by
test_dist_cpu.py."""
import datetime
import os

import pytest
import torch

from helpers import assert_close, assert_equal, gat_inputs, run_ranks

pytestmark = pytest.mark.gpu


def _single_gpu(rp, ci, ar, ac, x, g, p=0.0, seed=0):
    from dgnn_b200 import kernels
    cp, ri, pm = kernels.csr2csc(rp, ci)
    h = x.shape[1]
    mask = kernels.uniform_fill((ci.numel(), h), seed, 0, x.device) if p > 0 else None
    out, emax, esum, out_neg, a_neg = kernels.gat_forward(ar, ac, rp, ci, 0.2, x, p, mask, neg=True)
    pack, gr, _ = kernels.gat_rowstat_full(ar, emax, esum, out, g, 0.2, out_neg=out_neg, a_neg=a_neg)
    gf, _, gc = kernels.gat_backward_cols(None, cp, ri, pm if p > 0 else None, pack, mask, x, ac, g, 0.2, p, row_grad=False)
    return out, gf, gr, gc


@pytest.mark.parametrize("world,stages,p,mode", [(1, 1, 0.0, "dma"), (2, 1, 0.0, "dma"), (2, 2, 0.0, "pull"), (4, 3, 0.0, "dma"),
                                                 (3, 4, 0.3, "dma"), (3, 4, 0.3, "pull"), (8, 3, 0.0, "dma"), (8, 3, 0.0, "pull"),
                                                 (2, 0, 0.0, "dma"), (4, 0, 0.3, "dma"), (8, 0, 0.0, "pull")])
def test_emulated_ranks_equal_single_gpu(cuda, world, stages, p, mode):
    """stages = 0: the row-set schedule (every sweep finishes a range of rows; four ranges)."""
    from dgnn_b200 import dist as gdist
    from dgnn_b200 import kernels, synth
    n, e, h, f = 20_000, 600_000, 8, 32
    rp, ci = synth.rmat_graph(n, e, seed=9, device=cuda, ptr_dtype=torch.int64)
    _, _, x, g = [t.to(cuda) for t in gat_inputs(rp, n, h, f, 17)]
    gen = torch.Generator().manual_seed(3)
    al, ar_ = torch.randn(1, h, f, generator=gen).to(cuda), torch.randn(1, h, f, generator=gen).to(cuda)
    ar, ac = kernels.gat_logits_forward(x, al, ar_)        # the layer form: logits from the features
    out, gf, gr, gc = _single_gpu(rp, ci, ar, ac, x, g, p, seed=123)
    kw = dict(schedule="rowsets") if stages == 0 else dict(stages=stages)
    shards = [gdist.build_halo_shard(rp, ci, r, world, seed=5, edge_ids=p > 0, **kw) for r in range(world)]
    ctxs = [gdist.HaloContext(s, t, h, f, 0.2) for s, t in zip(shards, gdist.LocalTransport.for_all(shards, mode, pull_ctas=8))]
    loc = [[s.scatter_rows(t) for t in (x, g)] for s in shards]
    # phases in lockstep: own rows (the logits kernel and the row-statistics kernel also write the send buffers), then the sweeps
    rows = [gdist.halo_forward_prepare(c, h=l[0], attn_l=al, attn_r=ar_) for c, l in zip(ctxs, loc)]
    for c in ctxs:
        assert c.packed_fwd == (mode == "dma" and world > 1 and c.transport.plans[0].pack_idx.numel() > 0)
        c.transport.publish(c.shard.fwd, [c.X, c.AC], c.tags[0:2], packed=c.packed_fwd)
    fwd = [gdist.halo_forward_sweep(c, r, None, p, 123) for c, r in zip(ctxs, rows)]
    grow = [gdist.halo_backward_prepare(c, r, o[1], o[2], o[0], o[3], o[4], l[1])[0] for c, r, o, l in zip(ctxs, rows, fwd, loc)]
    for c in ctxs:
        c.transport.publish(c.shard.bwd, [c.G, c.PK], c.tags[2:4], packed=c.packed_bwd)
    bwd = [gdist.halo_backward_sweep(c, p, 123) for c in ctxs]
    torch.cuda.synchronize()
    seen = []
    for s, c, o, grw, b in zip(shards, ctxs, fwd, grow, bwd):
        c.transport.check()
        real = s.local_ids >= 0
        idx = s.local_ids[real]
        seen.append(idx)
        # Both sides are fp32 sums of the same terms in a different grouping (stages, chunk boundaries of long
        # rows); hub columns add ~10^4 terms of either sign, so an entry's rounding error scales with the sum of
        # the magnitudes, not with the entry: the absolute band is 1e-5 of the tensor's largest entry (at least 2e-5)
        band = lambda t: max(2e-5, 1e-5 * float(t.abs().max()))
        assert_close(o[0][real], out[idx], f"rank {s.rank} out")
        assert_close(b[0][real], gf[idx], f"rank {s.rank} grad_feat", atol=band(gf))
        assert_close(grw[real], gr[idx], f"rank {s.rank} grad_attn_row", atol=band(gr))
        assert_close(b[1][real], gc[idx], f"rank {s.rank} grad_attn_col", atol=band(gc))
        if mode == "dma" and world > 1 and c.transport.plans[0].pack_idx.numel():
            # what the producing kernels wrote into the send buffers is what a separate packing pass writes
            plan = c.transport.plans[0]
            k = plan.pack_idx.numel()
            assert_equal(c.transport.send[c.tags[0]][:k], c.X[:s.blk][plan.pack_idx.long()], "fused packing of the features")
            assert_equal(c.transport.send[c.tags[1]][:k], c.AC[:s.blk][plan.pack_idx.long()], "fused packing of attn_col")
            planb = c.transport.plans[1]
            kb = planb.pack_idx.numel()
            assert_equal(c.transport.send[c.tags[2]][:kb], c.G[:s.blk][planb.pack_idx.long()], "fused packing of grad_out")
            assert_equal(c.transport.send[c.tags[3]][:kb], c.PK[:s.blk][planb.pack_idx.long()], "fused packing of pack")
    assert torch.equal(torch.sort(torch.cat(seen)).values, torch.arange(n, device=cuda))


def test_halo_pull_and_edge_randoms(cuda):
    from dgnn_b200 import kernels
    g = torch.Generator().manual_seed(0)
    owners_a = [torch.randn(1000, 8, 32, generator=g).to(cuda) for _ in range(3)]
    owners_b = [torch.randn(1000, 8, generator=g).to(cuda) for _ in range(3)]
    rank = torch.randint(0, 3, (5000,), generator=g)
    idx = torch.randint(0, 1000, (5000,), generator=g)
    codes = ((rank << 27) | idx).to(torch.int32).to(cuda)
    dst_a = torch.zeros(5000, 8, 32, device=cuda)
    dst_b = torch.zeros(5000, 8, device=cuda)
    status = torch.zeros(1, dtype=torch.int32, device=cuda)
    kernels.halo_pull(codes, owners_a, dst_a, owners_b, dst_b, max_ctas=4, status=status)
    assert_equal(dst_a, torch.stack(owners_a)[rank.to(cuda), idx.to(cuda)], "halo rows a")
    assert_equal(dst_b, torch.stack(owners_b)[rank.to(cuda), idx.to(cuda)], "halo rows b")
    assert int(status.item()) == 0
    # a code outside the owners' blocks is skipped and reported, never dereferenced
    bad = torch.tensor([(1 << 27) | 5, (7 << 27) | 1, (2 << 27) | 1000], dtype=torch.int32, device=cuda)
    dst = torch.full((3, 8, 32), -1.0, device=cuda)
    kernels.halo_pull(bad, owners_a, dst, max_ctas=1, status=status)
    assert_equal(dst[0], owners_a[1][5], "valid row")
    assert bool((dst[1:] == -1.0).all()) and int(status.item()) == 1
    # the per-edge randoms are rows of the dense fill
    full = kernels.uniform_fill((4000, 8), 99, 0, cuda)
    pick = torch.randint(0, 4000, (700,), generator=g).to(torch.int32).to(cuda)
    assert_equal(kernels.uniform_fill_edges(pick, 8, 99), full[pick.long()], "edge randoms")
    for hh in (1, 3):
        full = kernels.uniform_fill((4000, hh), 5, 0, cuda)
        assert_equal(kernels.uniform_fill_edges(pick, hh, 5), full[pick.long()], f"edge randoms h={hh}")


def _layer_worker(rank, world, port, n, e, in_feats, heads, width, stages):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    torch.backends.cuda.matmul.allow_tf32 = False
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=120))
    try:
        from dgnn_b200 import dist as gdist
        from dgnn_b200 import kernels, synth
        from dgnn_b200.layers import GATConv
        rp, ci = synth.rmat_graph(n, e, seed=9, device=dev, ptr_dtype=torch.int64)
        cp, ri, pm = kernels.csr2csc(rp, ci)
        g = torch.Generator(device=dev).manual_seed(3)
        feat_in = torch.randn(n, in_feats, device=dev, generator=g)
        feat_wide = torch.randn(n, heads * width, device=dev, generator=g)
        cot = torch.randn(n, heads, width, device=dev, generator=g)
        report = {}
        for name, kw in (("plain", {}), ("residual_relu", dict(residual=True, activation=torch.relu)),
                         ("attn_drop", dict(attn_drop=0.3)), ("rowsets", {}), ("rowsets_attn_drop", dict(attn_drop=0.3))):
            torch.manual_seed(11)
            # the residual branch of the reference is applied to the projected features: identity when in_feats == H*F
            feat = feat_wide if "residual" in kw else feat_in
            in_feats = feat.shape[1]
            ref = GATConv(in_feats, width, heads, **kw).to(dev).train()
            with torch.no_grad():
                ref.bias.uniform_(-1.0, 1.0)
            sched = dict(schedule="rowsets") if name.startswith("rowsets") else dict(stages=stages)
            shard = gdist.build_halo_shard(rp, ci, rank, world, seed=5, edge_ids="attn_drop" in kw, **sched)
            layer = gdist.ShardedGATConv(in_feats, width, heads, shard, seed=42, **kw).to(dev).train()
            layer.load_state_dict(ref.state_dict())
            report[name + "_transport"] = type(layer.transport).__name__
            real = shard.local_ids >= 0
            ids = shard.local_ids[real]
            out = layer(shard.scatter_rows(feat))
            out.backward(shard.scatter_rows(cot))
            layer.allreduce_grads()
            if "attn_drop" in kw:
                # the single-GPU layer draws its mask from torch's generator; redo it with the sharded layer's seed
                from dgnn_b200.operators import fused_gatconv as op
                seed = layer.seed * 1000003 + layer.step
                orig = op.fused_gat.make_edge_mask
                op.fused_gat.make_edge_mask = lambda nnz, h_, p_, d_: kernels.uniform_fill((nnz, h_), seed, 0, d_)
                try:
                    ref_out = ref(rp, ci, cp, ri, pm, feat)
                    ref_out.backward(cot)
                finally:
                    op.fused_gat.make_edge_mask = orig
            else:
                ref_out = ref(rp, ci, cp, ri, pm, feat)
                ref_out.backward(cot)
            torch.cuda.synchronize()
            if hasattr(layer.transport, "check"):
                layer.transport.check()
            err = lambda a, b: float(((a - b).abs() / (1e-5 + 1e-4 * b.abs())).max())
            rel = lambda a, b: float((a - b).abs().max() / (b.abs().max() + 1e-12))
            ref_params = dict(ref.named_parameters())
            report[name] = dict(out=err(out.detach()[real], ref_out.detach()[ids]),
                                missing=[k for k, p in layer.named_parameters() if (p.grad is None) != (ref_params[k].grad is None)],
                                grads={k: rel(p.grad, ref_params[k].grad) for k, p in layer.named_parameters()
                                       if ref_params[k].grad is not None and p.grad is not None})
            # evaluation path: no statistics, no autograd
            layer.eval(); ref.eval()
            with torch.no_grad():
                report[name]["eval"] = err(layer(shard.scatter_rows(feat))[real], ref(rp, ci, cp, ri, pm, feat)[ids])
            del layer
        dist.barrier()
        return report
    finally:
        dist.destroy_process_group()


def test_sharded_layer_equals_single_gpu_layer(cuda):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    reports = run_ranks(_layer_worker, world, (50_000, 2_000_000, 100, 8, 32, 3), timeout=600)
    for rank, rep in enumerate(reports):
        for name in ("plain", "residual_relu", "attn_drop", "rowsets", "rowsets_attn_drop"):
            assert rep[name + "_transport"] == "SymmetricTransport", (rank, rep[name + "_transport"])
            r = rep[name]
            # outputs to 1e-4 relative / 1e-5 absolute; parameter gradients (sums over 50 k rows) within 1e-4 of their largest entry
            assert not r["missing"], (rank, name, r["missing"])
            assert r["out"] <= 1.0 and r["eval"] <= 1.0, (rank, name, r)
            assert all(v <= 1e-4 for v in r["grads"].values()), (rank, name, r)
