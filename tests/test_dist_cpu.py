"""Host logic of the sharded GAT layer on the CPU: the partition, the halo row lists, the staged
sweeps and the autograd plumbing, with the oracle standing in for the CUDA kernels as the per-rank
compute.  World-size 2 and 3 gloo runs (the halo rows travel through all-gathers there), a single-process
emulation of all ranks (the fetch path that indexes the owners' buffers), the EdgeConv batch split, and a
rank that fails on the host."""
import datetime
import os

import pytest
import torch
import torch.distributed as dist

from dgnn_b200 import dist as gdist
from dgnn_b200 import synth
from helpers import assert_close, assert_equal, gat_inputs, run_ranks
from oracle import dgnn_oracle as orc


class OracleBackend:
    """The staged entry points of dgnn_b200.kernels restated with tensor ops (state = dict)."""
    global_mask = None      # [nnz,H] uniform randoms of the whole graph's CSR, set by the dropout test

    @staticmethod
    def gat_forward_state(n_rows, h, f, device):
        return {}

    @staticmethod
    def gat_backward_state(n_cols, h, f, device):
        return {}

    @classmethod
    def uniform_fill_edges(cls, edge_id, h, seed):
        return cls.global_mask[edge_id.long()]

    @staticmethod
    def gat_forward_staged(attn_row, attn_col_buf, row_ptr, col_ind, slope, feat_buf, state, first, last, bias=None,
                           attn_drop=0.0, edge_mask=None, neg=False, save_stats=True, stage_mask=None, stage=0, outs=None):
        # every row takes part in every stage here (the per-row stage mask only saves work on the GPU)
        state = {} if state is None else state            # a single complete sweep (first = last) carries nothing
        n, h = attn_row.shape
        rows = orc.edge_rows(row_ptr)
        cols = col_ind.long()
        leaky = orc.leaky_relu(attn_row[rows] + attn_col_buf[cols], slope)
        m_p = torch.full((n, h), orc.NEG_INIT)
        if rows.numel():
            m_p = m_p.scatter_reduce(0, rows[:, None].expand(-1, h), leaky, "amax", include_self=True)
        e = torch.exp(leaky - m_p[rows])
        keep = torch.ones_like(e) if edge_mask is None else (edge_mask > attn_drop).float() / (1.0 - attn_drop)
        en = e * (leaky < 0).float()
        z_p = torch.zeros(n, h).index_add_(0, rows, e)
        zn_p = torch.zeros(n, h).index_add_(0, rows, en)
        feat = feat_buf[cols]
        acc_p = torch.zeros((n,) + tuple(feat_buf.shape[1:])).index_add_(0, rows, (e * keep)[:, :, None] * feat)
        accn_p = torch.zeros_like(acc_p).index_add_(0, rows, (en * keep)[:, :, None] * feat)
        if first:
            state.update(m=m_p, z=z_p, zn=zn_p, acc=acc_p, accn=accn_p)
        else:
            m = torch.maximum(state["m"], m_p)
            s1, s2 = torch.exp(state["m"] - m), torch.exp(m_p - m)
            state["z"] = state["z"] * s1 + z_p * s2
            state["zn"] = state["zn"] * s1 + zn_p * s2
            state["acc"] = state["acc"] * s1[:, :, None] + acc_p * s2[:, :, None]
            state["accn"] = state["accn"] * s1[:, :, None] + accn_p * s2[:, :, None]
            state["m"] = m
        if not last:
            return None
        z = state["z"]
        inv = torch.where(z > 0, 1.0 / z.clamp(min=1e-30), torch.zeros(()))
        out = state["acc"] * inv[:, :, None]
        if bias is not None:
            out = out + bias.view(1, h, -1)
        if not neg:
            res = (out, (state["m"] if save_stats else None), (z if save_stats else None))
        else:
            res = (out, state["m"], z, state["accn"] * inv[:, :, None], state["zn"] * inv)
        if outs is not None:                              # like the kernels: results land in the caller's tensors
            for dst, src in zip(outs, res):
                if dst is not None and src is not None:
                    dst.copy_(src)
        return res

    @staticmethod
    def gat_rowstat_full(attn_row, edge_max, edge_sum, out, grad_out, slope, bias=None, out_neg=None, a_neg=None,
                         pack=None, grad_copy=None):
        o = out if bias is None else out - bias.view(1, out.shape[1], -1)
        s = (grad_out * o).sum(-1)
        pk = torch.stack([attn_row, edge_max, 1.0 / edge_sum.clamp(min=1e-30), s], dim=-1)
        if pack is not None:
            pack.copy_(pk)
        if grad_copy is not None:
            grad_copy.copy_(grad_out)
        grad_row = (1.0 - slope) * (s * a_neg - (grad_out * out_neg).sum(-1)) if out_neg is not None else None
        grad_bias = grad_out.sum(0).reshape(-1) if bias is not None else None
        return (pk if pack is None else pack), grad_row, grad_bias

    @staticmethod
    def gat_backward_cols_staged(row_ptr, col_ptr, row_ind, permute, pack_buf, in_feat, attn_col, grad_buf, slope,
                                 state, first, last, attn_drop=0.0, edge_mask=None, row_grad=True, stage_mask=None, stage=0,
                                 outs=None):
        assert not row_grad and row_ptr is None and permute is None
        cols = orc.edge_rows(col_ptr)                     # local column of every CSC entry
        rows = row_ind.long()                             # buffer row of its destination
        pk = pack_buf[rows]                               # [E,H,4]
        leaky = orc.leaky_relu(pk[..., 0] + attn_col[cols], slope)
        alpha = torch.exp(leaky - pk[..., 1]) * pk[..., 2]
        keep = torch.ones_like(alpha) if edge_mask is None else (edge_mask > attn_drop).float() / (1.0 - attn_drop)
        g = (grad_buf[rows] * in_feat[cols]).sum(-1) * keep
        d = alpha * (g - pk[..., 3])
        d = torch.where(leaky < 0, d * slope, d)
        gf = torch.zeros_like(in_feat).index_add_(0, cols, (alpha * keep)[:, :, None] * grad_buf[rows])
        gc = torch.zeros_like(attn_col).index_add_(0, cols, d)
        state = {} if state is None else state
        if first:
            state["gf"], state["gc"] = gf, gc
        else:
            state["gf"], state["gc"] = state["gf"] + gf, state["gc"] + gc
        if last and outs is not None and outs[0] is not None:
            outs[0].copy_(state["gf"]); outs[1].copy_(state["gc"])
        return None, (state["gf"] if last else None), (state["gc"] if last else None)


GRAPH = dict(n=113, avg=6, seed=22, long_rows=[(2, 150), (112, 90)])


def _reference(h, f, p=0.0, mask=None):
    rp, ci = synth.random_graph(GRAPH["n"], GRAPH["avg"], seed=GRAPH["seed"], long_rows=GRAPH["long_rows"])
    n = rp.numel() - 1
    ar, ac, x, g = gat_inputs(rp, n, h, f, seed=5)
    o_ref, emax, esum = orc.gat_forward(ar, ac, rp, ci, 0.2, x, p, mask)
    gf, gr, gc = orc.gat_backward(0.2, p, rp, ci, emax, esum, mask, x, ar, ac, g)
    return rp, ci, (ar, ac, x, g), (o_ref, gf, gr, gc)


def _check_ranks(results, ref, n):
    o_ref, gf, gr, gc = ref
    seen = []
    for rank, (ids, out, (d_ar, d_ac, d_x)) in enumerate(results):
        real = ids >= 0
        idx = ids[real]
        seen.append(idx)
        assert_close(out[real], o_ref[idx], f"rank {rank} out")
        assert_close(d_ar[real], gr[idx], f"rank {rank} grad_attn_row", atol=2e-5)
        assert_close(d_ac[real], gc[idx], f"rank {rank} grad_attn_col", atol=2e-5)
        assert_close(d_x[real], gf[idx], f"rank {rank} grad_feat")
    assert torch.equal(torch.sort(torch.cat(seen)).values, torch.arange(n))     # every node owned exactly once


def _gloo_worker(rank, world, port, h, f, stages, p, schedule="staged"):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    try:
        mask = None
        rp, ci = synth.random_graph(GRAPH["n"], GRAPH["avg"], seed=GRAPH["seed"], long_rows=GRAPH["long_rows"])
        if p > 0:
            mask = torch.rand(ci.numel(), h, generator=torch.Generator().manual_seed(77))
            OracleBackend.global_mask = mask
        ar, ac, x, g = gat_inputs(rp, rp.numel() - 1, h, f, seed=5)
        shard = gdist.build_halo_shard(rp, ci, rank, world, stages=stages, seed=3, csr2csc=orc.csr2csc, edge_ids=p > 0,
                                       schedule=schedule, fractions=(0.1, 0.5, 1.0) if schedule == "rowsets" else None)
        hc = gdist.HaloContext(shard, gdist.GatherTransport(shard), h, f, 0.2, backend=OracleBackend)
        loc = [shard.scatter_rows(t).requires_grad_() for t in (ar, ac, x)]
        out = gdist.sharded_gat(*loc, hc, attn_drop=p, seed=1)
        out.backward(shard.scatter_rows(g))
        dist.barrier()
        return shard.local_ids.clone(), out.detach(), [t.grad for t in loc]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,stages,p,schedule", [(2, 1, 0.0, "staged"), (2, 3, 0.0, "staged"), (3, 2, 0.0, "staged"),
                                                     (2, 2, 0.4, "staged"), (2, 3, 0.0, "rowsets"), (3, 3, 0.4, "rowsets")])
def test_sharded_gat_gloo_equals_single(world, stages, p, schedule):
    h, f = 2, 4
    mask = torch.rand(0)
    rp, ci, _, _ = _reference(h, f)
    if p > 0:
        mask = torch.rand(ci.numel(), h, generator=torch.Generator().manual_seed(77))
    _, _, _, ref = _reference(h, f, p, mask if p > 0 else None)
    results = run_ranks(_gloo_worker, world, (h, f, stages, p, schedule), timeout=240)
    _check_ranks(results, ref, GRAPH["n"])


@pytest.mark.parametrize("mode", ["dma", "pull"])
@pytest.mark.parametrize("world,stages", [(1, 1), (2, 2), (4, 3), (3, 1), (1, 0), (2, 0), (4, 0)])
def test_all_ranks_emulated_in_one_process(world, stages, mode):
    """LocalTransport: every rank's buffers in one registry, phases run in lockstep.  "dma": owners pack what each
    peer needs into send buffers and the peers copy their contiguous ranges (the send plan); "pull": the halo rows
    are picked out of the owners' buffers by their codes."""
    h, f = 2, 4
    rp, ci, (ar, ac, x, g), ref = _reference(h, f)
    kw = dict(schedule="rowsets", fractions=(0.05, 0.3, 0.3, 1.0)) if stages == 0 else dict(stages=stages)   # 0: row sets (one empty)
    shards = [gdist.build_halo_shard(rp, ci, r, world, seed=9, csr2csc=orc.csr2csc, **kw) for r in range(world)]
    ctxs = [gdist.HaloContext(s, t, h, f, 0.2, backend=OracleBackend)
            for s, t in zip(shards, gdist.LocalTransport.for_all(shards, mode))]
    loc = [[s.scatter_rows(t) for t in (ar, ac, x, g)] for s in shards]
    rows = [gdist.halo_forward_prepare(c, h=l[2], attn_row=l[0], attn_col=l[1]) for c, l in zip(ctxs, loc)]
    for c in ctxs:
        c.transport.publish(c.shard.fwd, [c.X, c.AC], c.tags[0:2])
    fwd = [gdist.halo_forward_sweep(c, r) for c, r in zip(ctxs, rows)]
    grow = [gdist.halo_backward_prepare(c, r, o[1], o[2], o[0], o[3], o[4], l[3])[0] for c, r, o, l in zip(ctxs, rows, fwd, loc)]
    for c in ctxs:
        c.transport.publish(c.shard.bwd, [c.G, c.PK], c.tags[2:4])
    bwd = [gdist.halo_backward_sweep(c) for c in ctxs]
    results = [(s.local_ids, o[0], (gr, b[1], b[0])) for s, o, gr, b in zip(shards, fwd, grow, bwd)]
    _check_ranks(results, ref, GRAPH["n"])


@pytest.mark.parametrize("world,stages,relabel", [(1, 1, True), (3, 1, True), (4, 3, True), (2, 2, False), (3, 0, True)])
def test_halo_shard_invariants(world, stages, relabel):
    rp, ci = synth.random_graph(200, 5, seed=4, long_rows=[(7, 300)])
    n, nnz = rp.numel() - 1, ci.numel()
    cp, ri, pm = orc.csr2csc(rp, ci)
    owned, fwd_ids, bwd_ids = [], [], []
    kw = dict(schedule="rowsets", fractions=(0.1, 0.4, 1.0)) if stages == 0 else dict(stages=stages)   # 0: row sets
    shards = [gdist.build_halo_shard(rp, ci, r, world, seed=1, csr2csc=orc.csr2csc, edge_ids=True, relabel=relabel, **kw)
              for r in range(world)]
    for s in shards:
        owned.append(s.local_ids[s.local_ids >= 0])
        for side, glob_ptr, glob_ind in ((s.fwd, rp.long(), ci.long()), (s.bwd, cp, ri)):
            assert side.chunk_off[0] == 0 and side.chunk_off[-1] == side.n_halo and len(side.chunk_off) == s.chunks + 1
            owner, loc = gdist._decode(side.codes)
            assert bool((owner != s.rank).all()) and bool((loc < s.blk).all()) and bool((owner < world).all())
            # original id of every buffer row: own rows, then the halo rows named by their codes
            halo_orig = torch.stack([shards[int(o)].local_ids[int(l)] for o, l in zip(owner, loc)]) if side.n_halo else torch.zeros(0, dtype=torch.long)
            assert bool((halo_orig >= 0).all())
            assert halo_orig.unique().numel() == side.n_halo            # every halo row fetched once
            buf_orig = torch.cat([s.local_ids, halo_orig])
            for p in range(s.stages):
                ptr, ind, eid = side.ptr[p].long(), side.ind[p].long(), side.edge_id[p].long()
                assert ptr[0] == 0 and ptr[-1] == ind.numel() == eid.numel()
                seg = orc.edge_rows(ptr)
                if s.schedule == "rowsets":                            # stage p = all entries of segments bounds[p]:bounds[p+1]
                    assert ptr.numel() - 1 == side.bounds[p + 1] - side.bounds[p] and side.stage_mask is None
                    assert bool((ind < s.blk + side.chunk_off[p + 1]).all())      # only own rows and chunks 0..p
                    new = ind[ind >= s.blk + side.chunk_off[p]]                   # chunk p: first referenced by this set
                    assert new.unique().numel() == side.chunk_off[p + 1] - side.chunk_off[p]
                    seg = seg + side.bounds[p]
                else:
                    assert torch.equal(((side.stage_mask.long() >> p) & 1).bool(), (ptr[1:] - ptr[:-1]) > 0)   # bit p = has entries in stage p
                far = buf_orig[ind]                                    # original id of the far end of every entry
                near = s.local_ids[seg]
                if side is s.fwd:
                    assert torch.equal(far, ci.long()[eid]) and torch.equal(near, orc.edge_rows(rp)[eid])
                    assert bool(((ind < s.blk) == (p == 0)).all()) or s.stages == 1 or s.schedule == "rowsets"
                    fwd_ids.append(eid)
                else:
                    assert torch.equal(far, orc.edge_rows(rp)[eid]) and torch.equal(near, ci.long()[eid])
                    bwd_ids.append(eid)
                if s.schedule == "staged" and s.stages > 1 and p > 0:  # stage p holds exactly halo chunk p-1
                    lo, hi = s.blk + side.chunk_off[p - 1], s.blk + side.chunk_off[p]
                    assert bool(((ind >= lo) & (ind < hi)).all())
    assert torch.equal(torch.sort(torch.cat(owned)).values, torch.arange(n))
    assert torch.equal(torch.sort(torch.cat(fwd_ids)).values, torch.arange(nnz))   # every edge in exactly one forward piece
    assert torch.equal(torch.sort(torch.cat(bwd_ids)).values, torch.arange(nnz))   # ... and one backward piece


def test_split_clouds_by_batch():
    """EdgeConv on the per-rank cloud subsets, concatenated in rank order, equals EdgeConv on the whole batch."""
    b, p, k, f = 5, 64, 6, 8
    pts = synth.unit_sphere_clouds(b, p, seed=3)
    g = torch.Generator().manual_seed(0)
    h_src, h_dst = torch.randn(b * p, f, generator=g), torch.randn(b * p, f, generator=g)
    src_all = synth.knn_src_ind(pts, k)
    out_all, idx_all = orc.edgeconv_forward(k, src_all, h_src, h_dst)
    for world in (2, 3):
        outs, idxs, covered = [], [], 0
        for rank in range(world):
            loc, src, (b0, b1) = gdist.split_clouds(pts, k, rank, world, knn=synth.knn_src_ind)
            assert loc.shape[0] == b1 - b0 and src.numel() == (b1 - b0) * p * k
            assert src.numel() == 0 or (int(src.min()) >= 0 and int(src.max()) < (b1 - b0) * p)   # ids local to the rank
            o, i = orc.edgeconv_forward(k, src, h_src[b0 * p:b1 * p], h_dst[b0 * p:b1 * p]) if b1 > b0 else (torch.zeros(0, f), torch.zeros(0, f, dtype=torch.long))
            outs.append(o)
            idxs.append(i + b0 * p)
            covered += b1 - b0
        assert covered == b
        assert_equal(torch.cat(outs), out_all, f"world {world}: EdgeConv out")
        assert_equal(torch.cat(idxs), idx_all, f"world {world}: EdgeConv arg-max ids")


def _failing_worker(rank, world, port):
    """Rank 1 fails on the host before the halo exchange; rank 0 must get an error from its collective within
    the process-group timeout instead of waiting for ever."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    rp, ci = synth.random_graph(40, 4, seed=1)
    shard = gdist.build_halo_shard(rp, ci, rank, world, stages=2, seed=3, csr2csc=orc.csr2csc)
    hc = gdist.HaloContext(shard, gdist.GatherTransport(shard), 2, 4, 0.2, backend=OracleBackend)
    if rank == 1:
        raise RuntimeError("injected host-side failure on rank 1")
    ar, ac, x, _ = gat_inputs(rp, 40, 2, 4, seed=5)
    gdist.sharded_gat(*[shard.scatter_rows(t) for t in (ar, ac, x)], hc)
    return "finished"


def test_rank_failure_ends_the_peers_collective():
    results = run_ranks(_failing_worker, 2, (), timeout=120, expect_errors=True)
    assert results[1][0] == "error" and "injected host-side failure" in results[1][1]
    assert results[0][0] == "error", "rank 0 should have failed in its collective, not finished"
