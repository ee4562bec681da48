"""World-size-2 (and 3) gloo runs of the sharded GAT host logic on the CPU: the
partition, the padded id space, the collectives and the autograd plumbing, with
the oracle standing in for the CUDA kernels as the per-rank compute."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dgnn_b200 import dist as gdist
from dgnn_b200 import synth
from helpers import assert_close, gat_inputs
from oracle import dgnn_oracle as orc


class OracleBackend:
    """Same three entry points as dgnn_b200.kernels, computed by the oracle."""

    @staticmethod
    def gat_forward(attn_row, attn_col, row_ptr, col_ind, slope, in_feat):
        return orc.gat_forward(attn_row, attn_col, row_ptr, col_ind, slope, in_feat)

    @staticmethod
    def gat_rowstat(attn_row, edge_max, edge_sum, out, grad_out):
        return torch.stack([attn_row, edge_max, 1.0 / edge_sum.clamp(min=1e-30), (grad_out * out).sum(-1)], dim=-1).contiguous()

    @staticmethod
    def gat_backward_cols(row_ptr, col_ptr, row_ind, permute, pack, edge_mask, in_feat, attn_col, grad_out, slope):
        # CSR column ids of the block, recovered from the CSC arrays through permute
        cols = orc.edge_rows(col_ptr)
        col_ind = torch.empty_like(cols)
        col_ind[permute.long()] = cols
        rows_csr = torch.empty_like(cols)
        rows_csr[permute.long()] = row_ind.long()
        assert torch.equal(rows_csr, orc.edge_rows(row_ptr)), "permute / row_ptr inconsistent"
        safe_sum = 1.0 / pack[..., 2].clamp(min=1e-30)
        return orc.gat_backward(slope, 0.0, row_ptr, col_ind, pack[..., 1], safe_sum, None, in_feat,
                                pack[..., 0], attn_col, grad_out, s_row=pack[..., 3])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n, h, f, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rp, ci = synth.random_graph(n, 6, seed=21, long_rows=[(2, 150), (n - 1, 90)])
        ar, ac, x, g = gat_inputs(rp, n, h, f, seed=4)
        shard = gdist.build_shard(rp, ci, rank, world, csr2csc=orc.csr2csc)
        r0, r1 = shard.bounds[rank], shard.bounds[rank + 1]
        loc = [t[r0:r1].clone().requires_grad_() for t in (ar, ac, x)]
        out = gdist.sharded_gat(*loc, shard, 0.2, None, OracleBackend)
        out.backward(g[r0:r1])
        q.put((rank, r0, r1, out.detach(), [t.grad for t in loc]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_gat_equals_single(world):
    n, h, f = 120, 2, 4
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, h, f, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    rp, ci = synth.random_graph(n, 6, seed=21, long_rows=[(2, 150), (n - 1, 90)])
    ar, ac, x, g = gat_inputs(rp, n, h, f, seed=4)
    o_ref, emax, esum = orc.gat_forward(ar, ac, rp, ci, 0.2, x)
    gf, gr, gc = orc.gat_backward(0.2, 0.0, rp, ci, emax, esum, None, x, ar, ac, g)
    covered = 0
    for rank, r0, r1, out, (d_ar, d_ac, d_x) in results:
        covered += r1 - r0
        assert_close(out, o_ref[r0:r1], f"rank {rank} out")
        assert_close(d_ar, gr[r0:r1], f"rank {rank} grad_attn_row", atol=2e-5)
        assert_close(d_ac, gc[r0:r1], f"rank {rank} grad_attn_col", atol=2e-5)
        assert_close(d_x, gf[r0:r1], f"rank {rank} grad_feat")
    assert covered == n


def test_balanced_blocks():
    rp, _ = synth.random_graph(1000, 8, seed=2, long_rows=[(10, 3000)])
    for world in (1, 2, 4, 8):
        b = gdist.balanced_node_blocks(rp, world)
        b2 = gdist.balanced_node_blocks(rp, world, rp, 40.0)      # with out-degree and per-node terms
        assert b2[0] == 0 and b2[-1] == 1000 and all(x <= y for x, y in zip(b2, b2[1:]))
        assert b[0] == 0 and b[-1] == 1000 and all(x <= y for x, y in zip(b, b[1:]))
        nnz = int(rp[-1])
        loads = [int(rp[b[g + 1]] - rp[b[g]]) for g in range(world)]
        assert sum(loads) == nnz
        assert max(loads) <= nnz / world + 3000 + 50   # within one (heavy) row of the ideal split


# ---------------------------------------------------------------------------
# pipelined (relabelled, staged) sharding
# ---------------------------------------------------------------------------
class OracleStagedBackend(OracleBackend):
    """Staged entry points of dgnn_b200.kernels restated with tensor ops (state = dict)."""

    @staticmethod
    def gat_forward_state(n_rows, h, f, device):
        return {}

    @staticmethod
    def gat_backward_state(n_cols, h, f, device):
        return {}

    @staticmethod
    def gat_forward_staged(attn_row, attn_col_blk, row_ptr, col_ind, slope, feat_blk, state, first, last):
        n, h = attn_row.shape
        rows = orc.edge_rows(row_ptr)
        cols = col_ind.long()
        leaky = orc.leaky_relu(attn_row[rows] + attn_col_blk[cols], slope)
        m_p = torch.full((n, h), orc.NEG_INIT)
        if rows.numel():
            m_p = m_p.scatter_reduce(0, rows[:, None].expand(-1, h), leaky, "amax", include_self=True)
        e = torch.exp(leaky - m_p[rows])
        z_p = torch.zeros(n, h).index_add_(0, rows, e)
        acc_p = torch.zeros((n,) + tuple(feat_blk.shape[1:])).index_add_(0, rows, e[:, :, None] * feat_blk[cols])
        if first:
            state["m"], state["z"], state["acc"] = m_p, z_p, acc_p
        else:
            m = torch.maximum(state["m"], m_p)
            s1, s2 = torch.exp(state["m"] - m), torch.exp(m_p - m)
            state["z"] = state["z"] * s1 + z_p * s2
            state["acc"] = state["acc"] * s1[:, :, None] + acc_p * s2[:, :, None]
            state["m"] = m
        if not last:
            return None
        z = state["z"]
        out = torch.where(z[:, :, None] > 0, state["acc"] / z.clamp(min=1e-30)[:, :, None], torch.zeros(()))
        return out, state["m"], z

    @staticmethod
    def gat_backward_cols_staged(row_ptr, col_ptr, row_ind, permute, pack_blk, in_feat, attn_col, grad_blk, slope,
                                 state, first, last):
        gf, gr, gc = OracleBackend.gat_backward_cols(row_ptr, col_ptr, row_ind, permute, pack_blk, None, in_feat,
                                                     attn_col, grad_blk, slope)
        if first:
            state["gf"], state["gc"] = gf, gc
        else:
            state["gf"], state["gc"] = state["gf"] + gf, state["gc"] + gc
        return gr, (state["gf"] if last else None), (state["gc"] if last else None)


def _pipe_worker(rank, world, port, n, h, f, stages, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rp, ci = synth.random_graph(n, 6, seed=22, long_rows=[(2, 150), (n - 1, 90)])
        ar, ac, x, g = gat_inputs(rp, n, h, f, seed=5)
        shard = gdist.build_pipe_shard(rp, ci, rank, world, stages=stages, seed=3, csr2csc=orc.csr2csc)
        loc = [gdist.scatter_rows(t, shard).requires_grad_() for t in (ar, ac, x)]
        out = gdist.pipelined_gat(*loc, shard, 0.2, None, OracleStagedBackend)
        out.backward(gdist.scatter_rows(g, shard))
        q.put((rank, shard.local_ids.clone(), out.detach(), [t.grad for t in loc]))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,stages", [(2, 1), (2, 3), (3, 2)])
def test_pipelined_gat_equals_single(world, stages):
    n, h, f = 113, 2, 4
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pipe_worker, args=(r, world, port, n, h, f, stages, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    rp, ci = synth.random_graph(n, 6, seed=22, long_rows=[(2, 150), (n - 1, 90)])
    ar, ac, x, g = gat_inputs(rp, n, h, f, seed=5)
    o_ref, emax, esum = orc.gat_forward(ar, ac, rp, ci, 0.2, x)
    gf, gr, gc = orc.gat_backward(0.2, 0.0, rp, ci, emax, esum, None, x, ar, ac, g)
    seen = []
    for rank, ids, out, (d_ar, d_ac, d_x) in results:
        real = ids >= 0
        idx = ids[real]
        seen.append(idx)
        assert_close(out[real], o_ref[idx], f"rank {rank} out")
        assert_close(d_ar[real], gr[idx], f"rank {rank} grad_attn_row", atol=2e-5)
        assert_close(d_ac[real], gc[idx], f"rank {rank} grad_attn_col", atol=2e-5)
        assert_close(d_x[real], gf[idx], f"rank {rank} grad_feat")
    assert torch.equal(torch.sort(torch.cat(seen)).values, torch.arange(n))     # every node owned exactly once
