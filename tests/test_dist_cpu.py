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
