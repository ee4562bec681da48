"""Destination-row-block sharding of the fused GAT operator over torch.distributed.

The reference is single-GPU.  Here rank g owns a contiguous block of nodes:

  forward   rank g aggregates its destination rows A[block_g, :] and needs
            attn_col and in_feat of every source node  -> two all-gathers;
  backward  rank g owns the same nodes as SOURCE columns, A[:, block_g]: it
            needs grad_out and the row statistics pack of every destination
            row (two all-gathers) and produces grad_feat / grad_attn_col for
            its own nodes with no reduction; grad_attn_row comes out as
            per-rank partial sums over all rows -> one all-reduce of [N,H].

Blocks are chosen by a cost prefix (in-edges for the forward, out-edges for the
backward, a per-node term for the dense projection around the operator), so
they hold different node counts; the all-gathers therefore move uneven row
ranges straight into their place in one [N, ...] buffer (node ids stay global,
nothing is padded).  Gathered tensors land in this GPU's own memory before any
kernel reads them.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import kernels

# relative cost of one in-edge (forward gather), one out-edge (backward gather) and
# one node (projection GEMM + elementwise work of the layer), measured on a B200
COST_IN_EDGE, COST_OUT_EDGE, COST_NODE = 1.0, 2.8, 40.0


def balanced_node_blocks(row_ptr: torch.Tensor, world: int, col_ptr: torch.Tensor | None = None,
                         node_cost: float = 0.0) -> list[int]:
    """Boundaries b[0..world] of contiguous node blocks with about equal cost.
    With only `row_ptr` the cost of a node is its in-degree (equal in-edge counts);
    with `col_ptr` the out-degree and a per-node term are added with the weights above."""
    rp = row_ptr.long()
    n = rp.numel() - 1
    if col_ptr is None:
        prefix = rp.to(torch.float64)
    else:
        cp = col_ptr.long()
        ids = torch.arange(n + 1, device=rp.device, dtype=torch.float64)
        prefix = COST_IN_EDGE * rp.to(torch.float64) + COST_OUT_EDGE * cp.to(torch.float64) + node_cost * ids
    total = float(prefix[-1])
    targets = torch.tensor([total * g / world for g in range(1, world)], dtype=torch.float64, device=rp.device)
    inner = torch.searchsorted(prefix[:-1].contiguous(), targets, right=False).tolist() if world > 1 else []
    bounds = [0] + [min(max(int(b), 0), n) for b in inner] + [n]
    for i in range(1, len(bounds)):          # keep the boundaries monotone
        bounds[i] = max(bounds[i], bounds[i - 1])
    return bounds


@dataclass
class GatShard:
    """Per-rank graph pieces; node ids are global."""
    rank: int
    world: int
    bounds: list          # node block boundaries, len world+1
    n: int                # number of nodes of the whole graph
    n_loc: int
    # forward: local destination rows x all source columns
    fwd_row_ptr: torch.Tensor
    fwd_col_ind: torch.Tensor
    # backward: all destination rows x local source columns
    bwd_row_ptr: torch.Tensor   # CSR index pointer of the block, over all rows
    bwd_col_ptr: torch.Tensor   # CSC index pointer, local columns
    bwd_row_ind: torch.Tensor   # row id of each CSC entry
    bwd_permute: torch.Tensor   # CSR position (within the block) of each CSC entry


def build_shard(row_ptr, col_ind, rank, world, csr2csc=None, bounds=None) -> GatShard:
    """Cut rank's pieces out of the global CSR (rows = destinations).  `csr2csc`
    is the conversion routine (defaults to the CUDA kernel); every rank calls
    this with the same global graph."""
    csr2csc = csr2csc or kernels.csr2csc
    rp = row_ptr.long()
    n = rp.numel() - 1
    ptr_dtype = row_ptr.dtype
    col_ptr, row_ind, _ = csr2csc(row_ptr, col_ind)
    cp = col_ptr.long()
    bounds = bounds or balanced_node_blocks(rp, world, cp, COST_NODE)
    r0, r1 = bounds[rank], bounds[rank + 1]
    # forward piece: rows r0..r1 of the CSR
    lo, hi = int(rp[r0]), int(rp[r1])
    fwd_row_ptr = (rp[r0:r1 + 1] - lo).to(ptr_dtype).contiguous()
    fwd_col_ind = col_ind[lo:hi].to(torch.int32).contiguous()
    # backward piece: columns r0..r1 of the CSC
    clo, chi = int(cp[r0]), int(cp[r1])
    bwd_col_ptr = (cp[r0:r1 + 1] - clo).to(ptr_dtype).contiguous()
    bwd_row_ind = row_ind[clo:chi].to(torch.int32).contiguous()
    # CSR of the block = "CSC" of its transpose; perm[i] = CSC position of CSR entry i
    bwd_row_ptr, _, perm = csr2csc(bwd_col_ptr, bwd_row_ind, n)
    permute = torch.empty_like(perm)
    permute[perm.long()] = torch.arange(perm.numel(), dtype=perm.dtype, device=perm.device)
    return GatShard(rank, world, bounds, n, r1 - r0, fwd_row_ptr, fwd_col_ind,
                    bwd_row_ptr.to(ptr_dtype).contiguous(), bwd_col_ptr, bwd_row_ind, permute.to(torch.int32).contiguous())


def _all_gather_rows(x_loc: torch.Tensor, bounds: list, group) -> torch.Tensor:
    """[n_loc, ...] on every rank -> [N, ...]: rank g's rows land at bounds[g]:bounds[g+1]."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    out = x_loc.new_empty((bounds[-1],) + tuple(x_loc.shape[1:]))
    views = [out[bounds[g]: bounds[g + 1]] for g in range(world)]
    x_loc = x_loc.contiguous()
    if dist.get_backend(group) == "nccl":
        # uneven row ranges: NCCL runs this as one group of broadcasts straight into the views
        dist.all_gather(views, x_loc, group=group)
    else:
        views[rank].copy_(x_loc)
        for g in range(world):
            if views[g].numel():
                dist.broadcast(views[g], src=dist.get_global_rank(group, g) if group is not None else g, group=group)
    return out


def _sharded_forward(attn_row, attn_col, in_feat, shard, negative_slope, group, backend):
    attn_col_all = _all_gather_rows(attn_col, shard.bounds, group)
    feat_all = _all_gather_rows(in_feat, shard.bounds, group)
    return backend.gat_forward(attn_row, attn_col_all, shard.fwd_row_ptr, shard.fwd_col_ind, negative_slope, feat_all)


def _sharded_backward(attn_row, attn_col, in_feat, out, edge_max, edge_sum, grad_out, shard, negative_slope, group,
                      backend):
    pack = backend.gat_rowstat(attn_row, edge_max, edge_sum, out, grad_out)      # [n_loc,H,4]
    pack_all = _all_gather_rows(pack, shard.bounds, group)
    grad_all = _all_gather_rows(grad_out, shard.bounds, group)
    grad_feat, grad_row_part, grad_col = backend.gat_backward_cols(
        shard.bwd_row_ptr, shard.bwd_col_ptr, shard.bwd_row_ind, shard.bwd_permute, pack_all, None,
        in_feat, attn_col, grad_all, negative_slope)
    dist.all_reduce(grad_row_part, group=group)
    r0, r1 = shard.bounds[shard.rank], shard.bounds[shard.rank + 1]
    return grad_feat, grad_row_part[r0:r1].contiguous(), grad_col


class ShardedGATFunction(torch.autograd.Function):
    """Fused GAT on this rank's node block.  Inputs and outputs are the local
    rows: attn_row, attn_col [n_loc,H], in_feat [n_loc,H,F] -> out [n_loc,H,F]."""

    @staticmethod
    def forward(ctx, attn_row, attn_col, in_feat, shard, negative_slope, group, backend):
        out, edge_max, edge_sum = _sharded_forward(attn_row, attn_col, in_feat, shard, negative_slope, group, backend)
        ctx.save_for_backward(attn_row, attn_col, in_feat, out, edge_max, edge_sum)
        ctx.shard, ctx.slope, ctx.group, ctx.backend = shard, negative_slope, group, backend
        return out

    @staticmethod
    def backward(ctx, grad_out):
        attn_row, attn_col, in_feat, out, edge_max, edge_sum = ctx.saved_tensors
        grad_feat, grad_row, grad_col = _sharded_backward(attn_row, attn_col, in_feat, out, edge_max, edge_sum,
                                                         grad_out.contiguous(), ctx.shard, ctx.slope, ctx.group,
                                                         ctx.backend)
        return grad_row, grad_col, grad_feat, None, None, None, None


class ShardedGATLayerFunction(torch.autograd.Function):
    """Attention logits + sharded aggregation as one autograd node (CUDA only):
    h [n_loc,H,F], attn_l, attn_r [1,H,F] -> out [n_loc,H,F]."""

    @staticmethod
    def forward(ctx, h, attn_l, attn_r, shard, negative_slope, group):
        h = h.contiguous()
        attn_row, attn_col = kernels.gat_logits_forward(h, attn_l, attn_r)
        out, edge_max, edge_sum = _sharded_forward(attn_row, attn_col, h, shard, negative_slope, group, kernels)
        ctx.save_for_backward(attn_row, attn_col, h, out, edge_max, edge_sum, attn_l, attn_r)
        ctx.shard, ctx.slope, ctx.group = shard, negative_slope, group
        return out

    @staticmethod
    def backward(ctx, grad_out):
        attn_row, attn_col, h, out, edge_max, edge_sum, attn_l, attn_r = ctx.saved_tensors
        grad_h, grad_row, grad_col = _sharded_backward(attn_row, attn_col, h, out, edge_max, edge_sum,
                                                      grad_out.contiguous(), ctx.shard, ctx.slope, ctx.group, kernels)
        grad_l, grad_r = kernels.gat_logits_backward(h, attn_l, attn_r, grad_row, grad_col, grad_h)
        return grad_h, grad_l.view_as(attn_l), grad_r.view_as(attn_r), None, None, None


def sharded_gat(attn_row, attn_col, in_feat, shard, negative_slope=0.2, group=None, backend=kernels):
    """out_loc = fused GAT over the sharded graph; differentiable in the three tensors."""
    return ShardedGATFunction.apply(attn_row, attn_col, in_feat, shard, negative_slope, group, backend)


def sharded_gat_layer(h, attn_l, attn_r, shard, negative_slope=0.2, group=None):
    """Logits + sharded aggregation; differentiable in h and the attention vectors."""
    return ShardedGATLayerFunction.apply(h, attn_l, attn_r, shard, negative_slope, group)
