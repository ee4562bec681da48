"""Destination-row-block sharding of the fused GAT operator over torch.distributed.

The reference is single-GPU.  Here rank g owns a contiguous block of nodes,
chosen so that every block holds about the same number of in-edges:

  forward   rank g aggregates its destination rows A[block_g, :] and needs
            attn_col and in_feat of every source node  -> two all-gathers;
  backward  rank g owns the same nodes as SOURCE columns, A[:, block_g]: it
            needs grad_out and the row statistics pack of every destination
            row (two all-gathers) and produces grad_feat / grad_attn_col for
            its own nodes with no reduction; grad_attn_row comes out as
            per-rank partial sums over all rows -> one all-reduce of [N,H].

Blocks have different node counts, so node ids are remapped into a padded id
space (rank g' owns ids g'*n_max .. g'*n_max + n_g' - 1) in which the
all-gathers are plain equal-size `all_gather_into_tensor` calls.  Gathered
tensors land in this GPU's own memory before any kernel reads them.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import kernels


def balanced_node_blocks(row_ptr: torch.Tensor, world: int) -> list[int]:
    """Boundaries b[0..world] of contiguous node blocks with about nnz/world
    in-edges each (b[g] = first row whose edge offset reaches g*nnz/world)."""
    rp = row_ptr.long()
    n = rp.numel() - 1
    nnz = int(rp[-1])
    targets = torch.tensor([(nnz * g) // world for g in range(1, world)], dtype=torch.long, device=rp.device)
    inner = torch.searchsorted(rp[:-1].contiguous(), targets, right=False).tolist() if world > 1 else []
    bounds = [0] + [min(max(int(b), 0), n) for b in inner] + [n]
    for i in range(1, len(bounds)):          # keep the boundaries monotone
        bounds[i] = max(bounds[i], bounds[i - 1])
    return bounds


@dataclass
class GatShard:
    """Per-rank graph pieces, all in the padded id space."""
    rank: int
    world: int
    bounds: list          # node block boundaries, len world+1
    n_max: int            # padded block size
    n_loc: int
    # forward: local destination rows x all (padded) source columns
    fwd_row_ptr: torch.Tensor
    fwd_col_ind: torch.Tensor
    # backward: all (padded) destination rows x local source columns
    bwd_row_ptr: torch.Tensor   # CSR index pointer of the block, over padded rows
    bwd_col_ptr: torch.Tensor   # CSC index pointer, local columns
    bwd_row_ind: torch.Tensor   # padded row id of each CSC entry
    bwd_permute: torch.Tensor   # CSR position (within the block) of each CSC entry

    @property
    def n_pad(self) -> int:
        return self.world * self.n_max


def _pad_ids(ids: torch.Tensor, bounds: list, n_max: int) -> torch.Tensor:
    b = torch.tensor(bounds, dtype=torch.long, device=ids.device)
    blk = torch.searchsorted(b[1:].contiguous(), ids.long(), right=True)
    return (blk * n_max + (ids.long() - b[blk])).to(torch.int32)


def build_shard(row_ptr, col_ind, rank, world, csr2csc=None, bounds=None) -> GatShard:
    """Cut rank's pieces out of the global CSR (rows = destinations).  `csr2csc`
    is the conversion routine (defaults to the CUDA kernel); every rank calls
    this with the same global graph."""
    csr2csc = csr2csc or kernels.csr2csc
    rp = row_ptr.long()
    n = rp.numel() - 1
    bounds = bounds or balanced_node_blocks(rp, world)
    n_max = max(max(bounds[g + 1] - bounds[g] for g in range(world)), 1)
    r0, r1 = bounds[rank], bounds[rank + 1]
    ptr_dtype = row_ptr.dtype
    # forward piece
    lo, hi = int(rp[r0]), int(rp[r1])
    fwd_row_ptr = (rp[r0:r1 + 1] - lo).to(ptr_dtype).contiguous()
    fwd_col_ind = _pad_ids(col_ind[lo:hi], bounds, n_max)
    # backward piece: columns r0..r1 of the global CSC
    col_ptr, row_ind, _ = csr2csc(row_ptr, col_ind)
    cp = col_ptr.long()
    clo, chi = int(cp[r0]), int(cp[r1])
    bwd_col_ptr = (cp[r0:r1 + 1] - clo).to(ptr_dtype).contiguous()
    bwd_row_ind = _pad_ids(row_ind[clo:chi], bounds, n_max)
    # CSR of the block over padded rows = "CSC" of its transpose; perm[i] = CSC position of CSR entry i
    n_pad = world * n_max
    bwd_row_ptr, _, perm = csr2csc(bwd_col_ptr, bwd_row_ind, n_pad)
    permute = torch.empty_like(perm)
    permute[perm.long()] = torch.arange(perm.numel(), dtype=perm.dtype, device=perm.device)
    return GatShard(rank, world, bounds, n_max, r1 - r0, fwd_row_ptr, fwd_col_ind.contiguous(),
                    bwd_row_ptr.to(ptr_dtype).contiguous(), bwd_col_ptr, bwd_row_ind.contiguous(), permute.contiguous())


def _all_gather_padded(x_loc: torch.Tensor, n_max: int, group) -> torch.Tensor:
    """[n_loc, ...] -> [world*n_max, ...]; rows past n_loc of each block are zero."""
    world = dist.get_world_size(group)
    pad = x_loc.new_zeros((n_max,) + tuple(x_loc.shape[1:]))
    pad[: x_loc.shape[0]] = x_loc
    out = x_loc.new_empty((world * n_max,) + tuple(x_loc.shape[1:]))
    dist.all_gather_into_tensor(out, pad.contiguous(), group=group)
    return out


class ShardedGATFunction(torch.autograd.Function):
    """Fused GAT on this rank's node block.  Inputs and outputs are the local
    rows: attn_row, attn_col [n_loc,H], in_feat [n_loc,H,F] -> out [n_loc,H,F]."""

    @staticmethod
    def forward(ctx, attn_row, attn_col, in_feat, shard, negative_slope, group, backend):
        attn_col_all = _all_gather_padded(attn_col, shard.n_max, group)
        feat_all = _all_gather_padded(in_feat, shard.n_max, group)
        out, edge_max, edge_sum = backend.gat_forward(attn_row, attn_col_all, shard.fwd_row_ptr, shard.fwd_col_ind,
                                                      negative_slope, feat_all)
        ctx.save_for_backward(attn_row, attn_col, in_feat, out, edge_max, edge_sum)
        ctx.shard, ctx.slope, ctx.group, ctx.backend = shard, negative_slope, group, backend
        return out

    @staticmethod
    def backward(ctx, grad_out):
        attn_row, attn_col, in_feat, out, edge_max, edge_sum = ctx.saved_tensors
        shard, backend, group = ctx.shard, ctx.backend, ctx.group
        grad_out = grad_out.contiguous()
        pack = backend.gat_rowstat(attn_row, edge_max, edge_sum, out, grad_out)      # [n_loc,H,4]
        pack_all = _all_gather_padded(pack, shard.n_max, group)
        grad_all = _all_gather_padded(grad_out, shard.n_max, group)
        grad_feat, grad_row_part, grad_col = backend.gat_backward_cols(
            shard.bwd_row_ptr, shard.bwd_col_ptr, shard.bwd_row_ind, shard.bwd_permute, pack_all, None,
            in_feat, attn_col, grad_all, ctx.slope)
        dist.all_reduce(grad_row_part, group=group)
        lo = shard.rank * shard.n_max
        grad_row = grad_row_part[lo: lo + shard.n_loc].contiguous()
        return grad_row, grad_col, grad_feat, None, None, None, None


def sharded_gat(attn_row, attn_col, in_feat, shard, negative_slope=0.2, group=None, backend=kernels):
    """out_loc = fused GAT over the sharded graph; differentiable in the three tensors."""
    return ShardedGATFunction.apply(attn_row, attn_col, in_feat, shard, negative_slope, group, backend)
