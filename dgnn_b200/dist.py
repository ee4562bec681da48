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


# ---------------------------------------------------------------------------
# Pipelined sharding: random node relabelling, equal blocks, staged all-gathers
# ---------------------------------------------------------------------------
@dataclass
class PipeShard:
    """Pieces of the graph for one rank of the pipelined sharded operator.

    Nodes are relabelled by a seeded random permutation and dealt out in equal
    blocks of `blk` nodes per rank (ids past the real node count are padding
    without edges), so in-edges, out-edges and node counts are all balanced.
    Every block is cut into `stages` slices; stage p all-gathers slice p of every
    rank ([world*slice, ...] buffer, row g*slice + i = node i of rank g's slice p)
    while the kernels work on the edges of stage p-1."""
    rank: int
    world: int
    stages: int
    n: int
    blk: int
    slice: int
    local_ids: torch.Tensor       # original node id of every local row (-1 for padding)
    fwd: list                     # per stage: (row_ptr [blk+1], col_ind -> buffer row)
    bwd: list                     # per stage: (row_ptr [world*slice+1], col_ptr [blk+1], row_ind -> buffer row, permute)
    peer: object = None           # PeerGather when the slices travel as peer-to-peer copies instead of all-gathers


def _expand_segments(ptr, ids):
    """Positions and local segment index of all entries of the segments `ids` of a CSR/CSC pointer."""
    valid = ids >= 0
    safe = ids.clamp(min=0)
    start = ptr[safe]
    deg = torch.where(valid, ptr[safe + 1] - start, torch.zeros_like(start))
    seg = torch.repeat_interleave(torch.arange(ids.numel(), device=ids.device), deg)
    excl = torch.cumsum(deg, 0) - deg
    pos = start[seg] + (torch.arange(int(deg.sum()), device=ids.device) - excl[seg])
    return pos, seg


def build_pipe_shard(row_ptr, col_ind, rank, world, stages=4, seed=0, csr2csc=None) -> PipeShard:
    """Every rank calls this with the same global CSR (rows = destinations) and seed."""
    csr2csc = csr2csc or kernels.csr2csc
    dev = col_ind.device
    rp = row_ptr.long()
    n = rp.numel() - 1
    blk = -(-n // (world * stages)) * stages
    sl = blk // stages
    n_pad = world * blk
    g = torch.Generator(device="cpu").manual_seed(seed)
    order = torch.full((n_pad,), -1, dtype=torch.long)
    order[:n] = torch.randperm(n, generator=g)
    order = order[torch.randperm(n_pad, generator=g)].to(dev)        # padding spread over all blocks
    inv = torch.empty(n, dtype=torch.long, device=dev)
    real = order >= 0
    inv[order[real]] = torch.arange(n_pad, device=dev)[real]
    local_ids = order[rank * blk: (rank + 1) * blk].contiguous()

    def buffer_row(new_id):
        """(stage, row inside the stage's gathered buffer) of a relabelled node id."""
        owner, rem = new_id // blk, new_id % blk
        return rem // sl, owner * sl + rem % sl

    # forward: local destination rows, all sources, split by the stage of the source
    pos, row = _expand_segments(rp, local_ids)
    stage, buf = buffer_row(inv[col_ind[pos].long()])
    fwd = []
    for p in range(stages):
        m = stage == p
        ptr = torch.zeros(blk + 1, dtype=torch.long, device=dev)
        torch.cumsum(torch.bincount(row[m], minlength=blk), 0, out=ptr[1:])
        fwd.append((ptr.to(torch.int32), buf[m].to(torch.int32).contiguous()))
    del pos, row, stage, buf
    # backward: local source columns, all destinations, split by the stage of the destination
    col_ptr, row_ind, _ = csr2csc(row_ptr, col_ind)
    pos, col = _expand_segments(col_ptr.long(), local_ids)
    stage, buf = buffer_row(inv[row_ind[pos].long()])
    bwd = []
    for p in range(stages):
        m = stage == p
        cptr = torch.zeros(blk + 1, dtype=torch.long, device=dev)
        torch.cumsum(torch.bincount(col[m], minlength=blk), 0, out=cptr[1:])
        cptr = cptr.to(torch.int32)
        rind = buf[m].to(torch.int32).contiguous()
        # CSR of the sub-matrix = "CSC" of its transpose; perm[i] = CSC position of CSR entry i
        rptr, _, perm = csr2csc(cptr, rind, world * sl)
        permute = torch.empty_like(perm)
        permute[perm.long()] = torch.arange(perm.numel(), dtype=perm.dtype, device=perm.device)
        bwd.append((rptr.to(torch.int32).contiguous(), cptr, rind, permute.to(torch.int32).contiguous()))
    return PipeShard(rank, world, stages, n, blk, sl, local_ids, fwd, bwd)


class _StreamEvent:
    """Stands in for the Work object of an asynchronous collective: wait() orders the current stream after it."""

    def __init__(self, event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)


class PeerGather:
    """Slices fetched from the peers' memory by copy engines instead of an NCCL all-gather.

    Every rank keeps one staging buffer per gathered tensor in symmetric memory (torch.distributed's
    allocator: every rank can map every other rank's buffer over NVLink).  A gather is: copy the local
    block into the staging buffer, a one-element NCCL all-reduce as the barrier ("every rank's block is
    written"), then plain device-to-device copies of slice p of every peer into this rank's
    [world*slice, ...] buffer on a copy stream, peers visited in rotated order so that each peer serves
    one reader at a time.  The copies take no SM away from the kernels they overlap with and reach the
    NVLink rate of a peer copy; an all-reduce before the next overwrite of the staging buffer makes
    sure every peer has finished reading it.  No multicast, no kernel of this library touches peer memory."""

    def __init__(self, group):
        import os
        # the copies are plain peer reads: no multicast object is needed, and none should be bound to the buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group
        self.stream = torch.cuda.Stream()
        self.own_stream = torch.cuda.Stream()   # local rows go on their own stream, beside the peer copies
        self.staging = {}
        self.flag = None

    def _staging(self, tag, x_loc):
        import torch.distributed._symmetric_memory as symm
        key = (tag, tuple(x_loc.shape), x_loc.dtype)
        if key not in self.staging:          # collective: every rank reaches this in the same order
            buf = symm.empty(tuple(x_loc.shape), dtype=x_loc.dtype, device=x_loc.device)
            handle = symm.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
            self.staging[key] = (buf, handle, {})
        return self.staging[key]

    def _barrier(self, dev):
        if self.flag is None:
            self.flag = torch.zeros(1, dtype=torch.float32, device=dev)
        dist.all_reduce(self.flag, group=self.group)

    def gather_many(self, items, shard):
        """items: [(tag, x_loc [blk, ...]), ...] -> [(buffers, works), ...], one barrier pair for all of them."""
        dev = items[0][1].device
        cur = torch.cuda.current_stream()
        staged = [self._staging(tag, x) for tag, x in items]
        self._barrier(dev)                    # every peer has finished reading the previous content
        for (buf, _, _), (_, x) in zip(staged, items):
            buf.copy_(x)
        self._barrier(dev)                    # every rank's blocks are in place
        ready = torch.cuda.Event()
        ready.record(cur)
        results = []
        for _, x in items:
            tail = tuple(x.shape[1:])
            results.append(([x.new_empty((shard.world * shard.slice,) + tail) for _ in range(shard.stages)], []))
        lo, hi = shard.rank * shard.slice, (shard.rank + 1) * shard.slice
        entered = torch.cuda.Event()
        entered.record(cur)
        with torch.cuda.stream(self.own_stream):          # this rank's own rows of every stage buffer
            self.own_stream.wait_event(entered)
            for (_, x), (bufs, _) in zip(items, results):
                for p in range(shard.stages):
                    bufs[p][lo:hi].copy_(x[p * shard.slice:(p + 1) * shard.slice], non_blocking=True)
            own_done = torch.cuda.Event()
            own_done.record(self.own_stream)
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(ready)
            for p in range(shard.stages):
                sl = slice(p * shard.slice, (p + 1) * shard.slice)
                for (buf, handle, views), (_, x), (bufs, works) in zip(staged, items, results):
                    for i in range(1, shard.world):
                        q = (shard.rank + i) % shard.world
                        if q not in views:
                            views[q] = handle.get_buffer(q, tuple(x.shape), x.dtype)
                        bufs[p][q * shard.slice:(q + 1) * shard.slice].copy_(views[q][sl], non_blocking=True)
                    if p == 0:
                        self.stream.wait_event(own_done)
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
                    works.append(_StreamEvent(ev))
        for (_, x), (bufs, _) in zip(items, results):
            x.record_stream(self.own_stream)
            for bb in bufs:
                bb.record_stream(self.stream)
                bb.record_stream(self.own_stream)
        return results


def _gather_many(items, shard, group):
    """Start the gathers of the `stages` slices of several [blk, ...] tensors; [(buffers, works), ...]."""
    if shard.peer is not None and items[0][1].is_cuda and shard.world > 1:
        return shard.peer.gather_many([(tag, x.contiguous()) for tag, x in items], shard)
    return [_gather_slices(x, shard, group) for _, x in items]


def _gather_slices(x_loc, shard, group):
    """Start the all-gathers of the `stages` slices of x_loc [blk, ...]; returns (buffers, works)."""
    bufs, works = [], []
    for p in range(shard.stages):
        part = x_loc[p * shard.slice: (p + 1) * shard.slice]
        buf = x_loc.new_empty((shard.world * shard.slice,) + tuple(x_loc.shape[1:]))
        works.append(dist.all_gather_into_tensor(buf, part.contiguous(), group=group, async_op=True))
        bufs.append(buf)
    return bufs, works


def _pipe_forward(attn_row, attn_col, h, shard, slope, group, backend, bias=None):
    (col_bufs, col_works), (feat_bufs, feat_works) = _gather_many([("attn_col", attn_col), ("feat", h)], shard, group)
    state = backend.gat_forward_state(shard.blk, h.shape[1], h.shape[2], h.device)
    res = None
    for p in range(shard.stages):
        col_works[p].wait()
        feat_works[p].wait()
        ptr, col = shard.fwd[p]
        last = p == shard.stages - 1
        extra = {"bias": bias} if (bias is not None and last) else {}
        res = backend.gat_forward_staged(attn_row, col_bufs[p], ptr, col, slope, feat_bufs[p], state, p == 0, last, **extra)
    return res


def _pipe_backward(attn_row, attn_col, h, out, edge_max, edge_sum, grad_out, shard, slope, group, backend, pack=None):
    if pack is None:
        pack = backend.gat_rowstat(attn_row, edge_max, edge_sum, out, grad_out)
    (pack_bufs, pack_works), (grad_bufs, grad_works) = _gather_many([("pack", pack), ("grad_out", grad_out)], shard, group)
    state = backend.gat_backward_state(shard.blk, h.shape[1], h.shape[2], h.device)
    parts = []
    grad_feat = grad_col = None
    for p in range(shard.stages):
        pack_works[p].wait()
        grad_works[p].wait()
        rptr, cptr, rind, perm = shard.bwd[p]
        part, grad_feat, grad_col = backend.gat_backward_cols_staged(
            rptr, cptr, rind, perm, pack_bufs[p], h, attn_col, grad_bufs[p], slope, state, p == 0,
            p == shard.stages - 1)
        parts.append(part)                                     # [world*slice, H]: partial sums for the rows of stage p
    hh = h.shape[1]
    # [stages, world, slice, H] -> sum over ranks, keep the rows this rank owns
    allp = torch.stack(parts, 0).view(shard.stages, shard.world, shard.slice, hh)
    if dist.get_backend(group) == "nccl":
        send = allp.permute(1, 0, 2, 3).contiguous()           # [world, stages, slice, H]
        mine = send.new_empty((shard.stages, shard.slice, hh))
        dist.reduce_scatter_tensor(mine, send, group=group)
    else:
        allp = allp.contiguous()
        dist.all_reduce(allp, group=group)
        mine = allp[:, shard.rank]
    return grad_feat, mine.reshape(shard.blk, hh).contiguous(), grad_col


class PipelinedGATFunction(torch.autograd.Function):
    """Fused GAT on this rank's block of the relabelled graph, with the gathers of the
    source features (forward) and of grad_out (backward) overlapped with the kernels.
    attn_row, attn_col [blk,H], in_feat [blk,H,F] (rows in PipeShard.local_ids order)."""

    @staticmethod
    def forward(ctx, attn_row, attn_col, in_feat, shard, negative_slope, group, backend):
        out, edge_max, edge_sum = _pipe_forward(attn_row.contiguous(), attn_col.contiguous(), in_feat.contiguous(),
                                                shard, negative_slope, group, backend)
        ctx.save_for_backward(attn_row, attn_col, in_feat, out, edge_max, edge_sum)
        ctx.shard, ctx.slope, ctx.group, ctx.backend = shard, negative_slope, group, backend
        return out

    @staticmethod
    def backward(ctx, grad_out):
        attn_row, attn_col, in_feat, out, edge_max, edge_sum = ctx.saved_tensors
        grad_feat, grad_row, grad_col = _pipe_backward(attn_row, attn_col, in_feat, out, edge_max, edge_sum,
                                                      grad_out.contiguous(), ctx.shard, ctx.slope, ctx.group,
                                                      ctx.backend)
        return grad_row, grad_col, grad_feat, None, None, None, None


class PipelinedGATLayerFunction(torch.autograd.Function):
    """Attention logits + pipelined aggregation (+ bias in the last stage's epilogue) as one autograd
    node (CUDA only)."""

    @staticmethod
    def forward(ctx, h, attn_l, attn_r, bias, shard, negative_slope, group):
        h = h.contiguous()
        attn_row, attn_col = kernels.gat_logits_forward(h, attn_l, attn_r)
        out, edge_max, edge_sum = _pipe_forward(attn_row, attn_col, h, shard, negative_slope, group, kernels, bias=bias)
        ctx.save_for_backward(attn_row, attn_col, h, out, edge_max, edge_sum, attn_l, attn_r,
                              bias if bias is not None else h.new_empty(0))
        ctx.shard, ctx.slope, ctx.group, ctx.has_bias = shard, negative_slope, group, bias is not None
        return out

    @staticmethod
    def backward(ctx, grad_out):
        attn_row, attn_col, h, out, edge_max, edge_sum, attn_l, attn_r, bias = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        pack = grad_bias = None
        if ctx.has_bias:   # `out` carries the bias: the row statistics subtract it, its gradient falls out of the same pass
            pack, grad_bias = kernels.gat_rowstat_bias(attn_row, edge_max, edge_sum, out, grad_out, bias)
            grad_bias = grad_bias.view_as(bias)
        grad_h, grad_row, grad_col = _pipe_backward(attn_row, attn_col, h, out, edge_max, edge_sum, grad_out, ctx.shard,
                                                   ctx.slope, ctx.group, kernels, pack=pack)
        grad_l, grad_r = kernels.gat_logits_backward(h, attn_l, attn_r, grad_row, grad_col, grad_h)
        return grad_h, grad_l.view_as(attn_l), grad_r.view_as(attn_r), grad_bias, None, None, None


def pipelined_gat(attn_row, attn_col, in_feat, shard, negative_slope=0.2, group=None, backend=kernels):
    return PipelinedGATFunction.apply(attn_row, attn_col, in_feat, shard, negative_slope, group, backend)


def pipelined_gat_layer(h, attn_l, attn_r, shard, negative_slope=0.2, group=None, bias=None):
    """h [blk,H,F] -> logits, pipelined aggregation and (optionally) the bias add, one autograd node.  Rows that
    pad the last block also receive the bias; they carry no node."""
    return PipelinedGATLayerFunction.apply(h, attn_l, attn_r, bias, shard, negative_slope, group)


def enable_peer_copies(shard, group=None):
    """Switch a PipeShard on CUDA ranks of one NVLink domain from NCCL all-gathers to peer-to-peer copies
    (see PeerGather); returns the shard."""
    if shard.world > 1:
        peer = PeerGather(group)
        try:                                   # collective probe: symmetric memory may be unavailable on a platform
            peer._staging("probe", torch.zeros(16, dtype=torch.float32, device=shard.local_ids.device))
        except Exception as exc:               # every rank sees the same platform, so every rank falls back together
            import warnings
            warnings.warn(f"dgnn_b200: peer-to-peer slice copies unavailable ({exc}); using NCCL all-gathers")
            return shard
        shard.peer = peer
    return shard


def scatter_rows(x_global, shard):
    """Rows of a global [N, ...] tensor in this rank's local order (padding rows are zero)."""
    out = x_global.new_zeros((shard.blk,) + tuple(x_global.shape[1:]))
    real = shard.local_ids >= 0
    out[real] = x_global[shard.local_ids[real]]
    return out
