"""Row-block sharding of the fused GAT layer over the GPUs of one NVLink domain.

The reference is single-GPU.  Here the nodes are relabelled by a seeded random permutation and dealt
out in equal blocks, one per rank (in-edges, out-edges and node counts are balanced at once):

  forward   rank g aggregates the destination rows it owns, A[block_g, :], and needs the projected
            features and the source attention term of every node its in-edges reference;
  backward  rank g owns the same nodes as SOURCE columns, A[:, block_g], and needs grad_out and the
            row statistics `pack` of every destination its out-edges reference.  grad_feat and
            grad_attn_col come out column-owned; grad_attn_row is computed by the row owner from its
            own rows (kernels.gat_rowstat_full), so nothing is reduced across ranks.

Only the DISTINCT referenced rows travel ("halo"): on an R-MAT graph of 2.4 M nodes / 120 M edges a
rank of 8 references 0.88 M of the 2.1 M remote nodes (0.74 M of 1.2 M with 2 ranks).  Every rank
keeps, per gathered tensor, one buffer [own rows | halo rows]; its graph arrays index that buffer.
The own rows are written in place by the producing kernels (projection, logits, row statistics), a
barrier says "every rank's own rows are written", and the halo rows are then fetched from the owners'
buffers by kernels.halo_pull (plain loads over NVLink from symmetric memory, on a side stream) chunk
by chunk, while the aggregation kernels sweep the edges whose rows are already there: stage 0 = edges
between own nodes (no transfer needed), stage k = edges whose far end lies in halo chunk k.  The
per-row softmax state (forward) / per-column accumulators (backward) are carried between the sweeps
by the staged kernels.  No kernel waits on another rank; no multicast; no TMA on peer memory.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import kernels

HALO_SHIFT = 27          # codes = owner << 27 | row inside the owner's block (dgnn_halo_rank_shift)
HALO_MAX_RANKS = 16      # dgnn_halo_max_ranks


# ---------------------------------------------------------------------------
# graph pieces of one rank
# ---------------------------------------------------------------------------
@dataclass
class HaloSide:
    """One direction of a rank's sub-matrix, cut into sweeps (stages).

    forward:  segments = destination rows of the block, entries = their in-edges, `ind` = buffer row
              of the source;  backward: segments = source columns of the block, entries = their
              out-edges, `ind` = buffer row of the destination.  Buffer rows 0..blk-1 are the rank's
              own nodes, row blk+i is halo row i."""
    n_halo: int
    codes: torch.Tensor               # [n_halo] int32: owner << HALO_SHIFT | row in the owner's block
    chunk_off: list                   # halo rows of chunk c are chunk_off[c]:chunk_off[c+1]
    ptr: list                         # per stage: index pointer [blk+1] int32
    ind: list                         # per stage: buffer row of every entry, int32
    edge_id: list | None = None       # per stage: position of the entry in the CSR of the whole graph (int32)
    stage_mask: torch.Tensor = None   # [blk] uint8: bit p = the segment has entries in stage p
    bounds: list | None = None        # "rowsets" schedule: stage p holds ALL entries of the segments bounds[p]:bounds[p+1]


@dataclass
class HaloShard:
    rank: int
    world: int
    stages: int                       # sweeps per pass: stage 0 = own nodes, 1.. = halo chunks (1 stage: everything)
    n: int                            # nodes of the whole graph
    blk: int                          # nodes per rank (the last ids of the padded id space carry no node)
    local_ids: torch.Tensor           # original node id of every local row (-1 for padding)
    fwd: HaloSide = None
    bwd: HaloSide = None
    schedule: str = "staged"          # "staged": every sweep covers all segments and one slice of the far ends, the
                                      # per-segment state is carried between sweeps.  "rowsets": every sweep finishes
                                      # a range of segments (all their entries); halo chunk p = the halo rows that
                                      # ranges 0..p reference first.  No carried state; the first sweep waits for chunk 0

    @property
    def chunks(self):
        if self.schedule == "rowsets":
            return self.stages
        return max(self.stages - 1, 1)

    def chunk_stage(self, c):
        """The first stage that needs halo chunk c."""
        if self.schedule == "rowsets":
            return c
        return c + 1 if self.stages > 1 else 0

    def scatter_rows(self, x_global):
        """Rows of a global [N, ...] tensor in this rank's local order (padding rows are zero)."""
        out = x_global.new_zeros((self.blk,) + tuple(x_global.shape[1:]))
        real = self.local_ids >= 0
        out[real] = x_global[self.local_ids[real]]
        return out


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


def _set_bounds(seg, blk, fractions):
    """Segment ranges whose entry counts follow the cumulative `fractions` (the last one is 1)."""
    cnt = torch.bincount(seg, minlength=blk)
    cum = torch.cumsum(cnt, 0)
    total = int(cum[-1]) if blk else 0
    bounds = [0]
    for fr in fractions[:-1]:
        r = int(torch.searchsorted(cum, torch.tensor(int(fr * total), device=cum.device), right=True))
        bounds.append(min(max(r, bounds[-1]), blk))
    bounds.append(blk)
    return bounds, cnt


def _build_side(ptr, ind, edge_pos, local_ids, inv, rank, blk, n_pad, stages, want_ids, fractions=None) -> HaloSide:
    dev = ind.device
    rowsets = fractions is not None
    chunks = stages if rowsets else max(stages - 1, 1)
    pos, seg = _expand_segments(ptr, local_ids)
    other = inv[ind[pos].long()]                                   # relabelled id of the far end
    own = (other // blk) == rank
    uniq = torch.unique(other[~own])                               # ascending = (owner, row in block)
    if rowsets:
        bounds, seg_cnt = _set_bounds(seg, blk, fractions)
        set_of_seg = torch.bucketize(torch.arange(blk, device=dev), torch.tensor(bounds[1:-1], device=dev), right=True)
        set_of_entry = set_of_seg[seg]
        u_chunk = torch.full((uniq.numel(),), chunks, dtype=torch.long, device=dev)
        if uniq.numel():                                           # chunk = the first set that references the row
            u_chunk.scatter_reduce_(0, torch.searchsorted(uniq, other[~own]), set_of_entry[~own], reduce="amin")
    else:
        u_chunk = ((uniq % blk) * chunks) // blk                   # position slice inside the owner's block
    order = torch.argsort(u_chunk * n_pad + uniq)                  # chunk-major, then owner, then row
    place = torch.empty_like(order)
    place[order] = torch.arange(order.numel(), device=dev)         # halo row of uniq[i]
    codes = (((uniq // blk) << HALO_SHIFT) | (uniq % blk))[order].to(torch.int32).contiguous()
    counts = torch.bincount(u_chunk, minlength=chunks).tolist() if uniq.numel() else [0] * chunks
    chunk_off = [0]
    for c in counts:
        chunk_off.append(chunk_off[-1] + int(c))
    buf = other % blk
    stage = torch.zeros_like(other)
    if uniq.numel():
        rem = ~own
        hidx = torch.searchsorted(uniq, other[rem])
        buf[rem] = blk + place[hidx]
        if stages > 1 and not rowsets:
            stage[rem] = 1 + u_chunk[hidx]
    if rowsets:
        eid = pos if edge_pos is None else edge_pos[pos].long()
        ptrs, inds, ids = [], [], []
        for p_ in range(stages):
            r0, r1 = bounds[p_], bounds[p_ + 1]
            sp = torch.zeros(r1 - r0 + 1, dtype=torch.long, device=dev)
            torch.cumsum(seg_cnt[r0:r1], 0, out=sp[1:])
            m = set_of_entry == p_                                 # a contiguous run: entries are grouped by segment
            ptrs.append(sp.to(torch.int32))
            inds.append(buf[m].to(torch.int32).contiguous())
            if want_ids:
                ids.append(eid[m].to(torch.int32).contiguous())
        return HaloSide(int(uniq.numel()), codes, chunk_off, ptrs, inds, ids if want_ids else None, None, bounds)
    if stages > 8:
        raise ValueError("dgnn_b200: at most 8 stages (one bit per stage in the per-row stage mask)")
    ptrs, inds, ids = [], [], []
    smask = torch.zeros(blk, dtype=torch.long, device=dev)
    eid = pos if edge_pos is None else edge_pos[pos].long()
    for p in range(stages):
        m = stage == p
        cnt = torch.bincount(seg[m], minlength=blk)
        smask |= (cnt > 0).long() << p
        sp = torch.zeros(blk + 1, dtype=torch.long, device=dev)
        torch.cumsum(cnt, 0, out=sp[1:])
        ptrs.append(sp.to(torch.int32))
        inds.append(buf[m].to(torch.int32).contiguous())
        if want_ids:
            ids.append(eid[m].to(torch.int32).contiguous())
    return HaloSide(int(uniq.numel()), codes, chunk_off, ptrs, inds, ids if want_ids else None,
                    smask.to(torch.uint8).contiguous())


ROWSET_FRACTIONS = (0.08, 0.25, 0.55, 1.0)


def build_halo_shard(row_ptr, col_ind, rank, world, stages=3, seed=0, csr2csc=None, edge_ids=False,
                     relabel=True, schedule="staged", fractions=None) -> HaloShard:
    """Cut rank's pieces out of the global CSR (rows = destinations).  Every rank calls this with the same
    graph, seed and options.  `edge_ids` keeps, for every local entry, its position in the global CSR (needed
    for attention dropout: the mask of an edge is a function of that position, the same on the rank that
    holds the edge in its forward piece and on the rank that holds it in its backward piece).
    relabel=False keeps the node order (contiguous equal blocks).
    schedule="rowsets": sweep p finishes the rows (columns in the backward) of one range completely -- `fractions`
    = cumulative shares of the rank's entries per range, default ROWSET_FRACTIONS, `stages` is their number -- and
    needs the halo rows that ranges 0..p reference; nothing is carried between sweeps."""
    if schedule not in ("staged", "rowsets"):
        raise ValueError("dgnn_b200: schedule is 'staged' or 'rowsets'")
    if schedule == "rowsets":
        fractions = tuple(fractions) if fractions is not None else ROWSET_FRACTIONS
        if world == 1:
            fractions = (1.0,)
        if not fractions or abs(fractions[-1] - 1.0) > 1e-9 or any(b < a for a, b in zip(fractions, fractions[1:])):
            raise ValueError("dgnn_b200: fractions are cumulative shares ending in 1")
        stages = len(fractions)
    else:
        fractions = None
    if world > HALO_MAX_RANKS:
        raise ValueError(f"dgnn_b200: at most {HALO_MAX_RANKS} ranks")
    csr2csc = csr2csc or kernels.csr2csc
    dev = col_ind.device
    rp = row_ptr.long()
    n = rp.numel() - 1
    if col_ind.numel() >= 2**31:
        raise ValueError("dgnn_b200: edge positions are int32")
    blk = max(-(-n // world), 1)
    if blk > (1 << HALO_SHIFT):
        raise ValueError("dgnn_b200: block too large for the halo row codes")
    n_pad = world * blk
    order = torch.full((n_pad,), -1, dtype=torch.long)
    if relabel:
        g = torch.Generator(device="cpu").manual_seed(seed)
        order[:n] = torch.randperm(n, generator=g)
        order = order[torch.randperm(n_pad, generator=g)]            # padding spread over all blocks
    else:
        order[:n] = torch.arange(n)
    order = order.to(dev)
    inv = torch.empty(n, dtype=torch.long, device=dev)
    real = order >= 0
    inv[order[real]] = torch.arange(n_pad, device=dev)[real]
    local_ids = order[rank * blk: (rank + 1) * blk].contiguous()
    shard = HaloShard(rank, world, int(stages), n, blk, local_ids, schedule=schedule)
    shard.fwd = _build_side(rp, col_ind, None, local_ids, inv, rank, blk, n_pad, stages, edge_ids, fractions)
    col_ptr, row_ind, permute = csr2csc(row_ptr, col_ind)
    shard.bwd = _build_side(col_ptr.long(), row_ind, permute if edge_ids else None, local_ids, inv, rank, blk, n_pad,
                            stages, edge_ids, fractions)
    return shard


# ---------------------------------------------------------------------------
# transports: where the buffers live and how halo rows arrive
# ---------------------------------------------------------------------------
class _Done:
    def wait(self):
        pass


class _StreamEvent:
    """wait() orders the current stream after the event."""

    def __init__(self, event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)


def _decode(codes):
    c = codes.long()
    return c >> HALO_SHIFT, c & ((1 << HALO_SHIFT) - 1)


@dataclass
class SendPlan:
    """Who sends what to whom for one direction, derived from every rank's halo row list.

    The owner of a row packs it into its send buffer; the buffer is laid out chunk-major, then by
    requester, then in the requester's halo order, so that what rank g needs from owner s for chunk c is
    ONE contiguous range on both sides: send_off[s][c][g] in s's send buffer, recv rows in g's halo."""
    pack_idx: torch.Tensor      # [total_send] int32: rows of this rank's block in send-buffer order
    cap_send: int               # rows of the largest send buffer over all ranks
    recv: list                  # per chunk: [(owner, first halo row, rows, offset in the owner's send buffer)]
    fan_ptr: torch.Tensor = None   # [blk+1] int32: the inverse of pack_idx -- own row r goes to the send-buffer rows
    fan_pos: torch.Tensor = None   #   fan_pos[fan_ptr[r] : fan_ptr[r+1]] (kernels that produce the rows write them there)


def build_send_plan(me, world, chunks, codes_all, chunk_off_all, blk=None) -> SendPlan:
    """codes_all[g] / chunk_off_all[g]: HaloSide.codes and .chunk_off of every rank g (what g fetches); blk = rows
    per rank (for the inverse lists)."""
    dev = codes_all[me].device
    cnt = torch.zeros(world, chunks, world, dtype=torch.long)          # cnt[g][c][s]: rows g needs from s in chunk c
    mine = []                                                          # rows of my block, per (c, g)
    for g in range(world):
        owner, loc = _decode(codes_all[g])
        for c in range(chunks):
            lo, hi = int(chunk_off_all[g][c]), int(chunk_off_all[g][c + 1])
            o = owner[lo:hi]
            if hi > lo:
                cnt[g, c] = torch.bincount(o, minlength=world).cpu()
            mine.append((c, g, loc[lo:hi][o == me]))
    # send_off[s][c][g]: chunk-major, then requester
    per_sc = cnt.permute(2, 1, 0).contiguous()                         # [s][c][g]
    flat = per_sc.reshape(world, -1)
    send_off = (torch.cumsum(flat, 1) - flat).reshape(world, chunks, world)
    mine.sort(key=lambda t: (t[0], t[1]))
    pack_idx = torch.cat([t[2] for t in mine]).to(torch.int32).contiguous() if mine else torch.zeros(0, dtype=torch.int32, device=dev)
    recv = []
    for c in range(chunks):
        row = int(chunk_off_all[me][c])
        lst = []
        for s_ in range(world):                                        # halo rows of a chunk are sorted by owner
            k = int(cnt[me, c, s_])
            if k and s_ != me:
                lst.append((s_, row, k, int(send_off[s_, c, me])))
            row += k
        recv.append(lst)
    plan = SendPlan(pack_idx, int(flat.sum(1).max()), recv)
    if blk is not None:
        rows = pack_idx.long()
        order = torch.argsort(rows, stable=True)
        ptr = torch.zeros(blk + 1, dtype=torch.long, device=dev)
        if rows.numel():
            torch.cumsum(torch.bincount(rows, minlength=blk), 0, out=ptr[1:])
        plan.fan_ptr, plan.fan_pos = ptr.to(torch.int32).contiguous(), order.to(torch.int32).contiguous()
    return plan


class GatherTransport:
    """Fallback that needs nothing but torch.distributed collectives (gloo on CPU, NCCL without symmetric
    memory): the own blocks are all-gathered and the halo rows picked out of the result."""

    def __init__(self, shard, group=None):
        self.shard, self.group = shard, group
        self.caps = (shard.fwd.n_halo, shard.bwd.n_halo)

    def empty(self, tag, rows, tail, device):
        return torch.empty((rows,) + tuple(tail), dtype=torch.float32, device=device)

    def fan(self, side, bufs, tags):
        return None

    def publish(self, side, bufs, tags, packed=False):
        pass

    def start_pulls(self, side, bufs, tags):
        sh = self.shard
        owner, loc = _decode(side.codes)
        for buf in bufs:
            own = buf[:sh.blk].contiguous()
            full = own.new_empty((sh.world,) + tuple(own.shape))
            dist.all_gather_into_tensor(full.view(-1, *own.shape[1:]), own, group=self.group)
            buf[sh.blk: sh.blk + side.n_halo] = full[owner, loc]
        return [_Done() for _ in range(sh.chunks)]


class PeerTransport:
    """Halo rows taken out of the owners' memory, chunk by chunk, on a side stream.  Two modes:

    "dma"   the owner packs the rows each peer needs into a send buffer (kernels.halo_pull with itself as
            the only owner), a barrier follows, and every rank copies its contiguous ranges out of the
            peers' send buffers with plain device-to-device copies -- copy engines, no SM taken from the
            sweeps they run beside;
    "pull"  no packing: kernels.halo_pull reads the rows straight out of the owners' [own | halo] buffers
            with plain loads (over NVLink when the owner is another GPU).

    Sub-classes say where the peers' buffers are: `SymmetricTransport` (one process per GPU, torch.distributed
    symmetric memory) and `LocalTransport` (all ranks emulated in one process on one device, for tests)."""

    def __init__(self, shard, mode="dma", pull_ctas=0):
        if mode not in ("dma", "pull"):
            raise ValueError("mode must be 'dma' or 'pull'")
        self.shard, self.mode = shard, mode
        self.pull_ctas = int(pull_ctas)
        # True: packing and the barrier run on the side stream, beside the sweep over the own nodes (stage 0), instead
        # of in front of it on the compute stream
        self.overlap_publish = False
        self.stream = None
        self.status = None
        self.plans = None           # (forward SendPlan, backward SendPlan) in dma mode
        self.send = {}              # tag -> this rank's send buffer

    # -- provided by the sub-class --
    def peer_buffers(self, tag):
        """The buffer registered under `tag` on every rank (own tensor or peer mapping)."""
        raise NotImplementedError

    def shared_empty(self, tag, rows, tail, device):
        """A buffer that the other ranks can read; collective (same order on every rank)."""
        raise NotImplementedError

    def barrier(self):
        raise NotImplementedError

    # -- shared --
    def empty(self, tag, rows, tail, device):
        if self.mode == "pull":                                   # peers read the [own | halo] buffers themselves
            return self.shared_empty(tag, rows, tail, device)
        return torch.empty((rows,) + tuple(tail), dtype=torch.float32, device=device)

    def _plan(self, side):
        return self.plans[0] if side is self.shard.fwd else self.plans[1]

    def fan(self, side, bufs, tags):
        """For a kernel that produces the own rows of `bufs`: where each row goes in this rank's send buffers
        (kernels._fan_args), so that it can write the copies itself; None when nothing is to be packed this way.
        A caller that used it passes packed=True to publish()."""
        sh = self.shard
        if not (self.mode == "dma" and sh.world > 1 and bufs[0].is_cuda and len(bufs) == 2):
            return None
        plan = self._plan(side)
        if plan.fan_ptr is None or plan.pack_idx.numel() == 0:
            return None
        sends = self._sends(plan, bufs, tags)
        return dict(ptr=plan.fan_ptr, pos=plan.fan_pos, a=sends[0], b=sends[1])

    def _sends(self, plan, bufs, tags):
        out = []
        for buf, tag in zip(bufs, tags):
            if tag not in self.send:
                self.send[tag] = self.shared_empty(tag + ".send", max(plan.cap_send, 1), buf.shape[1:], buf.device)
            out.append(self.send[tag])
        return out

    def publish(self, side, bufs, tags, packed=False):
        """Own rows are written: make them available to the peers (pack in dma mode unless the producing kernel
        already did), then the barrier."""
        sh = self.shard
        cuda = bufs[0].is_cuda
        if packed:
            self.barrier()
            return
        if cuda and self.overlap_publish and sh.world > 1:
            dev = bufs[0].device
            if self.stream is None:
                self.stream = torch.cuda.Stream(device=dev, priority=-1)
            written = torch.cuda.Event()
            written.record(torch.cuda.current_stream(dev))
            with torch.cuda.stream(self.stream):
                self.stream.wait_event(written)
                self._pack(side, bufs, tags)
                self.barrier()
            return
        self._pack(side, bufs, tags)
        self.barrier()

    def _pack(self, side, bufs, tags):
        sh = self.shard
        if self.mode == "dma" and sh.world > 1:
            plan = self._plan(side)
            sends = self._sends(plan, bufs, tags)
            k = plan.pack_idx.numel()
            if k:
                if bufs[0].is_cuda:
                    own = [[b[:sh.blk]] for b in bufs]
                    kernels.halo_pull(plan.pack_idx, own[0], sends[0][:k], own[1] if len(bufs) > 1 else None,
                                      sends[1][:k] if len(bufs) > 1 else None, status=self._status(bufs[0].device))
                else:
                    for b, sbuf in zip(bufs, sends):
                        sbuf[:k] = b[:sh.blk][plan.pack_idx.long()]

    def _status(self, dev):
        if self.status is None:
            self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        return self.status

    def start_pulls(self, side, bufs, tags):
        sh = self.shard
        if side.n_halo == 0 or sh.world == 1:
            return [_Done() for _ in range(sh.chunks)]
        cuda = bufs[0].is_cuda
        if self.mode == "dma":
            srcs = [self.peer_buffers(t + ".send") for t in tags]
        else:
            srcs = [[s_[:sh.blk] for s_ in self.peer_buffers(t)] for t in tags]
        if not cuda:                                              # emulation on the CPU
            self._fetch_chunks(side, bufs, srcs, range(sh.chunks))
            return [_Done() for _ in range(sh.chunks)]
        dev = bufs[0].device
        if self.stream is None:
            self.stream = torch.cuda.Stream(device=dev, priority=-1)
        self._status(dev)
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(dev))
        works = []
        with torch.cuda.stream(self.stream):
            if not self.overlap_publish:
                self.stream.wait_event(ready)              # the barrier ran on the compute stream
            for c in range(sh.chunks):
                self._fetch_chunks(side, bufs, srcs, [c])
                ev = torch.cuda.Event()
                ev.record(self.stream)
                works.append(_StreamEvent(ev))
        return works

    def _fetch_chunks(self, side, bufs, srcs, chunks):
        sh = self.shard
        for c in chunks:
            if self.mode == "dma":
                lst = self._plan(side).recv[c]
                lst = lst[sh.rank % max(len(lst), 1):] + lst[:sh.rank % max(len(lst), 1)]   # ranks start at different owners
                for owner, row, k, off in lst:
                    for buf, src in zip(bufs, srcs):
                        buf[sh.blk + row: sh.blk + row + k].copy_(src[owner][off: off + k], non_blocking=True)
                continue
            lo, hi = side.chunk_off[c], side.chunk_off[c + 1]
            if hi <= lo:
                continue
            if bufs[0].is_cuda:
                dsts = [b[sh.blk + lo: sh.blk + hi] for b in bufs]
                kernels.halo_pull(side.codes[lo:hi], srcs[0], dsts[0], srcs[1] if len(bufs) > 1 else None,
                                  dsts[1] if len(bufs) > 1 else None, max_ctas=self.pull_ctas, status=self.status)
            else:
                owner, loc = _decode(side.codes[lo:hi])
                for buf, src in zip(bufs, srcs):
                    buf[sh.blk + lo: sh.blk + hi] = torch.stack(list(src), 0)[owner, loc]

    def check(self):
        """Raise if a fetch met a row code outside its owner's block (synchronises)."""
        if self.status is not None and int(self.status.item()) != 0:
            raise RuntimeError("dgnn_b200: a halo fetch skipped rows whose code lies outside the owner's block")


class LocalTransport(PeerTransport):
    """All ranks in one process on one device: `registry[rank][tag]` holds every emulated rank's buffers.  The
    caller runs the phases of all ranks in lockstep (prepare + publish on every rank, then sweep on every
    rank), which is what the barrier stands for.  Create one per rank with LocalTransport.for_all(shards)."""

    def __init__(self, shard, registry, mode="dma", pull_ctas=0):
        super().__init__(shard, mode, pull_ctas)
        self.registry = registry
        self.caps = None

    @classmethod
    def for_all(cls, shards, mode="dma", pull_ctas=0):
        registry = {}
        caps = (max(s.fwd.n_halo for s in shards), max(s.bwd.n_halo for s in shards))
        world, chunks = shards[0].world, shards[0].chunks
        out = []
        for s in shards:
            t = cls(s, registry, mode, pull_ctas)
            t.caps = caps
            if mode == "dma":
                t.plans = tuple(build_send_plan(s.rank, world, chunks, [getattr(x, d).codes for x in shards],
                                                [getattr(x, d).chunk_off for x in shards], s.blk) for d in ("fwd", "bwd"))
            out.append(t)
        return out

    def shared_empty(self, tag, rows, tail, device):
        buf = torch.empty((rows,) + tuple(tail), dtype=torch.float32, device=device)
        self.registry.setdefault(self.shard.rank, {})[tag] = buf
        return buf

    def peer_buffers(self, tag):
        return [self.registry[r][tag] for r in range(self.shard.world)]

    def barrier(self):
        pass


class SymmetricTransport(PeerTransport):
    """One process per GPU.  The buffers that peers read live in torch.distributed's symmetric memory (every
    rank maps every other rank's buffer over NVLink); the barrier is a one-element NCCL all-reduce on the compute
    stream.  Two barriers per training step (one per pass) also keep a rank from overwriting rows that a peer is
    still fetching: a rank's writes of pass k+1 come after its barrier of pass k, which every peer enters only
    after its own sweeps -- and therefore its fetches -- of the pass before.  No multicast object is created."""

    def __init__(self, shard, group=None, mode="dma", pull_ctas=0):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer reads only
        super().__init__(shard, mode, pull_ctas)
        self.group = group if group is not None else dist.group.WORLD
        dev = shard.local_ids.device
        world, chunks = shard.world, shard.chunks
        caps = torch.tensor([shard.fwd.n_halo, shard.bwd.n_halo], dtype=torch.int64, device=dev)
        dist.all_reduce(caps, op=dist.ReduceOp.MAX, group=self.group)     # symmetric buffers have one size on all ranks
        self.caps = (int(caps[0]), int(caps[1]))
        self.flag = torch.zeros(1, dtype=torch.float32, device=dev)
        self.peers = {}
        if mode == "dma":
            plans = []
            for side, cap in ((shard.fwd, self.caps[0]), (shard.bwd, self.caps[1])):
                # every rank learns every rank's halo row list (what it fetches, in which order)
                mine = torch.full((max(cap, 1),), -1, dtype=torch.int32, device=dev)
                mine[:side.n_halo] = side.codes
                codes = torch.empty((world, max(cap, 1)), dtype=torch.int32, device=dev)
                dist.all_gather_into_tensor(codes, mine, group=self.group)
                offs = torch.empty((world, chunks + 1), dtype=torch.int64, device=dev)
                dist.all_gather_into_tensor(offs, torch.tensor(side.chunk_off, dtype=torch.int64, device=dev), group=self.group)
                offs = offs.tolist()
                plans.append(build_send_plan(shard.rank, world, chunks, [codes[g, :offs[g][-1]] for g in range(world)], offs,
                                             shard.blk))
            self.plans = tuple(plans)

    def shared_empty(self, tag, rows, tail, device):
        import torch.distributed._symmetric_memory as symm
        shape = (rows,) + tuple(tail)
        buf = symm.empty(shape, dtype=torch.float32, device=device)
        handle = symm.rendezvous(buf, self.group)                          # collective: same order on every rank
        self.peers[tag] = [buf if q == self.shard.rank else handle.get_buffer(q, shape, torch.float32)
                           for q in range(self.shard.world)]
        return buf

    def peer_buffers(self, tag):
        return self.peers[tag]

    def barrier(self):
        dist.all_reduce(self.flag, group=self.group)


def make_transport(shard, group=None, mode="dma", pull_ctas=0):
    """SymmetricTransport on CUDA ranks when symmetric memory works on this platform, else GatherTransport."""
    if shard.world > 1 and shard.local_ids.is_cuda and dist.is_initialized() and dist.get_backend(group) == "nccl":
        try:
            t = SymmetricTransport(shard, group, mode, pull_ctas)
            t.shared_empty("probe", 16, (4,), shard.local_ids.device)      # collective probe: all ranks fail together
            return t
        except Exception as exc:
            import warnings
            warnings.warn(f"dgnn_b200: symmetric memory unavailable ({exc}); halo rows travel through all-gathers")
    return GatherTransport(shard, group)


# ---------------------------------------------------------------------------
# the sharded operator
# ---------------------------------------------------------------------------
class HaloContext:
    """Buffers and settings of one sharded GAT layer instance: [own | halo] buffers for the features and the
    source attention term (forward) and for grad_out and the row statistics (backward).  One forward may be
    in flight per context: the backward reads what the forward left in the buffers."""

    def __init__(self, shard, transport, heads, width, negative_slope=0.2, backend=kernels, tag="gat"):
        self.shard, self.transport, self.backend = shard, transport, backend
        self.h, self.f, self.slope = int(heads), int(width), float(negative_slope)
        dev = shard.local_ids.device
        cap_f, cap_b = transport.caps
        blk = shard.blk
        self.X = transport.empty(tag + ".x", blk + cap_f, (heads, width), dev)
        self.AC = transport.empty(tag + ".ac", blk + cap_f, (heads,), dev)
        self.G = transport.empty(tag + ".g", blk + cap_b, (heads, width), dev)
        self.PK = transport.empty(tag + ".pk", blk + cap_b, (heads, 4), dev)
        self.tags = (tag + ".x", tag + ".ac", tag + ".g", tag + ".pk")
        self.version = 0
        self.fuse_pack = True         # the kernels that produce the own rows also write their copies into the send buffers
        self.packed_fwd = self.packed_bwd = False
        self.exposed_ms = None        # a list: _timed_wait appends event pairs around every wait for a halo chunk

    @property
    def h_own(self):
        """[blk, H, F] tensor over the feature buffer's own rows: let the projection write here.  It shares the
        buffer's storage without being a view of it in autograd's eyes: an in-place write through a view makes
        autograd rebuild the gradient of the whole [own | halo] buffer in the backward (a zero fill and two copies
        of gigabytes); a tensor set on the storage has no base."""
        return self._own_rows((self.shard.blk,) + tuple(self.X.shape[1:]))

    @property
    def h_own_flat(self):
        """The same rows as [blk, H*F] (the shape the projection writes)."""
        return self._own_rows((self.shard.blk, self.h * self.f))

    def _own_rows(self, shape):
        X = self.X
        own = X.new_empty(0)
        stride = [1] * len(shape)
        for d in range(len(shape) - 2, -1, -1):
            stride[d] = stride[d + 1] * shape[d + 1]
        own.set_(X.untyped_storage(), X.storage_offset(), shape, tuple(stride))
        return own


def _masks(ctx, side, attn_drop, seed):
    if not attn_drop > 0.0:
        return [None] * len(side.ptr)
    if side.edge_id is None:
        raise RuntimeError("dgnn_b200: attention dropout on the sharded layer needs build_halo_shard(edge_ids=True)")
    return [ctx.backend.uniform_fill_edges(e, ctx.h, seed) for e in side.edge_id]


def halo_forward_prepare(ctx: HaloContext, h=None, attn_l=None, attn_r=None, attn_row=None, attn_col=None):
    """Write this rank's own rows of the forward buffers.  Layer form: h [blk,H,F] (copied unless it already is
    ctx.h_own) and the attention vectors -> logits computed here.  Operator form: attn_row / attn_col given."""
    blk = ctx.shard.blk
    if h.data_ptr() != ctx.X.data_ptr():
        ctx.X[:blk].copy_(h)
    ctx.packed_fwd = False
    if attn_l is not None:
        fan = ctx.transport.fan(ctx.shard.fwd, [ctx.X, ctx.AC], ctx.tags[0:2]) if ctx.fuse_pack else None
        kw = {"fan": fan} if fan is not None else {}
        attn_row, _ = ctx.backend.gat_logits_forward(ctx.X[:blk], attn_l, attn_r, out_col=ctx.AC[:blk], **kw)
        ctx.packed_fwd = fan is not None
    else:
        ctx.AC[:blk].copy_(attn_col)
    ctx.version += 1
    return attn_row


def halo_forward_sweep(ctx: HaloContext, attn_row, bias=None, attn_drop=0.0, seed=0, train=True):
    """Fetch the halo chunks and sweep the stages.  Returns (out, edge_max, edge_sum, out_neg, a_neg); the last
    four are None when train is False."""
    sh, be = ctx.shard, ctx.backend
    works = ctx.transport.start_pulls(sh.fwd, [ctx.X, ctx.AC], ctx.tags[0:2])
    masks = _masks(ctx, sh.fwd, attn_drop, seed)
    if sh.schedule == "rowsets":
        return _forward_rowsets(ctx, works, masks, attn_row, bias, attn_drop, train)
    state = be.gat_forward_state(sh.blk, ctx.h, ctx.f, ctx.X.device)
    waited, res = 0, None
    for p in range(sh.stages):
        while waited < sh.chunks and sh.chunk_stage(waited) <= p:
            _timed_wait(ctx, works[waited], "fwd", waited)
            waited += 1
        last = p == sh.stages - 1
        # rows are finished in the last stage in which they have edges (stage_mask), so the bias goes to every stage
        res = be.gat_forward_staged(attn_row, ctx.AC, sh.fwd.ptr[p], sh.fwd.ind[p], ctx.slope, ctx.X, state, p == 0, last,
                                    bias=bias, attn_drop=attn_drop, edge_mask=masks[p], neg=train,
                                    save_stats=train, stage_mask=sh.fwd.stage_mask, stage=p, outs=res)
    if train:
        return res
    return res[0], None, None, None, None


def _forward_rowsets(ctx, works, masks, attn_row, bias, attn_drop, train):
    """Sweep p finishes the rows bounds[p]:bounds[p+1] (all their edges) once halo chunks 0..p are there."""
    sh, be = ctx.shard, ctx.backend
    dev, blk, h, f = ctx.X.device, sh.blk, ctx.h, ctx.f
    out = torch.empty((blk, h, f), dtype=torch.float32, device=dev)
    stats = [torch.empty((blk, h), dtype=torch.float32, device=dev) for _ in range(2)] if train else [None, None]
    out_neg = torch.empty((blk, h, f), dtype=torch.float32, device=dev) if train else None
    a_neg = torch.empty((blk, h), dtype=torch.float32, device=dev) if train else None
    waited = 0
    for p in range(sh.stages):
        while waited < sh.chunks and sh.chunk_stage(waited) <= p:
            _timed_wait(ctx, works[waited], "fwd", waited)
            waited += 1
        r0, r1 = sh.fwd.bounds[p], sh.fwd.bounds[p + 1]
        if r1 == r0:
            continue
        cut = lambda t: None if t is None else t[r0:r1]
        be.gat_forward_staged(attn_row[r0:r1], ctx.AC, sh.fwd.ptr[p], sh.fwd.ind[p], ctx.slope, ctx.X, None, True, True,
                              bias=bias, attn_drop=attn_drop, edge_mask=masks[p], neg=train, save_stats=train,
                              outs=(out[r0:r1], cut(stats[0]), cut(stats[1]), cut(out_neg), cut(a_neg)))
    return out, stats[0], stats[1], out_neg, a_neg


def _backward_rowsets(ctx, works, masks, attn_drop):
    """Sweep p finishes the source columns bounds[p]:bounds[p+1] once halo chunks 0..p of grad_out / pack are there."""
    sh, be = ctx.shard, ctx.backend
    dev, blk, h, f = ctx.X.device, sh.blk, ctx.h, ctx.f
    grad_feat = torch.empty((blk, h, f), dtype=torch.float32, device=dev)
    grad_col = torch.empty((blk, h), dtype=torch.float32, device=dev)
    waited = 0
    for p in range(sh.stages):
        while waited < sh.chunks and sh.chunk_stage(waited) <= p:
            _timed_wait(ctx, works[waited], "bwd", waited)
            waited += 1
        c0, c1 = sh.bwd.bounds[p], sh.bwd.bounds[p + 1]
        if c1 == c0:
            continue
        be.gat_backward_cols_staged(None, sh.bwd.ptr[p], sh.bwd.ind[p], None, ctx.PK, ctx.X[c0:c1], ctx.AC[c0:c1], ctx.G,
                                    ctx.slope, None, True, True, attn_drop=attn_drop, edge_mask=masks[p], row_grad=False,
                                    outs=(grad_feat[c0:c1], grad_col[c0:c1]))
    return grad_feat, grad_col


def halo_backward_prepare(ctx: HaloContext, attn_row, edge_max, edge_sum, out, out_neg, a_neg, grad_out, bias=None):
    """Row statistics of the own rows into the backward buffers; returns (grad_attn_row, grad_bias)."""
    blk = ctx.shard.blk
    fan = ctx.transport.fan(ctx.shard.bwd, [ctx.G, ctx.PK], ctx.tags[2:4]) if ctx.fuse_pack else None
    kw = {"fan": fan} if fan is not None else {}
    _, grad_row, grad_bias = ctx.backend.gat_rowstat_full(attn_row, edge_max, edge_sum, out, grad_out, ctx.slope, bias=bias,
                                                          out_neg=out_neg, a_neg=a_neg, pack=ctx.PK[:blk],
                                                          grad_copy=ctx.G[:blk], **kw)
    ctx.packed_bwd = fan is not None
    return grad_row, grad_bias


def halo_backward_sweep(ctx: HaloContext, attn_drop=0.0, seed=0):
    """Fetch the halo chunks of grad_out / pack and sweep the stages over this rank's source columns.
    Returns (grad_feat [blk,H,F], grad_attn_col [blk,H])."""
    sh, be = ctx.shard, ctx.backend
    works = ctx.transport.start_pulls(sh.bwd, [ctx.G, ctx.PK], ctx.tags[2:4])
    masks = _masks(ctx, sh.bwd, attn_drop, seed)
    if sh.schedule == "rowsets":
        return _backward_rowsets(ctx, works, masks, attn_drop)
    state = be.gat_backward_state(sh.blk, ctx.h, ctx.f, ctx.X.device)
    waited = 0
    outs = None
    for p in range(sh.stages):
        while waited < sh.chunks and sh.chunk_stage(waited) <= p:
            _timed_wait(ctx, works[waited], "bwd", waited)
            waited += 1
        _, grad_feat, grad_col = be.gat_backward_cols_staged(
            None, sh.bwd.ptr[p], sh.bwd.ind[p], None, ctx.PK, ctx.X[:sh.blk], ctx.AC[:sh.blk], ctx.G, ctx.slope, state,
            p == 0, p == sh.stages - 1, attn_drop=attn_drop, edge_mask=masks[p], row_grad=False,
            stage_mask=sh.bwd.stage_mask, stage=p, outs=outs)
        outs = (grad_feat, grad_col)
    return outs


def _timed_wait(ctx, work, phase, chunk):
    """wait() for a halo chunk; with ctx.exposed_ms set, bracket it with events so that the time the compute
    stream spends waiting for the transfer can be reported."""
    if ctx.exposed_ms is None or not ctx.X.is_cuda:
        work.wait()
        return
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    work.wait()
    b.record()
    ctx.exposed_ms.append((phase, chunk, a, b))


def _timed_publish(ctx, phase, side, bufs, tags, packed):
    """transport.publish (packing, if it was not fused, and the barrier that makes the send buffers visible: the
    point where a rank waits for the slowest peer); bracketed like the chunk waits when ctx.exposed_ms is set."""
    if ctx.exposed_ms is None or not ctx.X.is_cuda:
        ctx.transport.publish(side, bufs, tags, packed=packed)
        return
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    ctx.transport.publish(side, bufs, tags, packed=packed)
    b.record()
    ctx.exposed_ms.append((phase, "publish_and_barrier", a, b))


class HaloGATFunction(torch.autograd.Function):
    """Fused GAT on this rank's block.  Layer form (logits=True): inputs (h, attn_l, attn_r, bias); operator form:
    (in_feat, attn_row, attn_col, None).  Output [blk,H,F] in HaloShard.local_ids order."""

    @staticmethod
    def forward(ctx, a, b, c, bias, hc, logits, attn_drop, seed):
        if logits:
            attn_row = halo_forward_prepare(hc, h=a.contiguous(), attn_l=b, attn_r=c)
        else:
            attn_row = halo_forward_prepare(hc, h=a.contiguous(), attn_row=b.contiguous(), attn_col=c.contiguous())
        _timed_publish(hc, "fwd", hc.shard.fwd, [hc.X, hc.AC], hc.tags[0:2], hc.packed_fwd)
        out, edge_max, edge_sum, out_neg, a_neg = halo_forward_sweep(hc, attn_row, bias, attn_drop, seed, train=True)
        ctx.save_for_backward(attn_row, edge_max, edge_sum, out, out_neg, a_neg, b, c,
                              bias if bias is not None else out.new_empty(0))
        ctx.hc, ctx.logits, ctx.has_bias, ctx.attn_drop, ctx.seed, ctx.version = hc, logits, bias is not None, attn_drop, seed, hc.version
        return out

    @staticmethod
    def backward(ctx, grad_out):
        hc = ctx.hc
        if hc.version != ctx.version:
            raise RuntimeError("dgnn_b200: the sharded layer ran another forward before this backward; its buffers "
                               "hold one forward at a time (use one HaloContext / layer per use in the graph)")
        attn_row, edge_max, edge_sum, out, out_neg, a_neg, b, c, bias = ctx.saved_tensors
        grad_row, grad_bias = halo_backward_prepare(hc, attn_row, edge_max, edge_sum, out, out_neg, a_neg,
                                                    grad_out.contiguous(), bias if ctx.has_bias else None)
        _timed_publish(hc, "bwd", hc.shard.bwd, [hc.G, hc.PK], hc.tags[2:4], hc.packed_bwd)
        grad_feat, grad_col = halo_backward_sweep(hc, ctx.attn_drop, ctx.seed)
        if grad_bias is not None:
            grad_bias = grad_bias.view_as(bias)
        if ctx.logits:
            grad_l, grad_r = hc.backend.gat_logits_backward(hc.h_own, b, c, grad_row, grad_col, grad_feat)
            return grad_feat, grad_l.view_as(b), grad_r.view_as(c), grad_bias, None, None, None, None
        return grad_feat, grad_row, grad_col, grad_bias, None, None, None, None


def sharded_gat(attn_row, attn_col, in_feat, hc: HaloContext, attn_drop=0.0, seed=0):
    """The fused operator (GATConvFuse of the reference, operators/fused_gatconv.py:6-34) on this rank's block:
    attn_row, attn_col [blk,H], in_feat [blk,H,F] in HaloShard.local_ids order; differentiable in all three."""
    return HaloGATFunction.apply(in_feat, attn_row, attn_col, None, hc, False, float(attn_drop), int(seed))


def sharded_gat_layer(h, attn_l, attn_r, hc: HaloContext, bias=None, attn_drop=0.0, seed=0):
    """Attention logits + sharded aggregation (+ bias in the last sweep's epilogue) as one autograd node."""
    return HaloGATFunction.apply(h, attn_l, attn_r, bias, hc, True, float(attn_drop), int(seed))


# ---------------------------------------------------------------------------
# the layer
# ---------------------------------------------------------------------------
class ShardedGATConv(torch.nn.Module):
    """GATConv of the reference (layers/gatconv_layer.py:7-92: same constructor arguments, parameter names,
    initialisation, residual / bias / activation order) on one rank's node block of a HaloShard.

    forward(feat) takes the input features of the rank's own nodes [blk, in_feats] in HaloShard.local_ids
    order (HaloShard.scatter_rows of a global tensor) and returns [blk, heads, out_feats] in the same order.
    Parameters are replicated: call allreduce_grads() after backward (one flat all-reduce).  Attention dropout
    draws the mask of an edge from (seed, step, position of the edge in the whole graph's CSR), so every rank
    sees the same mask for an edge; it needs build_halo_shard(edge_ids=True)."""

    def __init__(self, in_feats, out_feats, num_heads, shard, feat_drop=0., attn_drop=0., negative_slope=0.2,
                 residual=False, activation=None, bias=True, group=None, transport=None, seed=0):
        super().__init__()
        from .layers.gatconv_layer import GATConv
        proto = GATConv(in_feats, out_feats, num_heads, feat_drop, attn_drop, negative_slope, residual, activation, bias)
        self.in_feats, self.out_feats, self.num_heads = in_feats, out_feats, num_heads
        self.negative_slope, self.attn_drop, self.activation = negative_slope, attn_drop, activation
        self.W, self.attn_l, self.attn_r = proto.W, proto.attn_l, proto.attn_r
        self.feat_drop = proto.feat_drop
        if proto.bias is not None:
            self.bias = proto.bias
        else:
            self.register_buffer("bias", None)
        if proto.res_fc is not None:
            self.res_fc = proto.res_fc
        else:
            self.register_buffer("res_fc", None)
        self.shard, self.group = shard, group
        self.transport = transport if transport is not None else make_transport(shard, group)
        self.hc = None
        self.seed, self.step = int(seed), 0

    def _context(self):
        if self.hc is None:
            self.hc = HaloContext(self.shard, self.transport, self.num_heads, self.out_feats, self.negative_slope)
        return self.hc

    def forward(self, feat):
        from .operators.projection import project
        hc = self._context()
        heads, width = self.num_heads, self.out_feats
        plain = self.feat_drop.p == 0.0 or not self.training
        h = project(feat, self.W, out=hc.h_own_flat if plain else None)
        h = self.feat_drop(h.view(-1, heads, width))
        fuse_bias = self.bias is not None and self.res_fc is None
        self.step += 1
        if self.training and torch.is_grad_enabled():
            rst = sharded_gat_layer(h, self.attn_l, self.attn_r, hc, self.bias if fuse_bias else None,
                                    self.attn_drop, self.seed * 1000003 + self.step)
        else:
            with torch.no_grad():
                attn_row = halo_forward_prepare(hc, h=h.contiguous(), attn_l=self.attn_l, attn_r=self.attn_r)
                hc.transport.publish(hc.shard.fwd, [hc.X, hc.AC], hc.tags[0:2], packed=hc.packed_fwd)
                rst = halo_forward_sweep(hc, attn_row, self.bias if fuse_bias else None, train=False)[0]
        if self.res_fc is not None:
            rst = rst + self.res_fc(h).view(-1, heads, width)       # as in the reference: applied to the projected features
        if self.bias is not None and not fuse_bias:
            rst = rst + self.bias.view(-1, heads, width)
        return self.activation(rst) if self.activation else rst

    def allreduce_grads(self):
        """Sum the parameter gradients over the ranks with one all-reduce of a flat buffer."""
        ps = [p for p in self.parameters() if p.grad is not None]
        if not ps or self.shard.world == 1 or not dist.is_initialized():
            return
        flat = torch.cat([p.grad.reshape(-1) for p in ps])
        dist.all_reduce(flat, group=self.group)
        off = 0
        for p in ps:
            p.grad.copy_(flat[off: off + p.numel()].view_as(p.grad))
            off += p.numel()


# ---------------------------------------------------------------------------
# EdgeConv: batched point clouds are split by batch
# ---------------------------------------------------------------------------
def split_clouds(points, k, rank, world, knn=None):
    """Deal the clouds of a batch [B,P,D] to the ranks (contiguous, as equal as possible) and build this
    rank's kNN graph with ids local to its points: returns (points_loc [B_loc,P,D], src_ind [B_loc*P*k] int32,
    (b0, b1)).  Clouds never share edges (the caller-side loop of script/train/train_edgeconv.py:48-52 builds
    one kNN graph per batch), so EdgeConv on the pieces needs no exchange: the per-rank outputs concatenated in
    rank order equal the single-GPU result bit for bit."""
    from . import graph
    b = points.shape[0]
    b0, b1 = (b * rank) // world, (b * (rank + 1)) // world
    loc = points[b0:b1].contiguous()
    knn = knn or graph.knn_graph
    src = knn(loc, k) if b1 > b0 else torch.zeros(0, dtype=torch.int32, device=points.device)
    return loc, src, (b0, b1)
