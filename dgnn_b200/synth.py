"""Seeded synthetic graphs with the shapes of the benchmark configurations.

The public citation / Reddit / ModelNet40 data the reference trains on is not
available offline; these generators reproduce only sizes, degree skew and value
distributions.  CSR rows are destination nodes and columns are source nodes,
column ids sorted inside a row (the layout the reference builds with scipy,
script/train/train_gatconv.py:78-94).
"""
from __future__ import annotations

import math

import numpy as np
import torch


def csr_from_edges(dst: np.ndarray, src: np.ndarray, n: int, ptr_dtype=np.int32):
    """Sort (dst, src) pairs and build CSR; duplicates are kept."""
    order = np.lexsort((src, dst))
    dst, src = dst[order], src[order]
    row_ptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(dst, minlength=n), out=row_ptr[1:])
    return torch.from_numpy(row_ptr.astype(ptr_dtype)), torch.from_numpy(src.astype(np.int32))


def powerlaw_graph(n=2708, n_pairs=5278, seed=1, exponent=2.5, self_loops=True):
    """Undirected Chung-Lu style graph: `n_pairs` distinct node pairs drawn with
    power-law weights, symmetrised (2*n_pairs directed edges), self-loops removed
    and then added once per node.  Returns (row_ptr int32, col_ind int32)."""
    rng = np.random.default_rng(seed)
    w = (np.arange(1, n + 1, dtype=np.float64)) ** (-1.0 / (exponent - 1.0))
    w = rng.permutation(w / w.sum())
    pairs = set()
    while len(pairs) < n_pairs:
        need = n_pairs - len(pairs)
        a = rng.choice(n, size=2 * need + 16, p=w)
        b = rng.choice(n, size=2 * need + 16, p=w)
        for x, y in zip(a.tolist(), b.tolist()):
            if x != y:
                pairs.add((min(x, y), max(x, y)))
                if len(pairs) == n_pairs:
                    break
    p = np.array(sorted(pairs), dtype=np.int64)
    dst = np.concatenate([p[:, 0], p[:, 1]])
    src = np.concatenate([p[:, 1], p[:, 0]])
    if self_loops:
        dst = np.concatenate([dst, np.arange(n)])
        src = np.concatenate([src, np.arange(n)])
    return csr_from_edges(dst, src, n)


def random_graph(n, avg_deg, seed, long_rows=(), empty_rows=True, ptr_dtype=np.int32):
    """Uniform random multigraph for tests; `long_rows` = [(row, degree), ...] plants
    rows of a given degree (to cross the 32-edge tiles and the long-row split)."""
    rng = np.random.default_rng(seed)
    deg = rng.poisson(avg_deg, size=n).astype(np.int64)
    if empty_rows and n > 2:
        deg[rng.integers(0, n, size=max(1, n // 10))] = 0
    for r, d in long_rows:
        deg[r] = d
    dst = np.repeat(np.arange(n, dtype=np.int64), deg)
    src = rng.integers(0, n, size=int(deg.sum()), dtype=np.int64)
    return csr_from_edges(dst, src, n, ptr_dtype)


def rmat_edges(scale, n_edges, seed, a=0.57, b=0.19, c=0.19, device="cpu", chunk=1 << 24):
    """R-MAT edge list (dst, src) over 2^scale ids, generated in chunks on `device`."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    dst_parts, src_parts = [], []
    for start in range(0, n_edges, chunk):
        m = min(chunk, n_edges - start)
        dst = torch.zeros(m, dtype=torch.int64, device=device)
        src = torch.zeros(m, dtype=torch.int64, device=device)
        for _ in range(scale):
            u = torch.rand(m, generator=g, device=device)
            # quadrant a: (0,0)  b: (0,1)  c: (1,0)  d: (1,1)   [dst bit, src bit]
            dbit = (u >= a + b).to(torch.int64)
            sbit = (((u >= a) & (u < a + b)) | (u >= a + b + c)).to(torch.int64)
            dst = dst * 2 + dbit
            src = src * 2 + sbit
        dst_parts.append(dst)
        src_parts.append(src)
    return torch.cat(dst_parts), torch.cat(src_parts)


def rmat_graph(n_nodes, n_edges, seed, device="cpu", ptr_dtype=torch.int64):
    """R-MAT graph folded onto `n_nodes` ids (id mod n_nodes), sorted by (dst, src),
    duplicates kept.  Returns (row_ptr, col_ind int32) on `device`."""
    scale = max(1, math.ceil(math.log2(max(n_nodes, 2))))
    dst, src = rmat_edges(scale, n_edges, seed, device=device)
    dst %= n_nodes
    src %= n_nodes
    key = dst * n_nodes + src
    del dst, src
    key, _ = torch.sort(key)
    dst = torch.div(key, n_nodes, rounding_mode="floor")
    col = (key - dst * n_nodes).to(torch.int32)
    del key
    counts = torch.bincount(dst, minlength=n_nodes)
    del dst
    row_ptr = torch.zeros(n_nodes + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=row_ptr[1:])
    return row_ptr.to(ptr_dtype), col


def unit_sphere_clouds(batch, points, seed, device="cpu"):
    """`batch` clouds of `points` 3-D points, U(-1,1), centred and scaled into the unit sphere."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    x = torch.rand(batch, points, 3, generator=g) * 2 - 1
    x = x - x.mean(dim=1, keepdim=True)
    x = x / x.norm(dim=2).amax(dim=1)[:, None, None]
    return x.to(device)


def knn_src_ind(x, k):
    """Per-cloud kNN (self included); returns src_ind [B*P*k] int32 with global ids:
    neighbours of point i are src_ind[i*k:(i+1)*k]."""
    b, p, _ = x.shape
    d = torch.cdist(x, x)
    idx = d.topk(k, dim=2, largest=False).indices            # [B,P,k]
    idx = idx + (torch.arange(b, device=x.device) * p)[:, None, None]
    return idx.reshape(-1).to(torch.int32)


def monet_pseudo(row_ptr, col_ind):
    """pseudo[e] = (deg(src)^-1/2, deg(dst)^-1/2) in CSR edge order
    (recipe of script/train/train_gmmconv.py:120-122 of the reference)."""
    rp = row_ptr.long()
    n = rp.numel() - 1
    deg = (rp[1:] - rp[:-1]).clamp(min=1).float()
    rows = torch.repeat_interleave(torch.arange(n, device=rp.device), rp[1:] - rp[:-1])
    return torch.stack([deg[col_ind.long()].rsqrt(), deg[rows].rsqrt()], dim=1).contiguous()


def xavier_uniform(shape, fan_in, fan_out, gen):
    bound = math.sqrt(6.0 / (fan_in + fan_out))
    return (torch.rand(shape, generator=gen) * 2 - 1) * bound
