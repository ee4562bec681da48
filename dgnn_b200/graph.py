"""Graph preparation on the device: the arrays the fused operators take, built
from an edge list without leaving the GPU.  Replaces the scipy recipe of the
reference's training scripts (script/train/train_gatconv.py:78-94: CSR with
rows = destinations, tocsc(), permutation through a data array) and DGL's
KNNGraph for the point-cloud model (script/train/train_edgeconv.py:49)."""
from __future__ import annotations

from typing import NamedTuple

import torch

from . import kernels


class Graph(NamedTuple):
    row_ptr: torch.Tensor    # [N+1]  CSR over destination rows
    col_ind: torch.Tensor    # [E]    source id of every CSR entry, sorted inside a row
    col_ptr: torch.Tensor    # [N+1]  CSC over source columns
    row_ind: torch.Tensor    # [E]    destination id of every CSC entry
    permute: torch.Tensor    # [E]    CSR position of every CSC entry


def build_graph(src, dst, num_nodes, ptr_dtype=torch.int32, add_self_loops=False) -> Graph:
    """Edge list (src[e] -> dst[e], any order, duplicates kept) -> CSR + CSC + permute.
    The sort by (dst, src) is a torch sort of one 64-bit key per edge; the row pointer
    comes from dgnn_coo2csr and the CSC form from dgnn_csr2csc."""
    if not (src.is_cuda and dst.is_cuda):
        raise RuntimeError("dgnn_b200: build_graph works on CUDA tensors (there is no CPU path)")
    src, dst = src.long(), dst.long()
    if add_self_loops:
        keep = src != dst
        loops = torch.arange(num_nodes, device=src.device)
        src, dst = torch.cat([src[keep], loops]), torch.cat([dst[keep], loops])
    key, _ = torch.sort(dst * num_nodes + src)
    rows = torch.div(key, num_nodes, rounding_mode="floor")
    col_ind = (key - rows * num_nodes).to(torch.int32)
    row_ptr = kernels.coo2csr(rows.to(torch.int32), num_nodes, ptr_dtype)
    col_ptr, row_ind, permute = kernels.csr2csc(row_ptr, col_ind)
    return Graph(row_ptr, col_ind, col_ptr, row_ind, permute)


def knn_graph(points, k, chunk=8):
    """points [B,P,D] (one cloud per batch entry) -> src_ind [B*P*k] int32 with global ids;
    neighbours of point i are src_ind[i*k:(i+1)*k], the point itself included (distance 0).
    Brute force per cloud (cdist + topk), `chunk` clouds at a time."""
    b, p, _ = points.shape
    out = []
    for s in range(0, b, chunk):
        x = points[s: s + chunk]
        idx = torch.cdist(x, x).topk(k, dim=2, largest=False).indices
        idx = idx + (torch.arange(s, s + x.shape[0], device=points.device) * p)[:, None, None]
        out.append(idx.reshape(-1))
    return torch.cat(out).to(torch.int32)
