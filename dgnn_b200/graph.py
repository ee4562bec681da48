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
    """Edge list (src[e] -> dst[e], any order, duplicates kept) -> CSR + CSC + permute, all by this library's
    kernels: dgnn_coo_sort orders the edges by (dst, src), dgnn_coo2csr gives the row pointer and dgnn_csr2csc the
    CSC form."""
    if not (src.is_cuda and dst.is_cuda):
        raise RuntimeError("dgnn_b200: build_graph works on CUDA tensors (there is no CPU path)")
    if num_nodes >= 2**31:
        raise RuntimeError("dgnn_b200: node ids are int32")
    src, dst = src.to(torch.int32), dst.to(torch.int32)
    if add_self_loops:
        keep = src != dst
        loops = torch.arange(num_nodes, device=src.device, dtype=torch.int32)
        src, dst = torch.cat([src[keep], loops]), torch.cat([dst[keep], loops])
    rows, col_ind = kernels.coo_sort(dst, src, num_nodes)
    row_ptr = kernels.coo2csr(rows, num_nodes, ptr_dtype)
    col_ptr, row_ind, permute = kernels.csr2csc(row_ptr, col_ind)
    return Graph(row_ptr, col_ind, col_ptr, row_ind, permute)


def knn_graph(points, k):
    """points [B,P,D] (one cloud per batch entry) -> src_ind [B*P*k] int32 with global ids;
    neighbours of point i are src_ind[i*k:(i+1)*k] in ascending distance, the point itself first (distance 0),
    ties to the smaller index (dgnn_knn_graph)."""
    if not points.is_cuda:
        raise RuntimeError("dgnn_b200: knn_graph works on CUDA tensors (there is no CPU path)")
    return kernels.knn_graph(points.float().contiguous(), k)
