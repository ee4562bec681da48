"""ctypes binding of libdgnn_b200.so (the C ABI declared in include/dgnn_b200.h).

PyTorch is used only for device memory and streams: wrappers allocate outputs
and workspaces with torch.empty on the inputs' device and pass raw pointers and
the current stream.  There is no CPU path: a missing library or a non-CUDA
tensor raises.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.environ.get("DGNN_B200_LIB", os.path.join(_HERE, "libdgnn_b200.so"))
_lib = None
_lock = threading.Lock()

c_i64 = ctypes.c_int64
c_int = ctypes.c_int
c_f = ctypes.c_float
c_p = ctypes.c_void_p
c_sz = ctypes.c_size_t
c_u64 = ctypes.c_uint64

# name -> (restype, argtypes); must list every symbol of include/dgnn_b200.h
SIGNATURES = {
    "dgnn_version": (c_int, []),
    "dgnn_status_string": (ctypes.c_char_p, [c_int]),
    "dgnn_seg_chunk": (c_i64, []),
    "dgnn_check_ptr": (c_int, [c_i64, c_i64, c_p, c_int, c_p, c_p]),
    "dgnn_check_index": (c_int, [c_i64, c_p, c_i64, c_p, c_p]),
    "dgnn_gat_forward_workspace_bytes": (c_sz, [c_i64, c_i64, c_int, c_int]),
    "dgnn_gat_forward": (c_int, [c_i64, c_i64, c_int, c_int, c_p, c_int, c_p, c_p, c_p, c_p, c_f, c_f, c_p,
                                 c_p, c_p, c_p, c_p, c_sz, c_p]),
    "dgnn_gat_forward_state_bytes": (c_sz, [c_i64, c_int, c_int]),
    "dgnn_gat_fast_shape": (c_int, [c_int, c_int]),
    "dgnn_gat_forward_staged": (c_int, [c_i64, c_i64, c_int, c_int, c_p, c_int, c_p, c_p, c_p, c_p, c_f, c_f, c_p,
                                        c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_int, c_int, c_p, c_int, c_p, c_p, c_sz, c_p]),
    "dgnn_gat_rowstat_full": (c_int, [c_i64, c_int, c_int, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_f, c_p, c_p,
                                      c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_sz, c_p]),
    "dgnn_gat_logits_forward_fan": (c_int, [c_i64, c_int, c_int, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p]),
    "dgnn_gat_backward_cols_workspace_bytes": (c_sz, [c_i64, c_int, c_int, c_int]),
    "dgnn_gat_rowstat_bias_workspace_bytes": (c_sz, [c_int, c_int]),
    "dgnn_gat_rowstat_bias": (c_int, [c_i64, c_int, c_int, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_sz, c_p]),
    "dgnn_gat_backward_state_bytes": (c_sz, [c_i64, c_int, c_int]),
    "dgnn_gat_backward_cols_staged": (c_int, [c_i64, c_i64, c_i64, c_int, c_int, c_p, c_p, c_int, c_p, c_p, c_p, c_p,
                                              c_p, c_p, c_p, c_f, c_f, c_p, c_p, c_p, c_p, c_int, c_int, c_p, c_int, c_p, c_p, c_sz,
                                              c_p]),
    "dgnn_hot_rows_workspace_bytes": (c_sz, []),
    "dgnn_l2_set_aside": (c_i64, [c_i64]),
    "dgnn_hot_rows": (c_int, [c_i64, c_p, c_int, c_i64, c_p, c_p, c_sz, c_p]),
    "dgnn_gat_rowstat": (c_int, [c_i64, c_int, c_int, c_p, c_p, c_p, c_p, c_p, c_p, c_p]),
    "dgnn_gat_backward_workspace_bytes": (c_sz, [c_i64, c_i64, c_i64, c_int, c_int]),
    "dgnn_gat_backward_cols": (c_int, [c_i64, c_i64, c_i64, c_int, c_int, c_p, c_p, c_int, c_p, c_p, c_p, c_p,
                                       c_p, c_p, c_p, c_f, c_f, c_p, c_p, c_p, c_p, c_sz, c_p]),
    "dgnn_gat_backward": (c_int, [c_i64, c_i64, c_int, c_int, c_p, c_p, c_int, c_p, c_p, c_p, c_p, c_p, c_p, c_p,
                                  c_p, c_p, c_p, c_f, c_f, c_p, c_p, c_p, c_p, c_sz, c_p]),
    "dgnn_gat_logits_forward": (c_int, [c_i64, c_int, c_int, c_p, c_p, c_p, c_p, c_p, c_p]),
    "dgnn_gat_logits_backward_workspace_bytes": (c_sz, [c_int, c_int]),
    "dgnn_gat_logits_backward": (c_int, [c_i64, c_int, c_int, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_sz, c_p]),
    "dgnn_project_supported": (c_int, [c_i64, c_int, c_int]),
    "dgnn_project_workspace_bytes": (c_sz, [c_int]),
    "dgnn_project_forward": (c_int, [c_i64, c_int, c_int, c_p, c_p, c_int, c_p, c_p, c_sz, c_p]),
    "dgnn_project_wgrad_workspace_bytes": (c_sz, [c_int]),
    "dgnn_project_wgrad": (c_int, [c_i64, c_int, c_int, c_p, c_p, c_p, c_int, c_p, c_sz, c_p]),
    "dgnn_project_status": (c_int, [c_p, c_p, c_p]),
    "dgnn_project_sticky_status": (c_int, [c_p, c_p, c_p, c_int]),
    "dgnn_project_set_test_knobs": (c_int, [c_i64, c_int]),
    "dgnn_uniform_fill": (c_int, [c_u64, c_u64, c_i64, c_p, c_p]),
    "dgnn_uniform_fill_edges": (c_int, [c_u64, c_u64, c_i64, c_int, c_p, c_p, c_p]),
    "dgnn_halo_max_ranks": (c_int, []),
    "dgnn_halo_rank_shift": (c_int, []),
    "dgnn_halo_pull": (c_int, [c_i64, c_p, c_int, c_i64, c_p, c_p, c_int, c_p, c_p, c_int, c_int, c_p, c_p]),
    "dgnn_mhsddmm_workspace_bytes": (c_sz, []),
    "dgnn_mhsddmm": (c_int, [c_i64, c_i64, c_int, c_int, c_p, c_int, c_p, c_p, c_p, c_p, c_p, c_sz, c_p]),
    "dgnn_coo_sddmm": (c_int, [c_i64, c_int, c_p, c_p, c_p, c_p, c_p, c_p]),
    "dgnn_mhtranspose": (c_int, [c_i64, c_int, c_p, c_p, c_p, c_p]),
    "dgnn_gmm_forward_workspace_bytes": (c_sz, [c_i64, c_i64, c_int, c_int]),
    "dgnn_gmm_forward": (c_int, [c_i64, c_i64, c_int, c_int, c_int, c_p, c_int, c_p, c_p, c_p, c_p, c_p, c_p,
                                 c_p, c_sz, c_p]),
    "dgnn_gaussian": (c_int, [c_i64, c_int, c_int, c_p, c_p, c_p, c_p, c_p]),
    "dgnn_gaussian_bp_workspace_bytes": (c_sz, [c_i64, c_int, c_int]),
    "dgnn_gaussian_bp": (c_int, [c_i64, c_int, c_int, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_p, c_sz, c_p]),
    "dgnn_edgeconv_forward": (c_int, [c_i64, c_int, c_int, c_p, c_p, c_p, c_p, c_p, c_p]),
    "dgnn_edgeconv_backward": (c_int, [c_i64, c_int, c_p, c_p, c_p, c_p]),
    "dgnn_edgeconv_backward_ordered": (c_int, [c_i64, c_int, c_p, c_p, c_p, c_p, c_p, c_p]),
    "dgnn_csr2csc_workspace_bytes": (c_sz, [c_i64, c_i64, c_i64]),
    "dgnn_csr2csc": (c_int, [c_i64, c_i64, c_i64, c_p, c_int, c_p, c_p, c_p, c_p, c_p, c_sz, c_p]),
    "dgnn_csr2csc_static_max_nnz": (c_i64, []),
    "dgnn_csr2csc_static_max_cols": (c_i64, []),
    "dgnn_csr2csc_static": (c_int, [c_i64, c_i64, c_i64, c_p, c_int, c_p, c_p, c_p, c_p, c_p]),
    "dgnn_coo2csr": (c_int, [c_i64, c_i64, c_p, c_p, c_int, c_p]),
    "dgnn_coo_sort_workspace_bytes": (c_sz, [c_i64, c_i64]),
    "dgnn_coo_sort": (c_int, [c_i64, c_i64, c_p, c_p, c_p, c_p, c_p, c_sz, c_p]),
    "dgnn_knn_max_k": (c_int, []),
    "dgnn_knn_graph": (c_int, [c_i64, c_i64, c_int, c_int, c_p, c_p, c_p]),
}


def lib():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(_LIB_PATH):
                    raise RuntimeError(
                        f"dgnn_b200: CUDA library not found at {_LIB_PATH}; build it with "
                        "`python -m dgnn_b200.build` (there is no CPU fallback)")
                handle = ctypes.CDLL(_LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)  # AttributeError if the symbol is missing
                    fn.restype = res
                    fn.argtypes = args
                _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = lib().dgnn_status_string(status).decode()
        raise RuntimeError(f"dgnn_b200.{what} failed with status {status}: {msg}")


# ---------------------------------------------------------------------------
# argument helpers
# ---------------------------------------------------------------------------
def _cuda_f32(t: torch.Tensor, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"dgnn_b200: {name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != torch.float32:
        raise RuntimeError(f"dgnn_b200: {name} must be float32, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def _cuda_i32(t: torch.Tensor, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"dgnn_b200: {name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != torch.int32:
        raise RuntimeError(f"dgnn_b200: {name} must be int32, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


def _cuda_ptr(t: torch.Tensor, name: str):
    """Index-pointer array: int32 or int64; returns (tensor, idx_bits)."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"dgnn_b200: {name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype == torch.int32:
        bits = 32
    elif t.dtype == torch.int64:
        bits = 64
    else:
        raise RuntimeError(f"dgnn_b200: {name} must be int32 or int64, got {t.dtype}")
    return (t if t.is_contiguous() else t.contiguous()), bits


def _same_bits(a_bits: int, b: torch.Tensor, name: str) -> torch.Tensor:
    want = torch.int32 if a_bits == 32 else torch.int64
    if b.dtype != want:
        b = b.to(want)
    return b


def _p(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(dev) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _workspace(nbytes: int, dev) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=dev)


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NO_GUARD = _NoGuard()


def device_guard(dev):
    """Make `dev` current for allocations and launches; free when it already is (the usual case)."""
    if torch.cuda.current_device() == (dev.index if dev.index is not None else torch.cuda.current_device()):
        return _NO_GUARD
    return torch.cuda.device(dev)
