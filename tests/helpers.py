"""Shared helpers of the test-suite."""
import numpy as np
import torch

RTOL, ATOL = 1e-4, 1e-5   # fp32 tolerance of the reference's own functional scripts


def assert_close(a, b, what, rtol=RTOL, atol=ATOL):
    a = a.detach().cpu().double()
    b = b.detach().cpu().double()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    if a.numel() == 0:
        return
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    assert not bool(bad.any()), (f"{what}: {int(bad.sum())}/{a.numel()} elements differ; max abs err "
                                 f"{float(err.max()):.3e}, worst ratio {float((err / tol).max()):.2f}")


def assert_equal(a, b, what):
    a = a.detach().cpu()
    b = b.detach().cpu()
    assert a.shape == b.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    assert torch.equal(a.long() if not a.is_floating_point() else a, b.long() if not b.is_floating_point() else b), \
        f"{what}: not bit-equal"


def gat_inputs(row_ptr, n, h, f, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    attn_row = torch.randn(n, h, generator=g) * scale
    attn_col = torch.randn(n, h, generator=g) * scale
    in_feat = torch.randn(n, h, f, generator=g)
    grad_out = torch.randn(n, h, f, generator=g)
    return attn_row, attn_col, in_feat, grad_out


def scipy_csc(row_ptr, col_ind, n_cols=None):
    """col_ptr, row_ind, permute exactly as the reference's data preparation builds
    them (script/train/train_gatconv.py:78-94): scipy CSR with data = CSR position,
    then tocsc()."""
    import scipy.sparse as sp
    rp = row_ptr.cpu().numpy().astype(np.int64)
    ci = col_ind.cpu().numpy().astype(np.int64)
    n_rows = rp.shape[0] - 1
    n_cols = n_rows if n_cols is None else n_cols
    data = np.arange(ci.shape[0], dtype=np.int64)
    csr = sp.csr_matrix((data, ci, rp), shape=(n_rows, n_cols))
    csr.has_canonical_format = True   # keep duplicates: never sum them
    csc = csr.tocsc()
    return (torch.from_numpy(csc.indptr.astype(np.int64)), torch.from_numpy(csc.indices.astype(np.int64)),
            torch.from_numpy(csc.data.astype(np.int64)))


def free_port():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_entry(worker, rank, world, port, args, q, done):
    """Child process: run worker(rank, world, port, *args) and report its result or its traceback; then stay
    until the parent has read the results (tensors travel as shared-memory handles served by this process)."""
    import traceback
    try:
        q.put((rank, "ok", worker(rank, world, port, *args)))
    except BaseException:
        q.put((rank, "error", traceback.format_exc()))
    done.wait(timeout=600)


def run_ranks(worker, world, args=(), timeout=300, expect_errors=False):
    """Spawn `world` processes running worker(rank, world, port, *args) and return their results by rank.
    A rank that raises makes the call fail at once with its traceback (or, with expect_errors, is returned
    as ("error", traceback)); whatever happens, every child that is still alive afterwards is terminated
    and then killed, so no process stays behind blocked in a collective."""
    import queue as _queue
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    done = ctx.Event()
    port = free_port()
    procs = [ctx.Process(target=_rank_entry, args=(worker, r, world, port, tuple(args), q, done), daemon=True)
             for r in range(world)]
    results = {}
    try:
        for p in procs:
            p.start()
        while len(results) < world:
            try:
                rank, status, payload = q.get(timeout=timeout)
            except _queue.Empty:
                raise AssertionError(f"ranks {sorted(set(range(world)) - set(results))} gave no result within {timeout} s")
            if status == "error" and not expect_errors:
                raise AssertionError(f"rank {rank} failed:\n{payload}")
            results[rank] = payload if status == "ok" else ("error", payload)
        done.set()
        for p in procs:
            p.join(timeout=30)
    finally:
        done.set()
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]
