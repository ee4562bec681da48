"""TileBalanceScheduler (dgNN/operators/tile_balance_scheduler.py:3-11 of the
reference; the working copy is script/test/test_gat_tb.py:16-26): one row id per
32-edge tile of every row.  Kept for API compatibility; gat_forward_tb here does
not need it."""
import torch


def TileBalanceScheduler(row_ptr):
    rp = row_ptr.detach().to("cpu", torch.int64)
    deg = rp[1:] - rp[:-1]
    tiles = (deg + 31) // 32
    rows = torch.repeat_interleave(torch.arange(deg.numel(), dtype=torch.int64), tiles)
    return rows.int()
