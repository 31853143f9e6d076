"""Batch sharding across the GPUs of one node and the single collective of the
forward path: gathering the logits.

Inference has no cross-sample coupling (batch-norm uses stored statistics,
models/layers/convolutional_layer.cc:529-533; LSTM sequences are independent
across the batch axis), so rank r runs the whole network on a contiguous slice
of the batch with replicated weights and only the [rows, classes] outputs are
exchanged.  The reference itself is single-device (models/networks/network.cc:44-47).
"""
from __future__ import annotations

import numpy as np


def shard_bounds(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous slice [lo, hi) of `total` units for `rank`; the first
    total % world ranks get one extra unit."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_sizes(total: int, world: int) -> list[int]:
    return [hi - lo for lo, hi in (shard_bounds(total, world, r) for r in range(world))]


def shard_input(x, world: int, rank: int, recurrent: bool):
    """Slice of a host batch for `rank`: images [B,C,H,W] along B; sequences are
    time-major [T,B,in] (models/networks/recurrent.cc:197), sliced along axis 1
    and packed contiguous."""
    axis = 1 if recurrent else 0
    lo, hi = shard_bounds(x.shape[axis], world, rank)
    sl = [slice(None)] * x.ndim
    sl[axis] = slice(lo, hi)
    out = x[tuple(sl)]
    return np.ascontiguousarray(out) if isinstance(out, np.ndarray) else out.contiguous()


class _Gather:
    """An all-gather in flight: wait() returns the [total_rows, classes] tensor."""

    def __init__(self, work, out, sizes, mx):
        self.work, self.out, self.sizes, self.mx = work, out, sizes, mx

    def wait(self):
        import torch
        if self.work is not None:
            self.work.wait()        # orders the caller's current stream behind the collective; no host block
        if all(s == self.mx for s in self.sizes):
            return self.out
        return torch.cat([self.out[r * self.mx:r * self.mx + s] for r, s in enumerate(self.sizes)], 0)


def gather_rows(local, total_rows: int, world: int, rank: int, group=None, async_op: bool = False):
    """All-gathers per-rank [rows_r, classes] tensors into [total_rows, classes]
    on every rank (rows in global batch order).  Uneven shards are padded to the
    largest shard for the collective and trimmed afterwards.  With async_op the
    collective is only started (it overlaps whatever the caller queues next) and
    an object whose wait() gives the result is returned."""
    import torch
    import torch.distributed as dist
    sizes = shard_sizes(total_rows, world)
    assert local.shape[0] == sizes[rank], (local.shape, sizes, rank)
    if world == 1:
        return _Gather(None, local, sizes, sizes[0]) if async_op else local
    classes = local.shape[1]
    mx = max(sizes)
    if local.shape[0] != mx:
        pad = torch.zeros((mx - local.shape[0], classes), dtype=local.dtype, device=local.device)
        local = torch.cat([local, pad], 0)
    out = torch.empty((world * mx, classes), dtype=local.dtype, device=local.device)
    work = dist.all_gather_into_tensor(out, local.contiguous(), group=group, async_op=async_op)
    g = _Gather(work if async_op else None, out, sizes, mx)
    return g if async_op else g.wait()


def gather_time_major(local, total_batch: int, world: int, rank: int, group=None):
    """Gathers per-rank time-major outputs [T, B_r, classes] into [T, B, classes]."""
    T, b_r, classes = local.shape
    rows = gather_rows(local.permute(1, 0, 2).reshape(b_r, T * classes).contiguous(), total_batch, world, rank, group)
    return rows.reshape(total_batch, T, classes).permute(1, 0, 2).contiguous()
