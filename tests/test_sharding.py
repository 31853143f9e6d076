"""Batch sharding and the logits gather, on CPU: the arithmetic alone, and two
`gloo` ranks exchanging uneven shards."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nebula_b200 import sharding


def test_bounds_cover_the_batch_without_overlap():
    for total in (1, 7, 8, 256, 257):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_bounds(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1 and sizes == sharding.shard_sizes(total, world)
    with pytest.raises(ValueError):
        sharding.shard_bounds(4, 2, 2)


def test_time_major_inputs_are_sliced_along_the_batch_axis():
    x = np.arange(3 * 5 * 2, dtype=np.float32).reshape(3, 5, 2)
    a = sharding.shard_input(x, 2, 0, recurrent=True)
    b = sharding.shard_input(x, 2, 1, recurrent=True)
    assert a.shape == (3, 3, 2) and b.shape == (3, 2, 2) and a.flags["C_CONTIGUOUS"]
    assert np.array_equal(np.concatenate([a, b], 1), x)
    img = np.zeros((5, 3, 4, 4), np.float32)
    assert sharding.shard_input(img, 2, 1, recurrent=False).shape == (2, 3, 4, 4)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, total, classes, T, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(total * classes, dtype=torch.float32).view(total, classes)
        lo, hi = sharding.shard_bounds(total, world, rank)
        got = sharding.gather_rows(full[lo:hi].clone(), total, world, rank)
        ok = torch.equal(got, full)
        seq = torch.arange(T * total * classes, dtype=torch.float32).view(T, total, classes)
        got2 = sharding.gather_time_major(seq[:, lo:hi].contiguous(), total, world, rank)
        ok = ok and torch.equal(got2, seq)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [4, 5])
def test_gather_with_two_gloo_ranks(total):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, total, 3, 2, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res == [(0, True), (1, True)]
