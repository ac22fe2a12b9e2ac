"""Batch partition over ranks and the end-of-run gather, with CPU ranks (gloo, world size 2)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vesta_gpu_b200.shard import partition, gather_tokens


def test_even_lengths_split_contiguously():
    assert partition([384] * 8, 2) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert partition([1] * 4, 4) == [[0], [1], [2], [3]]
    assert partition([5, 5], 1) == [[0, 1]]


def test_ragged_lengths_are_balanced():
    rng = np.random.default_rng(0)
    lens = rng.integers(64, 513, size=256)
    for world in (2, 4, 8):
        parts = partition(lens, world)
        assert sorted(sum(parts, [])) == list(range(256))
        assert all(len(p) == 256 // world for p in parts)
        loads = [int(lens[p].sum()) for p in parts]
        assert max(loads) / min(loads) < 1.02


def test_uneven_split_is_refused():
    with pytest.raises(ValueError):
        partition([1, 2, 3], 2)


def _rank(rank, world, port, q):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    lens = np.array([70, 500, 64, 300, 128, 129, 400, 90])
    mine = partition(lens, world)[rank]
    local = torch.tensor([[i * 100 + s for s in range(5)] for i in mine], dtype=torch.int32)
    out = gather_tokens(local, mine, len(lens))
    if rank == 0:
        q.put(out.numpy())
    else:
        assert out is None
    dist.barrier()
    dist.destroy_process_group()


def test_gather_restores_sequence_order_world2():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    want = np.array([[i * 100 + s for s in range(5)] for i in range(8)], np.int32)
    assert np.array_equal(got, want)


def test_gather_single_process():
    local = torch.arange(6, dtype=torch.int32).view(3, 2)
    out = gather_tokens(local, [2, 0, 1], 3)
    assert out.tolist() == [[2, 3], [4, 5], [0, 1]]
