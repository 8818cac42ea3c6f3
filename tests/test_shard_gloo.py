"""The multi-GPU host logic (sharding, max-over-ranks timing, final gather) with two gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from vla_cpp_b200 import shard


def test_shard_range_covers_everything_once():
    for n, w in [(1024, 8), (1024, 1), (10, 4), (3, 8), (0, 2)]:
        seen = []
        for r in range(w):
            s, c = shard.shard_range(n, w, r)
            seen += list(range(s, s + c))
        assert seen == list(range(n))
    assert [shard.shard_range(1024, w, 0)[1] for w in (8, 4, 2, 1)] == [128, 256, 512, 1024]
    with pytest.raises(ValueError):
        shard.shard_range(4, 2, 2)


def _worker(rank, world, port, n_total, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        start, count = shard.shard_range(n_total, world, rank)
        # every rank "computes" chunks whose value encodes the observation index
        x = torch.arange(start, start + count, dtype=torch.float32).view(-1, 1, 1).expand(count, 5, 3).contiguous()
        full = shard.gather_action_chunks(x, n_total)
        ok = full.shape == (n_total, 5, 3) and torch.equal(full[:, 0, 0], torch.arange(n_total, dtype=torch.float32))
        times = shard.max_over_ranks([10.0 + rank, 3.0 - rank])
        ok = ok and times == [10.0 + world - 1, 3.0]
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_and_timing_over_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 7, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == {0: True, 1: True}


def test_single_process_paths_are_identities():
    x = torch.zeros(3, 2, 2)
    assert shard.gather_action_chunks(x, 3) is x
    assert shard.max_over_ranks([1.5, 2.5]) == [1.5, 2.5]
