"""CPU test of the multi-rank host logic with two gloo ranks: every batch row is owned by exactly
one rank, and the timing reduction is a max over ranks (what bench.py reports for N > 1)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jaxrwkv_b200.shard import shard_bounds, max_over_ranks, sum_over_ranks


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, global_batch, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = shard_bounds(global_batch, rank, world)
    owned = torch.zeros(global_batch, dtype=torch.int32)
    owned[lo:hi] = 1
    dist.all_reduce(owned)
    ms = max_over_ranks(10.0 + rank)               # the slowest rank defines the step time
    tokens = sum_over_ranks((hi - lo) * 4096)
    if rank == 0:
        out.put((owned.tolist(), ms, tokens))
    dist.destroy_process_group()


def test_two_rank_sharding_and_timing_reduction():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 7, q)) for r in range(2)]
    for p in procs:
        p.start()
    owned, ms, tokens = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert owned == [1] * 7
    assert ms == 11.0 and tokens == 7 * 4096


def test_shard_bounds_cover_and_balance():
    for gb in (1, 7, 8, 64):
        for world in (1, 2, 4, 8):
            spans = [shard_bounds(gb, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == gb
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
