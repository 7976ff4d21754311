"""CPU test (two gloo ranks) of the parameter-sharding helper: shard choice, gather-on-use, gradient
reduce-scatter with the mean convention, and averaging of replicated gradients."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jaxrwkv_b200.utils import fsdp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)                                  # same full parameters on both ranks
    full_w = torch.randn(6, 8, dtype=torch.float64)
    full_b = torch.randn(5, dtype=torch.float64)
    pw = fsdp.shard_param(full_w.clone(), min_weight_size=16)       # large: sharded along axis 1 (8 % 2 == 0, largest)
    pb = fsdp.shard_param(full_b.clone(), min_weight_size=16)       # small: replicated
    assert pw.idx == -1 and tuple(pw.v.shape) == (6, 4) and pb.idx == 0
    odd = fsdp.shard_param(torch.zeros(5, 7), min_weight_size=1)    # no divisible axis: replicated
    assert odd.idx == 0
    pw.v.requires_grad_(True); pb.v.requires_grad_(True)
    x = torch.arange(8, dtype=torch.float64) * (rank + 1)           # rank-dependent data
    params = fsdp.gather_params({"w": pw, "b": pb})
    assert torch.equal(params["w"].detach(), full_w)
    loss = (params["w"] @ x).sum() + (params["b"] * (rank + 1)).sum()
    loss.backward()
    fsdp.sync_grads(pb)
    # reference: mean over ranks of the per-rank gradients of the full parameters
    gw_full = sum(torch.ones(6, 1, dtype=torch.float64) * (torch.arange(8, dtype=torch.float64) * (r + 1)) for r in range(world)) / world
    gb_full = torch.full((5,), sum(r + 1 for r in range(world)) / world, dtype=torch.float64)
    ok = torch.allclose(pw.v.grad, gw_full[:, rank * 4:(rank + 1) * 4]) and torch.allclose(pb.v.grad, gb_full)
    cpu = fsdp.sharded_to_cpu({"w": pw})
    ok = ok and torch.equal(cpu["w"], full_w)
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag)
    if rank == 0:
        out.put(int(flag.item()))
    dist.destroy_process_group()


def test_two_rank_shard_gather_and_gradient_conventions():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    assert q.get(timeout=120) == 2
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
