"""NCCL test of the parameter-sharding helper on two GPUs of one node (skipped on a single-GPU box):
all-gather on use, reduce-scatter of the gradient with the mean convention."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jaxrwkv_b200.utils import fsdp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    torch.manual_seed(0)
    full = torch.randn(2048, 2048, dtype=torch.bfloat16).cuda()            # 8 MiB: config-4 sized weight
    pw = fsdp.shard_param(full.clone())
    assert pw.idx in (-1, -2) and pw.v.numel() == full.numel() // world
    pw.v.requires_grad_(True)
    x = torch.full((2048,), float(rank + 1), dtype=torch.bfloat16).cuda()
    w = fsdp.gather_param(pw)
    ok = torch.equal(w.detach(), full)
    (w.float() @ x.float()).sum().backward()
    expect = sum(r + 1 for r in range(world)) / world                       # mean over ranks of d/dw = x
    ok = ok and torch.allclose(pw.v.grad.float(), torch.full_like(pw.v.grad, expect).float(), rtol=1e-2)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag)
    if rank == 0:
        out.put(int(flag.item()))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_nccl_gather_and_reduce_scatter():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    assert q.get(timeout=300) == 2
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
