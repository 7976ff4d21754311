"""GPU test of b200wkv7_fwd_bwd_static, the entry point for hosts that cannot allocate device
memory where they need the gradients (a custom-call handler inside a rematerialised, compiled
training step: the framework's pool owns all device memory and the handler must not call the CUDA
allocator).  It keeps the backward's state checkpoints in a fixed array inside the library.

Checked through the C ABI against the regular forward + backward pair (caller-provided residual)
on two calls in a row with different inputs, which also shows that contents left behind by the
first call do not leak into the second.  Collected last so that a failure here cannot hide others.
"""
import ctypes

import numpy as np
import pytest
import torch

from jaxrwkv_b200 import rwkv7, _lib
from conftest import rel_err
from gpu_util import NAMES7, TOL, to_dev, flags, npf, wkv7_case

pytestmark = pytest.mark.gpu


def _static_call(t, length, ns, gy, gs, dtype):
    lib = _lib.load()
    code = _lib.dtype_code(dtype)
    B, T, H, N = t["k"].shape
    length = length.to(device="cuda", dtype=torch.int32).contiguous()
    ns = ns.to(device="cuda", dtype=torch.uint8).contiguous()
    y = torch.empty_like(t["k"]); s_out = torch.empty_like(t["s0"])
    grads = [torch.empty_like(t["k"]) for _ in range(6)] + [torch.empty_like(t["s0"])]
    p = lambda x: ctypes.c_void_p(x.data_ptr())
    st = lib.b200wkv7_fwd_bwd_static(torch.cuda.current_stream().cuda_stream, code, B, T, H, N,
                                     p(t["w"]), p(t["r"]), p(t["k"]), p(t["v"]), p(t["a"]), p(t["b"]), p(t["s0"]),
                                     p(length), p(ns), p(gy), p(gs), p(y), p(s_out), *[p(g) for g in grads], 0)
    _lib.check(st)
    return y, s_out, grads      # grads in ABI order: dw, dr, dk, dv, da, db, ds0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_matches_regular_pair_twice(dtype):
    for call, (T, seed) in enumerate(((200, 61), (130, 62))):
        d = wkv7_case(2, T, 2, seed=seed, s0_scale=0.4, p_start=0.02, random_length=True)
        t = to_dev(d, dtype)
        length, ns = flags(d)
        g = torch.Generator().manual_seed(seed)
        gy = torch.randn(t["k"].shape, generator=g).to(dtype).cuda()
        gs = torch.randn(t["s0"].shape, generator=g).to(dtype).cuda()
        (s_ref, y_ref), res = rwkv7.batched_wkv7_fwd(*[t[n] for n in NAMES7], length, ns, 2)
        gr, gw, gk, gv, ga, gb, g0 = rwkv7.batched_wkv7_bwd(res, (gs, gy), 2)
        y, s_out, grads = _static_call(t, length, ns, gy, gs, dtype)
        tol = TOL[dtype]
        assert rel_err(npf(y), npf(y_ref)) < tol and rel_err(npf(s_out), npf(s_ref)) < tol, call
        for name, got, ref in zip(("dw", "dr", "dk", "dv", "da", "db", "ds0"), grads, (gw, gr, gk, gv, ga, gb, g0)):
            assert rel_err(npf(got), npf(ref)) < tol, (call, name)


def test_static_scratch_rejects_oversized_problem():
    lib = _lib.load()
    cap = lib.b200wkv7_static_scratch_bytes()
    assert cap == 64 << 20
    B, T, H, N = 8, 4096, 32, 64
    assert lib.b200wkv7_residual_bytes(_lib.BF16, B, T, H, N) > cap
    one = ctypes.c_void_p(16)   # never dereferenced: the size check comes first
    st = lib.b200wkv7_fwd_bwd_static(None, _lib.BF16, B, T, H, N, *([one] * 9), one, one, one, one, *([one] * 7), 0)
    assert st == -7 and b"scratch" in lib.b200wkv_strerror(st)
