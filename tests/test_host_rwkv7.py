"""CPU tests of the host-side operator logic (leading-axis flattening, the batching
rules, broadcast of shared length/new_starts, cotangent order).  The two custom calls are
replaced by oracle-backed fakes, so no GPU is needed; what is under test is everything
between ``CudaRWKV.inner_loop`` and the C ABI."""
import numpy as np
import pytest
import torch

import oracle
from jaxrwkv_b200 import rwkv7
from conftest import rel_err


def _np(x):
    return x.detach().double().numpy()


@pytest.fixture
def fake_calls(monkeypatch):
    calls = {"fwd": [], "bwd": []}

    def fwd(r, w, k, v, a, b, s, length, new_starts, B, need_residual=True, flags=0):
        calls["fwd"].append(tuple(k.shape))
        assert k.dim() == 4 and k.shape[0] == B and length.shape == (B,) and new_starts.shape == (B, k.shape[1])
        so, y = oracle.wkv7_base_batched(*[_np(x) for x in (r, w, k, v, a, b, s)], length.numpy(), new_starts.numpy().astype(bool))
        res = (r, w, k, v, a, b, s, length, new_starts, torch.zeros(1, dtype=torch.uint8))
        return (torch.tensor(so, dtype=k.dtype), torch.tensor(y, dtype=k.dtype)), res

    def bwd(res, grads, B, flags=0):
        calls["bwd"].append(tuple(res[2].shape))
        r, w, k, v, a, b, s, length, new_starts, _ = res
        gs, gy = grads
        gs = np.zeros(s.shape) if gs is None else _np(gs)
        gy = np.zeros(k.shape) if gy is None else _np(gy)
        out = oracle.wkv7_bwd_batched(*[_np(x) for x in (r, w, k, v, a, b, s)], length.numpy(),
                                      new_starts.numpy().astype(bool), gy, gs)
        gr, gw, gk, gv, ga, gb, g0 = [torch.tensor(x, dtype=k.dtype) for x in out]
        return gr, gw, gk, gv, ga, gb, g0

    monkeypatch.setattr(rwkv7, "batched_wkv7_fwd", fwd)
    monkeypatch.setattr(rwkv7, "batched_wkv7_bwd", bwd)
    monkeypatch.setattr(rwkv7.CudaRWKV, "get_kernels", classmethod(lambda cls: None))
    return calls


def _data(lead, T=12, H=2, N=4, seed=0):
    B = int(np.prod(lead)) if lead else 1
    d = oracle.make_wkv7_inputs(B, T, H, N, seed=seed, s0_scale=0.5, p_start=0.2, random_length=True, dtype=np.float64)
    t = {n: torch.tensor(d[n]).reshape(tuple(lead) + d[n].shape[1:]) for n in ("r", "w", "k", "v", "a", "b", "s0")}
    length = torch.tensor(d["length"].astype(np.int64)).reshape(tuple(lead))
    ns = torch.tensor(d["new_starts"]).reshape(tuple(lead) + (T,))
    return d, t, length, ns


def test_single_sequence_and_leading_axes(fake_calls):
    for lead in [(), (3,), (2, 3)]:
        d, t, length, ns = _data(lead)
        s, y = rwkv7.CudaRWKV.inner_loop(t["r"], t["w"], t["k"], t["v"], t["a"], t["b"], t["s0"], length, ns)
        so, yo = oracle.wkv7_base_batched(*[d[n] for n in ("r", "w", "k", "v", "a", "b", "s0")], d["length"], d["new_starts"])
        assert s.shape == t["s0"].shape and y.shape == t["k"].shape
        assert rel_err(_np(y).reshape(yo.shape), yo) < 1e-12 and rel_err(_np(s).reshape(so.shape), so) < 1e-12
    assert [c[0] for c in fake_calls["fwd"]] == [1, 3, 6]


def test_vmap_nested_and_shared_flags(fake_calls):
    d, t, length, ns = _data((2, 3))
    f = rwkv7.CudaRWKV.inner_loop
    args = (t["r"], t["w"], t["k"], t["v"], t["a"], t["b"], t["s0"])
    s1, y1 = torch.vmap(torch.vmap(f))(*args, length, ns)
    s2, y2 = f(*args, length, ns)
    assert torch.equal(y1, y2) and torch.equal(s1, s2)
    # shared (unbatched) length and new_starts are broadcast, as in rwkv7.py:422-427
    sh_len, sh_ns = torch.tensor(7), ns[0, 0]
    s3, y3 = torch.vmap(torch.vmap(f, in_dims=(0,) * 7 + (None, None)), in_dims=(0,) * 7 + (None, None))(*args, sh_len, sh_ns)
    s4, y4 = f(*args, sh_len.expand(2, 3), sh_ns.expand(2, 3, -1))
    assert torch.equal(y3, y4) and torch.equal(s3, s4)
    with pytest.raises(Exception):
        torch.vmap(f, in_dims=(None,) + (0,) * 8)(t["r"][0], *args[1:], length, ns)


def test_gradients_all_inputs_both_outputs(fake_calls):
    d, t, length, ns = _data((2,))
    names = ("r", "w", "k", "v", "a", "b", "s0")
    leaves = [t[n].clone().requires_grad_(True) for n in names]
    s, y = rwkv7.wkv7_cuda(*leaves, length, ns)
    gy = torch.randn_like(y); gs = torch.randn_like(s)
    ((y * gy).sum() + (s * gs).sum()).backward()
    ref = oracle.wkv7_bwd_batched(*[d[n] for n in names], d["length"], d["new_starts"], _np(gy), _np(gs))
    for n, leaf, g in zip(names, leaves, ref):            # oracle returns (dr, dw, dk, dv, da, db, ds0)
        assert rel_err(_np(leaf.grad), g) < 1e-12, n
    # only the output is used: the state cotangent arrives as None
    leaves = [t[n].clone().requires_grad_(True) for n in names]
    s, y = rwkv7.wkv7_cuda(*leaves, length, ns)
    y.sum().backward()
    ref = oracle.wkv7_bwd_batched(*[d[n] for n in names], d["length"], d["new_starts"], np.ones(y.shape), np.zeros(s.shape))
    assert rel_err(_np(leaves[6].grad), ref[6]) < 1e-12


def test_vmap_of_grad(fake_calls):
    """Per-sequence value-and-grad under vmap (what tests/rand_grad_test.py of jaxrwkv does)."""
    d, t, length, ns = _data((3,))
    names = ("r", "w", "k", "v", "a", "b", "s0")

    def loss(r, w, k, v, a, b, s0, length, ns):
        s, y = rwkv7.wkv7_cuda(r, w, k, v, a, b, s0, length, ns)
        return (y * y).sum() + s.sum()

    g = torch.vmap(torch.func.grad(loss, argnums=(0, 6)))(*[t[n] for n in names], length, ns)
    leaves = [t[n].clone().requires_grad_(True) for n in names]
    s, y = rwkv7.wkv7_cuda(*leaves, length, ns)
    ((y * y).sum() + s.sum()).backward()
    assert rel_err(_np(g[0]), _np(leaves[0].grad)) < 1e-12 and rel_err(_np(g[1]), _np(leaves[6].grad)) < 1e-12
