"""GPU parity tests of the RWKV-4 kernels through the C ABI (host operator) against the CPU oracle,
the committed reference fixtures, and torch.autograd through the restated recurrence."""
import numpy as np
import pytest
import torch

import oracle
from oracle import torch_ref
from jaxrwkv_b200 import rwkv4
from conftest import rel_err
from gpu_util import TOL, flags, npf

pytestmark = pytest.mark.gpu
NAMES = ("r", "k", "v", "w", "u", "s0")


def dev(d, dtype):
    return {n: torch.tensor(d[n], dtype=torch.float32).to(dtype).cuda() for n in NAMES}


def state_loss(s, ga, gp):
    """A loss on the returned state that does not depend on how (aa, bb, pp) splits the magnitude
    between mantissas and exponent: aa/bb and log(bb)+pp are functions of the represented pair
    (aa e^pp, bb e^pp) only.  (A plain sum over the triple is discontinuous wherever the running
    maximum switches argument, so its gradient is ill-defined at near-ties.)  Empty states
    (bb == 0) are skipped."""
    aa, bb, pp = s[..., 0, :], s[..., 1, :], s[..., 2, :]
    ok = bb > 0
    safe = torch.where(ok, bb, torch.ones_like(bb))
    return (torch.where(ok, aa / safe, torch.zeros_like(aa)) * ga).sum() + \
           (torch.where(ok, torch.log(safe) + pp, torch.zeros_like(pp)) * gp).sum()


def check(d, dtype, seed=0):
    t = dev(d, dtype)
    length, ns = flags(d)
    leaves = [t[n].clone().requires_grad_(True) for n in NAMES]
    s, y = rwkv4.CudaRWKV.inner_loop(*leaves, length.cuda(), ns.cuda())
    g = torch.Generator().manual_seed(seed)
    gy = torch.randn(y.shape, generator=g).to(dtype)
    ga = torch.randn(s.shape[0], s.shape[2], generator=g).double()
    gp = torch.randn(s.shape[0], s.shape[2], generator=g).double()
    ((y.double() * gy.cuda().double()).sum() + state_loss(s.double(), ga.cuda(), gp.cuda())).backward()
    tol = TOL[dtype]
    B = t["k"].shape[0]
    cpu = [t[n].double().cpu().requires_grad_(True) for n in NAMES]
    tot = 0.0
    for i in range(B):
        so, yo = torch_ref.wkv4_base_torch(cpu[0][i], cpu[1][i], cpu[2][i], cpu[3], cpu[4], cpu[5][i], int(d["length"][i]),
                                           torch.tensor(d["new_starts"][i]))
        assert rel_err(npf(y[i]), yo.detach().numpy()) < tol, ("y", i)
        fin = np.abs(so.detach().numpy()) < 1e29
        assert rel_err(npf(s[i])[fin], so.detach().numpy()[fin]) < tol, ("s", i)
        tot = tot + (yo * gy[i].double()).sum() + state_loss(so, ga[i], gp[i])
    tot.backward()
    for n, leaf, ref in zip(NAMES, leaves, cpu):
        e = rel_err(npf(leaf.grad), ref.grad.numpy())
        assert e < tol, (n, e)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 5, 31, 32, 33, 70])
@pytest.mark.parametrize("default_state", [True, False])
def test_fwd_bwd_ragged(T, default_state, dtype):
    d = oracle.make_wkv4_inputs(3, T, 192, seed=500 + T, default_state=default_state)
    ns = np.zeros((3, T), dtype=bool)
    ns[0, 0] = True
    ns[1, [T // 2, min(T // 2 + 1, T - 1)]] = True
    d["new_starts"] = ns
    d["length"] = np.asarray([T, max(T - 2, 0), 0], dtype=np.uint32)
    check(d, dtype)


@pytest.mark.parametrize("case", ["v4_default_state", "v4_carried_state"])
def test_reference_fixtures(golden, case):
    g = golden(case)
    d = {n: g["in_" + n] for n in NAMES + ("length", "new_starts")}
    t = dev(d, torch.float32)
    length, ns = flags(d)
    s, y = rwkv4.CudaRWKV.inner_loop(t["r"], t["k"], t["v"], t["w"], t["u"], t["s0"], length.cuda(), ns.cuda())
    assert rel_err(npf(y), g["base_y"]) < 1e-4 and rel_err(npf(y), g["assoc_y"]) < 1e-4
    fin = np.abs(g["base_s"]) < 1e29
    assert rel_err(npf(s)[fin], g["base_s"][fin]) < 1e-4


def test_channel_count_4096_and_vmap():
    d = oracle.make_wkv4_inputs(2, 64, 4096, seed=7, p_start=0.05)
    t = dev(d, torch.bfloat16)
    length, ns = flags(d)
    f = rwkv4.CudaRWKV.inner_loop
    s1, y1 = f(t["r"], t["k"], t["v"], t["w"], t["u"], t["s0"], length.cuda(), ns.cuda())
    s2, y2 = torch.vmap(f, in_dims=(0, 0, 0, None, None, 0, 0, 0))(t["r"], t["k"], t["v"], t["w"], t["u"], t["s0"], length.cuda(), ns.cuda())
    assert torch.equal(y1, y2) and torch.equal(s1, s2) and torch.isfinite(y1.float()).all()
