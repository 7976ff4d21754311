"""GPU parity tests of the RWKV-5 / 5.2 / 6 kernels through the C ABI (host operator) against the
CPU oracle, the committed reference fixtures and autograd-checked reverse loops."""
import numpy as np
import pytest
import torch

import oracle
from jaxrwkv_b200 import rwkv5, rwkv5_2, rwkv6, _wkv6_family as fam
from conftest import rel_err
from gpu_util import TOL, flags, npf

pytestmark = pytest.mark.gpu
MODS = {"6": rwkv6, "5_2": rwkv5_2, "5": rwkv5}
NAMES = ("r", "k", "v", "w", "u", "s0")


def case(version, B, T, H, seed, p_start=0.0, random_length=False, s0_scale=0.3, starts=None, lengths=None):
    d = oracle.make_wkv6_inputs(B, T, H, 64, seed=seed, p_start=p_start, s0_scale=s0_scale,
                                random_length=random_length, version=version)
    if starts is not None:
        ns = np.zeros((B, T), dtype=bool)
        for i, row in enumerate(starts):
            ns[i, list(row)] = True
        d["new_starts"] = ns
    if lengths is not None:
        d["length"] = np.asarray(lengths, dtype=np.uint32)
    return d


def dev(d, dtype):
    return {n: torch.tensor(d[n], dtype=torch.float32).to(dtype).cuda() for n in NAMES}


def check(version, d, dtype, seed=0, tol_dw=None):
    t = dev(d, dtype)
    length, ns = flags(d)
    leaves = [t[n].clone().requires_grad_(True) for n in NAMES]
    s, y = MODS[version].CudaRWKV.inner_loop(*leaves[:5], leaves[5], length.cuda(), ns.cuda())
    rounded = [t[n].double().cpu().numpy() for n in NAMES]
    so, yo = oracle.wkv6_base_batched(*rounded, d["length"], d["new_starts"], version)
    tol = TOL[dtype]
    assert rel_err(npf(y), yo) < tol, ("y", rel_err(npf(y), yo))
    for i in range(so.shape[0]):
        assert rel_err(npf(s[i]), so[i]) < tol, ("s", i)
    g = torch.Generator().manual_seed(seed)
    gy = torch.randn(y.shape, generator=g).to(dtype).cuda()
    gs = torch.randn(s.shape, generator=g).to(dtype).cuda()
    ((y.float() * gy.float()).sum() + (s.float() * gs.float()).sum()).backward()
    ref = oracle.wkv6_bwd_batched(*rounded, d["length"], d["new_starts"], npf(gy), npf(gs), version)
    for n, leaf, gref in zip(("dr", "dk", "dv", "dw", "du", "ds0"), leaves, ref):
        e = rel_err(npf(leaf.grad).reshape(gref.shape), gref)
        assert e < (tol_dw if (n == "dw" and tol_dw is not None) else tol), (n, e)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("version", ["6", "5_2", "5"])
@pytest.mark.parametrize("T", [1, 7, 16, 17, 40, 70])
def test_fwd_bwd_ragged(version, T, dtype):
    rng = np.random.default_rng(T)
    starts = [sorted(set(rng.integers(0, T, size=2).tolist())), [0], [T // 2, min(T // 2 + 1, T - 1)]]
    lengths = [T, max(T - 3, 0), 0]
    check(version, case(version, 3, T, 2, seed=400 + T, starts=starts, lengths=lengths), dtype)


@pytest.mark.parametrize("version", ["6", "5_2", "5"])
def test_reference_fixtures(golden, version):
    g = golden(f"v{version}_resets")
    d = {n: g["in_" + n] for n in NAMES + ("length", "new_starts")}
    t = dev(d, torch.float32)
    length, ns = flags(d)
    s, y = MODS[version].CudaRWKV.inner_loop(t["r"], t["k"], t["v"], t["w"], t["u"], t["s0"], length.cuda(), ns.cuda())
    assert rel_err(npf(y), g["base_y"]) < 1e-4 and rel_err(npf(y), g["assoc_y"]) < 1e-4
    for i in range(s.shape[0]):
        assert rel_err(npf(s[i]), g["base_s"][i]) < 1e-4
        if not (int(d["length"][i]) < d["new_starts"].shape[1] and d["new_starts"][i][int(d["length"][i])]):
            assert rel_err(npf(s[i]), g["assoc_s"][i]) < 1e-4


def test_training_shape_v6_bf16():
    check("6", case("6", 2, 512, 4, seed=1236, p_start=1 / 128, random_length=True, s0_scale=0.1), torch.bfloat16)


def test_vmap_matches_batched():
    d = case("6", 3, 33, 2, seed=5, p_start=0.1)
    t = dev(d, torch.float32)
    length, ns = flags(d)
    f = rwkv6.CudaRWKV.inner_loop
    s1, y1 = torch.vmap(f, in_dims=(0, 0, 0, 0, None, 0, 0, 0))(t["r"], t["k"], t["v"], t["w"], t["u"], t["s0"], length.cuda(), ns.cuda())
    s2, y2 = f(t["r"], t["k"], t["v"], t["w"], t["u"], t["s0"], length.cuda(), ns.cuda())
    assert torch.equal(y1, y2) and torch.equal(s1, s2)


def test_config3_full_size_properties():
    """RWKV-6 training kernel at B=16, T=4096, H=32, bf16: finite, deterministic, and exactly
    homogeneous in (v, s0) under scaling by 2; one (batch, head) slice against the oracle."""
    B, T, H = 16, 4096, 32
    g = torch.Generator(device="cuda").manual_seed(1236)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")
    r, k, v = (rn(B, T, H, 64).bfloat16() for _ in range(3))
    w = (-torch.exp(-0.5 + 0.5 * rn(B, T, H, 64))).bfloat16().unsqueeze(-1)
    u = (0.1 * rn(H, 64, 1)).bfloat16()
    s0 = (0.1 * rn(B, H, 64, 64)).bfloat16()
    ns = torch.rand(B, T, generator=g, device="cuda") < 1 / 512
    length = torch.full((B,), T, device="cuda")
    s, y = rwkv6.CudaRWKV.inner_loop(r, k, v, w, u, s0, length, ns)
    s_b, y_b = rwkv6.CudaRWKV.inner_loop(r, k, v, w, u, s0, length, ns)
    s_2, y_2 = rwkv6.CudaRWKV.inner_loop(r, k, v * 2, w, u, s0 * 2, length, ns)
    assert torch.isfinite(y.float()).all() and torch.equal(y, y_b) and torch.equal(s, s_b)
    assert torch.equal(y_2, y * 2) and torch.equal(s_2, s * 2)
    bi, hh = 3, 17
    so, yo = oracle.wkv6_base(*[x[bi][:, hh:hh + 1].double().cpu().numpy() for x in (r, k, v, w)], u[hh:hh + 1].double().cpu().numpy(),
                              s0[bi][hh:hh + 1].double().cpu().numpy(), T, ns[bi].cpu().numpy(), "6")
    assert rel_err(npf(y[bi][:, hh:hh + 1]), yo) < 2e-2 and rel_err(npf(s[bi][hh:hh + 1]), so) < 2e-2


def test_config3_full_size_backward():
    """Config 3 exactly (B=16, T=4096, H=32, bf16, starts p=1/512, s0 ~ N(0, 0.1), dy and dstate ~ N(0,1)):
    forward + backward through the operator; gradients finite, deterministic and homogeneous of degree one in
    the cotangents; four (batch, head) slices against the oracle's reverse loop (du, a sum over the batch,
    against the oracle on those slices is not separable and is checked at small sizes instead)."""
    B, T, H = 16, 4096, 32
    g = torch.Generator(device="cuda").manual_seed(1236)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")
    r, k, v = (rn(B, T, H, 64).bfloat16() for _ in range(3))
    w = (-torch.exp(-0.5 + 0.5 * rn(B, T, H, 64))).bfloat16().unsqueeze(-1)
    u = (0.1 * rn(H, 64, 1)).bfloat16()
    s0 = (0.1 * rn(B, H, 64, 64)).bfloat16()
    ns = torch.rand(B, T, generator=g, device="cuda") < 1 / 512
    length = torch.full((B,), T, device="cuda")
    gy, gs = rn(B, T, H, 64).bfloat16(), rn(B, H, 64, 64).bfloat16()

    def grads(scale):
        leaves = [x.clone().requires_grad_(True) for x in (r, k, v, w, u, s0)]
        s, y = rwkv6.CudaRWKV.inner_loop(*leaves, length, ns)
        torch.autograd.backward((y, s), (gy * scale, gs * scale))
        return [x.grad for x in leaves]

    g1, g1b, g2 = grads(1), grads(1), grads(2)
    for n, a, b, c in zip(("dr", "dk", "dv", "dw", "du", "ds0"), g1, g1b, g2):
        assert torch.isfinite(a.float()).all(), n
        assert torch.equal(a, b), n
        if n != "du":                      # du is rounded to bf16 after the sum over the batch
            assert torch.equal(c, a * 2), n
    f64 = lambda x: x.double().cpu().numpy()
    for bi, hh in ((0, 0), (3, 17), (9, 5), (15, 31)):
        ins = [f64(x[bi:bi + 1, :, hh:hh + 1]) for x in (r, k, v, w)] + [f64(u[hh:hh + 1]), f64(s0[bi:bi + 1, hh:hh + 1])]
        ref = oracle.wkv6_bwd_batched(*ins, np.array([T], dtype=np.uint32), ns[bi:bi + 1].cpu().numpy(),
                                      f64(gy[bi:bi + 1, :, hh:hh + 1]), f64(gs[bi:bi + 1, hh:hh + 1]), "6")
        got = [g1[0][bi:bi + 1, :, hh:hh + 1], g1[1][bi:bi + 1, :, hh:hh + 1], g1[2][bi:bi + 1, :, hh:hh + 1],
               g1[3][bi:bi + 1, :, hh:hh + 1], None, g1[5][bi:bi + 1, hh:hh + 1]]
        for n, a, b in zip(("dr", "dk", "dv", "dw", "du", "ds0"), got, ref):
            if a is not None:
                e = rel_err(npf(a).reshape(b.shape), b)
                assert e < 2e-2, (n, bi, hh, e)


def _residual_mark(res):
    """Last 16 bytes of the bf16 residual: 0 = written by the chunked kernels, 1 = by the sequential ones."""
    return int(res[-1][-16:].view(torch.int32)[0].item())


def _fwd_mark(version, d):
    """Which kernels a bf16 forward of ``d`` uses (through the batched host call, which returns the residual)."""
    t = dev(d, torch.bfloat16)
    length, ns = flags(d)
    H = t["r"].shape[2]
    w = t["w"] if version == "6" else fam._expand_hn(t["w"], H, 64, torch.bfloat16)
    u = fam._expand_hn(t["u"], H, 64, torch.bfloat16)
    w = w.reshape(t["r"].shape) if version == "6" else w
    _, res = fam.batched_wkv6_fwd(version, t["r"], t["k"], t["v"], w, u, t["s0"], length.cuda(), ns.cuda(), t["r"].shape[0])
    return _residual_mark(res)


@pytest.mark.parametrize("version", ["6", "5_2", "5"])
@pytest.mark.parametrize("T", [16, 48, 70, 200])
def test_chunked_kernels_fwd_bwd(version, T):
    """The 16-token tensor-core kernels: start flags at chunk boundaries, inside chunks, adjacent, on the last token;
    lengths T, 0, on a chunk boundary and inside a chunk (the cotangent of the returned state then enters in the middle
    of a chunk, which is walked in two parts); T itself need not be a multiple of 16; all against the oracle, and the
    residual says which kernels ran."""
    rng = np.random.default_rng(T)
    starts = [sorted(set(rng.integers(0, T, size=3).tolist())), [0, 16 % T, T - 1], [T // 2, min(T // 2 + 1, T - 1)], [],
              [min(4, T - 1), min(5, T - 1)], []]
    lengths = [T, (T // 16) * 16 if T >= 32 else T, 0, 16, min(5, T), max(T - 3, 1)]
    d = case(version, 6, T, 2, seed=900 + T, starts=starts, lengths=lengths, s0_scale=0.5)
    # Version 6 trains on the chunked kernels.  Versions 5 / 5.2 train on the sequential ones (the gradient of a
    # CONSTANT decay, a sum over all tokens of terms that largely cancel, is only good to a few percent when taken
    # from bf16 tensor-core products) and use the chunked kernel for calls without a residual, checked below.
    assert _fwd_mark(version, d) == (0 if version == "6" else 1)
    check(version, d, torch.bfloat16)
    t = dev(d, torch.bfloat16)
    length, ns = flags(d)
    H = t["r"].shape[2]
    w = t["w"].reshape(t["r"].shape) if version == "6" else fam._expand_hn(t["w"], H, 64, torch.bfloat16)
    u = fam._expand_hn(t["u"], H, 64, torch.bfloat16)
    (s, y), _ = fam.batched_wkv6_fwd(version, t["r"], t["k"], t["v"], w, u, t["s0"], length.cuda(), ns.cuda(), t["r"].shape[0],
                                     need_residual=False)
    so, yo = oracle.wkv6_base_batched(*[t[n].double().cpu().numpy() for n in NAMES], d["length"], d["new_starts"], version)
    assert rel_err(npf(y), yo) < TOL[torch.bfloat16]
    for i in range(so.shape[0]):
        assert rel_err(npf(s[i]), so[i]) < TOL[torch.bfloat16], i


def test_chunked_kernels_fall_back_per_call():
    """A decay above 1 and a decay below exp(-10) per token are outside the chunked kernels' domain: the call is redone
    by the sequential kernels (mark 1) and still matches the oracle."""
    d = case("6", 2, 64, 2, seed=32)
    d["w"][1, 16:32] = -12.0                                   # log-decay: exp(-12) per token, -96 over eight tokens
    assert _fwd_mark("6", d) == 1
    check("6", d, torch.bfloat16)
    d = case("6", 2, 64, 2, seed=33)
    d["w"][0, 5] = 0.25                                        # a decay above 1
    assert _fwd_mark("6", d) == 1
    check("6", d, torch.bfloat16)
    d = case("6", 2, 64, 2, seed=34)
    d["w"][:] = np.maximum(d["w"], -9.0)                       # strong but representable decays stay chunked
    d["w"][0, 8:24] = -9.0
    assert _fwd_mark("6", d) == 0
    check("6", d, torch.bfloat16)


def test_chunked_forward_without_residual_matches_oracle():
    d = case("6", 3, 80, 2, seed=41, starts=[[7, 8, 50], [0], [79]], lengths=[80, 48, 0], s0_scale=0.5)
    t = dev(d, torch.bfloat16)
    length, ns = flags(d)
    u = fam._expand_hn(t["u"], 2, 64, torch.bfloat16)
    (s, y), _ = fam.batched_wkv6_fwd("6", t["r"], t["k"], t["v"], t["w"].reshape(t["r"].shape), u, t["s0"], length.cuda(), ns.cuda(), 3,
                                     need_residual=False)
    so, yo = oracle.wkv6_base_batched(*[t[n].double().cpu().numpy() for n in NAMES], d["length"], d["new_starts"], "6")
    assert rel_err(npf(y), yo) < TOL[torch.bfloat16]
    for i in range(3):
        assert rel_err(npf(s[i]), so[i]) < TOL[torch.bfloat16]


def test_run_parallel_backward_ragged():
    """From 32 chunks on, the backward is a state-gradient carry (64 tokens per step) plus the gradient kernel over runs of
    16 chunks.  T = 560 is 35 chunks, three runs and nine carry steps of which the last has 48 tokens; the lengths put
    the cotangent of the returned state on a step boundary, on a run boundary, one token short of each, inside a step and
    at 1, and start flags lie on, next to and far from those positions."""
    T = 560
    starts = [[0, 64, 65, 300, 511, 512, 559], [256, 257, 558], [513], [100, 511], [0, 299, 300, 301], [0]]
    lengths = [T, T - 1, 513, 512, 300, 1]
    d = case("6", 6, T, 2, seed=977, starts=starts, lengths=lengths, s0_scale=0.5)
    assert _fwd_mark("6", d) == 0
    check("6", d, torch.bfloat16)
