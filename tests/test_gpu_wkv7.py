"""GPU parity tests of the RWKV-7 kernels, called through the C ABI (ctypes) via the
host operator, against the CPU oracle and the committed reference fixtures."""
import numpy as np
import pytest
import torch

import oracle
from jaxrwkv_b200 import rwkv7, _lib
from conftest import rel_err
from gpu_util import NAMES7, TOL, to_dev, rounded, flags, npf, wkv7_case

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
# (element type, flags): fp32 -> sequential kernels; bf16 -> chunked tensor-core kernels, or the
# sequential ones when B200WKV_FLAG_SEQUENTIAL is set
KERNELS = [pytest.param(torch.float32, 0, id="f32-seq"), pytest.param(torch.bfloat16, 0, id="bf16-chunk"),
           pytest.param(torch.bfloat16, _lib.FLAG_SEQUENTIAL, id="bf16-seq")]


def run_fwd(t, length, ns, flags_=0):
    B = t["k"].shape[0]
    (s, y), res = rwkv7.batched_wkv7_fwd(t["r"], t["w"], t["k"], t["v"], t["a"], t["b"], t["s0"], length, ns, B, flags=flags_)
    return s, y, res


def check_fwd(d, dtype, flags_=0, tol=None):
    t = to_dev(d, dtype)
    length, ns = flags(d)
    s, y, _ = run_fwd(t, length, ns, flags_)
    so, yo = oracle.wkv7_base_batched(*rounded(t), d["length"], d["new_starts"])
    tol = tol or TOL[dtype]
    assert rel_err(npf(y), yo) < tol, ("y", rel_err(npf(y), yo))
    for i in range(so.shape[0]):     # per sequence: a zero state must come back as exact zeros
        e = rel_err(npf(s[i]), so[i])
        assert e < tol, ("s_out", i, e)
    return s, y


def check_bwd(d, dtype, seed=0, use_gy=True, use_gs=True, flags_=0, tol_dw=None):
    t = to_dev(d, dtype)
    length, ns = flags(d)
    B = t["k"].shape[0]
    s, y, res = run_fwd(t, length, ns, flags_)
    g = torch.Generator().manual_seed(seed)
    gy = torch.randn(y.shape, generator=g).to(dtype).cuda() if use_gy else None
    gs = torch.randn(s.shape, generator=g).to(dtype).cuda() if use_gs else None
    got = rwkv7.batched_wkv7_bwd(res, (gs, gy), B, flags=flags_)
    ref = oracle.wkv7_bwd_batched(*rounded(t), d["length"], d["new_starts"],
                                  npf(gy) if use_gy else np.zeros(y.shape), npf(gs) if use_gs else np.zeros(s.shape))
    for n, a, b in zip(("dr", "dw", "dk", "dv", "da", "db", "ds0"), got, ref):
        e = rel_err(npf(a), b)
        assert e < (tol_dw if (n == "dw" and tol_dw) else TOL[dtype]), (n, e)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["v7_plain", "v7_resets"])
def test_fwd_reference_fixtures(golden, case, dtype):
    """Against the outputs of jaxrwkv's own Base and AssociativeScan inner_loop."""
    g = golden(case)
    d = {n: g["in_" + n] for n in NAMES7 + ("length", "new_starts")}
    t = to_dev(d, dtype)
    length, ns = flags(d)
    s, y, _ = run_fwd(t, length, ns)
    tol = TOL[dtype] if dtype == torch.float32 else 3e-2   # fixtures were computed on unrounded inputs
    assert rel_err(npf(y), g["base_y"]) < tol
    for i in range(s.shape[0]):
        assert rel_err(npf(s[i]), g["base_s"][i]) < tol
        ym, sd = oracle.quirk_mask(d["new_starts"][i], int(d["length"][i]))
        # AssociativeScanRWKV, excluding the positions its index shift forces to zero
        assert rel_err(npf(y[i])[~ym], g["assoc_y"][i][~ym]) < tol
        if not sd:
            assert rel_err(npf(s[i]), g["assoc_s"][i]) < tol


def test_fwd_config1_fp32():
    """B=2, T=256, H=4, N=64, start only at t=0, zero initial state, length=T."""
    check_fwd(wkv7_case(2, 256, 4, seed=1234), torch.float32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [1, 2, 15, 16, 17, 31, 64, 65, 130])
def test_fwd_ragged_lengths_and_starts(T, dtype):
    rng = np.random.default_rng(T)
    starts = [sorted(set(rng.integers(0, T, size=3).tolist())), [0] + ([T - 1] if T > 1 else []), [], [min(1, T - 1)]]
    lengths = [T, max(T - 1, 0), 0, T + 5]
    check_fwd(wkv7_case(4, T, 2, seed=100 + T, s0_scale=0.5, starts=starts, lengths=lengths), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_fwd_adjacent_starts_every_position(dtype):
    T = 40
    d = wkv7_case(2, T, 1, seed=5, s0_scale=1.0, starts=[range(T), [7, 8, 9, 24, 25]], lengths=[T, 9])
    check_fwd(d, dtype)


def test_fwd_config2_shape_bf16():
    """B=8, T=1024, H=12 with Bernoulli(1/256) starts and lengths uniform in [T/2, T]."""
    d = wkv7_case(8, 1024, 12, seed=1235, p_start=1 / 256, random_length=True)
    check_fwd(d, torch.bfloat16)


@pytest.mark.parametrize("dtype,kflags", KERNELS)
@pytest.mark.parametrize("T", [1, 7, 8, 9, 16, 17, 24, 33, 64, 70, 130])
def test_bwd_ragged(T, dtype, kflags):
    rng = np.random.default_rng(T)
    starts = [sorted(set(rng.integers(0, T, size=2).tolist())), [0], [T // 2, min(T // 2 + 1, T - 1)]]
    lengths = [T, max(T - 3, 0), 0]
    check_bwd(wkv7_case(3, T, 2, seed=200 + T, s0_scale=0.5, starts=starts, lengths=lengths), dtype, flags_=kflags)


@pytest.mark.parametrize("dtype,kflags", KERNELS)
def test_bwd_missing_cotangents(dtype, kflags):
    d = wkv7_case(2, 40, 2, seed=9, s0_scale=0.5, starts=[[0, 20], [3]], lengths=[33, 40])
    check_bwd(d, dtype, use_gy=True, use_gs=False, flags_=kflags)
    check_bwd(d, dtype, use_gy=False, use_gs=True, flags_=kflags)


def test_bwd_chunk_single_full_chunk_no_state():
    """Smallest tensor-core case: one 64-token chunk, zero initial state, start at t=0."""
    check_bwd(wkv7_case(1, 64, 1, seed=51), torch.bfloat16)


def test_bwd_chunk_carried_state_two_chunks():
    check_bwd(wkv7_case(1, 128, 1, seed=52, s0_scale=0.5, starts=[[]], lengths=[128]), torch.bfloat16)


def test_bwd_chunk_adjacent_starts():
    T = 70
    check_bwd(wkv7_case(2, T, 1, seed=53, s0_scale=1.0, starts=[range(T), [7, 8, 9, 24, 25, 64, 65]], lengths=[T, 66]), torch.bfloat16)


@pytest.mark.parametrize("kflags", [0, _lib.FLAG_SEQUENTIAL])
def test_bwd_training_shape_bf16(kflags):
    check_bwd(wkv7_case(2, 512, 4, seed=11, p_start=1 / 128, random_length=True, s0_scale=0.1), torch.bfloat16, flags_=kflags)


def test_bwd_config1_fp32():
    check_bwd(wkv7_case(2, 256, 4, seed=1234), torch.float32)


def test_operator_autograd_and_vmap_on_gpu():
    """CudaRWKV.inner_loop end to end: vmap over batch, gradients for all inputs and the state."""
    d = wkv7_case(3, 48, 2, seed=21, s0_scale=0.5, p_start=0.05, random_length=True)
    t = to_dev(d, torch.float32)
    length, ns = flags(d)
    leaves = [t[n].clone().requires_grad_(True) for n in NAMES7]
    s, y = torch.vmap(rwkv7.CudaRWKV.inner_loop)(*leaves, length.cuda(), ns.cuda())
    gy, gs = torch.randn_like(y), torch.randn_like(s)
    ((y * gy).sum() + (s * gs).sum()).backward()
    ref = oracle.wkv7_bwd_batched(*rounded(t), d["length"], d["new_starts"], npf(gy), npf(gs))
    for n, leaf, g in zip(NAMES7, leaves, ref):
        assert rel_err(npf(leaf.grad), g) < 1e-4, n
    # a replicated batch gives identical rows (tests/vmap_test.py of jaxrwkv)
    rep = [x[:1].expand(3, *x.shape[1:]).contiguous() for x in (t[n] for n in NAMES7)]
    s2, y2 = torch.vmap(rwkv7.CudaRWKV.inner_loop, in_dims=(0,) * 7 + (None, None))(*rep, length[0].cuda(), ns[0].cuda())
    assert torch.equal(y2[0], y2[1]) and torch.equal(y2[0], y2[2]) and torch.equal(s2[0], s2[2])


def _residual_mark(res):
    """Last word pair of the bf16 residual: 0 = written by the chunked kernel, 1 = by the sequential fallback."""
    return int(res[-1][-16:].view(torch.int32)[0].item())


def test_decay_outside_the_chunked_range_is_still_exact_bf16():
    """BaseRWKV.inner_loop (rwkv7.py:201) applies exp(-exp(w)) to ANY w.  With w up to 2 the decay reaches
    6e-4 per token, and the cumulative decay inside a 64-token chunk leaves what the tensor-core products can
    carry; the forward must notice, and both directions must still match the oracle - without the caller
    asking for the sequential kernels."""
    d = wkv7_case(2, 200, 2, seed=77, s0_scale=0.5, starts=[[0, 90], []], lengths=[200, 150])
    d["w"] = np.random.default_rng(5).uniform(-0.5, 2.0, size=d["w"].shape).astype(np.float32)
    check_fwd(d, torch.bfloat16)
    check_bwd(d, torch.bfloat16)
    t = to_dev(d, torch.bfloat16)
    length, ns = flags(d)
    assert _residual_mark(run_fwd(t, length, ns)[2]) == 1
    # the model's own parametrisation (w <= -0.5) stays on the tensor-core kernels
    d2 = wkv7_case(2, 200, 2, seed=78, s0_scale=0.5)
    t2 = to_dev(d2, torch.bfloat16)
    length2, ns2 = flags(d2)
    assert _residual_mark(run_fwd(t2, length2, ns2)[2]) == 0
    # only one sequence of the batch out of range, inference call (no residual)
    d3 = wkv7_case(3, 130, 2, seed=79, s0_scale=0.5)
    d3["w"][1, 40:60] = 2.5
    t3 = to_dev(d3, torch.bfloat16)
    length3, ns3 = flags(d3)
    (s, y), _ = rwkv7.batched_wkv7_fwd(*[t3[n] for n in NAMES7], length3, ns3, 3, need_residual=False)
    so, yo = oracle.wkv7_base_batched(*rounded(t3), d3["length"], d3["new_starts"])
    assert rel_err(npf(y), yo) < TOL[torch.bfloat16] and rel_err(npf(s), so) < TOL[torch.bfloat16]


def test_operator_backward_with_strided_and_broadcast_operands():
    """Gradients through views the kernels cannot read directly: the vmapped axis in position 1
    (moved to the front as a strided view) and one int32 length / uint8 new_starts row shared by the
    whole batch (a stride-0 broadcast).  Both must give the oracle's gradients."""
    B, T, H = 3, 40, 2
    d = wkv7_case(B, T, H, seed=33, s0_scale=0.5, starts=[[0, 17]] * B, lengths=[29] * B)
    t = to_dev(d, torch.float32)
    # (T, B, H, N) storage, vmapped over axis 1; the state is (H, B, N, N), vmapped over axis 1
    leaves = [t[n].movedim(0, 1).contiguous().requires_grad_(True) for n in NAMES7]
    length = torch.tensor(29, dtype=torch.int32).cuda()
    ns = torch.tensor(d["new_starts"][0]).to(torch.uint8).cuda()
    s, y = torch.vmap(rwkv7.CudaRWKV.inner_loop, in_dims=(1,) * 7 + (None, None))(*leaves, length, ns)
    gy, gs = torch.randn_like(y), torch.randn_like(s)
    ((y * gy).sum() + (s * gs).sum()).backward()
    ref = oracle.wkv7_bwd_batched(*rounded(t), d["length"], d["new_starts"], npf(gy), npf(gs))
    so, yo = oracle.wkv7_base_batched(*rounded(t), d["length"], d["new_starts"])
    assert rel_err(npf(y), yo) < 1e-4 and rel_err(npf(s), so) < 1e-4
    for n, leaf, g in zip(NAMES7, leaves, ref):
        assert rel_err(npf(leaf.grad.movedim(1, 0)), g) < 1e-4, n


@pytest.mark.parametrize("dtype,kflags", KERNELS)
def test_run_to_run_determinism(dtype, kflags):
    d = wkv7_case(2, 100, 2, seed=31, p_start=0.05, s0_scale=0.3)
    t = to_dev(d, dtype)
    length, ns = flags(d)
    outs = []
    for _ in range(2):
        s, y, res = run_fwd(t, length, ns, kflags)
        g = rwkv7.batched_wkv7_bwd(res, (s.clone(), y.clone()), 2, flags=kflags)
        outs.append((s, y) + tuple(g))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_full_size_properties_bf16():
    """Headline shape B=8, T=4096, H=32, bf16, sequential kernel.  Size-independent properties instead of an
    oracle run: (1) a start flag at t splits the sequence into independent parts, so the
    tail equals a separate call on the tail; (2) y and s_out are linear in (v, s0), and
    scaling by 2 is exact in binary floating point, so the results must be bit-identical
    up to that factor; (3) the carried state composes: one call == two calls of half length."""
    B, T, H = 8, 4096, 32
    d = wkv7_case(B, T, H, seed=1237, s0_scale=0.1)
    d["new_starts"][:, 0] = False
    d["new_starts"][:, 1500] = True
    t = to_dev(d, torch.bfloat16)
    length, ns = flags(d)
    SEQ = _lib.FLAG_SEQUENTIAL
    s, y, _ = run_fwd(t, length, ns, SEQ)
    assert torch.isfinite(y.float()).all() and torch.isfinite(s.float()).all()
    # (1) tail after the start flag == fresh call on the tail with any initial state
    tail = {n: t[n][:, 1500:].contiguous() for n in NAMES7[:-1]}
    tail["s0"] = torch.randn_like(t["s0"])
    ns_tail = ns[:, 1500:].contiguous()
    s_t, y_t, _ = run_fwd(tail, torch.full((B,), T - 1500), ns_tail, SEQ)
    assert torch.equal(y_t, y[:, 1500:]) and torch.equal(s_t, s)
    # (2) exact homogeneity in (v, s0)
    t2 = dict(t); t2["v"] = t["v"] * 2; t2["s0"] = t["s0"] * 2
    s2, y2, _ = run_fwd(t2, length, ns, SEQ)
    assert torch.equal(y2, y * 2) and torch.equal(s2, s * 2)
    # (3) state carry across calls, in fp32 so that the hand-over is not rounded
    B3, H3 = 2, 4
    d3 = wkv7_case(B3, T, H3, seed=1238, s0_scale=0.1)
    t3 = to_dev(d3, torch.float32)
    l3, ns3 = flags(d3)
    s_full, y_full, _ = run_fwd(t3, l3, ns3)
    half = T // 2
    first = {n: t3[n][:, :half].contiguous() for n in NAMES7[:-1]}; first["s0"] = t3["s0"]
    s_a, y_a, _ = run_fwd(first, torch.full((B3,), half), ns3[:, :half].contiguous())
    second = {n: t3[n][:, half:].contiguous() for n in NAMES7[:-1]}; second["s0"] = s_a
    s_b, y_b, _ = run_fwd(second, torch.full((B3,), half), ns3[:, half:].contiguous())
    assert torch.equal(torch.cat([y_a, y_b], 1), y_full) and torch.equal(s_b, s_full)


def test_calls_fail_loudly_on_bad_input():
    d = wkv7_case(1, 16, 1, seed=1)
    t = to_dev(d, torch.float32)
    length, ns = flags(d)
    bad = dict(t); bad["w"] = t["w"].to(torch.bfloat16)
    with pytest.raises(_lib.B200WKVError):
        run_fwd(bad, length, ns)
    cpu = {n: x.cpu() for n, x in t.items()}
    with pytest.raises(_lib.B200WKVError, match="no CPU path"):
        run_fwd(cpu, length, ns)


# ---------------------------------------------------------------- tensor-core (chunked) forward
def run_fwd_infer(t, length, ns):
    """bf16 forward without a residual: dispatches to the chunked tcgen05 kernel."""
    B = t["k"].shape[0]
    (s, y), _ = rwkv7.batched_wkv7_fwd(t["r"], t["w"], t["k"], t["v"], t["a"], t["b"], t["s0"], length, ns, B,
                                       need_residual=False)
    return s, y


def check_fwd_chunk(d, tol=TOL[torch.bfloat16]):
    t = to_dev(d, torch.bfloat16)
    length, ns = flags(d)
    s, y = run_fwd_infer(t, length, ns)
    so, yo = oracle.wkv7_base_batched(*rounded(t), d["length"], d["new_starts"])
    ey = rel_err(npf(y), yo)
    assert ey < tol, ("y", ey)
    for i in range(so.shape[0]):
        e = rel_err(npf(s[i]), so[i])
        assert e < tol, ("s_out", i, e)
    # and against the sequential fp32-arithmetic kernel on the same bf16 inputs
    s2, y2, _ = run_fwd(t, length, ns, _lib.FLAG_SEQUENTIAL)
    assert rel_err(npf(y), npf(y2)) < tol


def test_chunk_fwd_single_full_chunk():
    check_fwd_chunk(wkv7_case(1, 64, 1, seed=41))


def test_chunk_fwd_carried_state_multi_chunk():
    check_fwd_chunk(wkv7_case(2, 256, 2, seed=42, s0_scale=0.5, starts=[[], [0]], lengths=[256, 256]))


@pytest.mark.parametrize("T", [1, 2, 15, 16, 17, 63, 65, 130, 200])
def test_chunk_fwd_ragged_lengths_and_starts(T):
    rng = np.random.default_rng(T)
    starts = [sorted(set(rng.integers(0, T, size=3).tolist())), [0] + ([T - 1] if T > 1 else []), [], [min(1, T - 1)]]
    lengths = [T, max(T - 1, 0), 0, T + 5]
    check_fwd_chunk(wkv7_case(4, T, 2, seed=300 + T, s0_scale=0.5, starts=starts, lengths=lengths))


def test_chunk_fwd_adjacent_starts_every_position():
    T = 70
    check_fwd_chunk(wkv7_case(2, T, 1, seed=45, s0_scale=1.0, starts=[range(T), [7, 8, 9, 24, 25, 64, 65]], lengths=[T, 9]))


def test_chunk_fwd_config2_shape():
    check_fwd_chunk(wkv7_case(8, 1024, 12, seed=1235, p_start=1 / 256, random_length=True))


def test_chunk_fwd_reference_fixtures(golden):
    for case in ("v7_plain", "v7_resets"):
        g = golden(case)
        d = {n: g["in_" + n] for n in NAMES7 + ("length", "new_starts")}
        t = to_dev(d, torch.bfloat16)
        length, ns = flags(d)
        s, y = run_fwd_infer(t, length, ns)
        assert rel_err(npf(y), g["base_y"]) < 3e-2       # fixtures were computed on unrounded inputs
        for i in range(s.shape[0]):
            assert rel_err(npf(s[i]), g["base_s"][i]) < 3e-2


def test_chunk_fwd_full_size_properties():
    """Headline shape on the tensor-core kernel: finite, deterministic, exactly homogeneous in
    (v, s0) under scaling by 2, and start flags / state hand-over agree with separate calls to
    within the bf16 tolerance (chunk boundaries differ between the two runs, so not bit-equal)."""
    B, T, H = 8, 4096, 32
    d = wkv7_case(B, T, H, seed=1237, s0_scale=0.1)
    d["new_starts"][:, 0] = False
    d["new_starts"][:, 1500] = True
    t = to_dev(d, torch.bfloat16)
    length, ns = flags(d)
    s, y = run_fwd_infer(t, length, ns)
    s_again, y_again = run_fwd_infer(t, length, ns)
    assert torch.isfinite(y.float()).all() and torch.isfinite(s.float()).all()
    assert torch.equal(y, y_again) and torch.equal(s, s_again)
    t2 = dict(t); t2["v"] = t["v"] * 2; t2["s0"] = t["s0"] * 2
    s2, y2 = run_fwd_infer(t2, length, ns)
    assert torch.equal(y2, y * 2) and torch.equal(s2, s * 2)
    tail = {n: t[n][:, 1500:].contiguous() for n in NAMES7[:-1]}
    tail["s0"] = torch.randn_like(t["s0"])
    s_t, y_t = run_fwd_infer(tail, torch.full((B,), T - 1500), ns[:, 1500:].contiguous())
    assert rel_err(npf(y_t), npf(y[:, 1500:])) < 1e-2 and rel_err(npf(s_t), npf(s)) < 1e-2
    # sequential kernel on the same inputs
    s_q, y_q, _ = run_fwd(t, length, ns, _lib.FLAG_SEQUENTIAL)
    assert rel_err(npf(y), npf(y_q)) < TOL[torch.bfloat16] and rel_err(npf(s), npf(s_q)) < TOL[torch.bfloat16]
    # and the oracle itself on four (batch, head) slices: y and the returned state
    for bi, hh in ((0, 0), (2, 9), (5, 30), (7, 31)):
        ins = [t[n][bi, :, hh:hh + 1].double().cpu().numpy() for n in NAMES7[:-1]] + [t["s0"][bi, hh:hh + 1].double().cpu().numpy()]
        so, yo = oracle.wkv7_base(*ins, int(d["length"][bi]), d["new_starts"][bi])
        assert rel_err(npf(y[bi, :, hh:hh + 1]), yo) < TOL[torch.bfloat16], ("y", bi, hh)
        assert rel_err(npf(s[bi, hh:hh + 1]), so) < TOL[torch.bfloat16], ("s_out", bi, hh)


def test_chunk_bwd_full_size_properties():
    """Headline shape through the tensor-core forward + backward: finite, deterministic, and the
    gradients are exactly homogeneous of degree one in the cotangents (scaling dy and ds by 2)."""
    B, T, H = 8, 4096, 32
    d = wkv7_case(B, T, H, seed=1239, s0_scale=0.1, p_start=1 / 512)
    t = to_dev(d, torch.bfloat16)
    length, ns = flags(d)
    s, y, res = run_fwd(t, length, ns)
    gy = torch.randn_like(y); gs = torch.randn_like(s)
    g1 = rwkv7.batched_wkv7_bwd(res, (gs, gy), B)
    g1b = rwkv7.batched_wkv7_bwd(res, (gs, gy), B)
    g2 = rwkv7.batched_wkv7_bwd(res, (gs * 2, gy * 2), B)
    for a, b, c in zip(g1, g1b, g2):
        assert torch.isfinite(a.float()).all()
        assert torch.equal(a, b)
        assert torch.equal(c, a * 2)
    # spot-check two (batch, head) slices against the oracle
    for bi, hh in ((0, 0), (0, 1), (0, 3), (7, 31)):   # (0, 1) and (0, 3) are walked by two CTAs each on 148 SMs
        ins = [t[n][bi:bi + 1, :, hh:hh + 1].double().cpu().numpy() for n in NAMES7[:-1]] + [t["s0"][bi:bi + 1, hh:hh + 1].double().cpu().numpy()]
        ref = oracle.wkv7_bwd_batched(*ins, d["length"][bi:bi + 1], d["new_starts"][bi:bi + 1],
                                      npf(gy[bi:bi + 1, :, hh:hh + 1]), npf(gs[bi:bi + 1, hh:hh + 1]))
        got = [g1[i][bi:bi + 1, :, hh:hh + 1] for i in range(6)] + [g1[6][bi:bi + 1, hh:hh + 1]]
        for n, a, b in zip(("dr", "dw", "dk", "dv", "da", "db", "ds0"), got, ref):
            assert rel_err(npf(a), b) < TOL[torch.bfloat16], (n, bi, hh, rel_err(npf(a), b))


@pytest.mark.parametrize("T", [64, 192, 512])
def test_bwd_carry_and_gradient_kernels(T):
    """Sequences made of whole 64-token blocks (start flags only at multiples of 64, `length` 0, a multiple of 64
    or beyond T) take the two-kernel backward: the sequential state-gradient carry, then the gradients of all
    blocks in parallel.  Rows of other kinds in the same call (a flag or `length` inside a block) take the
    one-kernel backward; every gradient of every row against the oracle."""
    nb = T // 64
    starts = [[0], [], [0, 64 * (nb // 2)], [64 * (nb - 1)], [0, 5], []]
    lengths = [T, T + 7, 64 * max(nb - 1, 0), 0, T, T - 3]
    d = wkv7_case(6, T, 3, seed=600 + T, s0_scale=0.5, starts=starts, lengths=lengths)
    check_bwd(d, torch.bfloat16)
    check_bwd(d, torch.bfloat16, use_gy=True, use_gs=False)
    # With dy = 0 and a 64 x 64 state cotangent the decay gradient is the small difference of large running sums
    # D_t = sum_i dS_t S_t (|dw| is a tenth of |dk|): every tensor-core backward here, one-kernel or split, lands
    # near 2.5 % on it (the fp32 sequential kernels at 0.2 %), so this one gradient gets 4e-2 in this one variant.
    check_bwd(d, torch.bfloat16, use_gy=False, use_gs=True, tol_dw=4e-2)


def test_bwd_carry_and_gradient_kernels_many_sequences():
    """More (sequence, block) pairs than resident CTAs, so that every CTA of the gradient kernel walks several
    blocks of several sequences; run twice for bit-identical results."""
    B, T, H = 6, 1024, 40
    d = wkv7_case(B, T, H, seed=77, s0_scale=0.3, starts=[[0], [], [0, 512], [], [0], [256]], lengths=[T, T, 768, T, 0, T])
    t = to_dev(d, torch.bfloat16)
    length, ns = flags(d)
    s, y, res = run_fwd(t, length, ns)
    gy, gs = torch.randn_like(y), torch.randn_like(s)
    g1 = rwkv7.batched_wkv7_bwd(res, (gs, gy), B)
    g2 = rwkv7.batched_wkv7_bwd(res, (gs, gy), B)
    for a, b in zip(g1, g2):
        assert torch.isfinite(a.float()).all() and torch.equal(a, b)
    for bi, hh in ((0, 0), (1, 39), (2, 7), (4, 20), (5, 13)):
        ins = [t[n][bi:bi + 1, :, hh:hh + 1].double().cpu().numpy() for n in NAMES7[:-1]] + [t["s0"][bi:bi + 1, hh:hh + 1].double().cpu().numpy()]
        ref = oracle.wkv7_bwd_batched(*ins, d["length"][bi:bi + 1], d["new_starts"][bi:bi + 1],
                                      npf(gy[bi:bi + 1, :, hh:hh + 1]), npf(gs[bi:bi + 1, hh:hh + 1]))
        got = [g1[i][bi:bi + 1, :, hh:hh + 1] for i in range(6)] + [g1[6][bi:bi + 1, hh:hh + 1]]
        for n, a, b in zip(("dr", "dw", "dk", "dv", "da", "db", "ds0"), got, ref):
            assert rel_err(npf(a), b) < TOL[torch.bfloat16], (n, bi, hh, rel_err(npf(a), b))


def test_bwd_carry_ring_depths_agree():
    """With more sequences than two per SM the state-gradient carry runs a shallower copy ring at four CTAs per SM; the
    same rows in two calls of half the batch take the deeper ring: every gradient must be bit-identical."""
    B, T, H = 10, 256, 32
    starts = [[0], [], [0, 128], [64], [0], [192], [], [0, 64, 128, 192], [], [0]]
    lengths = [T, T, 128, T, 0, T, 64, T, T + 5, 192]
    d = wkv7_case(B, T, H, seed=91, s0_scale=0.4, starts=starts, lengths=lengths)
    t = to_dev(d, torch.bfloat16)
    length, ns = flags(d)
    s, y, res = run_fwd(t, length, ns)
    gy, gs = torch.randn_like(y), torch.randn_like(s)
    whole = rwkv7.batched_wkv7_bwd(res, (gs, gy), B)
    for lo in (0, 5):
        th = {n: v[lo:lo + 5].contiguous() for n, v in t.items()}
        s_h, y_h, res_h = run_fwd(th, length[lo:lo + 5].contiguous(), ns[lo:lo + 5].contiguous())
        assert torch.equal(y_h, y[lo:lo + 5]) and torch.equal(s_h, s[lo:lo + 5])
        half = rwkv7.batched_wkv7_bwd(res_h, (gs[lo:lo + 5].contiguous(), gy[lo:lo + 5].contiguous()), 5)
        for a, b in zip(half, whole):
            assert torch.equal(a, b[lo:lo + 5])


def test_bwd_headline_shape_against_oracle_slices():
    """The benchmark's own shape and flags (B=8, T=4096, H=32, a start at t=0 only, length = T): the path the
    headline number times.  Four (batch, head) slices of every gradient against the oracle."""
    B, T, H = 8, 4096, 32
    d = wkv7_case(B, T, H, seed=1240, s0_scale=0.1)
    t = to_dev(d, torch.bfloat16)
    length, ns = flags(d)
    s, y, res = run_fwd(t, length, ns)
    gy, gs = torch.randn_like(y), torch.randn_like(s)
    g1 = rwkv7.batched_wkv7_bwd(res, (gs, gy), B)
    for a in g1:
        assert torch.isfinite(a.float()).all()
    for bi, hh in ((0, 0), (3, 1), (5, 17), (7, 31)):
        ins = [t[n][bi:bi + 1, :, hh:hh + 1].double().cpu().numpy() for n in NAMES7[:-1]] + [t["s0"][bi:bi + 1, hh:hh + 1].double().cpu().numpy()]
        ref = oracle.wkv7_bwd_batched(*ins, d["length"][bi:bi + 1], d["new_starts"][bi:bi + 1],
                                      npf(gy[bi:bi + 1, :, hh:hh + 1]), npf(gs[bi:bi + 1, hh:hh + 1]))
        got = [g1[i][bi:bi + 1, :, hh:hh + 1] for i in range(6)] + [g1[6][bi:bi + 1, hh:hh + 1]]
        for n, a, b in zip(("dr", "dw", "dk", "dv", "da", "db", "ds0"), got, ref):
            assert rel_err(npf(a), b) < TOL[torch.bfloat16], (n, bi, hh, rel_err(npf(a), b))


@pytest.mark.parametrize("T", [300, 512])
def test_chunk_bwd_sequences_split_across_ctas(T):
    """More sequences than SMs and not a multiple of them: the tensor-core backward cuts sequences
    into runs of blocks owned by neighbouring CTAs.  Ragged lengths and start flags; every gradient
    against the token-sequential kernels on the same inputs."""
    B, H = 5, 37
    d = wkv7_case(B, T, H, seed=4321 + T, s0_scale=0.3, p_start=1 / 100, random_length=True)
    t = to_dev(d, torch.bfloat16)
    length, ns = flags(d)
    s, y, res = run_fwd(t, length, ns)
    gy = torch.randn_like(y); gs = torch.randn_like(s)
    g1 = rwkv7.batched_wkv7_bwd(res, (gs, gy), B)
    g1b = rwkv7.batched_wkv7_bwd(res, (gs, gy), B)
    s_q, y_q, res_q = run_fwd(t, length, ns, _lib.FLAG_SEQUENTIAL)
    g2 = rwkv7.batched_wkv7_bwd(res_q, (gs, gy), B, flags=_lib.FLAG_SEQUENTIAL)
    for n, a, a2, b in zip(("dr", "dw", "dk", "dv", "da", "db", "ds0"), g1, g1b, g2):
        assert torch.equal(a, a2), n
        for bi in range(B):
            assert rel_err(npf(a[bi]), npf(b[bi])) < TOL[torch.bfloat16], (n, bi, rel_err(npf(a[bi]), npf(b[bi])))


def test_forward_backward_replay_from_a_cuda_graph():
    """The calls only enqueue work (kernels, one small memset), so a forward + backward pair can be captured
    into a CUDA graph and replayed on new data; shape chosen so that the backward runs in its split mode."""
    B, T, H = 5, 256, 37
    d = wkv7_case(B, T, H, seed=77, s0_scale=0.3, p_start=1 / 100, random_length=True)
    t = to_dev(d, torch.bfloat16)
    length, ns = (x.cuda() for x in flags(d))
    length, ns = length.to(torch.int32), ns.to(torch.uint8)
    gy = torch.randn_like(t["r"]); gs = torch.randn_like(t["s0"])
    rwkv7.batched_wkv7_bwd(run_fwd(t, length, ns)[2], (gs, gy), B)     # first calls outside the capture
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            s, y, res = run_fwd(t, length, ns)
            grads = rwkv7.batched_wkv7_bwd(res, (gs, gy), B)
    torch.cuda.current_stream().wait_stream(side)
    # new data in the captured input buffers, then replay
    for n in NAMES7[:-1]:
        t[n].copy_(torch.roll(t[n], 1, dims=0))
    gy.copy_(torch.roll(gy, 1, dims=0))
    graph.replay()
    torch.cuda.synchronize()
    s2, y2, res2 = run_fwd(t, length, ns)
    grads2 = rwkv7.batched_wkv7_bwd(res2, (gs, gy), B)
    assert torch.equal(y, y2) and torch.equal(s, s2)
    for a, b in zip(grads, grads2):
        assert torch.equal(a, b)


def test_host_pipeline_matches_device_path():
    """wkv7_fwd_bwd_host (pinned host tensors in and out, batch sliced over three streams) returns
    exactly what the device-resident forward + backward return."""
    from jaxrwkv_b200.host import wkv7_fwd_bwd_host
    d = wkv7_case(5, 200, 2, seed=71, s0_scale=0.3, p_start=0.02, random_length=True)
    t = to_dev(d, torch.bfloat16)
    length, ns = flags(d)
    g = torch.Generator().manual_seed(1)
    gy = torch.randn(t["k"].shape, generator=g).bfloat16().cuda(); gs = torch.randn(t["s0"].shape, generator=g).bfloat16().cuda()
    s, y, res = run_fwd(t, length, ns)
    grads = rwkv7.batched_wkv7_bwd(res, (gs, gy), 5)
    host_in = {n: t[n].cpu().pin_memory() for n in NAMES7}
    host_in["dy"] = gy.cpu().pin_memory(); host_in["ds"] = gs.cpu().pin_memory()
    for rows in (1, 2):
        out = wkv7_fwd_bwd_host(host_in, length, ns, slice_rows=rows)
        assert torch.equal(out["y"], y.cpu()) and torch.equal(out["s_out"], s.cpu())
        for n, ref in zip(("dr", "dw", "dk", "dv", "da", "db", "ds0"), grads):
            assert torch.equal(out[n], ref.cpu()), n


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_step_kernel(dtype):
    """T == 1 without a residual takes the single-pass step kernel: carried state, start flags on
    some rows, length 0 on one row; then 6 chained steps against the oracle run over the 6 tokens."""
    B, H = 5, 3
    d = wkv7_case(B, 1, H, seed=81, s0_scale=0.7, starts=[[], [0], [], [0], []], lengths=[1, 1, 0, 0, 1])
    t = to_dev(d, dtype)
    length, ns = flags(d)
    (s, y), _ = rwkv7.batched_wkv7_fwd(*[t[n] for n in NAMES7], length, ns, B, need_residual=False)
    so, yo = oracle.wkv7_base_batched(*rounded(t), d["length"], d["new_starts"])
    assert rel_err(npf(y), yo) < TOL[dtype]
    for i in range(B):
        assert rel_err(npf(s[i]), so[i]) < TOL[dtype], i
    d = wkv7_case(2, 6, 2, seed=82, s0_scale=0.5, starts=[[3], []], lengths=[6, 6])
    t = to_dev(d, torch.float32)
    st = t["s0"]
    outs = []
    for tt in range(6):
        st, o = rwkv7.wkv7_step(*[t[n][:, tt] for n in NAMES7[:-1]], st, new_starts=torch.tensor(d["new_starts"][:, tt]).cuda())
        outs.append(o)
    so, yo = oracle.wkv7_base_batched(*rounded(t), d["length"], d["new_starts"])
    assert rel_err(npf(torch.stack(outs, 1)), yo) < 1e-4 and rel_err(npf(st), so) < 1e-4


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_step_many_pairs_ring_wraps(dtype):
    """More (batch, head) pairs than resident CTAs times ring stages, so every CTA refills each
    stage of its ring several times; compared with the T-loop kernels on the same one-token inputs."""
    B, H = 192, 40
    g = torch.Generator(device="cuda").manual_seed(5)
    shp = (B, 1, H, 64)
    r, k, v = (torch.randn(shp, device="cuda", generator=g).to(dtype) for _ in range(3))
    w = (-0.5 - torch.nn.functional.softplus(torch.randn(shp, device="cuda", generator=g))).to(dtype)
    kk = torch.nn.functional.normalize(torch.randn(shp, device="cuda", generator=g), dim=-1)
    a, b = (-kk).to(dtype), (kk * torch.rand(shp, device="cuda", generator=g)).to(dtype)
    s0 = (0.5 * torch.randn(B, H, 64, 64, device="cuda", generator=g)).to(dtype)
    length = torch.ones(B, dtype=torch.int32, device="cuda")
    length[7] = 0
    ns = torch.zeros(B, 1, dtype=torch.uint8, device="cuda")
    ns[3] = 1
    ns[190] = 1
    (s1, y1), _ = rwkv7.batched_wkv7_fwd(r, w, k, v, a, b, s0, length, ns, B, need_residual=False)
    # the recurrence of one token in float64 (rwkv7.py:199-220), state indexed [value][key]
    f = lambda x: x.double().squeeze(1)
    S = torch.where(ns.bool()[:, :, None, None], torch.zeros_like(s0, dtype=torch.float64), s0.double())
    sa = torch.einsum("bhij,bhj->bhi", S, f(a))
    S = S * torch.exp(-torch.exp(f(w)))[:, :, None, :] + f(v)[..., :, None] * f(k)[..., None, :] + sa[..., :, None] * f(b)[..., None, :]
    y2 = torch.einsum("bhij,bhj->bhi", S, f(r)).unsqueeze(1)
    s2 = torch.where((length > 0)[:, None, None, None], S, s0.double())
    rows = [(i, rel_err(npf(y1[i]), y2[i].cpu().numpy())) for i in range(B)]
    assert max(e for _, e in rows) < TOL[dtype], sorted(rows, key=lambda t: -t[1])[:5]
    assert rel_err(npf(s1), s2.cpu().numpy()) < TOL[dtype]
    assert torch.equal(s1[7], s0[7])
    # the T-loop kernels on the same one-token problem
    (s3, y3), _ = rwkv7.batched_wkv7_fwd(r, w, k, v, a, b, s0, length, ns, B, need_residual=True,
                                         flags=_lib.FLAG_SEQUENTIAL)
    rows = [(i, rel_err(npf(y3[i]), y2[i].cpu().numpy())) for i in range(B)]
    assert max(e for _, e in rows) < TOL[dtype], sorted(rows, key=lambda t: -t[1])[:5]
    assert rel_err(npf(s3), s2.cpu().numpy()) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_step_on_packed_state_in_place(dtype):
    """The step that updates the (H, N, N) block inside the model's packed (B, L, 2+N, D) state where
    it lies equals the step on a copied-out block, and touches nothing else in the container."""
    B, H, L, N = 6, 5, 3, 64
    g = torch.Generator(device="cuda").manual_seed(17)
    shp = (B, 1, H, N)
    r, k, v = (torch.randn(shp, device="cuda", generator=g).to(dtype) for _ in range(3))
    w = (-0.5 - torch.nn.functional.softplus(torch.randn(shp, device="cuda", generator=g))).to(dtype)
    kk = torch.nn.functional.normalize(torch.randn(shp, device="cuda", generator=g), dim=-1)
    a, b = (-kk).to(dtype), (kk * torch.rand(shp, device="cuda", generator=g)).to(dtype)
    state = (0.5 * torch.randn(B, L, 2 + N, H * N, device="cuda", generator=g)).to(dtype)
    ns = torch.zeros(B, 1, dtype=torch.uint8, device="cuda"); ns[2] = 1
    length = torch.ones(B, dtype=torch.int32, device="cuda"); length[4] = 0
    layer = 1
    before = state.clone()
    # the reference reshapes state[1:] (N, H*N) to (H, N, N) as a raw reshape (rwkv7.py:255)
    s_in = before[:, layer, 2:].reshape(B, H, N, N)
    s_ref, y_ref = rwkv7.wkv7_step(r, w, k, v, a, b, s_in, new_starts=ns, length=length)
    y = rwkv7.wkv7_step_packed(r, w, k, v, a, b, state, layer, new_starts=ns, length=length)
    assert torch.equal(y, y_ref)
    assert torch.equal(state[:, layer, 2:].reshape(B, H, N, N), s_ref)
    untouched = torch.ones(L, 2 + N, dtype=torch.bool); untouched[layer, 2:] = False
    assert torch.equal(state[:, untouched], before[:, untouched])


def test_no_bounded_wait_ran_out_during_the_suite():
    """Every mbarrier wait in the tensor-core kernels is bounded and records a failure in a device
    word; after the tensor-core tests above that word must still be clear."""
    assert _lib.load().b200wkv_device_status() == 0


def test_inference_forward_cut_at_start_flags():
    """Few sequences, calls without a residual: the forward offers every sequence to several CTAs, which cut it at start
    flags (a flag cuts every dependence).  Lengths on a cut, before it, behind it, zero; sequences without any flag;
    flags only near the ends; all against the oracle."""
    T = 1024
    # cuts are looked for near k T / 8: flags exactly there, just beside, and far away
    starts = [[128, 256, 384, 640, 900], [], [5, 1020], [127, 129, 511, 513, 514], [0, 300, 301, 767], [512]]
    lengths = [T, T, 700, 513, 0, 512]
    d = wkv7_case(6, T, 2, seed=501, s0_scale=0.5, starts=starts, lengths=lengths)
    check_fwd_chunk(d)
    # the benchmark's inference configuration in small: Bernoulli(1/256) flags, ragged lengths
    d = wkv7_case(3, 2048, 2, seed=502, s0_scale=0.0, p_start=1 / 256, random_length=True)
    check_fwd_chunk(d)
