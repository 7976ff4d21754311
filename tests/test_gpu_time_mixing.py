"""GPU tests of the elementwise stages around the RWKV-7 operator (b200wkv7_mix_pre / _post) and of the
whole time-mixing function built from them, the token-shift kernel and the WKV operator."""
import numpy as np
import pytest
import torch

from conftest import rel_err
from test_oracle import unflatten_params

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    from jaxrwkv_b200 import time_mixing as tm


def ref_pre(k, wl, al, v, vf, vl, w0, a0, v0, k_k, k_a, H):
    """rwkv7.py:238-252, :257 in plain torch (differentiable)."""
    C = k.shape[-1]
    w = -torch.nn.functional.softplus(-(w0.reshape(C) + wl)) - 0.5
    if vf is not None:
        v = v + (vf - v) * torch.sigmoid(v0.reshape(C) + vl)
    a = torch.sigmoid(a0.reshape(C) + al)
    kk = (k * k_k.reshape(C)).reshape(*k.shape[:-1], H, -1)
    kk = kk / torch.clamp(torch.linalg.norm(kk, dim=-1, keepdim=True), min=1e-12)
    kk = kk.reshape(k.shape)
    return w, k * (1 + (a - 1) * k_a.reshape(C)), v, -kk, kk * a


def ref_post(y, r, k, v, g, ln_w, ln_b, r_k, H, eps=64e-5):
    """rwkv7.py:263-265 in plain torch."""
    C = y.shape[-1]
    yh = y.reshape(*y.shape[:-1], H, -1)
    mean = yh.mean(dim=-1, keepdim=True)
    var = yh.var(dim=-1, unbiased=False, keepdim=True)
    x = ((yh - mean) / torch.sqrt(var + eps)).reshape(y.shape) * ln_w.reshape(C) + ln_b.reshape(C)
    hs = lambda t: t.reshape(*t.shape[:-1], H, -1)
    bonus = (hs(r) * hs(k) * r_k.reshape(H, -1)).sum(dim=-1, keepdim=True)
    return (x + (bonus * hs(v)).reshape(y.shape)) * g


def _leaves(gen, shapes, dtype, dev, scale=1.0):
    return [(scale * torch.randn(s, generator=gen, dtype=torch.float64)).to(dtype).to(dev).requires_grad_(True) for s in shapes]


CASES = [(2, 37, 2), (1, 300, 32), (3, 50, 40), (2, 33, 3)]      # (B, T, H): 16 rows per block; 1; 320-thread blocks; 240


@pytest.mark.parametrize("B,T,H", CASES)
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("use_vmix", [True, False])
def test_mix_pre_forward_backward(B, T, H, dtype, tol, use_vmix):
    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(5 + H)
    C = H * 64
    k, wl, al, v, vf, vl = _leaves(gen, [(B, T, C)] * 6, dtype, dev)
    w0, a0, v0, k_k, k_a = _leaves(gen, [(1, 1, C)] * 5, dtype, dev)
    cot = [torch.randn(B, T, C, generator=gen, dtype=torch.float64).to(dtype).to(dev) for _ in range(5)]
    if use_vmix:
        outs = tm.mix_pre(k, wl, al, v, vf, vl, w0, a0, v0, k_k, k_a, H)
    else:
        outs = tm.mix_pre(k, wl, al, v, None, None, w0, a0, None, k_k, k_a, H)
    leaves = [k, wl, al, v, w0, a0, k_k, k_a] + ([vf, vl, v0] if use_vmix else [])
    grads = torch.autograd.grad(outs, leaves, cot)
    d = [t.detach().double().cpu().requires_grad_(True) for t in (k, wl, al, v, vf, vl, w0, a0, v0, k_k, k_a)]
    ref = ref_pre(d[0], d[1], d[2], d[3], d[4] if use_vmix else None, d[5], d[6], d[7], d[8], d[9], d[10], H)
    ref_leaves = [d[0], d[1], d[2], d[3], d[6], d[7], d[9], d[10]] + ([d[4], d[5], d[8]] if use_vmix else [])
    ref_grads = torch.autograd.grad(ref, ref_leaves, [c.double().cpu() for c in cot])
    for name, got, want in zip(("w", "k", "v", "a_i", "b_i"), outs, ref):
        assert rel_err(got.detach().float().cpu().numpy(), want.detach().numpy()) < tol, name
    # parameter gradients are sums over B*T rows of products rounded to bf16 once at the end: same tolerance
    for i, (got, want) in enumerate(zip(grads, ref_grads)):
        assert got.shape == want.shape
        assert rel_err(got.float().cpu().numpy(), want.numpy()) < 2 * tol, i


@pytest.mark.parametrize("B,T,H", CASES)
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1.5e-2)])
def test_mix_post_forward_backward(B, T, H, dtype, tol):
    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(11 + H)
    C = H * 64
    y, r, k, v, g = _leaves(gen, [(B, T, C)] * 5, dtype, dev)
    ln_w, ln_b = _leaves(gen, [(C,)] * 2, dtype, dev)
    (r_k,) = _leaves(gen, [(H, 64)], dtype, dev, scale=0.3)
    cot = torch.randn(B, T, C, generator=gen, dtype=torch.float64).to(dtype).to(dev)
    out = tm.mix_post(y, r, k, v, g, ln_w, ln_b, r_k, H)
    leaves = [y, r, k, v, g, ln_w, ln_b, r_k]
    grads = torch.autograd.grad(out, leaves, cot)
    d = [t.detach().double().cpu().requires_grad_(True) for t in leaves]
    ref = ref_post(*d, H)
    ref_grads = torch.autograd.grad(ref, d, cot.double().cpu())
    assert rel_err(out.detach().float().cpu().numpy(), ref.detach().numpy()) < tol
    for i, (got, want) in enumerate(zip(grads, ref_grads)):
        assert got.shape == want.shape
        assert rel_err(got.float().cpu().numpy(), want.numpy()) < 2 * tol, i


def test_mix_pre_zero_key_rows_hit_the_norm_floor():
    """k == 0 for a whole head: the reference divides by max(norm, 1e-12), so kk is exactly zero and its gradient
    is the cotangent times 1e12 (rwkv7.py:250)."""
    dev = torch.device("cuda")
    gen = torch.Generator().manual_seed(3)
    H, C = 2, 128
    k, wl, al, v = _leaves(gen, [(1, 5, C)] * 4, torch.float32, dev)
    with torch.no_grad():
        k[0, 2, :64] = 0
    w0, a0, k_k, k_a = _leaves(gen, [(C,)] * 4, torch.float32, dev)
    outs = tm.mix_pre(k, wl, al, v, None, None, w0, a0, None, k_k, k_a, H)
    assert torch.all(outs[3][0, 2, :64] == 0) and torch.all(outs[4][0, 2, :64] == 0)
    assert all(torch.isfinite(o).all() for o in outs)
    cot = [torch.zeros_like(k) for _ in range(5)]
    cot[3] = torch.full_like(k, 1e-12)
    (gk,) = torch.autograd.grad(outs, [k], cot)
    want = -(k_k.detach())[:64]                # d a_i / d k = -k_k / 1e-12 below the floor
    assert rel_err(gk[0, 2, :64].cpu().numpy(), want.cpu().numpy()) < 1e-5


def test_abi_rejects_bad_shapes_and_alignment():
    from jaxrwkv_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(64 * 4 + 8, dtype=torch.float32, device="cuda")
    p = x.data_ptr()
    args = [p] * 16
    assert lib.b200wkv7_mix_pre_fwd(None, _lib.F32, 1, 1, 32, 0, *args) == -2          # N != 64
    assert lib.b200wkv7_mix_pre_fwd(None, _lib.F32, 0, 1, 64, 0, *args) == -2          # no rows
    assert lib.b200wkv7_mix_pre_fwd(None, 7, 1, 1, 64, 0, *args) == -1                 # dtype
    bad = [p + 4] + [p] * 15
    assert lib.b200wkv7_mix_pre_fwd(None, _lib.F32, 1, 1, 64, 0, *bad) == -6           # misaligned (B200WKV_EUNSUPPORTED)
    assert lib.b200wkv7_mix_post_fwd(None, _lib.F32, 1, 1, 64, 1e-3, *([p] * 8 + [None])) == -3   # NULL result


@pytest.mark.parametrize("layer_id", [0, 1])
def test_time_mixing_layer_matches_reference_fixture(golden, layer_id):
    """The reference's own time_mixing_seq (fixture) against token-shift kernel + GEMMs + mix_pre kernel + WKV
    operator + mix_post kernel in fp32; tolerance 1e-4 (the fp32 bar of the operator)."""
    g = golden("v7_time_mixing")
    dev = torch.device("cuda")
    to = lambda a: torch.as_tensor(np.asarray(a, dtype=np.float32), device=dev)
    att = unflatten_params(g)
    att = {k: ({kk: to(vv) for kk, vv in v.items()} if isinstance(v, dict) else to(v)) for k, v in att.items()}
    H, S = int(g["H"]), int(g["S"])
    out, state, vf = tm.time_mixing_seq(to(g["in_x"]), to(g["in_state"]), to(g["in_v_first"]), att,
                                        torch.as_tensor(g["in_length"].astype(np.int32), device=dev),
                                        torch.as_tensor(g["in_new_starts"], device=dev), H, S, layer_id)
    # (the fixture's parameters are (1, 1, C) as in the reference's checkpoints, which leaves a unit axis in its results)
    assert rel_err(out.detach().cpu().numpy(), g[f"out_l{layer_id}"].reshape(out.shape)) < 1e-4
    assert rel_err(state.detach().cpu().numpy(), g[f"state_l{layer_id}"].reshape(state.shape)) < 1e-4
    assert rel_err(vf.detach().cpu().numpy(), g[f"v_first_l{layer_id}"].reshape(vf.shape)) < 1e-5


def test_time_mixing_layer_gradients_match_cpu_autograd(golden):
    """d(sum of out * cot)/d(x, state, every parameter) through the kernels' backward passes against torch autograd of
    the same function written with plain torch ops and the differentiable CPU restatement of the operator (fp64)."""
    from oracle import torch_ref
    g = golden("v7_time_mixing")
    dev = torch.device("cuda")
    H, S = int(g["H"]), int(g["S"])
    att_np = unflatten_params(g)
    B, T, C = g["in_x"].shape
    length = g["in_length"].astype(np.int64)
    ns = g["in_new_starts"]
    gen = torch.Generator().manual_seed(9)
    cot = torch.randn(B, T, C, generator=gen, dtype=torch.float64)

    def leaves(device, dtype):
        mk = lambda a: torch.as_tensor(np.asarray(a), dtype=dtype, device=device).requires_grad_(True)
        att = {k: ({kk: mk(vv) for kk, vv in v.items()} if isinstance(v, dict) else mk(v)) for k, v in att_np.items()}
        flat = [att[k] if not isinstance(att[k], dict) else None for k in sorted(att)]
        flat = [t for t in flat if t is not None] + [att[k][kk] for k in sorted(att) if isinstance(att[k], dict) for kk in sorted(att[k])]
        return att, flat, mk(g["in_x"]), mk(g["in_state"]), mk(g["in_v_first"])

    att, flat, x, state, vf = leaves(dev, torch.float32)
    out, new_state, _ = tm.time_mixing_seq(x, state, vf, att, torch.as_tensor(length.astype(np.int32), device=dev),
                                           torch.as_tensor(ns, device=dev), H, S, 1)
    loss = (out * cot.to(dev).float()).sum() + 0.1 * new_state.sum()
    got = torch.autograd.grad(loss, [x, state, vf] + flat, allow_unused=True)

    att_r, flat_r, x_r, state_r, vf_r = leaves("cpu", torch.float64)
    outs, states = [], []
    for i in range(B):
        mix = torch.stack([att_r[n].reshape(C) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")])
        sx = torch.cat([state_r[i, :1], x_r[i, :-1]], dim=0)
        sx = torch.where(torch.as_tensor(ns[i])[:, None], torch.zeros_like(sx), sx) - x_r[i]
        xr, xw, xk, xv, xa, xg = (x_r[i] + sx * mix[j] for j in range(6))
        r = xr @ att_r["receptance"]["weight"].T
        wl = torch.tanh(xw @ att_r["w1"]) @ att_r["w2"]
        k = xk @ att_r["key"]["weight"].T
        v = xv @ att_r["value"]["weight"].T
        al = (xa @ att_r["a1"]) @ att_r["a2"]
        gg = torch.sigmoid(xg @ att_r["g1"]) @ att_r["g2"]
        vl = (xv @ att_r["v1"]) @ att_r["v2"]
        w, kp, vp, a_i, b_i = ref_pre(k, wl, al, v, vf_r[i], vl, att_r["w0"], att_r["a0"], att_r["v0"], att_r["k_k"], att_r["k_a"], H)
        sh = (T, H, S)
        s_new, y = torch_ref.wkv7_base_torch(r.reshape(sh), w.reshape(sh), kp.reshape(sh), vp.reshape(sh), a_i.reshape(sh),
                                             b_i.reshape(sh), state_r[i, 1:].reshape(H, S, S), int(length[i]), torch.as_tensor(ns[i]))
        xo = ref_post(y.reshape(T, C), r, kp, vp, gg, att_r["ln_x"]["weight"], att_r["ln_x"]["bias"], att_r["r_k"], H)
        outs.append(xo @ att_r["output"]["weight"].T)
        states.append(torch.cat([x_r[i, int(length[i]) - 1][None], s_new.reshape(S, C)], dim=0))
    loss_r = (torch.stack(outs) * cot).sum() + 0.1 * torch.stack(states).sum()
    want = torch.autograd.grad(loss_r, [x_r, state_r, vf_r] + flat_r, allow_unused=True)
    for i, (a, b) in enumerate(zip(got, want)):
        assert (a is None) == (b is None), i
        if a is not None:
            assert rel_err(a.cpu().numpy(), b.numpy()) < 2e-4, i


def test_mix_kernels_at_benchmark_size_on_row_slices():
    """8 x 4096 tokens, 32 heads, bf16 (every thread walks ~28 rows): forward results and stream gradients on a
    random subset of rows against the plain-torch rendition; parameter gradients, which sum over all rows, against
    the same sums accumulated in fp64 over row blocks."""
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(21)
    B, T, H = 8, 4096, 32
    C = H * 64
    rn = lambda *s: torch.randn(*s, generator=gen, device=dev).to(torch.bfloat16)
    k, wl, al, v, vf, vl, y, r, g = (rn(B, T, C).requires_grad_(True) for _ in range(9))
    w0, a0, v0, k_k, k_a, ln_w, ln_b = (rn(C).requires_grad_(True) for _ in range(7))
    r_k = (0.3 * rn(H, 64)).detach().requires_grad_(True)
    cot = [rn(B, T, C) for _ in range(6)]
    pre = tm.mix_pre(k, wl, al, v, vf, vl, w0, a0, v0, k_k, k_a, H)
    post = tm.mix_post(y, r, pre[1], pre[2], g, ln_w, ln_b, r_k, H)
    leaves = [k, wl, al, v, vf, vl, y, r, g, w0, a0, v0, k_k, k_a, ln_w, ln_b, r_k]
    grads = torch.autograd.grad(list(pre) + [post], leaves, cot)
    rows = torch.randperm(B * T, generator=torch.Generator().manual_seed(3))[:257].to(dev)
    flat = lambda t: t.reshape(B * T, C)
    # streams: the subset of rows only (every op is row-wise)
    sub = [flat(t.detach())[rows].double().cpu().requires_grad_(True) for t in leaves[:9]]
    par = [t.detach().double().cpu().requires_grad_(True) for t in leaves[9:]]
    pre_r = ref_pre(sub[0], sub[1], sub[2], sub[3], sub[4], sub[5], par[0], par[1], par[2], par[3], par[4], H)
    post_r = ref_post(sub[6], sub[7], pre_r[1], pre_r[2], sub[8], par[5], par[6], par[7], H)
    cot_r = [flat(c)[rows].double().cpu() for c in cot]
    grads_r = torch.autograd.grad(list(pre_r) + [post_r], sub, cot_r)
    for i, (got, want) in enumerate(zip(list(pre) + [post], list(pre_r) + [post_r])):
        assert rel_err(flat(got.detach())[rows].float().cpu().numpy(), want.detach().numpy()) < 1.5e-2, ("out", i)
    for i, (got, want) in enumerate(zip(grads[:9], grads_r)):
        assert rel_err(flat(got)[rows].float().cpu().numpy(), want.numpy()) < 3e-2, ("stream grad", i)
    # parameters: fp64 sums over all rows, in blocks
    acc = [torch.zeros(p.shape, dtype=torch.float64) for p in par]
    for lo in range(0, B * T, 4096):
        blk = [flat(t.detach())[lo:lo + 4096].double() for t in leaves[:9]]
        pb = [t.detach().double().requires_grad_(True) for t in leaves[9:]]
        pr = ref_pre(blk[0], blk[1], blk[2], blk[3], blk[4], blk[5], pb[0], pb[1], pb[2], pb[3], pb[4], H)
        po = ref_post(blk[6], blk[7], pr[1], pr[2], blk[8], pb[5], pb[6], pb[7], H)
        gb = torch.autograd.grad(list(pr) + [po], pb, [flat(c)[lo:lo + 4096].double() for c in cot])
        for a_, g_ in zip(acc, gb):
            a_ += g_.cpu()
    for i, (got, want) in enumerate(zip(grads[9:], acc)):
        assert rel_err(got.float().cpu().numpy(), want.numpy()) < 3e-2, ("param grad", i)
