"""GPU parity of the fused token shift against the NumPy restatement and a torch autograd reference."""
import numpy as np
import pytest
import torch

from oracle import token_shift as oracle_shift
from conftest import rel_err

pytestmark = pytest.mark.gpu


def _inputs(B, T, D, M, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, D, generator=g)
    prev = torch.randn(B, D, generator=g)
    mix = torch.rand(M, D, generator=g)
    length = torch.randint(0, T + 1, (B,), generator=g)
    length[0] = T
    ns = torch.rand(B, T, generator=g) < 0.05
    ns[-1, 0] = True
    return [t.to(dtype) for t in (x, prev, mix)] + [length, ns]


def _torch_ref(x, prev, mix, length, ns):
    B, T, D = x.shape
    sx = torch.cat([prev[:, None], x[:, :-1]], dim=1)
    sx = torch.where(ns[:, :, None], torch.zeros_like(sx), sx) - x
    out = x[None] + sx[None] * mix[:, None, None, :]
    idx = (length - 1) % T
    return out, x[torch.arange(B), idx]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("B,T,D,M", [(3, 37, 64, 6), (2, 300, 128, 1), (1, 1, 256, 6), (2, 513, 2048, 6)])
def test_token_shift_forward_matches_oracle(B, T, D, M, dtype, tol):
    from jaxrwkv_b200.token_shift import token_shift
    x, prev, mix, length, ns = _inputs(B, T, D, M, dtype, 5)
    out, st = token_shift(x.cuda(), prev.cuda(), mix.cuda(), length.cuda(), ns.cuda())
    for bi in range(B):
        ref, rst = oracle_shift.token_shift(x[bi].float().numpy(), prev[bi].float().numpy(), mix.float().numpy(),
                                            int(length[bi]), ns[bi].numpy())
        assert rel_err(out[:, bi].float().cpu().numpy(), ref) <= tol
        np.testing.assert_array_equal(st[bi].float().cpu().numpy(), rst)      # a copied row: exact


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("B,T,D,M", [(3, 37, 64, 6), (2, 300, 128, 1), (1, 1, 256, 6)])
def test_token_shift_backward_matches_autograd(B, T, D, M, dtype, tol):
    from jaxrwkv_b200.token_shift import token_shift
    x, prev, mix, length, ns = _inputs(B, T, D, M, dtype, 9)
    g = torch.Generator().manual_seed(1)
    gout = torch.randn(M, B, T, D, generator=g).to(dtype)
    gst = torch.randn(B, D, generator=g).to(dtype)
    xr, pr, mr = (t.float().clone().requires_grad_(True) for t in (x, prev, mix))
    ro, rs = _torch_ref(xr, pr, mr, length, ns)
    ((ro * gout.float()).sum() + (rs * gst.float()).sum()).backward()
    xc, pc, mc = (t.cuda().requires_grad_(True) for t in (x, prev, mix))
    o, s = token_shift(xc, pc, mc, length.cuda(), ns.cuda())
    ((o.float() * gout.cuda().float()).sum() + (s.float() * gst.cuda().float()).sum()).backward()
    assert rel_err(xc.grad.float().cpu().numpy(), xr.grad.numpy()) <= tol
    assert rel_err(pc.grad.float().cpu().numpy(), pr.grad.numpy()) <= tol
    assert rel_err(mc.grad.float().cpu().numpy(), mr.grad.numpy()) <= tol


def test_token_shift_rejects_bad_shapes():
    from jaxrwkv_b200 import _lib
    lib = _lib.load()
    assert lib.b200wkv_token_shift_fwd(None, 0, 1, 1, 6, 1, None, None, None, None, None, None, None) == -2   # D % 4
    assert lib.b200wkv_token_shift_fwd(None, 0, 1, 1, 8, 9, None, None, None, None, None, None, None) == -2   # M > 8
    assert lib.b200wkv_token_shift_fwd(None, 0, 1, 1, 8, 1, None, None, None, None, None, None, None) == -3   # NULL


def test_token_shift_matches_reference_fixture(golden):
    from jaxrwkv_b200.token_shift import token_shift
    g = golden("v7_token_shift")
    x, prev, mix = (torch.from_numpy(g["in_" + n]).cuda() for n in ("x", "prev", "mix"))
    out, st = token_shift(x, prev, mix, torch.from_numpy(g["in_length"].astype(np.int64)).cuda(),
                          torch.from_numpy(g["in_new_starts"]).cuda())
    assert rel_err(out[0].cpu().numpy(), g["xk"]) <= 1e-6
    np.testing.assert_array_equal(st.cpu().numpy().astype(np.float64), g["last"])
