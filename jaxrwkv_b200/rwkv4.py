"""RWKV-4 WKV operator on B200: host side of jaxrwkv's ``CudaRWKV`` seam for version 4.

Mirrors src/jaxrwkv/rwkv4.py:311-406: ``batched_wkv4_fwd`` / ``batched_wkv4_bwd`` issue the two
custom calls, ``wkv4_cuda(k, v, w, time_first, s, length, new_starts)`` is the differentiable
operator (``w`` is the raw decay parameter; ``-exp(w)`` is applied here, rwkv4.py:312), and
``CudaRWKV.inner_loop(r, k, v, w, time_first, s, length, new_starts)`` returns ``(s_out, r * out)``
(rwkv4.py:403-406).  k, v, r are (..., T, C); w, time_first (C,); the state (..., 3, C).
"""
import torch

from . import _lib
from .rwkv7 import _ptr, _stream, _vmap_front


def batched_wkv4_fwd(k, v, w_neg, time_first, s, length, new_starts, B, need_residual=True):
    lib = _lib.load()
    dtype = k.dtype
    if not all(x.dtype == dtype for x in (k, v, w_neg, time_first, s)):
        raise _lib.B200WKVError("wkv4: k, v, w, time_first and s must share one element type")
    if not all(x.is_cuda for x in (k, v, w_neg, time_first, s)):
        raise _lib.B200WKVError("wkv4: tensors must live on a CUDA device (there is no CPU path)")
    code = _lib.dtype_code(dtype)
    _, T, C = k.shape
    k, v, w_neg, time_first, s = (x.contiguous() for x in (k, v, w_neg, time_first, s))
    length = length.to(device=k.device, dtype=torch.int32).contiguous()
    new_starts = new_starts.to(device=k.device, dtype=torch.uint8).contiguous()
    out, new_s = torch.empty_like(k), torch.empty_like(s)
    residual, rbytes = None, 0
    if need_residual:
        rbytes = lib.b200wkv4_residual_bytes(code, B, T, C)
        residual = torch.empty(rbytes, dtype=torch.uint8, device=k.device)
    _lib.check(lib.b200wkv4_fwd(_stream(), code, B, T, C, _ptr(w_neg), _ptr(time_first), _ptr(k), _ptr(v), _ptr(s),
                                _ptr(length), _ptr(new_starts), _ptr(new_s), _ptr(out), _ptr(residual), rbytes, 0))
    return (new_s, out), (k, v, w_neg, time_first, s, length, new_starts, residual)


def batched_wkv4_bwd(res, grads, B):
    """Returns (gk, gv, gw_neg, gu, gs) with gw_neg, gu summed over the batch (rwkv4.py:351)."""
    lib = _lib.load()
    k, v, w_neg, u, s, length, new_starts, residual = res
    gs_new, gy = grads
    # dense C-order buffers for the kernel (see batched_wkv7_bwd): views and broadcasts are materialised
    k, v, w_neg, u, s = (x.contiguous() for x in (k, v, w_neg, u, s))
    length = length.to(device=k.device, dtype=torch.int32).contiguous()
    new_starts = new_starts.to(device=k.device, dtype=torch.uint8).contiguous()
    code = _lib.dtype_code(k.dtype)
    _, T, C = k.shape
    assert length.shape == (B,) and new_starts.shape == (B, T)
    gy = None if gy is None else gy.to(k.dtype).contiguous()
    gs_new = None if gs_new is None else gs_new.to(k.dtype).contiguous()
    gk, gv, gs = torch.empty_like(k), torch.empty_like(v), torch.empty_like(s)
    gw = torch.empty(B, C, dtype=torch.float32, device=k.device)
    gu = torch.empty(B, C, dtype=torch.float32, device=k.device)
    _lib.check(lib.b200wkv4_bwd(_stream(), code, B, T, C, _ptr(w_neg), _ptr(u), _ptr(k), _ptr(v), _ptr(gy), _ptr(s),
                                _ptr(length), _ptr(new_starts), _ptr(gs_new), _ptr(residual), residual.numel(),
                                _ptr(gw), _ptr(gu), _ptr(gk), _ptr(gv), _ptr(gs), 0))
    return gk, gv, gw.sum(0), gu.sum(0), gs


def _lead(k):
    lead = tuple(k.shape[:-2])
    B = 1
    for d in lead:
        B *= d
    return lead, B


class _WKV4Bwd(torch.autograd.Function):
    @staticmethod
    def forward(k, v, w, u, s, length, new_starts, residual, gs_new, gy):
        lead, B = _lead(k)
        T, C = k.shape[-2:]
        length = torch.as_tensor(length, device=k.device).expand(lead).reshape(B)
        new_starts = torch.as_tensor(new_starts, device=k.device).expand(lead + (T,)).reshape(B, T)
        w_neg = -torch.exp(w.float()).to(k.dtype)
        res = (k.reshape(B, T, C), v.reshape(B, T, C), w_neg, u, s.reshape(B, 3, C), length.to(torch.int32),
               new_starts.to(torch.uint8), residual)
        gs_new = None if gs_new is None else gs_new.reshape(B, 3, C)
        gy = None if gy is None else gy.reshape(B, T, C)
        gk, gv, gwn, gu, gs = batched_wkv4_bwd(res, (gs_new, gy), B)
        gw = (gwn * w_neg.float()).to(w.dtype)          # d(-exp(w))/dw = -exp(w)
        return gk.reshape(lead + (T, C)), gv.reshape(lead + (T, C)), gw, gu.to(u.dtype), gs.reshape(lead + (3, C))

    @staticmethod
    def setup_context(ctx, inputs, output):
        pass

    @staticmethod
    def backward(ctx, *g):
        raise _lib.B200WKVError("wkv4: second-order differentiation is not supported")

    @staticmethod
    def vmap(info, in_dims, k, v, w, u, s, length, new_starts, residual, gs_new, gy):
        n = info.batch_size
        if in_dims[2] is not None or in_dims[3] is not None:
            raise _lib.B200WKVError("wkv4 under vmap: w and time_first cannot be batched")     # rwkv4.py:362-363
        k, v = _vmap_front(n, (k, v), in_dims[:2], (False, False))
        s, length, new_starts = _vmap_front(n, (s, length, new_starts), in_dims[4:7], (False, False, False))
        gs_new, gy = _vmap_front(n, (gs_new, gy), in_dims[8:], (False, False))
        outs = _WKV4Bwd.apply(k, v, w, u, s, length, new_starts, residual, gs_new, gy)
        return outs, (0, 0, None, None, 0)


class _WKV4(torch.autograd.Function):
    """custom_vjp + custom_vmap of the reference (rwkv4.py:353-382) in torch terms."""

    @staticmethod
    def forward(k, v, w, u, s, length, new_starts):
        lead, B = _lead(k)
        T, C = k.shape[-2:]
        length = torch.as_tensor(length, device=k.device).expand(lead).reshape(B)
        new_starts = torch.as_tensor(new_starts, device=k.device).expand(lead + (T,)).reshape(B, T)
        w_neg = -torch.exp(w.float()).to(k.dtype)                                          # rwkv4.py:312
        (new_s, out), res = batched_wkv4_fwd(k.reshape(B, T, C), v.reshape(B, T, C), w_neg, u, s.reshape(B, 3, C),
                                             length, new_starts, B)
        return new_s.reshape(lead + (3, C)), out.reshape(lead + (T, C)), res[-1]

    @staticmethod
    def setup_context(ctx, inputs, output):
        k, v, w, u, s, length, new_starts = inputs
        ctx.save_for_backward(k, v, w, u, s, torch.as_tensor(length), torch.as_tensor(new_starts), output[2])
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(output[2])

    @staticmethod
    def backward(ctx, gs_new, gy, _gres):
        k, v, w, u, s, length, new_starts, residual = ctx.saved_tensors
        gk, gv, gw, gu, gs = _WKV4Bwd.apply(k, v, w, u, s, length, new_starts, residual, gs_new, gy)
        return gk, gv, gw, gu, gs, None, None

    @staticmethod
    def vmap(info, in_dims, k, v, w, u, s, length, new_starts):
        n = info.batch_size
        if in_dims[2] is not None or in_dims[3] is not None:
            raise _lib.B200WKVError("wkv4 under vmap: w and time_first cannot be batched")
        k, v = _vmap_front(n, (k, v), in_dims[:2], (False, False))
        s, length, new_starts = _vmap_front(n, (s, length, new_starts), in_dims[4:7], (False, False, False))
        new_s, out, residual = _WKV4.apply(k, v, w, u, s, length, new_starts)
        return (new_s, out, residual), (0, 0, None)


def wkv4_cuda(k, v, w, time_first, s, length, new_starts):
    new_s, out, _ = _WKV4.apply(k, v, w, time_first, s, length, new_starts)
    return new_s, out


class CudaRWKV:
    """The ``rwkv_type="CudaRWKV"`` operator seam (rwkv4.py:385-406)."""

    @classmethod
    def get_kernels(cls):
        return _lib.load()

    @classmethod
    def inner_loop(cls, r, k, v, w, time_first, s, length, new_starts):
        cls.get_kernels()
        s, out = wkv4_cuda(k, v, w, time_first, s, length, new_starts)
        return s, r * out
