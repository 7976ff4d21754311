"""Host side of the RWKV-5 / 5.2 / 6 WKV operator (shared by rwkv5.py, rwkv5_2.py, rwkv6.py).

jaxrwkv has no CudaRWKV class for these versions; this adds one behind the same seam, with the
argument shapes the reference's ``inner_loop`` receives (src/jaxrwkv/rwkv6.py:174-191,
rwkv5_2.py:164-180, rwkv5.py:161-177): r, k, v (..., T, H, N); the state (..., H, N, N) indexed
[key, value]; ``w`` (..., T, H, N, 1) log-decay for version 6, (H, N, 1) / (H, 1, 1) constant
decay for 5.2 / 5; ``time_first`` (H, N, 1) or (H, 1, 1).  The shared operands (time_first, the
constant decay) are never batched, as under ``jax.vmap(..., in_axes=None)``.
"""
import torch

from . import _lib
from .rwkv7 import _ptr, _stream, _flatten_lead, _bcast_flags, _vmap_front


def _expand_hn(x, H, N, dtype):
    return x.reshape(x.shape[0], -1).expand(H, N).to(dtype).contiguous()


def batched_wkv6_fwd(version, r, k, v, w, u, s, length, new_starts, B, need_residual=True):
    """One ``b200wkv6_fwd`` call on (B,T,H,N) tensors; ``w`` is (B,T,H,N) for version 6, (H,N) else;
    ``u`` is (H,N).  Returns ((new_s, out), residuals)."""
    lib = _lib.load()
    dtype = k.dtype
    if not all(x.dtype == dtype for x in (r, k, v, w, u, s)):
        raise _lib.B200WKVError("wkv6: r, k, v, w, time_first and s must share one element type")
    if not all(x.is_cuda for x in (r, k, v, w, u, s)):
        raise _lib.B200WKVError("wkv6: tensors must live on a CUDA device (there is no CPU path)")
    code = _lib.dtype_code(dtype)
    _, T, H, N = k.shape
    r, k, v, w, u, s = (x.contiguous() for x in (r, k, v, w, u, s))
    length = length.to(device=k.device, dtype=torch.int32).contiguous()
    new_starts = new_starts.to(device=k.device, dtype=torch.uint8).contiguous()
    out, new_s = torch.empty_like(k), torch.empty_like(s)
    residual, rbytes = None, 0
    if need_residual:
        rbytes = lib.b200wkv6_residual_bytes(code, B, T, H, N)
        residual = torch.empty(rbytes, dtype=torch.uint8, device=k.device)
    _lib.check(lib.b200wkv6_fwd(_stream(), code, 6 if version == "6" else 5, B, T, H, N, _ptr(r), _ptr(k), _ptr(v),
                                _ptr(w), _ptr(u), _ptr(s), _ptr(length), _ptr(new_starts), _ptr(out), _ptr(new_s),
                                _ptr(residual), rbytes, 0))
    return (new_s, out), (r, k, v, w, u, s, length, new_starts, residual)


def batched_wkv6_bwd(version, res, grads, B):
    """One ``b200wkv6_bwd`` call.  Returns (gr, gk, gv, gw, gu, gs); gw is (B,T,H,N) for version 6,
    else (H,N) summed over the batch; gu is (H,N) summed over the batch (fp32)."""
    lib = _lib.load()
    r, k, v, w, u, s, length, new_starts, residual = res
    gs_out, gy = grads
    # dense C-order buffers for the kernel (see batched_wkv7_bwd): views and broadcasts are materialised
    r, k, v, w, u, s = (x.contiguous() for x in (r, k, v, w, u, s))
    length = length.to(device=k.device, dtype=torch.int32).contiguous()
    new_starts = new_starts.to(device=k.device, dtype=torch.uint8).contiguous()
    code = _lib.dtype_code(k.dtype)
    _, T, H, N = k.shape
    assert length.shape == (B,) and new_starts.shape == (B, T)
    gy = None if gy is None else gy.to(k.dtype).contiguous()
    gs_out = None if gs_out is None else gs_out.to(k.dtype).contiguous()
    gr, gk, gv = (torch.empty_like(k) for _ in range(3))
    gs = torch.empty_like(s)
    gw = torch.empty_like(k) if version == "6" else torch.empty(B, H, N, dtype=torch.float32, device=k.device)
    gu = torch.empty(B, H, N, dtype=torch.float32, device=k.device)
    _lib.check(lib.b200wkv6_bwd(_stream(), code, 6 if version == "6" else 5, B, T, H, N, _ptr(r), _ptr(k), _ptr(v),
                                _ptr(w), _ptr(u), _ptr(s), _ptr(length), _ptr(new_starts), _ptr(gy), _ptr(gs_out),
                                _ptr(residual), residual.numel(), _ptr(gr), _ptr(gk), _ptr(gv), _ptr(gw), _ptr(gu),
                                _ptr(gs), 0))
    if version != "6":
        gw = gw.sum(0)
    return gr, gk, gv, gw, gu.sum(0), gs


def _make_functions(version):
    per_token = version == "6"

    class Bwd(torch.autograd.Function):
        @staticmethod
        def forward(r, k, v, w, u, s, length, new_starts, residual, gs_out, gy):
            lead, B = _flatten_lead(k)
            T, H, N = k.shape[-3:]
            fr, fk, fv = (x.reshape(B, T, H, N) for x in (r, k, v))
            fw = w.reshape(B, T, H, N) if per_token else _expand_hn(w, H, N, k.dtype)
            fu = _expand_hn(u, H, N, k.dtype)
            length, new_starts = _bcast_flags(length, new_starts, lead, B, T, k.device)
            res = (fr, fk, fv, fw, fu, s.reshape(B, H, N, N), length.to(torch.int32), new_starts.to(torch.uint8), residual)
            gs_out = None if gs_out is None else gs_out.reshape(B, H, N, N)
            gy = None if gy is None else gy.reshape(B, T, H, N)
            gr, gk, gv, gw, gu, gs = batched_wkv6_bwd(version, res, (gs_out, gy), B)
            shp = lead + (T, H, N)
            gw = gw.reshape(w.shape) if per_token else gw.reshape(H, N, 1).sum(1, keepdim=True).reshape(w.shape) if w.shape[1] == 1 else gw.reshape(w.shape)
            gu = gu.reshape(H, N, 1)
            if u.shape[1] == 1:
                gu = gu.sum(1, keepdim=True)
            return (gr.reshape(shp), gk.reshape(shp), gv.reshape(shp), gw.to(w.dtype), gu.to(u.dtype),
                    gs.reshape(lead + (H, N, N)))

        @staticmethod
        def setup_context(ctx, inputs, output):
            pass

        @staticmethod
        def backward(ctx, *g):
            raise _lib.B200WKVError("wkv6: second-order differentiation is not supported")

        @staticmethod
        def vmap(info, in_dims, r, k, v, w, u, s, length, new_starts, residual, gs_out, gy):
            n = info.batch_size
            if in_dims[4] is not None or (not per_token and in_dims[3] is not None):
                raise _lib.B200WKVError("wkv6 under vmap: time_first (and a constant decay) cannot be batched")
            r, k, v = _vmap_front(n, (r, k, v), in_dims[:3], (True,) * 3)
            if per_token:
                w, = _vmap_front(n, (w,), in_dims[3:4], (True,))
            s, length, new_starts = _vmap_front(n, (s, length, new_starts), in_dims[5:8], (True, False, False))
            gs_out, gy = _vmap_front(n, (gs_out, gy), in_dims[9:], (False, False))
            outs = Bwd.apply(r, k, v, w, u, s, length, new_starts, residual, gs_out, gy)
            # gradients of the shared operands are already summed over the batch
            return outs, (0, 0, 0, 0 if per_token else None, None, 0)

    class Fwd(torch.autograd.Function):
        @staticmethod
        def forward(r, k, v, w, u, s, length, new_starts):
            lead, B = _flatten_lead(k)
            T, H, N = k.shape[-3:]
            fr, fk, fv = (x.reshape(B, T, H, N) for x in (r, k, v))
            fw = w.reshape(B, T, H, N) if per_token else _expand_hn(w, H, N, k.dtype)
            fu = _expand_hn(u, H, N, k.dtype)
            length, new_starts = _bcast_flags(length, new_starts, lead, B, T, k.device)
            (new_s, out), res = batched_wkv6_fwd(version, fr, fk, fv, fw, fu, s.reshape(B, H, N, N), length, new_starts, B)
            return new_s.reshape(lead + (H, N, N)), out.reshape(lead + (T, H, N)), res[-1]

        @staticmethod
        def setup_context(ctx, inputs, output):
            r, k, v, w, u, s, length, new_starts = inputs
            ctx.save_for_backward(r, k, v, w, u, s, torch.as_tensor(length), torch.as_tensor(new_starts), output[2])
            ctx.set_materialize_grads(False)
            ctx.mark_non_differentiable(output[2])

        @staticmethod
        def backward(ctx, gs_out, gy, _gres):
            r, k, v, w, u, s, length, new_starts, residual = ctx.saved_tensors
            gr, gk, gv, gw, gu, gs = Bwd.apply(r, k, v, w, u, s, length, new_starts, residual, gs_out, gy)
            return gr, gk, gv, gw, gu, gs, None, None

        @staticmethod
        def vmap(info, in_dims, r, k, v, w, u, s, length, new_starts):
            n = info.batch_size
            if in_dims[4] is not None or (not per_token and in_dims[3] is not None):
                raise _lib.B200WKVError("wkv6 under vmap: time_first (and a constant decay) cannot be batched")
            r, k, v = _vmap_front(n, (r, k, v), in_dims[:3], (True,) * 3)
            if per_token:
                w, = _vmap_front(n, (w,), in_dims[3:4], (True,))
            s, length, new_starts = _vmap_front(n, (s, length, new_starts), in_dims[5:8], (True, False, False))
            new_s, out, residual = Fwd.apply(r, k, v, w, u, s, length, new_starts)
            return (new_s, out, residual), (0, 0, None)

    return Fwd, Bwd


_FUNCS = {ver: _make_functions(ver) for ver in ("6", "5_2", "5")}


def wkv_cuda(version, r, k, v, w, time_first, s, length, new_starts):
    """Differentiable operator; returns (s_out, out)."""
    new_s, out, _ = _FUNCS[version][0].apply(r, k, v, w, time_first, s, length, new_starts)
    return new_s, out


def make_class(version):
    class CudaRWKV:
        """The ``rwkv_type="CudaRWKV"`` operator seam for this RWKV version."""
        VERSION = version

        @classmethod
        def get_kernels(cls):
            return _lib.load()

        @classmethod
        def inner_loop(cls, r, k, v, w, time_first, s, length, new_starts):
            cls.get_kernels()
            return wkv_cuda(version, r, k, v, w, time_first, s, length, new_starts)
    return CudaRWKV
