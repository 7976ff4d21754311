"""RWKV-7 time mixing around the WKV operator, batched.

``time_mixing_seq`` mirrors jaxrwkv's ``BaseRWKV.time_mixing_seq`` (src/jaxrwkv/rwkv7.py:222-266) with a
leading batch axis (the reference vmaps the per-sequence function): the token shift (rwkv7.py:226-235,
:254), the projections and LoRAs (matrix products, done by the framework's GEMMs: ``torch.matmul``), the
elementwise stage in front of the operator (:238-252, :257) as ONE kernel, the operator (:259), and the
elementwise stage behind it (:263-265) as ONE kernel.  The two elementwise stages are
``b200wkv7_mix_pre_{fwd,bwd}`` and ``b200wkv7_mix_post_{fwd,bwd}`` of the C ABI; ``mix_pre`` and ``mix_post``
are their differentiable host wrappers.  Arrays are CUDA ``torch`` tensors; there is no CPU path.
"""
import torch

from . import _lib
from .rwkv7 import CudaRWKV
from .token_shift import token_shift

GROUP_NORM_EPS = 64e-5   # rwkv7.py:263


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _rows(x, H, N):
    if not x.is_cuda:
        raise _lib.B200WKVError("time mixing: tensors must live on a CUDA device (there is no CPU path)")
    C = H * N
    assert x.shape[-1] == C, (x.shape, H, N)
    return x.numel() // C


def _same(ref, *ts):
    """Contiguous copies of ``ts`` in ``ref``'s dtype and shape (parameters are flattened to (C,))."""
    return [None if t is None else t.to(ref.dtype).expand(ref.shape).contiguous() for t in ts]


def _params(ref, C, *ps):
    return [None if p is None else p.to(ref.dtype).reshape(C).contiguous() for p in ps]


class _MixPre(torch.autograd.Function):
    @staticmethod
    def forward(k, wl, al, v, v_first, vl, w0, a0, v0, k_k, k_a, H, N):
        lib = _lib.load()
        C = H * N
        rows = _rows(k, H, N)
        use_vmix = v_first is not None
        k, wl, al, v, v_first, vl = _same(k, k, wl, al, v, v_first, vl)
        w0, a0, v0, k_k, k_a = _params(k, C, w0, a0, v0, k_k, k_a)
        w, kp, vp, ai, bi = (torch.empty_like(k) for _ in range(5))
        _lib.check(lib.b200wkv7_mix_pre_fwd(_stream(), _lib.dtype_code(k.dtype), rows, H, N, int(use_vmix), _ptr(k), _ptr(wl),
                                            _ptr(al), _ptr(v), _ptr(v_first), _ptr(vl), _ptr(w0), _ptr(a0), _ptr(v0),
                                            _ptr(k_k), _ptr(k_a), _ptr(w), _ptr(kp), _ptr(vp), _ptr(ai), _ptr(bi)))
        return w, kp, vp, ai, bi

    @staticmethod
    def setup_context(ctx, inputs, output):
        k, wl, al, v, v_first, vl, w0, a0, v0, k_k, k_a, H, N = inputs
        ctx.dims = (H, N)
        ctx.use_vmix = v_first is not None
        ctx.param_shapes = [None if p is None else p.shape for p in (w0, a0, v0, k_k, k_a)]
        ctx.param_dtypes = [None if p is None else p.dtype for p in (w0, a0, v0, k_k, k_a)]
        empty = k.new_empty(0)
        ctx.save_for_backward(*[empty if t is None else t for t in (k, wl, al, v, v_first, vl, w0, a0, v0, k_k, k_a)])

    @staticmethod
    def backward(ctx, gw, gkp, gvp, gai, gbi):
        lib = _lib.load()
        H, N = ctx.dims
        C = H * N
        k, wl, al, v, v_first, vl, w0, a0, v0, k_k, k_a = ctx.saved_tensors
        if not ctx.use_vmix:
            v_first = vl = v0 = None
        rows = _rows(k, H, N)
        k_c, wl, al, v, v_first, vl = _same(k, k, wl, al, v, v_first, vl)
        w0, a0, v0, k_k, k_a = _params(k_c, C, w0, a0, v0, k_k, k_a)
        gw, gkp, gvp, gai, gbi = _same(k_c, *[torch.zeros_like(k_c) if g is None else g for g in (gw, gkp, gvp, gai, gbi)])
        dk, dwl, dal, dv = (torch.empty_like(k_c) for _ in range(4))
        dvf = torch.empty_like(k_c) if ctx.use_vmix else None
        dvl = torch.empty_like(k_c) if ctx.use_vmix else None
        n_part = lib.b200wkv7_mix_partial_rows(rows, H, N)
        partial = torch.empty((n_part, 5, C), dtype=torch.float32, device=k.device)
        _lib.check(lib.b200wkv7_mix_pre_bwd(_stream(), _lib.dtype_code(k_c.dtype), rows, H, N, int(ctx.use_vmix), _ptr(k_c),
                                            _ptr(wl), _ptr(al), _ptr(v), _ptr(v_first), _ptr(vl), _ptr(w0), _ptr(a0), _ptr(v0),
                                            _ptr(k_k), _ptr(k_a), _ptr(gw), _ptr(gkp), _ptr(gvp), _ptr(gai), _ptr(gbi),
                                            _ptr(dk), _ptr(dwl), _ptr(dal), _ptr(dv), _ptr(dvf), _ptr(dvl), _ptr(partial)))
        sums = partial.sum(dim=0)
        pg = [None if shp is None else sums[i].to(dt).reshape(shp)
              for i, (shp, dt) in enumerate(zip(ctx.param_shapes, ctx.param_dtypes))]
        return dk, dwl, dal, dv, dvf, dvl, pg[0], pg[1], pg[2], pg[3], pg[4], None, None


class _MixPost(torch.autograd.Function):
    @staticmethod
    def forward(y, r, k, v, g, ln_w, ln_b, r_k, H, N, eps):
        lib = _lib.load()
        C = H * N
        rows = _rows(y, H, N)
        y, r, k, v, g = _same(y, y, r, k, v, g)
        ln_w, ln_b, r_k = _params(y, C, ln_w, ln_b, r_k)
        x = torch.empty_like(y)
        _lib.check(lib.b200wkv7_mix_post_fwd(_stream(), _lib.dtype_code(y.dtype), rows, H, N, float(eps), _ptr(y), _ptr(r),
                                             _ptr(k), _ptr(v), _ptr(g), _ptr(ln_w), _ptr(ln_b), _ptr(r_k), _ptr(x)))
        return x

    @staticmethod
    def setup_context(ctx, inputs, output):
        y, r, k, v, g, ln_w, ln_b, r_k, H, N, eps = inputs
        ctx.dims = (H, N, eps)
        ctx.param_shapes = [p.shape for p in (ln_w, ln_b, r_k)]
        ctx.param_dtypes = [p.dtype for p in (ln_w, ln_b, r_k)]
        ctx.save_for_backward(y, r, k, v, g, ln_w, ln_b, r_k)

    @staticmethod
    def backward(ctx, gx):
        lib = _lib.load()
        H, N, eps = ctx.dims
        C = H * N
        y, r, k, v, g, ln_w, ln_b, r_k = ctx.saved_tensors
        rows = _rows(y, H, N)
        y, r, k, v, g, gx = _same(y, y, r, k, v, g, gx)
        ln_w, ln_b, r_k = _params(y, C, ln_w, ln_b, r_k)
        dy, dr, dk, dv, dg = (torch.empty_like(y) for _ in range(5))
        n_part = lib.b200wkv7_mix_partial_rows(rows, H, N)
        partial = torch.empty((n_part, 3, C), dtype=torch.float32, device=y.device)
        _lib.check(lib.b200wkv7_mix_post_bwd(_stream(), _lib.dtype_code(y.dtype), rows, H, N, float(eps), _ptr(y), _ptr(r),
                                             _ptr(k), _ptr(v), _ptr(g), _ptr(ln_w), _ptr(ln_b), _ptr(r_k), _ptr(gx), _ptr(dy),
                                             _ptr(dr), _ptr(dk), _ptr(dv), _ptr(dg), _ptr(partial)))
        sums = partial.sum(dim=0)
        pg = [sums[i].to(dt).reshape(shp) for i, (shp, dt) in enumerate(zip(ctx.param_shapes, ctx.param_dtypes))]
        return dy, dr, dk, dv, dg, pg[0], pg[1], pg[2], None, None, None


def mix_pre(k, wl, al, v, v_first, vl, w0, a0, v0, k_k, k_a, H, N=64):
    """Streams ``(..., H*N)``; parameters with ``H*N`` elements.  Returns ``(w, k', v', a_i, b_i)`` as the
    operator takes them (rwkv7.py:238, :243, :245, :248-252, :257).  ``v_first=None`` (with ``vl``, ``v0``) is
    the first layer, whose value stream passes through unchanged."""
    return _MixPre.apply(k, wl, al, v, v_first, vl, w0, a0, v0, k_k, k_a, H, N)


def mix_post(y, r, k, v, g, ln_w, ln_b, r_k, H, N=64, eps=GROUP_NORM_EPS):
    """``(group_norm(y) * ln_w + ln_b + (sum_n r k r_k) v) * g`` per token and head (rwkv7.py:263-265);
    ``k`` and ``v`` are the operator's operands (``k'``, ``v'`` of :func:`mix_pre`)."""
    return _MixPost.apply(y, r, k, v, g, ln_w, ln_b, r_k, H, N, eps)


def time_mixing_seq(x, state, v_first, att, length, new_starts, H, S, layer_id):
    """Batched ``BaseRWKV.time_mixing_seq`` (rwkv7.py:222-266).

    ``x`` (B, T, C); ``state`` (B, 1 + S, C): row 0 the token-shift row, rows 1.. the (H, S, S) WKV state
    (rwkv7.py:254-255); ``v_first`` (B, T, C); ``att`` the layer's parameter dict with the reference's keys;
    ``length`` (B,), ``new_starts`` (B, T).  Returns ``(out (B, T, C), new_state, v_first)``.
    """
    B, T, C = x.shape
    mix = torch.stack([att[n].reshape(C) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")]).to(x.dtype)
    mixed, shift_row = token_shift(x, state[:, 0], mix, length, new_starts)
    xr, xw, xk, xv, xa, xg = mixed.unbind(0)

    r = xr @ att["receptance"]["weight"].T
    wl = torch.tanh(xw @ att["w1"]) @ att["w2"]
    k = xk @ att["key"]["weight"].T
    v = xv @ att["value"]["weight"].T
    al = (xa @ att["a1"]) @ att["a2"]
    g = torch.sigmoid(xg @ att["g1"]) @ att["g2"]
    if layer_id == 0:
        v_first = v
        w, kp, vp, a_i, b_i = mix_pre(k, wl, al, v, None, None, att["w0"], att["a0"], None, att["k_k"], att["k_a"], H, S)
    else:
        vl = (xv @ att["v1"]) @ att["v2"]
        w, kp, vp, a_i, b_i = mix_pre(k, wl, al, v, v_first, vl, att["w0"], att["a0"], att["v0"], att["k_k"], att["k_a"], H, S)

    s = state[:, 1:].reshape(B, H, S, S)
    shape = (B, T, H, S)
    s_new, out = CudaRWKV.inner_loop(r.reshape(shape), w.reshape(shape), kp.reshape(shape), vp.reshape(shape),
                                     a_i.reshape(shape), b_i.reshape(shape), s, length, new_starts)
    new_state = torch.cat([shift_row[:, None], s_new.reshape(B, S, C)], dim=1)

    xo = mix_post(out.reshape(B, T, C), r, kp, vp, g, att["ln_x"]["weight"], att["ln_x"]["bias"], att["r_k"], H, S)
    return xo @ att["output"]["weight"].T, new_state, v_first
