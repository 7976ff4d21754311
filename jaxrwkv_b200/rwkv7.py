"""RWKV-7 WKV operator on B200: host side of jaxrwkv's ``CudaRWKV`` seam.

Mirrors the names and argument meaning of the FFI glue in jaxrwkv
(src/jaxrwkv/rwkv7.py:356-473): ``batched_wkv7_fwd`` / ``batched_wkv7_bwd`` issue
the two custom calls, ``wkv7_cuda`` is the differentiable operator, and
``CudaRWKV.inner_loop(r, w, k, v, a, b, s, length, new_starts) -> (s_out, out)``
is the seam the model code calls (rwkv7.py:259).  Arrays are CUDA ``torch``
tensors (JAX is not part of this build; torch only provides device memory,
streams and the autograd/vmap hooks that ``jax.custom_vjp`` /
``jax.custom_batching.custom_vmap`` provide in the reference).

Differences from the reference kernels, all in the direction of the reference's
own Base/Scan semantics: gradients flow from the returned state and into the
input state, start flags in the middle of a sequence are exact in forward and
backward, T need not be a multiple of 16, and T == 1 runs on the GPU kernel too.
"""
import torch

from . import _lib


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _check_inputs(r, w, k, v, a, b, s):
    dtype = k.dtype
    if not all(x.dtype == dtype for x in (r, w, k, v, a, b, s)):          # rwkv7.py:361
        raise _lib.B200WKVError("wkv7: r, w, k, v, a, b and s must share one element type")
    if not all(x.is_cuda for x in (r, w, k, v, a, b, s)):
        raise _lib.B200WKVError("wkv7: tensors must live on a CUDA device (there is no CPU path)")
    if not all(x.shape == k.shape for x in (r, w, v, a, b)):
        raise _lib.B200WKVError("wkv7: r, w, k, v, a, b must have identical shapes")
    return _lib.dtype_code(dtype)


def batched_wkv7_fwd(r, w, k, v, a, b, s, length, new_starts, B, need_residual=True, flags=0, buffers=None):
    """One ``wkv7-fwd`` call on (B,T,H,N) tensors (rwkv7.py:356-376).

    Returns ``((new_s, out), residuals)``; ``residuals`` carries the inputs and the
    opaque buffer the backward kernel needs (None when ``need_residual`` is False).
    ``buffers`` may hold preallocated results ``out``, ``new_s`` and ``residual`` (the way XLA hands a
    custom call its result buffers); what is missing is allocated here.
    """
    lib = _lib.load()
    code = _check_inputs(r, w, k, v, a, b, s)
    Bk, T, H, N = k.shape
    assert Bk == B and s.shape == (B, H, N, N), (k.shape, s.shape, B)
    r, w, k, v, a, b, s = (x.contiguous() for x in (r, w, k, v, a, b, s))
    length = length.to(device=k.device, dtype=torch.int32).contiguous()      # uint32 bit pattern
    new_starts = new_starts.to(device=k.device, dtype=torch.uint8).contiguous()
    assert length.shape == (B,) and new_starts.shape == (B, T)
    buffers = buffers or {}
    out = buffers.get("out")
    new_s = buffers.get("new_s")
    out = torch.empty_like(k) if out is None else out
    new_s = torch.empty_like(s) if new_s is None else new_s
    residual, rbytes = None, 0
    if need_residual:
        rbytes = lib.b200wkv7_residual_bytes(code, B, T, H, N)
        residual = buffers.get("residual")
        if residual is None:
            residual = torch.empty(rbytes, dtype=torch.uint8, device=k.device)
        elif residual.numel() * residual.element_size() < rbytes or not residual.is_contiguous():
            raise _lib.B200WKVError("wkv7: the preallocated residual is too small")
    _lib.check(lib.b200wkv7_fwd(_stream(), code, B, T, H, N, _ptr(w), _ptr(r), _ptr(k), _ptr(v), _ptr(a), _ptr(b),
                                _ptr(s), _ptr(length), _ptr(new_starts), _ptr(out), _ptr(new_s),
                                _ptr(residual), rbytes, flags))
    return (new_s, out), (r, w, k, v, a, b, s, length, new_starts, residual)


def batched_wkv7_bwd(res, grads, B, flags=0, buffers=None):
    """One ``wkv7-bwd`` call (rwkv7.py:378-411).  ``grads`` is ``(gs_out, gy)``; either may be
    None.  Returns ``(gr, gw, gk, gv, ga, gb, gs)`` in the operator's argument order.  ``buffers`` may
    hold preallocated results under those seven names."""
    lib = _lib.load()
    r, w, k, v, a, b, s, length, new_starts, residual = res
    gs_out, gy = grads
    # the kernels read dense C-order buffers: a vmapped axis moved to the front, a permuted view or a
    # broadcast (stride-0) length / new_starts must be materialised exactly as the forward does
    r, w, k, v, a, b, s = (x.contiguous() for x in (r, w, k, v, a, b, s))
    length = length.to(device=k.device, dtype=torch.int32).contiguous()
    new_starts = new_starts.to(device=k.device, dtype=torch.uint8).contiguous()
    code = _lib.dtype_code(k.dtype)
    _, T, H, N = k.shape
    assert length.shape == (B,) and new_starts.shape == (B, T)
    gy = None if gy is None else gy.to(k.dtype).contiguous()
    gs_out = None if gs_out is None else gs_out.to(k.dtype).contiguous()
    buffers = buffers or {}
    gw, gr, gk, gv, ga, gb = (buffers[n] if n in buffers else torch.empty_like(k) for n in ("gw", "gr", "gk", "gv", "ga", "gb"))
    gs = buffers["gs"] if "gs" in buffers else torch.empty_like(s)
    _lib.check(lib.b200wkv7_bwd(_stream(), code, B, T, H, N, _ptr(w), _ptr(r), _ptr(k), _ptr(v), _ptr(a), _ptr(b),
                                _ptr(s), _ptr(length), _ptr(new_starts), _ptr(gy), _ptr(gs_out),
                                _ptr(residual), residual.numel() * residual.element_size(), _ptr(gw), _ptr(gr), _ptr(gk), _ptr(gv),
                                _ptr(ga), _ptr(gb), _ptr(gs), flags))
    return gr, gw, gk, gv, ga, gb, gs


def _flatten_lead(k):
    lead = tuple(k.shape[:-3])
    B = 1
    for d in lead:
        B *= d
    return lead, B


def _bcast_flags(length, new_starts, lead, B, T, device):
    length = torch.as_tensor(length, device=device).expand(lead).reshape(B)
    new_starts = torch.as_tensor(new_starts, device=device).expand(lead + (T,)).reshape(B, T)
    return length, new_starts


def _vmap_front(n, xs, dims, required):
    """Move each batched argument's vmapped axis to the front; broadcast the others."""
    out = []
    for x, d, req in zip(xs, dims, required):
        if x is None:
            out.append(None)
        elif d is not None:
            out.append(x.movedim(d, 0))
        elif req:
            raise _lib.B200WKVError("wkv7 under vmap: r, w, k, v, a, b and s must all be batched")
        else:
            x = torch.as_tensor(x)
            out.append(x.expand((n,) + tuple(x.shape)))
    return out


class _WKV7Bwd(torch.autograd.Function):
    """The ``wkv7-bwd`` call as its own function so that it has a batching rule too
    (rwkv7.py:434-440).  Not differentiable a second time."""

    @staticmethod
    def forward(r, w, k, v, a, b, s, length, new_starts, residual, gs_out, gy):
        lead, B = _flatten_lead(k)
        T, H, N = k.shape[-3:]
        flat = [x.reshape(B, T, H, N) for x in (r, w, k, v, a, b)]
        length, new_starts = _bcast_flags(length, new_starts, lead, B, T, k.device)
        res = (*flat, s.reshape(B, H, N, N), length.to(torch.int32), new_starts.to(torch.uint8), residual)
        gs_out = None if gs_out is None else gs_out.reshape(B, H, N, N)
        gy = None if gy is None else gy.reshape(B, T, H, N)
        gr, gw, gk, gv, ga, gb, gs = batched_wkv7_bwd(res, (gs_out, gy), B)
        shp = lead + (T, H, N)
        return (gr.reshape(shp), gw.reshape(shp), gk.reshape(shp), gv.reshape(shp), ga.reshape(shp),
                gb.reshape(shp), gs.reshape(lead + (H, N, N)))

    @staticmethod
    def setup_context(ctx, inputs, output):
        pass

    @staticmethod
    def backward(ctx, *g):
        raise _lib.B200WKVError("wkv7: second-order differentiation is not supported")

    @staticmethod
    def vmap(info, in_dims, r, w, k, v, a, b, s, length, new_starts, residual, gs_out, gy):
        n = info.batch_size
        args = _vmap_front(n, (r, w, k, v, a, b, s, length, new_starts), in_dims[:9], (True,) * 7 + (False, False))
        gs_out, gy = _vmap_front(n, (gs_out, gy), in_dims[10:], (False, False))
        outs = _WKV7Bwd.apply(*args, residual, gs_out, gy)
        return outs, (0,) * 7


class _WKV7(torch.autograd.Function):
    """custom_vjp + custom_vmap of the reference (rwkv7.py:414-446) in torch terms."""

    @staticmethod
    def forward(r, w, k, v, a, b, s, length, new_starts):
        lead, B = _flatten_lead(k)                # any number of leading batch axes, possibly none
        T, H, N = k.shape[-3:]
        flat = [x.reshape(B, T, H, N) for x in (r, w, k, v, a, b)]
        length, new_starts = _bcast_flags(length, new_starts, lead, B, T, k.device)
        (new_s, out), res = batched_wkv7_fwd(*flat, s.reshape(B, H, N, N), length, new_starts, B)
        return new_s.reshape(lead + (H, N, N)), out.reshape(lead + (T, H, N)), res[-1]

    @staticmethod
    def setup_context(ctx, inputs, output):
        r, w, k, v, a, b, s, length, new_starts = inputs
        ctx.save_for_backward(r, w, k, v, a, b, s, torch.as_tensor(length), torch.as_tensor(new_starts), output[2])
        ctx.set_materialize_grads(False)
        ctx.mark_non_differentiable(output[2])

    @staticmethod
    def backward(ctx, gs_out, gy, _gres):
        r, w, k, v, a, b, s, length, new_starts, residual = ctx.saved_tensors
        gr, gw, gk, gv, ga, gb, gs = _WKV7Bwd.apply(r, w, k, v, a, b, s, length, new_starts, residual, gs_out, gy)
        return gr, gw, gk, gv, ga, gb, gs, None, None              # order of rwkv7.py:411

    @staticmethod
    def vmap(info, in_dims, r, w, k, v, a, b, s, length, new_starts):
        """Batching rule (rwkv7.py:419-431): the seven tensors must be batched, ``length`` and
        ``new_starts`` are broadcast when they are not; the new axis becomes one more leading
        batch axis, which ``forward`` flattens — so nesting works to any depth."""
        args = _vmap_front(info.batch_size, (r, w, k, v, a, b, s, length, new_starts), in_dims,
                           (True,) * 7 + (False, False))
        new_s, out, residual = _WKV7.apply(*args)
        return (new_s, out, residual), (0, 0, None)


_STEP_FLAGS = {}


def wkv7_step(r, w, k, v, a, b, s, new_starts=None, length=None):
    """One decoding step without autograd bookkeeping: tensors (B, 1, H, N) or (B, H, N), state
    (B, H, N, N).  Returns (s_out, out) with out shaped like r.  This is the T == 1 call that
    jaxrwkv routes to the Python loop (rwkv7.py:469-470); here it is one pass over the state."""
    shp = r.shape
    B, H, N = shp[0], shp[-2], shp[-1]
    flat = [x.reshape(B, 1, H, N) for x in (r, w, k, v, a, b)]
    key = (B, r.device)
    if key not in _STEP_FLAGS:      # default flags are constants: build them once per batch size
        _STEP_FLAGS[key] = (torch.zeros(B, 1, dtype=torch.uint8, device=r.device),
                            torch.ones(B, dtype=torch.int32, device=r.device))
    if new_starts is None:
        new_starts = _STEP_FLAGS[key][0]
    if length is None:
        length = _STEP_FLAGS[key][1]
    (new_s, out), _ = batched_wkv7_fwd(*flat, s, length, new_starts.reshape(B, 1), B, need_residual=False)
    return new_s, out.reshape(shp)


def wkv7_step_packed(r, w, k, v, a, b, state, layer, new_starts=None, length=None):
    """One decoding step on the model's packed state, updated in place.

    ``state`` is jaxrwkv's per-sequence container under a batch, ``(B, L, 2 + N, D)`` with
    ``D = H * N`` (``default_state``, rwkv7.py:175-180); rows ``2:`` of layer ``layer`` are this
    operator's ``(H, N, N)`` block (rwkv7.py:255, :260).  The kernel reads and writes that block
    where it lies: no slice is copied out or back.  Returns ``out`` shaped like ``r``.
    """
    lib = _lib.load()
    shp = r.shape
    B, H, N = shp[0], shp[-2], shp[-1]
    Bs, L, rows, D = state.shape
    if not (Bs == B and rows == 2 + N and D == H * N and state.is_contiguous() and state.dtype == r.dtype):
        raise _lib.B200WKVError("wkv7_step_packed: state must be a contiguous (B, L, 2+N, H*N) tensor of the streams' dtype")
    flat = [x.reshape(B, 1, H, N).contiguous() for x in (r, w, k, v, a, b)]
    code = _check_inputs(*flat, state)
    key = (B, r.device)
    if key not in _STEP_FLAGS:
        _STEP_FLAGS[key] = (torch.zeros(B, 1, dtype=torch.uint8, device=r.device),
                            torch.ones(B, dtype=torch.int32, device=r.device))
    new_starts = _STEP_FLAGS[key][0] if new_starts is None else new_starts.to(device=r.device, dtype=torch.uint8).reshape(B, 1).contiguous()
    length = _STEP_FLAGS[key][1] if length is None else length.to(device=r.device, dtype=torch.int32).contiguous()
    out = torch.empty_like(flat[0])
    block = state[:, layer, 2:]                 # (B, N, D) view: B blocks of H*N*N elements, L*(2+N)*D apart
    rr, ww, kk, vv, aa, bb = flat
    _lib.check(lib.b200wkv7_step_inplace(_stream(), code, B, H, N, _ptr(ww), _ptr(rr), _ptr(kk), _ptr(vv), _ptr(aa),
                                         _ptr(bb), block.data_ptr(), state.stride(0), _ptr(length), _ptr(new_starts),
                                         _ptr(out)))
    return out.reshape(shp)


def wkv7_cuda(r, w, k, v, a, b, s, length, new_starts):
    """Differentiable WKV-7 operator (rwkv7.py:442-446).  Tensors are (..., T, H, N) with any
    number of leading batch axes, the state (..., H, N, N); ``length`` and ``new_starts`` may
    carry the same leading axes or be shared.  Returns ``(s_out, out)``."""
    new_s, out, _ = _WKV7.apply(r, w, k, v, a, b, s, length, new_starts)
    return new_s, out


class CudaRWKV:
    """The ``rwkv_type="CudaRWKV"`` operator seam (rwkv7.py:450-473)."""

    @classmethod
    def get_kernels(cls):
        return _lib.load()

    @classmethod
    def inner_loop(cls, r, w, k, v, a, b, s, length, new_starts):
        cls.get_kernels()
        s, out = wkv7_cuda(r, w, k, v, a, b, s, length, new_starts)
        return s, out
