"""Token shift with start flags and the carried last row, fused with the mix interpolations.

Host side of ``b200wkv_token_shift_{fwd,bwd}``.  It covers the lines around the WKV operator in
jaxrwkv's RWKV-7 layers: ``time_mixing_seq`` (src/jaxrwkv/rwkv7.py:226-235 builds the six mixed
inputs, :254 stores ``x[length-1]`` as the new shift row) and ``channel_mixing_seq``
(rwkv7.py:192-197, one mix).  Arrays are CUDA ``torch`` tensors with a leading batch axis (the
reference vmaps the per-sequence function over it).
"""
import torch

from . import _lib

SHIFT_TILE = 64   # B200WKV_SHIFT_TILE of the C header


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _prep(x, prev, mix, length, new_starts):
    if not (x.is_cuda and prev.is_cuda and mix.is_cuda):
        raise _lib.B200WKVError("token_shift: tensors must live on a CUDA device (there is no CPU path)")
    if not (x.dtype == prev.dtype == mix.dtype):
        raise _lib.B200WKVError("token_shift: x, prev and mix must share one element type")
    B, T, D = x.shape
    M = mix.shape[0]
    assert prev.shape == (B, D) and mix.shape == (M, D), (x.shape, prev.shape, mix.shape)
    length = torch.as_tensor(length, device=x.device).expand(B).to(torch.int32).contiguous()
    new_starts = torch.as_tensor(new_starts, device=x.device).expand(B, T).to(torch.uint8).contiguous()
    return x.contiguous(), prev.contiguous(), mix.contiguous(), length, new_starts, (B, T, D, M)


class _TokenShift(torch.autograd.Function):
    @staticmethod
    def forward(x, prev, mix, length, new_starts):
        lib = _lib.load()
        x, prev, mix, length, new_starts, (B, T, D, M) = _prep(x, prev, mix, length, new_starts)
        out = torch.empty((M, B, T, D), dtype=x.dtype, device=x.device)
        state_out = torch.empty_like(prev)
        _lib.check(lib.b200wkv_token_shift_fwd(_stream(), _lib.dtype_code(x.dtype), B, T, D, M, _ptr(x), _ptr(prev),
                                               _ptr(mix), _ptr(length), _ptr(new_starts), _ptr(out), _ptr(state_out)))
        return out, state_out

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, prev, mix, length, new_starts = inputs
        x, prev, mix, length, new_starts, dims = _prep(x, prev, mix, length, new_starts)
        ctx.save_for_backward(x, prev, mix, length, new_starts)
        ctx.dims = dims

    @staticmethod
    def backward(ctx, gout, gstate):
        lib = _lib.load()
        x, prev, mix, length, new_starts = ctx.saved_tensors
        B, T, D, M = ctx.dims
        gout = gout.to(x.dtype).contiguous()
        gstate = None if gstate is None else gstate.to(x.dtype).contiguous()
        gx, gprev = torch.empty_like(x), torch.empty_like(prev)
        ntile = (T + SHIFT_TILE - 1) // SHIFT_TILE
        gmix = torch.empty((B, ntile, M, D), dtype=torch.float32, device=x.device)
        _lib.check(lib.b200wkv_token_shift_bwd(_stream(), _lib.dtype_code(x.dtype), B, T, D, M, _ptr(x), _ptr(prev),
                                               _ptr(mix), _ptr(length), _ptr(new_starts), _ptr(gout), _ptr(gstate),
                                               _ptr(gx), _ptr(gprev), _ptr(gmix)))
        return gx, gprev, gmix.sum(dim=(0, 1)).to(mix.dtype), None, None


def token_shift(x, prev, mix, length, new_starts):
    """``x`` (B,T,D), ``prev`` (B,D), ``mix`` (M,D) -> ``(mixed (M,B,T,D), new_prev (B,D))``.

    ``mixed[m] = x + (shifted - x) * mix[m]`` with ``shifted[t] = 0`` at a start flag, ``prev`` at
    t = 0 and ``x[t-1]`` otherwise; ``new_prev = x[length-1]`` (rwkv7.py:226-235, :254, :192-197).
    """
    return _TokenShift.apply(x, prev, mix, length, new_starts)
