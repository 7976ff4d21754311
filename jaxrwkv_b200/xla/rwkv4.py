"""RWKV-4 ``CudaRWKV`` for JAX on the B200 kernels: replacement for src/jaxrwkv/rwkv4.py:305-406
(same names, operand order and batching behaviour: ``w`` and ``time_first`` are never batched)."""
import jax
import jax.numpy as jnp
import numpy as np

from .. import _lib
from ._ffi import register_targets, dtype_str, dtype_code, float0_like, merge_leading, split_leading, to_front


def _attrs(B, T, C):
    return dict(B=np.uint64(B), T=np.uint64(T), C=np.uint64(C))


def batched_wkv4_fwd(k, v, w, time_first, s, length, new_starts, B):
    w = -jnp.exp(w)                                                                        # rwkv4.py:312
    T, C = k.shape[-2:]
    dtype = k.dtype
    assert all(x.dtype == dtype for x in (k, v, w, time_first, s))
    nbytes = int(_lib.load().b200wkv4_residual_bytes(dtype_code(dtype), B, T, C))
    new_s, out, residual = jax.ffi.ffi_call(
        f"wkv4-fwd-{dtype_str(dtype)}",
        (jax.ShapeDtypeStruct(s.shape, dtype), jax.ShapeDtypeStruct(k.shape, dtype), jax.ShapeDtypeStruct((nbytes,), jnp.uint8)),
    )(w, time_first, k, v, s, length, new_starts, **_attrs(B, T, C))
    return (new_s, out), (k, v, w, time_first, s, length, new_starts, residual)


def batched_wkv4_bwd(res, grads, B):
    k, v, w, u, s, length, new_starts, residual = res       # w is already -exp(w_raw)
    gs_new, gy = grads
    T, C = k.shape[-2:]
    like = lambda x: jax.ShapeDtypeStruct(x.shape, x.dtype)
    part = jax.ShapeDtypeStruct((B, C), jnp.float32)        # per-batch partial sums, added below (rwkv4.py:351)
    gw, gu, gk, gv, gs = jax.ffi.ffi_call(f"wkv4-bwd-{dtype_str(k.dtype)}", (part, part, like(k), like(v), like(s)))(
        w, u, k, v, gy.astype(k.dtype), s, length, new_starts, gs_new.astype(s.dtype), residual, **_attrs(B, T, C))
    gw_raw = (jnp.sum(gw, axis=0) * w.astype(jnp.float32)).astype(w.dtype)      # d(-exp(w_raw)) / d(w_raw) = -exp(w_raw) = w
    return gk, gv, gw_raw, jnp.sum(gu, axis=0).astype(u.dtype), gs, float0_like(length), float0_like(new_starts)


@jax.custom_batching.custom_vmap
def _fwd_b(k, v, w, time_first, s, length, new_starts):
    return batched_wkv4_fwd(k, v, w, time_first, s, jnp.uint32(length), new_starts, k.shape[0])


@_fwd_b.def_vmap
def _fwd_b_rule(axis_size, in_batched, k, v, w, time_first, s, length, new_starts):
    assert not in_batched[2] and not in_batched[3], "w and time_first cannot be batched"    # rwkv4.py:362-363
    k, v, s, length, new_starts = [merge_leading(x) for x in
                                   to_front(axis_size, [in_batched[i] for i in (0, 1, 4, 5, 6)], (k, v, s, length, new_starts))]
    (new_s, out), res = _fwd_b(k, v, w, time_first, s, length, new_starts)
    sp = lambda x: split_leading(x, axis_size)
    rk, rv, rw, ru, rs, rl, rn, residual = res
    return ((sp(new_s), sp(out)), (sp(rk), sp(rv), rw, ru, sp(rs), sp(rl), sp(rn), residual)), \
        ((True, True), (True, True, False, False, True, True, True, False))


@jax.custom_batching.custom_vmap
def _bwd_b(res, grads):
    return batched_wkv4_bwd(res, grads, res[0].shape[0])


@_bwd_b.def_vmap
def _bwd_b_rule(axis_size, in_batched, res, grads):
    rb, gb = in_batched
    k, v, s, length, new_starts = [merge_leading(x) for x in
                                   to_front(axis_size, [rb[i] for i in (0, 1, 4, 5, 6)], [res[i] for i in (0, 1, 4, 5, 6)])]
    grads_m = tuple(merge_leading(x) for x in to_front(axis_size, gb, grads))
    gk, gv, gw, gu, gs, _, _ = _bwd_b((k, v, res[2], res[3], s, length, new_starts, res[7]), grads_m)
    sp = lambda x: split_leading(x, axis_size)
    outs = (sp(gk), sp(gv), gw, gu, sp(gs), float0_like(sp(length)), float0_like(sp(new_starts)))
    return outs, (True, True, False, False, True, True, True)      # gw, gu are already summed over the batch


@jax.custom_vjp
def wkv4_cuda(k, v, w, time_first, s, length, new_starts):
    return wkv4_fwd(k, v, w, time_first, s, length, new_starts)[0]


def wkv4_fwd(k, v, w, time_first, s, length, new_starts):
    (new_s, out), res = _fwd_b(k[None], v[None], w, time_first, s[None], jnp.uint32(length)[None], new_starts[None])
    return (new_s[0], out[0]), res


def wkv4_bwd(res, grads):
    gs_new, gy = grads
    gk, gv, gw, gu, gs, _, _ = _bwd_b(res, (gs_new[None], gy[None]))
    return gk[0], gv[0], gw, gu, gs[0], float0_like(res[5][0]), float0_like(res[6][0])


wkv4_cuda.defvjp(wkv4_fwd, wkv4_bwd)


def make_cuda_rwkv():
    """``CudaRWKV(BaseRWKV)`` of rwkv4.py:385-406; assign it to ``jaxrwkv.rwkv4.CudaRWKV``."""
    from jaxrwkv.rwkv4 import BaseRWKV

    class CudaRWKV(BaseRWKV):
        @classmethod
        def get_kernels(cls):
            register_targets()

        @classmethod
        def inner_loop(cls, r, k, v, w, time_first, s, length, new_starts):
            cls.get_kernels()
            s, out = wkv4_cuda(k, v, w, time_first, s, length, new_starts)
            return s, r * out                                                             # rwkv4.py:406

    return CudaRWKV


def __getattr__(name):
    if name == "CudaRWKV":
        cls = make_cuda_rwkv()
        globals()["CudaRWKV"] = cls
        return cls
    raise AttributeError(name)
