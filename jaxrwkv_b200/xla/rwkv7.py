"""RWKV-7 ``CudaRWKV`` for JAX on the B200 kernels: replacement for the FFI glue of jaxrwkv
(src/jaxrwkv/rwkv7.py:349-473), same names and argument meaning.

Differences from the reference glue: one opaque ``residual`` result instead of ``s_restore`` /
``sa_restore`` (rwkv7.py:362-365); both cotangents are used and the gradient of the input state is
returned; ``length`` / ``new_starts`` get ``float0`` cotangents; the batching rule merges the mapped
axis into the kernels' batch dimension and applies to its own result, so ``vmap`` nests to any depth
(the reference's rule survives one level, rwkv7.py:419-431); T need not be a multiple of 16 and T == 1
runs on the GPU (the reference falls back to the Python loop, rwkv7.py:469-470).
"""
import jax
import jax.numpy as jnp
import numpy as np

from .. import _lib
from ._ffi import register_targets, dtype_str, dtype_code, float0_like, merge_leading, split_leading, to_front


def _attrs(B, T, H):
    return dict(B=np.uint64(B), T=np.uint64(T), H=np.uint64(H))


def batched_wkv7_fwd(r, w, k, v, a, b, s, length, new_starts, B):
    """One "wkv7-fwd" custom call on (B,T,H,C) arrays (rwkv7.py:356-376)."""
    T, H, C = k.shape[-3:]
    dtype = k.dtype
    assert all(x.dtype == dtype for x in (r, w, k, v, a, b, s))                         # rwkv7.py:361
    nbytes = int(_lib.load().b200wkv7_residual_bytes(dtype_code(dtype), B, T, H, C))     # host call at trace time
    out, residual, new_s = jax.ffi.ffi_call(
        f"wkv7-fwd-{dtype_str(dtype)}",
        (jax.ShapeDtypeStruct(k.shape, dtype), jax.ShapeDtypeStruct((nbytes,), jnp.uint8), jax.ShapeDtypeStruct(s.shape, dtype)),
    )(w, r, k, v, a, b, s, length, new_starts, **_attrs(B, T, H))
    return (new_s, out), (r, w, k, v, a, b, s, length, new_starts, residual)


def batched_wkv7_infer(r, w, k, v, a, b, s, length, new_starts, B):
    """The forward when nothing will be differentiated: no residual is produced."""
    T, H, C = k.shape[-3:]
    out, new_s = jax.ffi.ffi_call(
        f"wkv7-infer-{dtype_str(k.dtype)}", (jax.ShapeDtypeStruct(k.shape, k.dtype), jax.ShapeDtypeStruct(s.shape, s.dtype)),
    )(w, r, k, v, a, b, s, length, new_starts, **_attrs(B, T, H))
    return new_s, out


def batched_wkv7_bwd(res, grads, B):
    """One "wkv7-bwd" custom call (rwkv7.py:378-411); returns cotangents in the operator's argument order."""
    r, w, k, v, a, b, s, length, new_starts, residual = res
    gs_out, gy = grads
    T, H, C = k.shape[-3:]
    like = lambda x: jax.ShapeDtypeStruct(x.shape, x.dtype)
    # the kernel uses part of the residual as scratch: operand 10 is donated to an eighth result
    gw, gr, gk, gv, ga, gb, gs, _ = jax.ffi.ffi_call(
        f"wkv7-bwd-{dtype_str(k.dtype)}", (like(w), like(r), like(k), like(v), like(a), like(b), like(s), like(residual)),
        input_output_aliases={10: 7},
    )(w, r, k, v, a, b, s, length, new_starts, gy.astype(k.dtype), residual, gs_out.astype(s.dtype), **_attrs(B, T, H))
    return gr, gw, gk, gv, ga, gb, gs, float0_like(length), float0_like(new_starts)


# ---- batching: every function below takes arrays WITH a leading batch axis and is its own vmap rule's target
@jax.custom_batching.custom_vmap
def _fwd_b(r, w, k, v, a, b, s, length, new_starts):
    return batched_wkv7_fwd(r, w, k, v, a, b, s, jnp.uint32(length), new_starts, k.shape[0])


@_fwd_b.def_vmap
def _fwd_b_rule(axis_size, in_batched, *args):
    args = [merge_leading(x) for x in to_front(axis_size, in_batched, args)]
    (new_s, out), res = _fwd_b(*args)
    sp = lambda x: split_leading(x, axis_size)
    res_out = tuple(sp(x) for x in res[:-1]) + (res[-1],)      # the residual is one opaque buffer for the merged batch
    return ((sp(new_s), sp(out)), res_out), ((True, True), (True,) * 9 + (False,))


@jax.custom_batching.custom_vmap
def _infer_b(r, w, k, v, a, b, s, length, new_starts):
    return batched_wkv7_infer(r, w, k, v, a, b, s, jnp.uint32(length), new_starts, k.shape[0])


@_infer_b.def_vmap
def _infer_b_rule(axis_size, in_batched, *args):
    args = [merge_leading(x) for x in to_front(axis_size, in_batched, args)]
    new_s, out = _infer_b(*args)
    return (split_leading(new_s, axis_size), split_leading(out, axis_size)), (True, True)


@jax.custom_batching.custom_vmap
def _bwd_b(res, grads):
    return batched_wkv7_bwd(res, grads, res[2].shape[0])


@_bwd_b.def_vmap
def _bwd_b_rule(axis_size, in_batched, res, grads):
    res_b, grads_b = in_batched
    res_m = [merge_leading(x) for x in to_front(axis_size, res_b[:-1], res[:-1])] + [res[-1]]
    grads_m = [merge_leading(x) for x in to_front(axis_size, grads_b, grads)]
    outs = _bwd_b(tuple(res_m), tuple(grads_m))
    outs = tuple(split_leading(x, axis_size) for x in outs[:7]) + tuple(float0_like(split_leading(x, axis_size)) for x in res_m[7:9])
    return outs, (True,) * 9


def _lead1(xs):
    return [x[None] for x in xs]


@jax.custom_vjp
def wkv7_cuda(r, w, k, v, a, b, s, length, new_starts):
    """Differentiable operator on one sequence (rwkv7.py:442-446): tensors (T,H,C), state (H,C,C)."""
    new_s, out = _infer_b(*_lead1((r, w, k, v, a, b, s, jnp.uint32(length), new_starts)))
    return new_s[0], out[0]


def wkv7_fwd(r, w, k, v, a, b, s, length, new_starts):
    (new_s, out), res = _fwd_b(*_lead1((r, w, k, v, a, b, s, jnp.uint32(length), new_starts)))
    return (new_s[0], out[0]), res


def wkv7_bwd(res, grads):
    gs_out, gy = grads
    outs = _bwd_b(res, (gs_out[None], gy[None]))
    return tuple(x[0] for x in outs[:7]) + (float0_like(res[7][0]), float0_like(res[8][0]))


wkv7_cuda.defvjp(wkv7_fwd, wkv7_bwd)


def _base_class():
    from jaxrwkv.rwkv7 import BaseRWKV            # the reference package: weights, init, token shift, projections
    return BaseRWKV


def make_cuda_rwkv():
    """``CudaRWKV(BaseRWKV)`` (rwkv7.py:450-473): only ``inner_loop`` differs from the base class, so
    ``get_model`` / ``get_rand_model`` / ``forward`` / ``default_state`` are inherited unchanged.
    Assign the result to ``jaxrwkv.rwkv7.CudaRWKV`` so that ``getattr(module, rwkv_type)`` finds it
    (src/jaxrwkv/auto.py:62, :89)."""
    Base = _base_class()

    class CudaRWKV(Base):
        @classmethod
        def get_kernels(cls):
            register_targets()

        @classmethod
        def inner_loop(cls, r, w, k, v, a, b, s, length, new_starts):
            cls.get_kernels()
            return wkv7_cuda(r, w, k, v, a, b, s, length, new_starts)

    return CudaRWKV


def __getattr__(name):
    if name == "CudaRWKV":
        cls = make_cuda_rwkv()
        globals()["CudaRWKV"] = cls
        return cls
    raise AttributeError(name)
