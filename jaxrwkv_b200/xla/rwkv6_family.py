"""``CudaRWKV`` for RWKV-5, 5.2 and 6 in JAX on the B200 kernels.  jaxrwkv has no such class for these
versions; this adds one behind the same seam, ``inner_loop(r, k, v, w, time_first, s, length, new_starts)``
of src/jaxrwkv/rwkv6.py:174-191, rwkv5_2.py:164-180 and rwkv5.py:161-177.  r, k, v are (T,H,N); the state
(H,N,N) is indexed [key, value]; ``w`` is the (T,H,N,1) log-decay for version 6 and the constant decay
(H,N,1) / (H,1,1) for 5.2 / 5; ``time_first`` is (H,N,1) or (H,1,1).  The shared operands are never batched.

    CudaRWKV6 = make_cuda_rwkv("6")     # assign to jaxrwkv.rwkv6.CudaRWKV; likewise "5_2", "5"
"""
import jax
import jax.numpy as jnp
import numpy as np

from .. import _lib
from ._ffi import register_targets, dtype_str, dtype_code, float0_like, merge_leading, split_leading, to_front


def _hn(x, H, N, dtype):
    return jnp.broadcast_to(x.reshape(x.shape[0], -1), (H, N)).astype(dtype)


def make_operator(version):
    per_token = version == "6"
    vcode = 6 if per_token else 5

    def attrs(B, T, H):
        return dict(B=np.uint64(B), T=np.uint64(T), H=np.uint64(H), version=np.uint64(vcode))

    def batched_fwd(r, k, v, w, u, s, length, new_starts, B):
        T, H, N = k.shape[-3:]
        dtype = k.dtype
        fw = w.reshape(k.shape) if per_token else _hn(w, H, N, dtype)
        nbytes = int(_lib.load().b200wkv6_residual_bytes(dtype_code(dtype), B, T, H, N))
        out, residual, new_s = jax.ffi.ffi_call(
            f"wkv6-fwd-{dtype_str(dtype)}",
            (jax.ShapeDtypeStruct(k.shape, dtype), jax.ShapeDtypeStruct((nbytes,), jnp.uint8), jax.ShapeDtypeStruct(s.shape, dtype)),
        )(r, k, v, fw, _hn(u, H, N, dtype), s, length, new_starts, **attrs(B, T, H))
        return (new_s, out), (r, k, v, w, u, s, length, new_starts, residual)

    def batched_bwd(res, grads, B):
        r, k, v, w, u, s, length, new_starts, residual = res
        gs_out, gy = grads
        T, H, N = k.shape[-3:]
        dtype = k.dtype
        like = lambda x: jax.ShapeDtypeStruct(x.shape, x.dtype)
        part = jax.ShapeDtypeStruct((B, H, N), jnp.float32)      # per-batch partial sums of the shared operands' gradients
        fw = w.reshape(k.shape) if per_token else _hn(w, H, N, dtype)
        # the kernel uses part of the residual as scratch: operand 9 is donated to a seventh result
        gr, gk, gv, gw, gu, gs, _ = jax.ffi.ffi_call(
            f"wkv6-bwd-{dtype_str(dtype)}", (like(r), like(k), like(v), like(k) if per_token else part, part, like(s), like(residual)),
            input_output_aliases={9: 6},
        )(r, k, v, fw, _hn(u, H, N, dtype), s, length, new_starts, gy.astype(dtype), residual, gs_out.astype(dtype), **attrs(B, T, H))
        fold = lambda g, ref: (g.sum(0).reshape(H, N, 1).sum(1, keepdims=True) if ref.shape[1] == 1 else g.sum(0).reshape(H, N, 1)).astype(ref.dtype)
        gw = gw.reshape(w.shape) if per_token else fold(gw, w)
        return gr, gk, gv, gw, fold(gu, u), gs, float0_like(length), float0_like(new_starts)

    @jax.custom_batching.custom_vmap
    def fwd_b(r, k, v, w, u, s, length, new_starts):
        return batched_fwd(r, k, v, w, u, s, jnp.uint32(length), new_starts, k.shape[0])

    batched_idx = (0, 1, 2, 3, 5, 6, 7) if per_token else (0, 1, 2, 5, 6, 7)

    @fwd_b.def_vmap
    def fwd_b_rule(axis_size, in_batched, *args):
        assert not in_batched[4] and (per_token or not in_batched[3]), "time_first (and a constant decay) cannot be batched"
        args = list(args)
        merged = [merge_leading(x) for x in to_front(axis_size, [in_batched[i] for i in batched_idx], [args[i] for i in batched_idx])]
        for i, x in zip(batched_idx, merged):
            args[i] = x
        (new_s, out), res = fwd_b(*args)
        sp = lambda x: split_leading(x, axis_size)
        res_out = tuple(sp(x) if i in batched_idx else x for i, x in enumerate(res[:-1])) + (res[-1],)
        return ((sp(new_s), sp(out)), res_out), ((True, True), tuple(i in batched_idx for i in range(8)) + (False,))

    @jax.custom_batching.custom_vmap
    def bwd_b(res, grads):
        return batched_bwd(res, grads, res[1].shape[0])

    @bwd_b.def_vmap
    def bwd_b_rule(axis_size, in_batched, res, grads):
        rb, gb = in_batched
        res = list(res)
        merged = [merge_leading(x) for x in to_front(axis_size, [rb[i] for i in batched_idx], [res[i] for i in batched_idx])]
        for i, x in zip(batched_idx, merged):
            res[i] = x
        grads_m = tuple(merge_leading(x) for x in to_front(axis_size, gb, grads))
        gr, gk, gv, gw, gu, gs, _, _ = bwd_b(tuple(res), grads_m)
        sp = lambda x: split_leading(x, axis_size)
        outs = (sp(gr), sp(gk), sp(gv), sp(gw) if per_token else gw, gu, sp(gs), float0_like(sp(res[6])), float0_like(sp(res[7])))
        return outs, (True, True, True, per_token, False, True, True, True)

    @jax.custom_vjp
    def wkv_cuda(r, k, v, w, u, s, length, new_starts):
        return wkv_fwd(r, k, v, w, u, s, length, new_starts)[0]

    def wkv_fwd(r, k, v, w, u, s, length, new_starts):
        (new_s, out), res = fwd_b(r[None], k[None], v[None], w[None] if per_token else w, u, s[None],
                                  jnp.uint32(length)[None], new_starts[None])
        return (new_s[0], out[0]), res

    def wkv_bwd(res, grads):
        gs_out, gy = grads
        gr, gk, gv, gw, gu, gs, _, _ = bwd_b(res, (gs_out[None], gy[None]))
        return gr[0], gk[0], gv[0], gw[0] if per_token else gw, gu, gs[0], float0_like(res[6][0]), float0_like(res[7][0])

    wkv_cuda.defvjp(wkv_fwd, wkv_bwd)
    return wkv_cuda


def make_cuda_rwkv(version):
    """``CudaRWKV(BaseRWKV)`` for version "6", "5_2" or "5"."""
    import importlib
    Base = importlib.import_module({"6": "jaxrwkv.rwkv6", "5_2": "jaxrwkv.rwkv5_2", "5": "jaxrwkv.rwkv5"}[version]).BaseRWKV
    op = make_operator(version)

    class CudaRWKV(Base):
        @classmethod
        def get_kernels(cls):
            register_targets()

        @classmethod
        def inner_loop(cls, r, k, v, w, time_first, s, length, new_starts):
            cls.get_kernels()
            return op(r, k, v, w, time_first, s, length, new_starts)

    return CudaRWKV
