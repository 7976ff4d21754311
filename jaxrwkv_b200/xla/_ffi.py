"""Loading of the XLA FFI adapter library and registration of its targets with JAX."""
import ctypes
import os
import threading

import jax
import jax.numpy as jnp
import numpy as np

from .. import _lib

XLA_LIB_PATH = os.path.join(os.path.dirname(_lib.LIB_PATH), "libb200wkv_xla.so")

# FFI target name -> handler symbol exported by csrc/xla_ffi_adapter.cc.  The first eight are the names and
# symbols jaxrwkv itself registers (rwkv7.py:461-465, rwkv4.py:396-400).
TARGETS = {}
for _dt, _sym in (("fp32", "F32"), ("bf16", "BF16")):
    TARGETS.update({
        f"wkv7-fwd-{_dt}": f"WKV7Fwd{_sym}", f"wkv7-bwd-{_dt}": f"WKV7Bwd{_sym}",
        f"wkv4-fwd-{_dt}": f"WKV4Fwd{_sym}", f"wkv4-bwd-{_dt}": f"WKV4Bwd{_sym}",
        f"wkv7-infer-{_dt}": f"WKV7Infer{_sym}", f"wkv7-step-{_dt}": f"WKV7Step{_sym}",
        f"wkv6-fwd-{_dt}": f"WKV6Fwd{_sym}", f"wkv6-bwd-{_dt}": f"WKV6Bwd{_sym}",
        f"token-shift-fwd-{_dt}": f"TokenShiftFwd{_sym}", f"token-shift-bwd-{_dt}": f"TokenShiftBwd{_sym}",
    })

_lock = threading.Lock()
_registered = False


def register_targets():
    """Load the kernels and the adapter once and register every target for platform "CUDA"
    (the counterpart of CudaRWKV.get_kernels in jaxrwkv, rwkv7.py:453-465)."""
    global _registered
    with _lock:
        if _registered:
            return
        _lib.load()                                             # raises if libb200wkv.so has not been built
        ctypes.CDLL(_lib.LIB_PATH, mode=ctypes.RTLD_GLOBAL)     # the adapter's undefined b200wkv* symbols resolve here
        if not os.path.exists(XLA_LIB_PATH):
            raise _lib.B200WKVError(f"{XLA_LIB_PATH} is missing: run `python -m jaxrwkv_b200.build` where the XLA FFI "
                                    "headers are installed (jax.ffi.include_dir()). There is no fallback.")
        adapter = ctypes.cdll.LoadLibrary(XLA_LIB_PATH)
        for name, symbol in TARGETS.items():
            jax.ffi.register_ffi_target(name, jax.ffi.pycapsule(getattr(adapter, symbol)), platform="CUDA")
        _registered = True


def dtype_str(dtype):
    if dtype == jnp.float32:
        return "fp32"
    if dtype == jnp.bfloat16:
        return "bf16"
    raise _lib.B200WKVError(f"b200wkv: element type {dtype} is not supported (float32 or bfloat16)")


def dtype_code(dtype):
    return _lib.F32 if dtype == jnp.float32 else _lib.BF16


def float0_like(x):
    """Cotangent of an integer or boolean operand."""
    return np.zeros(jnp.shape(x), dtype=jax.dtypes.float0)


def merge_leading(x):
    """(A, B, ...) -> (A*B, ...)"""
    return x.reshape((x.shape[0] * x.shape[1],) + x.shape[2:])


def split_leading(x, a):
    """(A*B, ...) -> (A, B, ...)"""
    return x.reshape((a, x.shape[0] // a) + x.shape[1:])


def to_front(axis_size, in_batched, args):
    """custom_vmap hands batched operands with the mapped axis first; the others are broadcast to it."""
    return [x if bat else jnp.broadcast_to(x[None], (axis_size,) + jnp.shape(x)) for x, bat in zip(args, in_batched)]
