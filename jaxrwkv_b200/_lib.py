"""ctypes binding of libb200wkv.so (the C ABI declared in include/b200wkv.h)."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libb200wkv.so")

F32, BF16 = 0, 1
FLAG_SEQUENTIAL = 1

_P = ctypes.c_void_p
_I = ctypes.c_int
_SZ = ctypes.c_size_t
_U = ctypes.c_uint

# name -> (restype, argtypes); must list every symbol the header declares
PROTOTYPES = {
    "b200wkv_strerror": (ctypes.c_char_p, [_I]),
    "b200wkv_abi_version": (_I, []),
    "b200wkv_device_status": (_I, []),
    "b200wkv_debug_split_plan": (_I, [_I, _I, _I, _P, _P]),
    "b200wkv_debug_runs": (_I, [_I, _I, _I, _I, _P, _I]),
    "b200wkv7_residual_bytes": (_SZ, [_I, _I, _I, _I, _I]),
    "b200wkv7_fwd": (_I, [_P, _I, _I, _I, _I, _I] + [_P] * 9 + [_P, _P, _P, _SZ, _U]),
    "b200wkv7_step_inplace": (_I, [_P, _I, _I, _I, _I] + [_P] * 6 + [_P, ctypes.c_longlong, _P, _P, _P]),
    "b200wkv7_bwd": (_I, [_P, _I, _I, _I, _I, _I] + [_P] * 9 + [_P, _P, _P, _SZ] + [_P] * 7 + [_U]),
    "b200wkv6_residual_bytes": (_SZ, [_I, _I, _I, _I, _I]),
    "b200wkv6_fwd": (_I, [_P, _I, _I, _I, _I, _I, _I] + [_P] * 8 + [_P, _P, _P, _SZ, _U]),
    "b200wkv6_bwd": (_I, [_P, _I, _I, _I, _I, _I, _I] + [_P] * 8 + [_P, _P, _P, _SZ] + [_P] * 6 + [_U]),
    "b200wkv4_residual_bytes": (_SZ, [_I, _I, _I, _I]),
    "b200wkv4_fwd": (_I, [_P, _I, _I, _I, _I] + [_P] * 7 + [_P, _P, _P, _SZ, _U]),
    "b200wkv4_bwd": (_I, [_P, _I, _I, _I, _I] + [_P] * 9 + [_P, _SZ] + [_P] * 5 + [_U]),
    "b200wkv_token_shift_fwd": (_I, [_P, _I, _I, _I, _I, _I] + [_P] * 7),
    "b200wkv_token_shift_bwd": (_I, [_P, _I, _I, _I, _I, _I] + [_P] * 10),
    "b200wkv7_mix_partial_rows": (_I, [ctypes.c_longlong, _I, _I]),
    "b200wkv7_mix_pre_fwd": (_I, [_P, _I, ctypes.c_longlong, _I, _I, _I] + [_P] * 16),
    "b200wkv7_mix_pre_bwd": (_I, [_P, _I, ctypes.c_longlong, _I, _I, _I] + [_P] * 23),
    "b200wkv7_mix_post_fwd": (_I, [_P, _I, ctypes.c_longlong, _I, _I, ctypes.c_float] + [_P] * 9),
    "b200wkv7_mix_post_bwd": (_I, [_P, _I, ctypes.c_longlong, _I, _I, ctypes.c_float] + [_P] * 15),
    "b200wkv7_static_scratch_bytes": (_SZ, []),
    "b200wkv7_fwd_bwd_static": (_I, [_P, _I, _I, _I, _I, _I] + [_P] * 9 + [_P, _P] + [_P, _P] + [_P] * 7 + [_U]),
}

_lib = None


class B200WKVError(RuntimeError):
    pass


def load():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200WKVError(
                f"{LIB_PATH} is missing: build it with `python -m jaxrwkv_b200.build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback for the WKV operators.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status):
    if status != 0:
        raise B200WKVError(f"b200wkv: {load().b200wkv_strerror(status).decode()} (status {status})")


def dtype_code(torch_dtype):
    import torch
    if torch_dtype == torch.float32:
        return F32
    if torch_dtype == torch.bfloat16:
        return BF16
    raise B200WKVError(f"b200wkv: element type {torch_dtype} is not supported (float32 or bfloat16)")
