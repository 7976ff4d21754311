"""RWKV-5 WKV operator on B200 behind the ``CudaRWKV`` seam (see _wkv6_family)."""
from ._wkv6_family import make_class, wkv_cuda as _wkv_cuda

CudaRWKV = make_class("5")


def wkv_cuda(r, k, v, w, time_first, s, length, new_starts):
    return _wkv_cuda("5", r, k, v, w, time_first, s, length, new_starts)
