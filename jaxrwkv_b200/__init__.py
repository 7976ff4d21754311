"""B200-native WKV state-recurrence operators behind jaxrwkv's ``CudaRWKV`` seam.

The compute lives in ``lib/libb200wkv.so`` (hand-written sm_100a CUDA behind the
C ABI of ``include/b200wkv.h``); this package is the thin host side that mirrors
jaxrwkv's operator interface (``CudaRWKV.inner_loop`` and the ``wkv*_cuda``
functions of src/jaxrwkv/rwkv7.py:356-473).  There is no CPU fallback: importing
an operator without the built library, or calling one without a CUDA device,
raises.
"""
from . import _lib  # noqa: F401

__all__ = ["rwkv7", "_lib"]
__version__ = "0.1.0"
