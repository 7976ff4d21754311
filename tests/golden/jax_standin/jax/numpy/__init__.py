"""``jax.numpy`` stand-in: thin NumPy wrappers returning arrays that support the
functional-update syntax ``x.at[idx].set(value)``."""
import numpy as _np

try:
    from ml_dtypes import bfloat16
except Exception:  # pragma: no cover
    bfloat16 = _np.float32
float32 = _np.float32
float64 = _np.float64
uint32 = _np.uint32
int32 = _np.int32


class _AtIdx:
    def __init__(self, arr, idx):
        self.arr, self.idx = arr, idx

    def set(self, value):
        out = _np.array(self.arr, copy=True)
        out[self.idx] = value
        return out.view(Arr)


class _At:
    def __init__(self, arr):
        self.arr = arr

    def __getitem__(self, idx):
        return _AtIdx(self.arr, idx)


class Arr(_np.ndarray):
    @property
    def at(self):
        return _At(self)


def _wrap(x):
    return _np.asarray(x).view(Arr)


def _lift(name):
    f = getattr(_np, name)

    def g(*a, **kw):
        return _wrap(f(*a, **kw))
    g.__name__ = name
    return g


for _n in ("exp", "zeros", "zeros_like", "ones", "ones_like", "empty_like", "expand_dims",
           "concatenate", "where", "arange", "diag", "outer", "stack", "maximum", "repeat",
           "sqrt", "mean", "var", "sum", "square", "tanh", "abs", "sign", "reshape", "pow"):
    globals()[_n] = _lift(_n) if hasattr(_np, _n) else None
pow = _lift("power")


def astype(x, dtype):
    return _wrap(_np.asarray(x).astype(dtype))


def size(x, axis=None):
    return _np.size(x, axis)


def asarray(x, dtype=None):
    return _wrap(_np.asarray(x, dtype=dtype))


array = asarray


class linalg:
    @staticmethod
    def norm(x, axis=None, keepdims=False):
        return _wrap(_np.linalg.norm(_np.asarray(x), axis=axis, keepdims=keepdims))
