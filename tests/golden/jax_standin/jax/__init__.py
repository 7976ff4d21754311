"""A NumPy stand-in for the few ``jax`` entry points that jaxrwkv's WKV
``inner_loop`` functions touch.  It exists only so that
``tests/golden/make_golden.py`` can execute the reference's own operator source
(unmodified) in an image where JAX cannot be installed.  Eager, CPU, NumPy
semantics; no tracing, no autodiff.  Not a general JAX replacement and never
imported by the library.
"""
import numpy as _np

from . import numpy  # noqa: F401  (jax.numpy)
from .numpy import Arr, _wrap


def vmap(fn, in_axes=0, out_axes=0):
    """Map ``fn`` over axis 0 of every (mapped) argument and stack the results."""
    def mapped(*args):
        axes = in_axes if isinstance(in_axes, (tuple, list)) else (in_axes,) * len(args)
        n = next(a.shape[0] for a, ax in zip(args, axes) if ax is not None)
        outs = [fn(*[(a if ax is None else a[i]) for a, ax in zip(args, axes)]) for i in range(n)]
        if isinstance(outs[0], tuple):
            return tuple(_wrap(_np.stack([o[j] for o in outs])) for j in range(len(outs[0])))
        return _wrap(_np.stack(outs))
    return mapped


def _tree_index(tree, i):
    if isinstance(tree, (tuple, list)):
        return tuple(_tree_index(t, i) for t in tree)
    return tree[i]


def _tree_stack(items):
    if isinstance(items[0], (tuple, list)):
        return tuple(_tree_stack([it[j] for it in items]) for j in range(len(items[0])))
    return _wrap(_np.stack([_np.asarray(it) for it in items]))


def _tree_len(tree):
    if isinstance(tree, (tuple, list)):
        return _tree_len(tree[0])
    return tree.shape[0]


class lax:
    @staticmethod
    def select(pred, on_true, on_false):
        """Scalar-predicate select (the only form jaxrwkv uses)."""
        return on_true if bool(pred) else on_false

    @staticmethod
    def scan(f, init, xs, length=None, unroll=1):
        carry = init
        ys = []
        for i in range(_tree_len(xs)):
            carry, y = f(carry, _tree_index(xs, i))
            ys.append(y)
        return carry, _tree_stack(ys)

    @staticmethod
    def associative_scan(fn, elems):
        """Inclusive scan by its definition: a sequential left fold.  ``fn`` is
        called on length-1 slices, which is a valid batch for the vectorised
        combine functions jaxrwkv passes."""
        elems = tuple(elems)
        n = elems[0].shape[0]
        acc = tuple(e[0:1] for e in elems)
        outs = [acc]
        for i in range(1, n):
            acc = tuple(_wrap(_np.asarray(x)) for x in fn(acc, tuple(e[i:i + 1] for e in elems)))
            outs.append(acc)
        return tuple(_wrap(_np.concatenate([o[j] for o in outs], axis=0)) for j in range(len(elems)))


class nn:
    @staticmethod
    def sigmoid(x):
        return _wrap(1.0 / (1.0 + _np.exp(-_np.asarray(x))))

    @staticmethod
    def relu(x):
        return _wrap(_np.maximum(_np.asarray(x), 0))

    @staticmethod
    def softplus(x):
        return _wrap(_np.logaddexp(0.0, _np.asarray(x)))


class _Decorated:
    """What custom_vjp / custom_vmap return here: the plain function plus the
    registration hooks, which are accepted and ignored."""
    def __init__(self, fn):
        self.fn = fn

    def __call__(self, *a, **kw):
        return self.fn(*a, **kw)

    def defvjp(self, *a, **kw):
        return None

    def def_vmap(self, rule):
        return rule


def custom_vjp(fn, *a, **kw):
    return _Decorated(fn)


class custom_batching:
    @staticmethod
    def custom_vmap(fn):
        return _Decorated(fn)


def checkpoint(fn=None, **kw):
    return fn if fn is not None else (lambda f: f)


class checkpoint_policies:
    dots_with_no_batch_dims_saveable = None


class ShapeDtypeStruct:
    def __init__(self, shape, dtype):
        self.shape, self.dtype = shape, dtype
