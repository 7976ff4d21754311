"""Work-efficient inclusive associative scan over the leading axis.

Test infrastructure (part of the CPU oracle).  ``jax.lax.associative_scan`` is
what jaxrwkv's AssociativeScanRWKV classes call (src/jaxrwkv/rwkv7.py:342,
rwkv6.py:297, rwkv5.py:272, rwkv4.py:285).  This is a restatement of the
published odd/even recursive-doubling scheme: combine neighbouring pairs, scan
the half-length sequence of pair results recursively, then fill in the even
positions with one more combine.  It performs about 2T combines, each applied
to a whole slice at once, so the ``fn`` it is given must be vectorised over the
leading axis exactly like the functions jaxrwkv passes to JAX.

Works on NumPy arrays and on torch tensors (anything that supports slicing
plus the two small helpers below).
"""
import numpy as np


def _cat(parts):
    if isinstance(parts[0], np.ndarray):
        return np.concatenate(parts, axis=0)
    import torch
    return torch.cat(parts, dim=0)


def _interleave(even, odd):
    """even has ceil(n/2) rows (positions 0,2,4..), odd has floor(n/2) rows."""
    n = even.shape[0] + odd.shape[0]
    if isinstance(even, np.ndarray):
        out = np.empty((n,) + even.shape[1:], dtype=even.dtype)
    else:
        out = even.new_empty((n,) + tuple(even.shape[1:]))
    out[0::2] = even
    out[1::2] = odd
    return out


def associative_scan(fn, elems):
    """Inclusive scan of a tuple of arrays along axis 0 with associative ``fn``.

    ``fn(left, right)`` takes two tuples of equally shaped slices and returns a
    tuple; ``left`` is always the earlier (lower index) operand.
    """
    elems = tuple(elems)
    n = elems[0].shape[0]
    if n < 2:
        return elems
    # pairs (0,1), (2,3), ... -> inclusive totals at odd positions of each pair
    pair = fn(tuple(e[0:n - 1:2] for e in elems), tuple(e[1:n:2] for e in elems))
    odd = associative_scan(fn, pair)           # scanned value at positions 1,3,5,...
    if n % 2 == 0:
        left = tuple(o[:-1] for o in odd)
    else:
        left = odd
    right = tuple(e[2:n:2] for e in elems)
    if right[0].shape[0] > 0:
        even_tail = fn(left, right)            # positions 2,4,6,...
        even = tuple(_cat([e[0:1], t]) for e, t in zip(elems, even_tail))
    else:
        even = tuple(e[0:1] for e in elems)
    return tuple(_interleave(ev, od) for ev, od in zip(even, odd))
