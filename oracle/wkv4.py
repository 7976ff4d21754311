"""RWKV-4 WKV recurrence: NumPy restatement (test infrastructure only).

Per channel the state is the triple (aa, bb, pp): a numerator, a denominator
and the running maximum exponent they are both scaled by.  With ``w' = -exp(w)``
and ``u`` = time_first::

    (aa, bb, pp) <- (0, 0, -1e30)                      if new_starts[t]
    q  = max(pp, u + k_t)
    y_t = r_t * (e^{pp-q} aa + e^{u+k_t-q} v_t) / (e^{pp-q} bb + e^{u+k_t-q})
    q' = max(pp + w', k_t)
    aa <- e^{pp+w'-q'} aa + e^{k_t-q'} v_t ;  bb <- e^{pp+w'-q'} bb + e^{k_t-q'} ;  pp <- q'
    s_out = state of the last t < length               (the input state if length == 0)

r, k, v are (T, C); w, u are (C,); the state is (3, C).
"""
import numpy as np

from .scan import associative_scan


def wkv4_base(r, k, v, w, u, s, length, new_starts):
    """Restates BaseRWKV.inner_loop, src/jaxrwkv/rwkv4.py:143-172.
    Returns (s_out (3,C), y (T,C))."""
    T = r.shape[0]
    wneg = -np.exp(w)                                           # rwkv4.py:144
    S = np.array(s, copy=True)
    out_s = np.array(s, copy=True)
    y = np.empty_like(r)
    for t in range(T):
        if new_starts[t]:                                       # rwkv4.py:148-152
            S = np.zeros_like(S)
            S[2] = -1e30
        aa, bb, pp = S
        ww = u + k[t]                                           # rwkv4.py:155-162
        qq = np.maximum(pp, ww)
        e1 = np.exp(pp - qq)
        e2 = np.exp(ww - qq)
        y[t] = r[t] * ((e1 * aa + e2 * v[t]) / (e1 * bb + e2))
        ww = pp + wneg                                          # rwkv4.py:164-169
        qq = np.maximum(ww, k[t])
        e1 = np.exp(ww - qq)
        e2 = np.exp(k[t] - qq)
        S = np.stack([e1 * aa + e2 * v[t], e1 * bb + e2, qq]).astype(r.dtype)
        if t < length:                                          # rwkv4.py:170
            out_s = S.copy()
    return out_s, y


def wkv4_assoc(r, k, v, w, u, s, length, new_starts):
    """Restates AssociativeScanRWKV.inner_loop, src/jaxrwkv/rwkv4.py:251-300.

    Scan element i (i >= 1) is token i-1 as (v, 1, k) stamped with position i;
    combining decays the left element by the position gap.  As in the other
    versions the reference resets element i for a start at token i, so the
    returned state is the reset state when ``new_starts[length]`` (length < T).
    """
    T, C = r.shape
    wneg = -np.exp(w)
    AA = np.concatenate((s[0:1], v)).astype(r.dtype)
    BB = np.ones_like(AA)
    BB[0] = s[1]
    PP = np.concatenate((s[2:3], k)).astype(r.dtype)
    EI = np.arange(T + 1)[:, None]
    ns = np.concatenate((np.asarray(new_starts, dtype=bool), np.zeros(1, dtype=bool)))[:, None]
    AA = np.where(ns, np.zeros_like(AA), AA)
    BB = np.where(ns, np.zeros_like(BB), BB)
    PP = np.where(ns, np.ones_like(PP) * (-1e30), PP)

    def combine(e1, e2):
        A1, B1, P1, E1, r1 = e1
        A2, B2, P2, E2, r2 = e2
        d = E2 - E1
        ww = P1 + d * wneg
        qq = np.maximum(ww, P2)
        AN = A1 * np.exp(ww - qq) + A2 * np.exp(P2 - qq)
        BN = B1 * np.exp(ww - qq) + B2 * np.exp(P2 - qq)
        return (np.where(r2, A2, AN), np.where(r2, B2, BN), np.where(r2, P2, qq), E2,
                np.where(r2, r2, r1))

    AA, BB, PP, _, _ = associative_scan(combine, (AA, BB, PP, EI, ns))
    aa, bb, pp = AA[:T], BB[:T], PP[:T]
    ww = u[None] + k
    qq = np.maximum(pp, ww)
    e1 = np.exp(pp - qq)
    e2 = np.exp(ww - qq)
    y = r * ((e1 * aa + e2 * v) / (e1 * bb + e2))
    L = int(length)
    return np.stack([AA[L], BB[L], PP[L]]).astype(r.dtype), y.astype(r.dtype)


def wkv4_base_batched(r, k, v, w, u, s, length, new_starts):
    """Batch axis in front of r, k, v, s, length, new_starts; w and u shared."""
    B = r.shape[0]
    outs = [wkv4_base(r[i], k[i], v[i], w, u, s[i], length[i], new_starts[i]) for i in range(B)]
    return np.stack([o[0] for o in outs]), np.stack([o[1] for o in outs])
