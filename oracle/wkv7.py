"""RWKV-7 WKV recurrence: NumPy restatement (test infrastructure only).

Per head, with decay ``d_t = exp(-exp(w_t))`` and a state ``S`` indexed
``[value i, key j]``::

    S   <- 0                      if new_starts[t]
    sa   = S a_t
    S   <- S * d_t[None, :] + v_t k_t^T + sa b_t^T
    y_t  = S r_t
    s_out = S of the last t < length          (the input state if length == 0)

Shapes follow jaxrwkv's single-sequence operator: r, w, k, v, a, b are
(T, H, N), the state is (H, N, N), ``length`` an integer, ``new_starts`` (T,)
booleans.  The ``*_batched`` helpers add a leading batch axis, which is what
``jax.vmap`` does around the reference operator.

All arithmetic is carried out in the dtype of the inputs (use float64 inputs
for an exact oracle).
"""
import numpy as np

from .scan import associative_scan


def wkv7_base(r, w, k, v, a, b, s, length, new_starts):
    """Restates BaseRWKV.inner_loop, src/jaxrwkv/rwkv7.py:199-220 (the token loop).

    ScanRWKV.inner_loop (rwkv7.py:294-317) is the same arithmetic inside lax.scan.
    Returns (s_out (H,N,N), y (T,H,N)).
    """
    T = r.shape[0]
    decay = np.exp(-np.exp(w))                                  # rwkv7.py:201
    S = np.array(s, copy=True)
    out_s = np.array(s, copy=True)                              # rwkv7.py:203
    y = np.empty_like(r)
    for t in range(T):
        if new_starts[t]:                                       # rwkv7.py:207
            S = np.zeros_like(S)
        sa = np.einsum('hij,hj->hi', S, a[t])                   # rwkv7.py:216
        S = (S * decay[t][:, None, :]
             + v[t][:, :, None] * k[t][:, None, :]
             + sa[:, :, None] * b[t][:, None, :])               # rwkv7.py:217
        y[t] = np.einsum('hij,hj->hi', S, r[t])                 # rwkv7.py:218
        if t < length:                                          # rwkv7.py:219
            out_s = S.copy()
    return out_s, y


def wkv7_assoc(r, w, k, v, a, b, s, length, new_starts):
    """Restates AssociativeScanRWKV.inner_loop, src/jaxrwkv/rwkv7.py:319-346.

    Element 0 of the scanned sequence is ``(s, 0)``, element i >= 1 is token
    i-1 as ``(v k^T, diag(d) + a b^T)``.  The reference zeroes element i where
    ``new_starts_ext[i]`` holds (new_starts with one False appended), i.e. it
    zeroes token i-1 when token i is a start.  Consequences reproduced here:
    ``y[t-1] == 0`` whenever ``new_starts[t]``, and the returned state is zero
    when ``new_starts[length]`` (length < T).
    """
    T, H, N = r.shape
    decay = np.exp(-np.exp(w))                                                  # :322
    W = (decay[..., :, None] * np.eye(N, dtype=r.dtype)) + a[..., :, None] * b[..., None, :]   # :324,327
    A = v[..., :, None] * k[..., None, :]                                       # :325,328
    all_A = np.concatenate((np.asarray(s, dtype=r.dtype)[None], A))             # :329
    all_W = np.concatenate((np.zeros_like(W[0:1]), W))                          # :330
    ns = np.concatenate((np.asarray(new_starts, dtype=bool), np.zeros(1, dtype=bool)))
    ns = ns[:, None, None, None]                                                # :331
    all_A = np.where(ns, np.zeros_like(all_A), all_A)                           # :332
    all_W = np.where(ns, np.zeros_like(all_W), all_W)                           # :333

    def combine(e1, e2):                                                        # :335-341
        A1, W1 = e1
        A2, W2 = e2
        return A2 + A1 @ W2, W1 @ W2

    scan_s, _ = associative_scan(combine, (all_A, all_W))                       # :342
    y = (scan_s[1:] @ r[..., None])[..., 0]                                     # :344
    return scan_s[int(length)].astype(r.dtype), y.astype(r.dtype)               # :345-346


def quirk_mask(new_starts, length):
    """Positions where AssociativeScanRWKV (v7) departs from Base/Scan semantics.

    Returns (y_mask (T,) bool, state_differs bool): ``y_mask[t]`` is True where
    the associative-scan output is forced to zero (``new_starts[t+1]``), and
    ``state_differs`` is True when the returned state is forced to zero
    (``new_starts[length]`` with length < T).  See wkv7_assoc.
    """
    ns = np.asarray(new_starts, dtype=bool)
    T = ns.shape[0]
    y_mask = np.zeros(T, dtype=bool)
    y_mask[:-1] = ns[1:]
    state_differs = bool(length < T and ns[int(length)])
    return y_mask, state_differs


def wkv7_bwd(r, w, k, v, a, b, s, length, new_starts, dy, ds_out):
    """Reverse-mode derivative of wkv7_base (what jax.grad computes through
    BaseRWKV.inner_loop, rwkv7.py:199-220), written as an explicit reverse loop.

    Returns (dr, dw, dk, dv, da, db, ds0), each shaped like its primal; ``dw``
    is with respect to the raw ``w`` (before exp(-exp(.))).  Checked against
    torch.autograd in the test-suite.
    """
    T, H, N = r.shape
    ew = np.exp(w)
    decay = np.exp(-ew)
    # forward sweep: keep the state entering each token (after a reset) and leaving it
    S = np.array(s, copy=True)
    S_in = np.empty((T, H, N, N), dtype=r.dtype)
    S_out = np.empty((T, H, N, N), dtype=r.dtype)
    for t in range(T):
        if new_starts[t]:
            S = np.zeros_like(S)
        S_in[t] = S
        sa = np.einsum('hij,hj->hi', S, a[t])
        S = S * decay[t][:, None, :] + v[t][:, :, None] * k[t][:, None, :] + sa[:, :, None] * b[t][:, None, :]
        S_out[t] = S
    dr = np.zeros_like(r); dw = np.zeros_like(r); dk = np.zeros_like(r)
    dv = np.zeros_like(r); da = np.zeros_like(r); db = np.zeros_like(r)
    dS = np.zeros_like(S)
    L = min(int(length), T)      # `out_s <- S if t < length`: a length beyond T returns the last state
    for t in range(T - 1, -1, -1):
        if t == L - 1:
            dS = dS + ds_out
        dS = dS + dy[t][:, :, None] * r[t][:, None, :]
        dr[t] = np.einsum('hij,hi->hj', S_out[t], dy[t])
        dv[t] = np.einsum('hij,hj->hi', dS, k[t])
        dk[t] = np.einsum('hij,hi->hj', dS, v[t])
        sa = np.einsum('hij,hj->hi', S_in[t], a[t])
        db[t] = np.einsum('hij,hi->hj', dS, sa)
        dsa = np.einsum('hij,hj->hi', dS, b[t])
        da[t] = np.einsum('hij,hi->hj', S_in[t], dsa)
        dw[t] = np.einsum('hij,hij->hj', dS, S_in[t]) * (-ew[t]) * decay[t]
        dS = dS * decay[t][:, None, :] + dsa[:, :, None] * a[t][:, None, :]
        if new_starts[t]:
            dS = np.zeros_like(dS)
    ds0 = dS
    if L == 0:
        ds0 = ds0 + ds_out
    return dr, dw, dk, dv, da, db, ds0


def _batched(fn, n_out):
    def run(*args):
        B = args[0].shape[0]
        outs = [fn(*[x[i] for x in args]) for i in range(B)]
        return tuple(np.stack([o[j] for o in outs]) for j in range(n_out))
    return run


wkv7_base_batched = _batched(wkv7_base, 2)
wkv7_assoc_batched = _batched(wkv7_assoc, 2)
wkv7_bwd_batched = _batched(wkv7_bwd, 7)
