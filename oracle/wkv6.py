"""RWKV-5 / 5.2 / 6 WKV recurrence: NumPy restatement (test infrastructure only).

State ``S`` is indexed ``[key, value]`` (transposed with respect to RWKV-7)::

    S   <- 0                                   if new_starts[t]
    y_t  = r_t^T (u * (k_t v_t^T) + S)         (uses the state *before* the update)
    S   <- k_t v_t^T + d_t[:, None] * S
    s_out = S of the last t < length           (the input state if length == 0)

``version`` selects where the decay comes from, mirroring the three reference
modules:

* ``"6"``   – ``w`` is (T, H, N, 1) and holds log-decay; d_t = exp(w_t)
              (src/jaxrwkv/rwkv6.py:174-191; the caller passes w = -exp(.), rwkv6.py:217-218)
* ``"5_2"`` – ``w`` is (H, N, 1) and already is the decay (src/jaxrwkv/rwkv5_2.py:164-180, :198)
* ``"5"``   – ``w`` is (H, 1, 1) and already is the decay (src/jaxrwkv/rwkv5.py:161-177, :194)

``u`` ("time_first") is (H, N, 1), or (H, 1, 1) for version 5.
"""
import numpy as np

from .scan import associative_scan


def _decay_seq(w, T, version):
    if version == "6":
        return np.exp(w)                                   # rwkv6.py:176
    return np.broadcast_to(w[None], (T,) + w.shape)        # time-constant decay


def wkv6_base(r, k, v, w, u, s, length, new_starts, version="6"):
    """Restates BaseRWKV.inner_loop of rwkv6.py:174-191 / rwkv5.py:161-177 /
    rwkv5_2.py:164-180.  Returns (s_out (H,N,N), y (T,H,N))."""
    T = r.shape[0]
    d = _decay_seq(w, T, version)
    S = np.array(s, copy=True)
    out_s = np.array(s, copy=True)
    y = np.empty_like(r)
    for t in range(T):
        if new_starts[t]:
            S = np.zeros_like(S)
        at = k[t][:, :, None] * v[t][:, None, :]                      # kt @ vt
        y[t] = np.einsum('hk,hkv->hv', r[t], u * at + S)
        S = at + d[t] * S
        if t < length:
            out_s = S.copy()
    return out_s, y


def wkv6_assoc(r, k, v, w, u, s, length, new_starts, version="6"):
    """Restates AssociativeScanRWKV.inner_loop of rwkv6.py:276-302 (and
    rwkv5.py:251-277, rwkv5_2.py:255-281).  Outputs agree with wkv6_base at every
    position; the returned state is zero when ``new_starts[length]`` (length < T),
    because the reference zeroes scan element i for a start at token i."""
    T, H, N = r.shape
    d = _decay_seq(w, T, version)
    d = np.broadcast_to(d, (T, H, N, 1)) if d.shape[-2] != N else d
    A = k[..., :, None] * v[..., None, :]
    all_A = np.concatenate((np.asarray(s, dtype=r.dtype)[None], A))
    all_W = np.concatenate((np.zeros_like(d[0:1]), d))
    ns = np.concatenate((np.asarray(new_starts, dtype=bool), np.zeros(1, dtype=bool)))[:, None, None, None]
    all_A = np.where(ns, np.zeros_like(all_A), all_A)
    all_W = np.where(ns, np.zeros_like(all_W), all_W)

    def combine(e1, e2):
        A1, W1, r1 = e1
        A2, W2, r2 = e2
        return (np.where(r2, A2, A2 + W2 * A1), np.where(r2, W2, W2 * W1), np.where(r2, r2, r1))

    scan_s, _, _ = associative_scan(combine, (all_A, all_W, ns))
    y = np.einsum('thk,thkv->thv', r, u * A + scan_s[:-1])
    return scan_s[int(length)].astype(r.dtype), y.astype(r.dtype)


def wkv6_bwd(r, k, v, w, u, s, length, new_starts, dy, ds_out, version="6"):
    """Reverse-mode derivative of wkv6_base as an explicit reverse loop.

    Returns (dr, dk, dv, dw, du, ds0).  ``dw`` has the shape of ``w``: for
    version 6 it is with respect to the log-decay, for 5/5.2 with respect to the
    time-constant decay itself (summed over tokens, and over the key axis for
    version 5).  ``du`` has the shape of ``u``.  Checked against torch.autograd
    in the test-suite.
    """
    T, H, N = r.shape
    d = np.broadcast_to(_decay_seq(w, T, version), (T, H, N, 1))
    ub = np.broadcast_to(u, (H, N, 1))
    S = np.array(s, copy=True)
    S_in = np.empty((T, H, N, N), dtype=r.dtype)
    for t in range(T):
        if new_starts[t]:
            S = np.zeros_like(S)
        S_in[t] = S
        S = k[t][:, :, None] * v[t][:, None, :] + d[t] * S
    dr = np.zeros_like(r); dk = np.zeros_like(r); dv = np.zeros_like(r)
    dd = np.zeros((T, H, N, 1), dtype=r.dtype)
    du = np.zeros((H, N, 1), dtype=r.dtype)
    dS = np.zeros_like(S)
    L = min(int(length), T)      # `out_s <- S if t < length`: a length beyond T returns the last state
    for t in range(T - 1, -1, -1):
        if t == L - 1:
            dS = dS + ds_out
        dyv = np.einsum('hv,hv->h', dy[t], v[t])[:, None]                 # (H,1)
        dr[t] = ub[..., 0] * k[t] * dyv + np.einsum('hkv,hv->hk', S_in[t], dy[t])
        du[..., 0] += r[t] * k[t] * dyv
        dk[t] = r[t] * ub[..., 0] * dyv + np.einsum('hkv,hv->hk', dS, v[t])
        ruk = np.einsum('hk,hk->h', r[t] * ub[..., 0], k[t])[:, None]
        dv[t] = ruk * dy[t] + np.einsum('hkv,hk->hv', dS, k[t])
        dd[t, ..., 0] = np.einsum('hkv,hkv->hk', dS, S_in[t])
        dS = d[t] * dS + r[t][:, :, None] * dy[t][:, None, :]
        if new_starts[t]:
            dS = np.zeros_like(dS)
    ds0 = dS
    if L == 0:
        ds0 = ds0 + ds_out
    if version == "6":
        dw = dd * d                              # d = exp(w)
    elif version == "5_2":
        dw = dd.sum(axis=0)
    else:
        dw = dd.sum(axis=(0, 2, 3))[:, None, None]
    if u.shape[1] == 1:
        du = du.sum(axis=1, keepdims=True)
    return dr, dk, dv, dw, du, ds0


def wkv6_base_batched(r, k, v, w, u, s, length, new_starts, version="6"):
    """Batch axis in front of r, k, v, s, length, new_starts (and of w for version 6);
    u (and the constant decay of 5/5.2) are shared, as under jax.vmap(in_axes=None)."""
    B = r.shape[0]
    outs = [wkv6_base(r[i], k[i], v[i], w[i] if version == "6" else w, u, s[i],
                      length[i], new_starts[i], version) for i in range(B)]
    return np.stack([o[0] for o in outs]), np.stack([o[1] for o in outs])


def wkv6_bwd_batched(r, k, v, w, u, s, length, new_starts, dy, ds_out, version="6"):
    """As wkv6_bwd with a batch axis; gradients of the shared u (and of the shared
    decay for 5/5.2) are summed over the batch."""
    B = r.shape[0]
    outs = [wkv6_bwd(r[i], k[i], v[i], w[i] if version == "6" else w, u, s[i],
                     length[i], new_starts[i], dy[i], ds_out[i], version) for i in range(B)]
    dr, dk, dv = (np.stack([o[j] for o in outs]) for j in range(3))
    if version == "6":
        dw = np.stack([o[3] for o in outs])
    else:
        dw = sum(o[3] for o in outs)
    du = sum(o[4] for o in outs)
    ds0 = np.stack([o[5] for o in outs])
    return dr, dk, dv, dw, du, ds0
