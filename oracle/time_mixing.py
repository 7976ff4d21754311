"""CPU restatement (test infrastructure, not a product path) of RWKV-7 time mixing around the WKV operator:
jaxrwkv src/jaxrwkv/rwkv7.py:222-266.  ``mix_pre`` / ``mix_post`` are the two elementwise stages that the
CUDA kernels ``b200wkv7_mix_pre_*`` / ``b200wkv7_mix_post_*`` implement; ``time_mixing_seq`` is the whole
per-sequence function with the operator taken from ``oracle.wkv7``."""
import numpy as np

from .token_shift import token_shift
from .wkv7 import wkv7_base


def _sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def _softplus(x):
    return np.logaddexp(0.0, x)


def mix_pre(k, wl, al, v, v_first, vl, w0, a0, v0, k_k, k_a, H):
    """Streams (T, C), parameters broadcastable to (C,).  Returns (w, k', v', a_i, b_i) as (T, C)."""
    T, C = k.shape
    w = -_softplus(-(np.reshape(w0, C) + wl)) - 0.5                                   # rwkv7.py:238
    if v_first is not None:
        v = v + (v_first - v) * _sigmoid(np.reshape(v0, C) + vl)                      # rwkv7.py:243
    a = _sigmoid(np.reshape(a0, C) + al)                                              # rwkv7.py:245
    kk = (k * np.reshape(k_k, C)).reshape(T, H, -1)                                   # rwkv7.py:248-249
    kk = kk / np.maximum(np.linalg.norm(kk, axis=-1, keepdims=True), 1e-12)           # rwkv7.py:250
    kk = kk.reshape(T, C)
    kp = k * (1 + (a - 1) * np.reshape(k_a, C))                                       # rwkv7.py:252
    return w, kp, v, -kk, kk * a                                                      # rwkv7.py:257


def mix_post(y, r, k, v, g, ln_w, ln_b, r_k, H, eps=64e-5):
    """(T, C) streams; group norm over each head's channels, the r-k bonus and the gate (rwkv7.py:263-265)."""
    T, C = y.shape
    yh = y.reshape(T, H, -1)
    mean = yh.mean(axis=-1, keepdims=True)
    var = yh.var(axis=-1, keepdims=True)
    x = ((yh - mean) / np.sqrt(var + eps)).reshape(T, C) * np.reshape(ln_w, C) + np.reshape(ln_b, C)
    bonus = np.sum(r.reshape(T, H, -1) * k.reshape(T, H, -1) * np.reshape(r_k, (H, -1)), axis=-1, keepdims=True)
    x = x + (bonus * v.reshape(T, H, -1)).reshape(T, C)
    return x * g


def time_mixing_seq(x, state, v_first, att, length, new_starts, H, S, layer_id):
    """x (T, C), state (1 + S, C), v_first (T, C); ``att`` holds the reference's parameter names."""
    T, C = x.shape
    mix = np.stack([np.reshape(att[n], C) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")])
    (xr, xw, xk, xv, xa, xg), shift_row = token_shift(x, state[0], mix, length, new_starts)
    r = xr @ att["receptance"]["weight"].T
    wl = np.tanh(xw @ att["w1"]) @ att["w2"]
    k = xk @ att["key"]["weight"].T
    v = xv @ att["value"]["weight"].T
    al = (xa @ att["a1"]) @ att["a2"]
    g = _sigmoid(xg @ att["g1"]) @ att["g2"]
    if layer_id == 0:
        v_first = v
        w, kp, vp, a_i, b_i = mix_pre(k, wl, al, v, None, None, att["w0"], att["a0"], None, att["k_k"], att["k_a"], H)
    else:
        vl = (xv @ att["v1"]) @ att["v2"]
        w, kp, vp, a_i, b_i = mix_pre(k, wl, al, v, v_first, vl, att["w0"], att["a0"], att["v0"], att["k_k"], att["k_a"], H)
    s = state[1:].reshape(H, S, S)
    sh = (T, H, S)
    s_new, out = wkv7_base(r.reshape(sh), w.reshape(sh), kp.reshape(sh), vp.reshape(sh), a_i.reshape(sh), b_i.reshape(sh),
                           s, length, new_starts)
    new_state = np.concatenate([shift_row[None], np.asarray(s_new).reshape(S, C)], axis=0)
    xo = mix_post(np.asarray(out).reshape(T, C), r, kp, vp, g, att["ln_x"]["weight"], att["ln_x"]["bias"], att["r_k"], H)
    return xo @ att["output"]["weight"].T, new_state, v_first
