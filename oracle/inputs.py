"""Seeded synthetic inputs with the value distributions of the benchmark configs
(test infrastructure; shared by tests, the smoke check and the benchmark).

The RWKV-7 generator follows how jaxrwkv's time-mixing block produces the six
operands of the WKV operator (src/jaxrwkv/rwkv7.py:238 raw decay
``w = -softplus(-x) - 0.5``, :248-252 per-head L2-normalised ``kk``, :257
``a = -kk`` and ``b = kk * sigmoid(.)``), with N(0,1) stand-ins for the
projection outputs.  All draws come from a counter-based Philox generator so a
(seed, shape) pair always yields the same tensors.
"""
import numpy as np


def _rng(seed):
    return np.random.Generator(np.random.Philox(int(seed)))


def make_wkv7_inputs(B, T, H, N=64, seed=1234, p_start=0.0, random_length=False,
                     s0_scale=0.0, dtype=np.float32):
    """Returns a dict with r,w,k,v,a,b (B,T,H,N), s0 (B,H,N,N), length (B,) uint32,
    new_starts (B,T) bool.  ``new_starts[:,0]`` is always set, further starts are
    Bernoulli(p_start); ``length`` is T, or uniform in [T/2, T] when random_length."""
    g = _rng(seed)
    shp = (B, T, H, N)
    r = g.standard_normal(shp)
    k = g.standard_normal(shp)
    v = g.standard_normal(shp)
    x = g.standard_normal(shp)
    w = -np.logaddexp(0.0, -x) - 0.5                  # exp(w) = 0.606531 * sigmoid(x)
    kk = g.standard_normal(shp)
    kk = kk / np.maximum(np.linalg.norm(kk, axis=-1, keepdims=True), 1e-12)
    asig = 1.0 / (1.0 + np.exp(-g.standard_normal(shp)))
    a = -kk
    b = kk * asig
    s0 = s0_scale * g.standard_normal((B, H, N, N))
    ns = g.random((B, T)) < p_start
    ns[:, 0] = True
    if random_length:
        length = g.integers(T // 2, T + 1, size=B)
    else:
        length = np.full(B, T)
    out = dict(r=r, w=w, k=k, v=v, a=a, b=b, s0=s0)
    out = {n: np.ascontiguousarray(t, dtype=dtype) for n, t in out.items()}
    out["length"] = length.astype(np.uint32)
    out["new_starts"] = ns
    return out


def make_wkv6_inputs(B, T, H, N=64, seed=1236, p_start=1.0 / 512, s0_scale=0.1,
                     random_length=False, version="6", dtype=np.float32):
    """RWKV-6 training-kernel inputs: r,k,v ~ N(0,1); log-decay w = -exp(x) with
    x ~ N(-0.5, 0.5) per token (rwkv6.py:217-218 convention); bonus u ~ N(0, 0.1);
    s0 ~ N(0, s0_scale).  For version "5_2"/"5" the decay is time-constant:
    exp(-exp(x)) of shape (H,N,1) / (H,1,1)."""
    g = _rng(seed)
    shp = (B, T, H, N)
    r = g.standard_normal(shp)
    k = g.standard_normal(shp)
    v = g.standard_normal(shp)
    if version == "6":
        w = -np.exp(-0.5 + 0.5 * g.standard_normal(shp))[..., None]
        u = 0.1 * g.standard_normal((H, N, 1))
    elif version == "5_2":
        w = np.exp(-np.exp(-0.5 + 0.5 * g.standard_normal((H, N, 1))))
        u = 0.1 * g.standard_normal((H, N, 1))
    else:
        w = np.exp(-np.exp(-0.5 + 0.5 * g.standard_normal((H, 1, 1))))
        u = np.exp(0.1 * g.standard_normal((H, 1, 1)))
    s0 = s0_scale * g.standard_normal((B, H, N, N))
    ns = g.random((B, T)) < p_start
    length = g.integers(T // 2, T + 1, size=B) if random_length else np.full(B, T)
    out = dict(r=r, k=k, v=v, w=w, u=u, s0=s0)
    out = {n: np.ascontiguousarray(t, dtype=dtype) for n, t in out.items()}
    out["length"] = length.astype(np.uint32)
    out["new_starts"] = ns
    return out


def make_wkv4_inputs(B, T, C, seed=1238, p_start=0.0, random_length=False,
                     default_state=True, dtype=np.float32):
    """RWKV-4 inputs: r = sigmoid(N(0,1)), k,v ~ N(0,1); w (pre -exp) and u ~ N(0, 0.5)
    per channel; the state is jaxrwkv's default (0, 0, -1e30) (rwkv4.py:117-123) or a
    random valid triple."""
    g = _rng(seed)
    r = 1.0 / (1.0 + np.exp(-g.standard_normal((B, T, C))))
    k = g.standard_normal((B, T, C))
    v = g.standard_normal((B, T, C))
    w = -1.0 + 0.5 * g.standard_normal(C)
    u = 0.5 * g.standard_normal(C)
    s0 = np.zeros((B, 3, C))
    if default_state:
        s0[:, 2] = -1e30
    else:
        s0[:, 0] = g.standard_normal((B, C))
        s0[:, 1] = 0.5 + g.random((B, C))
        s0[:, 2] = g.standard_normal((B, C))
    ns = g.random((B, T)) < p_start
    length = g.integers(T // 2, T + 1, size=B) if random_length else np.full(B, T)
    out = dict(r=r, k=k, v=v, w=w, u=u, s0=s0)
    out = {n: np.ascontiguousarray(t, dtype=dtype) for n, t in out.items()}
    out["length"] = length.astype(np.uint32)
    out["new_starts"] = ns
    return out
