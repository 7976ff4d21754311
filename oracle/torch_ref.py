"""torch-CPU versions of the restated recurrences (test infrastructure only).

Two uses: (1) the token loops below are differentiable, so ``torch.autograd``
supplies an independent backward oracle for the hand-written reverse loops in
``oracle.wkv7`` / ``oracle.wkv6`` and for the CUDA backward kernels;
(2) ``wkv7_assoc_torch`` materialises the per-token transition matrices and runs
the same associative scan as jaxrwkv's AssociativeScanRWKV, which is the
formulation timed as the CPU baseline.
"""
import torch

from .scan import associative_scan


def wkv7_base_torch(r, w, k, v, a, b, s, length, new_starts):
    """Differentiable restatement of BaseRWKV.inner_loop, src/jaxrwkv/rwkv7.py:199-220.
    Tensors (T,H,N), state (H,N,N)."""
    T = r.shape[0]
    decay = torch.exp(-torch.exp(w))
    S = s
    out_s = s
    ys = []
    for t in range(T):
        if bool(new_starts[t]):
            S = torch.zeros_like(S)
        sa = torch.einsum('hij,hj->hi', S, a[t])
        S = S * decay[t][:, None, :] + v[t][:, :, None] * k[t][:, None, :] + sa[:, :, None] * b[t][:, None, :]
        ys.append(torch.einsum('hij,hj->hi', S, r[t]))
        if t < int(length):
            out_s = S
    return out_s, torch.stack(ys)


def wkv7_assoc_torch(r, w, k, v, a, b, s, length, new_starts):
    """Restates AssociativeScanRWKV.inner_loop, src/jaxrwkv/rwkv7.py:319-346, with
    the (T+1, H, N, N) transition tensors materialised exactly as the reference does."""
    T, H, N = r.shape
    decay = torch.exp(-torch.exp(w))
    W = torch.diag_embed(decay) + a[..., :, None] * b[..., None, :]
    A = v[..., :, None] * k[..., None, :]
    all_A = torch.cat((s[None].to(r.dtype), A))
    all_W = torch.cat((torch.zeros_like(W[0:1]), W))
    ns = torch.cat((new_starts.bool(), torch.zeros(1, dtype=torch.bool)))[:, None, None, None]
    all_A = torch.where(ns, torch.zeros_like(all_A), all_A)
    all_W = torch.where(ns, torch.zeros_like(all_W), all_W)

    def combine(e1, e2):
        A1, W1 = e1
        A2, W2 = e2
        return A2 + A1 @ W2, W1 @ W2

    scan_s, _ = associative_scan(combine, (all_A, all_W))
    y = (scan_s[1:] @ r[..., None])[..., 0]
    return scan_s[int(length)], y


def wkv6_base_torch(r, k, v, w, u, s, length, new_starts, version="6"):
    """Differentiable restatement of BaseRWKV.inner_loop of rwkv6.py:174-191
    (version "6": w (T,H,N,1) log-decay) and rwkv5_2.py:164-180 / rwkv5.py:161-177
    (w is the time-constant decay, (H,N,1) / (H,1,1))."""
    T = r.shape[0]
    d = torch.exp(w) if version == "6" else w
    S = s
    out_s = s
    ys = []
    for t in range(T):
        if bool(new_starts[t]):
            S = torch.zeros_like(S)
        at = k[t][:, :, None] * v[t][:, None, :]
        ys.append(torch.einsum('hk,hkv->hv', r[t], u * at + S))
        S = at + (d[t] if version == "6" else d) * S
        if t < int(length):
            out_s = S
    return out_s, torch.stack(ys)


def wkv4_base_torch(r, k, v, w, u, s, length, new_starts):
    """Differentiable restatement of BaseRWKV.inner_loop, src/jaxrwkv/rwkv4.py:143-172."""
    T = r.shape[0]
    wneg = -torch.exp(w)
    aa, bb, pp = s[0], s[1], s[2]
    out = (aa, bb, pp)
    ys = []
    for t in range(T):
        if bool(new_starts[t]):
            aa = torch.zeros_like(aa); bb = torch.zeros_like(bb); pp = torch.full_like(pp, -1e30)
        ww = u + k[t]
        qq = torch.maximum(pp, ww)
        e1 = torch.exp(pp - qq); e2 = torch.exp(ww - qq)
        ys.append(r[t] * ((e1 * aa + e2 * v[t]) / (e1 * bb + e2)))
        ww = pp + wneg
        qq = torch.maximum(ww, k[t])
        e1 = torch.exp(ww - qq); e2 = torch.exp(k[t] - qq)
        aa, bb, pp = e1 * aa + e2 * v[t], e1 * bb + e2, qq
        if t < int(length):
            out = (aa, bb, pp)
    return torch.stack(out), torch.stack(ys)
