"""Seeded synthetic operands of the WKV operators, drawn on the device.

RWKV-7: the distributions jaxrwkv's time-mixing block feeds the operator (src/jaxrwkv/rwkv7.py:238 raw
decay ``-softplus(-x) - 0.5``, :248-252 per-head L2-normalised ``kk``, :257 ``a = -kk``,
``b = kk * sigmoid(.)``), with N(0,1) stand-ins for the projection outputs.  RWKV-6: r, k, v ~ N(0,1),
log-decay ``-exp(x)`` with x ~ N(-0.5, 0.5) (the caller convention of rwkv6.py:217-218), bonus
u ~ N(0, 0.1).  Used by the benchmark; the tests draw the same distributions on the host
(``oracle.inputs``).
"""
import torch


def _flags(g, B, T, device, p_start, random_length, first=True):
    ns = (torch.rand(B, T, generator=g, device=device) < p_start).to(torch.uint8)
    if first:
        ns[:, 0] = 1
    if random_length:
        length = torch.randint(T // 2, T + 1, (B,), generator=g, device=device, dtype=torch.int32)
    else:
        length = torch.full((B,), T, dtype=torch.int32, device=device)
    return ns, length


def make_wkv7_device_inputs(B, T, H, N, dtype, device, seed, p_start=0.0, random_length=False, s0_scale=0.1,
                            grads=True):
    g = torch.Generator(device=device).manual_seed(seed)
    shp = (B, T, H, N)
    rn = lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32)
    ten = {}
    for n in ("r", "k", "v"):
        ten[n] = rn(*shp).to(dtype)
    ten["w"] = (-torch.nn.functional.softplus(-rn(*shp)) - 0.5).to(dtype)
    kk = torch.nn.functional.normalize(rn(*shp), dim=-1, eps=1e-12)
    ten["a"] = (-kk).to(dtype)
    ten["b"] = (kk * torch.sigmoid(rn(*shp))).to(dtype)
    del kk
    ten["s0"] = (s0_scale * rn(B, H, N, N)).to(dtype)
    if grads:
        ten["dy"] = rn(*shp).to(dtype)
        ten["ds"] = rn(B, H, N, N).to(dtype)
    ten["new_starts"], ten["length"] = _flags(g, B, T, device, p_start, random_length)
    return ten


def make_wkv6_device_inputs(B, T, H, N, dtype, device, seed, p_start=1.0 / 512, s0_scale=0.1):
    g = torch.Generator(device=device).manual_seed(seed)
    shp = (B, T, H, N)
    rn = lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32)
    ten = {n: rn(*shp).to(dtype) for n in ("r", "k", "v")}
    ten["w"] = (-torch.exp(-0.5 + 0.5 * rn(*shp))).to(dtype).reshape(B, T, H, N, 1)
    ten["u"] = (0.1 * rn(H, N, 1)).to(dtype)
    ten["s0"] = (s0_scale * rn(B, H, N, N)).to(dtype)
    ten["dy"] = rn(*shp).to(dtype)
    ten["ds"] = rn(B, H, N, N).to(dtype)
    ten["new_starts"], ten["length"] = _flags(g, B, T, device, p_start, False, first=False)
    return ten
