"""Seeded synthetic operands of the RWKV-7 WKV operator, drawn on the device.

Same distributions as jaxrwkv's time-mixing block feeds the operator (src/jaxrwkv/rwkv7.py:238 raw
decay ``-softplus(-x) - 0.5``, :248-252 per-head L2-normalised ``kk``, :257 ``a = -kk``,
``b = kk * sigmoid(.)``), with N(0,1) stand-ins for the projection outputs.  Used by the benchmark
and by ``python -m jaxrwkv_b200.run_case``.
"""
import torch


def make_wkv7_device_inputs(B, T, H, N, dtype, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    shp = (B, T, H, N)
    rn = lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32)
    r, k, v = rn(*shp), rn(*shp), rn(*shp)
    w = -torch.nn.functional.softplus(-rn(*shp)) - 0.5
    kk = torch.nn.functional.normalize(rn(*shp), dim=-1, eps=1e-12)
    a = -kk
    b = kk * torch.sigmoid(rn(*shp))
    s0 = 0.1 * rn(B, H, N, N)
    dy = rn(*shp)
    ds = rn(B, H, N, N)
    ten = {n: x.to(dtype).contiguous() for n, x in dict(r=r, w=w, k=k, v=v, a=a, b=b, s0=s0, dy=dy, ds=ds).items()}
    ns = torch.zeros(B, T, dtype=torch.uint8, device=device)
    ns[:, 0] = 1
    ten["new_starts"] = ns
    ten["length"] = torch.full((B,), T, dtype=torch.int32, device=device)
    return ten
