"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import oracle

NAMES7 = ("r", "w", "k", "v", "a", "b", "s0")
# Stated tolerances (Frobenius-relative): fp32 against the float64 oracle, bf16 against the
# float64 oracle evaluated on the bf16-rounded inputs.
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}


def to_dev(d, dtype, names=NAMES7):
    return {n: torch.tensor(d[n], dtype=torch.float32).to(dtype).cuda() for n in names}


def rounded(t, names=NAMES7):
    """What the kernel actually sees, as float64 NumPy."""
    return [t[n].double().cpu().numpy() for n in names]


def flags(d):
    return torch.tensor(d["length"].astype(np.int64)), torch.tensor(d["new_starts"])


def npf(x):
    return x.detach().double().cpu().numpy()


def wkv7_case(B, T, H, seed, p_start=0.0, random_length=False, s0_scale=0.0, starts=None, lengths=None):
    d = oracle.make_wkv7_inputs(B, T, H, 64, seed=seed, p_start=p_start, random_length=random_length, s0_scale=s0_scale)
    if starts is not None:
        ns = np.zeros((B, T), dtype=bool)
        for i, row in enumerate(starts):
            ns[i, list(row)] = True
        d["new_starts"] = ns
    if lengths is not None:
        d["length"] = np.asarray(lengths, dtype=np.uint32)
    return d
