"""Generate the golden fixtures in this directory by running jaxrwkv's own
``inner_loop`` source.

    python tests/golden/make_golden.py --reference-src <jaxrwkv checkout>/src

JAX cannot be installed in the build image, so the reference modules
(src/jaxrwkv/rwkv{4,5,5_2,6,7}.py and llm.py, loaded unmodified from the
checkout) are executed against ``tests/golden/jax_standin`` — a NumPy
implementation of the handful of jax calls those functions make.  The package
``__init__`` of jaxrwkv (tokenizers, HuggingFace hub) is bypassed by registering
an empty package object and importing the version modules directly.

For every case the Base, Scan and AssociativeScan classes are all run in
float64 on float32-representable inputs; the Base and AssociativeScan results
are stored (Scan is asserted equal to Base and only its max deviation is
recorded).  Inputs are stored as float32, outputs as float64.
"""
import argparse
import importlib
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def load_reference(src):
    sys.path.insert(0, os.path.join(HERE, "jax_standin"))
    pkg = types.ModuleType("jaxrwkv")
    pkg.__path__ = [os.path.join(src, "jaxrwkv")]
    sys.modules["jaxrwkv"] = pkg
    return {v: importlib.import_module(f"jaxrwkv.rwkv{v}") for v in ("4", "5", "5_2", "6", "7")}


def f64(d, names):
    return [np.asarray(d[n], dtype=np.float64) for n in names]


def run_v7(mod, d):
    import jax.numpy as jnp
    out = {}
    B = d["r"].shape[0]
    for cls in ("BaseRWKV", "ScanRWKV", "AssociativeScanRWKV"):
        ss, ys = [], []
        for i in range(B):
            args = [jnp.asarray(x[i]) for x in f64(d, ["r", "w", "k", "v", "a", "b", "s0"])]
            s, y = getattr(mod, cls).inner_loop(*args, int(d["length"][i]), jnp.asarray(d["new_starts"][i]))
            ss.append(np.asarray(s)); ys.append(np.asarray(y))
        out[cls] = (np.stack(ss), np.stack(ys))
    return out


def run_v6(mod, d, version):
    import jax.numpy as jnp
    out = {}
    B = d["r"].shape[0]
    for cls in ("BaseRWKV", "ScanRWKV", "AssociativeScanRWKV"):
        ss, ys = [], []
        for i in range(B):
            r, k, v, s0 = [jnp.asarray(x[i]) for x in f64(d, ["r", "k", "v", "s0"])]
            w = np.asarray(d["w"], dtype=np.float64)
            w = jnp.asarray(w[i] if version == "6" else w)
            u = jnp.asarray(np.asarray(d["u"], dtype=np.float64))
            s, y = getattr(mod, cls).inner_loop(r, k, v, w, u, s0, int(d["length"][i]),
                                                jnp.asarray(d["new_starts"][i]))
            ss.append(np.asarray(s)); ys.append(np.asarray(y))
        out[cls] = (np.stack(ss), np.stack(ys))
    return out


def run_v4(mod, d):
    import jax.numpy as jnp
    out = {}
    B = d["r"].shape[0]
    for cls in ("BaseRWKV", "ScanRWKV", "AssociativeScanRWKV"):
        ss, ys = [], []
        for i in range(B):
            r, k, v, s0 = [jnp.asarray(x[i]) for x in f64(d, ["r", "k", "v", "s0"])]
            w, u = [jnp.asarray(x) for x in f64(d, ["w", "u"])]
            s, y = getattr(mod, cls).inner_loop(r, k, v, w, u, s0, int(d["length"][i]),
                                                jnp.asarray(d["new_starts"][i]))
            ss.append(np.asarray(s)); ys.append(np.asarray(y))
        out[cls] = (np.stack(ss), np.stack(ys))
    return out


def run_shift(mod, name, seed):
    """Token shift of RWKV-7 through the reference's own ``channel_mixing_seq`` (rwkv7.py:192-197).

    With identity key/value matrices the function returns ``relu(xk)**2``; inputs are positive and the
    mix lies in [0, 1], so ``xk >= 0`` and its square root is the shifted-and-mixed input itself.
    """
    import jax.numpy as jnp
    rng = np.random.default_rng(seed)
    B, T, D = 3, 19, 16
    x = rng.uniform(0.1, 2.0, (B, T, D)).astype(np.float32)
    prev = rng.uniform(0.1, 2.0, (B, D)).astype(np.float32)
    mix = rng.uniform(0.0, 1.0, (1, D)).astype(np.float32)
    ns = np.zeros((B, T), bool)
    ns[0, [0, 7]] = True; ns[1, [5, 6, 18]] = True
    length = np.asarray([19, 12, 0], dtype=np.uint32)
    eye = jnp.asarray(np.eye(D))
    xk, last = [], []
    for i in range(B):
        ffn = {"x_k": jnp.asarray(mix[0].astype(np.float64)), "key": {"weight": eye}, "value": {"weight": eye}}
        out, row = mod.BaseRWKV.channel_mixing_seq(jnp.asarray(x[i].astype(np.float64)), jnp.asarray(prev[i:i + 1].astype(np.float64)),
                                                   ffn, int(length[i]), jnp.asarray(ns[i]))
        xk.append(np.sqrt(np.asarray(out))); last.append(np.asarray(row))
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, in_x=x, in_prev=prev, in_mix=mix, in_new_starts=ns, in_length=length,
                        xk=np.stack(xk), last=np.stack(last))
    print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


def time_mixing_params(rng, C, H, lora=8):
    """Random parameters of one RWKV-7 attention block with the reference's names and shapes (rwkv7.py:222-266)."""
    u = lambda *shape, lo=-1.0, hi=1.0: rng.uniform(lo, hi, shape).astype(np.float32)
    sq = lambda: {"weight": (u(C, C) / np.sqrt(C)).astype(np.float32)}
    att = {n: u(1, 1, C, lo=0.0, hi=1.0) for n in ("x_r", "x_w", "x_k", "x_v", "x_a", "x_g")}
    att.update(receptance=sq(), key=sq(), value=sq(), output=sq())
    att.update(w0=u(1, 1, C, lo=-2.0, hi=1.0), w1=u(C, lora) / np.sqrt(C), w2=u(lora, C),
               a0=u(1, 1, C), a1=u(C, lora) / np.sqrt(C), a2=u(lora, C),
               v0=u(1, 1, C), v1=u(C, lora) / np.sqrt(C), v2=u(lora, C),
               g1=u(C, lora) / np.sqrt(C), g2=u(lora, C),
               k_k=u(1, 1, C, lo=0.5, hi=1.5), k_a=u(1, 1, C, lo=0.5, hi=1.5), r_k=u(H, C // H),
               ln_x={"weight": u(C, lo=0.5, hi=1.5), "bias": u(C)})
    return att


def flatten_params(att, prefix="p_"):
    out = {}
    for k, v in att.items():
        if isinstance(v, dict):
            out.update({f"{prefix}{k}.{kk}": vv for kk, vv in v.items()})
        else:
            out[prefix + k] = v
    return out


def run_time_mixing(mod, name, seed):
    """The whole time-mixing function of RWKV-7 (rwkv7.py:222-266) on random parameters, per sequence, for the first
    layer (the value stream passes through) and a later one (mixed with ``v_first``), in float64."""
    import jax.numpy as jnp
    rng = np.random.default_rng(seed)
    B, T, H, S = 3, 21, 2, 64
    C = H * S
    att = time_mixing_params(rng, C, H)
    x = rng.standard_normal((B, T, C)).astype(np.float32)
    state = (0.3 * rng.standard_normal((B, 1 + S, C))).astype(np.float32)
    v_first = rng.standard_normal((B, T, C)).astype(np.float32)
    ns = np.zeros((B, T), bool)
    ns[0, [0, 9]] = True; ns[1, [4, 5, 20]] = True
    length = np.asarray([21, 13, 21], dtype=np.uint32)
    to64 = lambda t: ({k: to64(v) for k, v in t.items()} if isinstance(t, dict) else jnp.asarray(np.asarray(t, np.float64)))
    att64 = to64(att)
    arrays = dict(in_x=x, in_state=state, in_v_first=v_first, in_new_starts=ns, in_length=length, H=np.int64(H), S=np.int64(S))
    arrays.update(flatten_params(att))
    for layer_id in (0, 1):
        outs, states, vfs = [], [], []
        for i in range(B):
            o, st, vf = mod.BaseRWKV.time_mixing_seq(to64(x[i]), to64(state[i]), to64(v_first[i]), att64, int(length[i]),
                                                     jnp.asarray(ns[i]), H, S, layer_id)
            outs.append(np.asarray(o)); states.append(np.asarray(st)); vfs.append(np.asarray(vf))
        arrays.update({f"out_l{layer_id}": np.stack(outs), f"state_l{layer_id}": np.stack(states),
                       f"v_first_l{layer_id}": np.stack(vfs)})
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


def save(name, d, res):
    base_s, base_y = res["BaseRWKV"]
    scan_s, scan_y = res["ScanRWKV"]
    dev = max(np.abs(scan_s - base_s).max(), np.abs(scan_y - base_y).max())
    assert dev < 1e-9, (name, dev)
    arrays = {f"in_{k}": v for k, v in d.items()}
    arrays.update(base_s=base_s, base_y=base_y, assoc_s=res["AssociativeScanRWKV"][0],
                  assoc_y=res["AssociativeScanRWKV"][1], scan_vs_base_maxdev=np.float64(dev))
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}: scan-vs-base {dev:.2e}, {os.path.getsize(path) / 1024:.0f} KiB")


def set_starts(d, starts, lengths):
    ns = np.zeros_like(d["new_starts"])
    for i, row in enumerate(starts):
        ns[i, list(row)] = True
    d["new_starts"] = ns
    d["length"] = np.asarray(lengths, dtype=np.uint32)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-src", required=True, help="path to the jaxrwkv checkout's src/ directory")
    a = ap.parse_args()
    mods = load_reference(a.reference_src)
    sys.path.insert(0, ROOT)
    from oracle.inputs import make_wkv7_inputs, make_wkv6_inputs, make_wkv4_inputs

    # RWKV-7 -----------------------------------------------------------------------------
    d = make_wkv7_inputs(2, 40, 2, 64, seed=101)                      # config-1 style: start at t=0 only
    save("v7_plain", d, run_v7(mods["7"], d))
    d = make_wkv7_inputs(3, 48, 1, 64, seed=102, s0_scale=0.5)
    # row 0: carried state (no start at 0), adjacent starts, length lands on a start (state quirk)
    # row 1: start at 0 and mid-sequence, length mid-chunk; row 2: length == 0
    set_starts(d, [(17, 18, 30), (0, 16, 33), (5,)], [30, 41, 0])
    save("v7_resets", d, run_v7(mods["7"], d))
    d = make_wkv7_inputs(2, 21, 3, 8, seed=103, s0_scale=1.0)         # small head size, oracle-only
    set_starts(d, [(0, 7), (3, 20)], [21, 13])
    save("v7_small", d, run_v7(mods["7"], d))

    run_shift(mods["7"], "v7_token_shift", 104)
    run_time_mixing(mods["7"], "v7_time_mixing", 105)

    # RWKV-6 / 5.2 / 5 -------------------------------------------------------------------
    for version, seed in (("6", 201), ("5_2", 202), ("5", 203)):
        d = make_wkv6_inputs(2, 40, 2, 64, seed=seed, s0_scale=0.5, version=version)
        set_starts(d, [(11, 12, 25), (0,)], [25, 33])
        save(f"v{version}_resets", d, run_v6(mods[version], d, version))

    # RWKV-4 -----------------------------------------------------------------------------
    d = make_wkv4_inputs(2, 40, 128, seed=301, default_state=True)
    set_starts(d, [(0,), (9, 10, 31)], [40, 31])
    save("v4_default_state", d, run_v4(mods["4"], d))
    d = make_wkv4_inputs(2, 33, 128, seed=302, default_state=False)
    set_starts(d, [(), (20,)], [0, 27])
    save("v4_carried_state", d, run_v4(mods["4"], d))


if __name__ == "__main__":
    main()
