"""CPU tests: the restated recurrences against the fixtures produced by running
jaxrwkv's own inner_loop source (tests/golden/make_golden.py), and the explicit
reverse loops against torch.autograd."""
import numpy as np
import pytest
import torch

import oracle
from oracle import torch_ref
from conftest import rel_err

TOL = 1e-12


def _inputs(g, names):
    return [np.asarray(g["in_" + n], dtype=np.float64) for n in names]


@pytest.mark.parametrize("case", ["v7_plain", "v7_resets", "v7_small"])
def test_wkv7_matches_reference_fixtures(golden, case):
    g = golden(case)
    args = _inputs(g, ["r", "w", "k", "v", "a", "b", "s0"])
    length, ns = g["in_length"], g["in_new_starts"]
    s, y = oracle.wkv7_base_batched(*args, length, ns)
    assert rel_err(y, g["base_y"]) < TOL and rel_err(s, g["base_s"]) < TOL
    s2, y2 = oracle.wkv7_assoc_batched(*args, length, ns)
    assert rel_err(y2, g["assoc_y"]) < 1e-10 and rel_err(s2, g["assoc_s"]) < 1e-10


def test_wkv7_assoc_quirk_positions(golden):
    """AssociativeScan == Base except y[t-1] where new_starts[t], and the state when
    new_starts[length]; there the associative scan returns exact zeros."""
    g = golden("v7_resets")
    for i in range(g["in_r"].shape[0]):
        ym, sd = oracle.quirk_mask(g["in_new_starts"][i], int(g["in_length"][i]))
        assert rel_err(g["assoc_y"][i][~ym], g["base_y"][i][~ym]) < 1e-10
        assert np.all(g["assoc_y"][i][ym] == 0)
        if sd:
            assert np.all(g["assoc_s"][i] == 0)
        else:
            assert rel_err(g["assoc_s"][i], g["base_s"][i]) < 1e-10
    assert oracle.quirk_mask(g["in_new_starts"][0], int(g["in_length"][0]))[1]   # row 0 exercises it
    assert int(g["in_length"][2]) == 0 and np.array_equal(g["base_s"][2], g["in_s0"][2].astype(np.float64))


@pytest.mark.parametrize("version", ["6", "5_2", "5"])
def test_wkv6_family_matches_reference_fixtures(golden, version):
    g = golden(f"v{version}_resets")
    r, k, v, w, u, s0 = _inputs(g, ["r", "k", "v", "w", "u", "s0"])
    length, ns = g["in_length"], g["in_new_starts"]
    s, y = oracle.wkv6_base_batched(r, k, v, w, u, s0, length, ns, version)
    assert rel_err(y, g["base_y"]) < TOL and rel_err(s, g["base_s"]) < TOL
    for i in range(r.shape[0]):
        s2, y2 = oracle.wkv6_assoc(r[i], k[i], v[i], w[i] if version == "6" else w, u, s0[i],
                                   length[i], ns[i], version)
        assert rel_err(y2, g["assoc_y"][i]) < 1e-10 and rel_err(s2, g["assoc_s"][i]) < 1e-10


@pytest.mark.parametrize("case", ["v4_default_state", "v4_carried_state"])
def test_wkv4_matches_reference_fixtures(golden, case):
    g = golden(case)
    r, k, v, w, u, s0 = _inputs(g, ["r", "k", "v", "w", "u", "s0"])
    length, ns = g["in_length"], g["in_new_starts"]
    s, y = oracle.wkv4_base_batched(r, k, v, w, u, s0, length, ns)
    assert rel_err(y, g["base_y"]) < TOL and rel_err(s, g["base_s"]) < TOL
    for i in range(r.shape[0]):
        s2, y2 = oracle.wkv4_assoc(r[i], k[i], v[i], w, u, s0[i], length[i], ns[i])
        assert rel_err(y2, g["assoc_y"][i]) < 1e-10
        assert rel_err(s2[:2], g["assoc_s"][i][:2]) < 1e-10 and rel_err(s2[2], g["assoc_s"][i][2]) < 1e-10


def test_associative_scan_equals_left_fold():
    rng = np.random.default_rng(0)
    for n in (1, 2, 3, 7, 8, 33):
        A = rng.standard_normal((n, 3, 3))
        out, = oracle.associative_scan(lambda a, b: (a[0] @ b[0],), (A,))
        acc = A[0]
        for i in range(n):
            acc = A[0] if i == 0 else acc @ A[i]
            assert np.allclose(out[i], acc, rtol=1e-12, atol=1e-12)


def _t(x):
    return torch.tensor(np.asarray(x, dtype=np.float64), requires_grad=True)


def test_wkv7_reverse_loop_matches_autograd():
    d = oracle.make_wkv7_inputs(1, 20, 2, 8, seed=7, s0_scale=1.0, dtype=np.float64)
    ns = np.zeros(20, dtype=bool); ns[[7, 8, 15]] = True
    rng = np.random.default_rng(1)
    dy = rng.standard_normal((20, 2, 8)); ds = rng.standard_normal((2, 8, 8))
    for length in (13, 20, 0, 8, 25):
        names = ["r", "w", "k", "v", "a", "b", "s0"]
        ts = [_t(d[n][0]) for n in names]
        s_out, y = torch_ref.wkv7_base_torch(*ts, length, torch.tensor(ns))
        ((y * torch.tensor(dy)).sum() + (s_out * torch.tensor(ds)).sum()).backward()
        got = oracle.wkv7_bwd(*[d[n][0] for n in names], length, ns, dy, ds)
        for g_, t_, n in zip(got, ts, names):
            assert rel_err(g_, t_.grad.numpy()) < 1e-11, (n, length)


@pytest.mark.parametrize("version", ["6", "5_2", "5"])
def test_wkv6_reverse_loop_matches_autograd(version):
    d = oracle.make_wkv6_inputs(1, 18, 2, 8, seed=9, s0_scale=1.0, version=version, dtype=np.float64)
    ns = np.zeros(18, dtype=bool); ns[[5, 6, 12]] = True
    rng = np.random.default_rng(2)
    dy = rng.standard_normal((18, 2, 8)); ds = rng.standard_normal((2, 8, 8))
    for length in (11, 18, 0, 23):
        r, k, v, s0 = [_t(d[n][0]) for n in ["r", "k", "v", "s0"]]
        w = _t(d["w"][0] if version == "6" else d["w"]); u = _t(d["u"])
        s_out, y = torch_ref.wkv6_base_torch(r, k, v, w, u, s0, length, torch.tensor(ns), version)
        ((y * torch.tensor(dy)).sum() + (s_out * torch.tensor(ds)).sum()).backward()
        got = oracle.wkv6_bwd(d["r"][0], d["k"][0], d["v"][0], d["w"][0] if version == "6" else d["w"],
                              d["u"], d["s0"][0], length, ns, dy, ds, version)
        for g_, t_, n in zip(got, [r, k, v, w, u, s0], "r k v w u s0".split()):
            assert rel_err(g_, t_.grad.numpy()) < 1e-11, (n, length)


def test_torch_restatements_match_numpy():
    d = oracle.make_wkv7_inputs(1, 24, 2, 16, seed=3, s0_scale=0.3, dtype=np.float64)
    ns = np.zeros(24, dtype=bool); ns[[0, 9]] = True
    names = ["r", "w", "k", "v", "a", "b", "s0"]
    s_np, y_np = oracle.wkv7_assoc(*[d[n][0] for n in names], 20, ns)
    s_t, y_t = torch_ref.wkv7_assoc_torch(*[torch.tensor(d[n][0]) for n in names], 20, torch.tensor(ns))
    assert rel_err(y_t.numpy(), y_np) < 1e-11 and rel_err(s_t.numpy(), s_np) < 1e-11
    d4 = oracle.make_wkv4_inputs(1, 17, 32, seed=4, default_state=False, dtype=np.float64)
    s_np, y_np = oracle.wkv4_base(d4["r"][0], d4["k"][0], d4["v"][0], d4["w"], d4["u"], d4["s0"][0], 12, ns[:17])
    s_t, y_t = torch_ref.wkv4_base_torch(*[torch.tensor(x) for x in (d4["r"][0], d4["k"][0], d4["v"][0], d4["w"], d4["u"], d4["s0"][0])], 12, torch.tensor(ns[:17]))
    assert rel_err(y_t.numpy(), y_np) < 1e-12 and rel_err(s_t.numpy(), s_np) < 1e-12


def test_token_shift_matches_reference_fixture(golden):
    """Fixture made by the reference's own channel_mixing_seq with identity matrices (make_golden.run_shift)."""
    from oracle import token_shift as ts
    g = golden("v7_token_shift")
    for i in range(g["in_x"].shape[0]):
        mixed, last = ts.token_shift(g["in_x"][i].astype(np.float64), g["in_prev"][i].astype(np.float64),
                                     g["in_mix"].astype(np.float64), int(g["in_length"][i]), g["in_new_starts"][i])
        assert rel_err(mixed[0], g["xk"][i]) < 1e-12
        np.testing.assert_array_equal(last, g["last"][i])


def unflatten_params(g, prefix="p_"):
    """The parameter dict of tests/golden/make_golden.flatten_params, rebuilt (float64)."""
    att = {}
    for key, val in g.items():
        if not key.startswith(prefix):
            continue
        name = key[len(prefix):]
        val = np.asarray(val, dtype=np.float64)
        if "." in name:
            outer, inner = name.split(".")
            att.setdefault(outer, {})[inner] = val
        else:
            att[name] = val
    return att


@pytest.mark.parametrize("layer_id", [0, 1])
def test_time_mixing_matches_reference_fixture(golden, layer_id):
    """Fixture made by the reference's own time_mixing_seq (make_golden.run_time_mixing): the token shift, the
    elementwise stages on both sides of the operator and the operator, composed as rwkv7.py:222-266 composes them."""
    from oracle import time_mixing as tm
    g = golden("v7_time_mixing")
    att = unflatten_params(g)
    H, S = int(g["H"]), int(g["S"])
    for i in range(g["in_x"].shape[0]):
        out, state, vf = tm.time_mixing_seq(g["in_x"][i].astype(np.float64), g["in_state"][i].astype(np.float64),
                                            g["in_v_first"][i].astype(np.float64), att, int(g["in_length"][i]),
                                            g["in_new_starts"][i], H, S, layer_id)
        assert rel_err(out, g[f"out_l{layer_id}"][i]) < 1e-11
        assert rel_err(state, g[f"state_l{layer_id}"][i]) < 1e-11
        assert rel_err(vf, g[f"v_first_l{layer_id}"][i]) < 1e-12
