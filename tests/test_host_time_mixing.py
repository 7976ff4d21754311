"""CPU test of the host-side composition of RWKV-7 time mixing (jaxrwkv_b200/time_mixing.py): the token shift, the two
elementwise stages and the operator are replaced by oracle-backed fakes, so what is under test is everything the module
does itself - the projections, the parameter reshapes, the state packing, the first-layer branch - against the fixture
made by the reference's own time_mixing_seq."""
import numpy as np
import pytest
import torch

from oracle import time_mixing as otm
from oracle import token_shift as ots
from oracle.wkv7 import wkv7_base
from jaxrwkv_b200 import time_mixing as tm
from conftest import rel_err
from test_oracle import unflatten_params


def _np(x):
    return None if x is None else x.detach().double().numpy()


@pytest.fixture
def fakes(monkeypatch):
    def token_shift(x, prev, mix, length, new_starts):
        outs = [ots.token_shift(_np(x[i]), _np(prev[i]), _np(mix), int(length[i]), new_starts[i].numpy().astype(bool)) for i in range(x.shape[0])]
        mixed = torch.tensor(np.stack([o[0] for o in outs], axis=1))
        return mixed, torch.tensor(np.stack([o[1] for o in outs]))

    def mix_pre(k, wl, al, v, v_first, vl, w0, a0, v0, k_k, k_a, H, N=64):
        outs = [otm.mix_pre(_np(k[i]), _np(wl[i]), _np(al[i]), _np(v[i]), None if v_first is None else _np(v_first[i]),
                            None if vl is None else _np(vl[i]), _np(w0), _np(a0), _np(v0), _np(k_k), _np(k_a), H) for i in range(k.shape[0])]
        return tuple(torch.tensor(np.stack([o[j] for o in outs])) for j in range(5))

    def mix_post(y, r, k, v, g, ln_w, ln_b, r_k, H, N=64, eps=64e-5):
        return torch.tensor(np.stack([otm.mix_post(_np(y[i]), _np(r[i]), _np(k[i]), _np(v[i]), _np(g[i]), _np(ln_w), _np(ln_b), _np(r_k), H, eps)
                                      for i in range(y.shape[0])]))

    def inner_loop(cls, r, w, k, v, a, b, s, length, new_starts):
        outs = [wkv7_base(*[_np(x[i]) for x in (r, w, k, v, a, b, s)], int(length[i]), new_starts[i].numpy().astype(bool)) for i in range(r.shape[0])]
        return torch.tensor(np.stack([o[0] for o in outs])), torch.tensor(np.stack([o[1] for o in outs]))

    monkeypatch.setattr(tm, "token_shift", token_shift)
    monkeypatch.setattr(tm, "mix_pre", mix_pre)
    monkeypatch.setattr(tm, "mix_post", mix_post)
    monkeypatch.setattr(tm.CudaRWKV, "inner_loop", classmethod(inner_loop))


@pytest.mark.parametrize("layer_id", [0, 1])
def test_time_mixing_composition_matches_reference_fixture(golden, fakes, layer_id):
    g = golden("v7_time_mixing")
    to = lambda a: torch.as_tensor(np.asarray(a, dtype=np.float64))
    att = unflatten_params(g)
    att = {k: ({kk: to(vv) for kk, vv in v.items()} if isinstance(v, dict) else to(v)) for k, v in att.items()}
    H, S = int(g["H"]), int(g["S"])
    out, state, vf = tm.time_mixing_seq(to(g["in_x"]), to(g["in_state"]), to(g["in_v_first"]), att,
                                        torch.as_tensor(g["in_length"].astype(np.int64)), torch.as_tensor(g["in_new_starts"]), H, S, layer_id)
    assert rel_err(out.numpy(), g[f"out_l{layer_id}"].reshape(out.shape)) < 1e-11
    assert rel_err(state.numpy(), g[f"state_l{layer_id}"].reshape(state.shape)) < 1e-11
    assert rel_err(vf.numpy(), g[f"v_first_l{layer_id}"].reshape(vf.shape)) < 1e-12
