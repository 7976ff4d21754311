"""CPU tests of the work split of the tensor-core backward: which thread block walks which piece of
which sequence, and in what order (the order is what keeps the hand-over waits free of cycles)."""
import ctypes

import pytest

from jaxrwkv_b200 import _lib


def _runs(lib, chains, seg, grid, cta):
    buf = (ctypes.c_int * (3 * 64))()
    n = lib.b200wkv_debug_runs(chains, seg, grid, cta, buf, 64)
    assert 0 < n <= 64
    return [(buf[3 * i], buf[3 * i + 1], buf[3 * i + 2]) for i in range(n)]


@pytest.mark.parametrize("chains,seg,grid", [(256, 4, 148), (185, 4, 148), (149, 8, 148), (1000, 2, 148),
                                             (296, 1, 148), (7, 1, 7), (300, 8, 296), (513, 4, 512)])
def test_every_segment_is_walked_once_and_waits_cannot_cycle(chains, seg, grid):
    lib = _lib.load()
    seen = {}
    for cta in range(grid):
        runs = _runs(lib, chains, seg, grid, cta)
        partial_head = [r for r in runs if r[1] > 0]      # begins inside a sequence: takes a carry from cta - 1
        partial_tail = [r for r in runs if r[2] < seg]    # ends inside a sequence: hands a carry to cta + 1
        assert len(partial_head) <= 1 and len(partial_tail) <= 1
        if partial_tail:
            assert runs[0] == partial_tail[0]             # produced before anything that might wait
        if partial_head:
            assert runs[-1] == partial_head[0]            # consumed last
        assert len({r[0] for r in runs}) == len(runs)     # one run per sequence
        for chain, a, b in runs:
            assert 0 <= chain < chains and 0 <= a < b <= seg
            for j in range(a, b):
                assert (chain, j) not in seen
                seen[(chain, j)] = cta
    assert len(seen) == chains * seg
    # the piece that continues a sequence belongs to the next thread block, segments in order
    for (chain, j), cta in seen.items():
        if j > 0:
            assert seen[(chain, j - 1)] in (cta, cta - 1)


def test_split_is_chosen_only_when_it_shortens_the_schedule():
    lib = _lib.load()
    g, s = ctypes.c_int(), ctypes.c_int()

    def plan(chains, n_blk, per_sm=1):
        assert lib.b200wkv_debug_split_plan(chains, n_blk, per_sm, ctypes.byref(g), ctypes.byref(s)) == 0
        return g.value, s.value

    assert plan(64, 64) == (64, 1)            # fewer sequences than SMs: one thread block each
    sms = plan(10 ** 6, 64)[0]                # the grid of a saturated launch is the SM count
    assert plan(2 * sms, 64) == (sms, 1)      # divides evenly: whole sequences, no hand-over
    grid, seg = plan(sms + sms // 2 + 7, 64)
    assert grid == sms and seg in (2, 4, 8)
    assert plan(sms + 1, 1)[1] == 1           # a single block cannot be cut
    chains = 256 if sms == 148 else sms + sms // 2 + 7
    grid, seg = plan(chains, 64)
    units = -(-chains * seg // grid)
    assert units / seg < -(-chains // grid)   # strictly shorter than whole-sequence waves
