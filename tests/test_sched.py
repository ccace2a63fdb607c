"""The skew-aware schedulers of the product library (mini_mega_b200/csrc/mxk_sched.cuh through the
C ABI) against the schedules recorded from the reference's own functions (tests/golden/sched.npz:
gs_schedule_member of src/group_sched.cuh:164-205, lpt_assign of src/balance_partition.cuh:62-115):
exact on the host, and the device evaluation of the same source must agree with the host."""
import ctypes as C
import os

import numpy as np
import pytest

from mini_mega_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
I32 = C.POINTER(C.c_int32)


def _p(a):
    return a.ctypes.data_as(I32)


@pytest.fixture(scope="module")
def lib():
    _lib.build()
    return _lib.lib()


@pytest.fixture(scope="module")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "sched.npz"))


def test_member_windows_match_reference_schedules(lib, golden):
    g = golden
    EPR, GR = int(g["consts"][0]), int(g["consts"][4])
    assert lib.mxk_group_ranks() == GR
    for ci in range(6):
        for win in (32, 64, 128):
            for m in range(GR):
                cg = np.ascontiguousarray(g[f"gs_{ci}_{win}_{m}_cg"])
                ge, w = np.zeros(512, np.int32), np.zeros(512, np.int32)
                n = lib.mxk_gs_schedule_member(_p(cg), EPR, GR, win, m, _p(ge), _p(w), 512)
                assert n == g[f"gs_{ci}_{win}_{m}_ge"].size
                assert np.array_equal(ge[:n], g[f"gs_{ci}_{win}_{m}_ge"]) and np.array_equal(w[:n], g[f"gs_{ci}_{win}_{m}_w"])
    # every window of the group lands on exactly one member; run-time group sizes other than the reference's 4
    rng = np.random.default_rng(0)
    for gr, epr, win in ((2, 32, 128), (8, 4, 64), (1, 8, 32)):
        cg = rng.integers(0, 700, gr * epr).astype(np.int32)
        seen = set()
        for m in range(gr):
            ge, w = np.zeros(4096, np.int32), np.zeros(4096, np.int32)
            n = lib.mxk_gs_schedule_member(_p(cg), epr, gr, win, m, _p(ge), _p(w), 4096)
            for i in range(n):
                assert (int(ge[i]), int(w[i])) not in seen
                seen.add((int(ge[i]), int(w[i])))
        assert len(seen) == int(sum((int(c) + win - 1) // win for c in cg))


def test_skew_test_and_bad_arguments(lib):
    flat = np.full(32, 10, np.int32)
    hot = flat.copy()
    hot[3] = 400
    assert lib.mxk_gs_group_skewed(_p(flat), 32, 2) == 0
    assert lib.mxk_gs_group_skewed(_p(hot), 32, 2) == 1
    assert lib.mxk_gs_group_skewed(_p(flat), 32, 0) == 1      # skew_num 0: always on
    out = np.zeros(8, np.int32)
    assert lib.mxk_gs_schedule_member(_p(flat), 8, 4, 128, 4, _p(out), _p(out), 8) == -1   # member outside the group
    assert lib.mxk_gs_schedule_member(_p(flat), 8, 17, 128, 0, _p(out), _p(out), 8) == -1  # group too large


def test_lpt_assign_matches_reference(lib, golden):
    g = golden
    for ci in range(6):
        counts = g[f"win_{ci}_counts"].astype(np.int32)
        for grp in (0, 5):
            experts = np.arange(grp * 32, grp * 32 + 32, dtype=np.int32)
            tasks, mo, ld = np.zeros((8192, 3), np.int32), np.zeros(8192, np.int32), np.zeros(4, np.int64)
            n = lib.mxk_lpt_assign(_p(counts), _p(experts), 32, 64, 4, 4, _p(tasks), _p(mo),
                                   ld.ctypes.data_as(C.POINTER(C.c_int64)), 8192)
            assert np.array_equal(tasks[:n], g[f"lpt_{ci}_{grp}_tasks"])
            assert np.array_equal(mo[:n], g[f"lpt_{ci}_{grp}_member"])
            assert np.array_equal(ld, g[f"lpt_{ci}_{grp}_load"])


@pytest.mark.gpu
def test_device_schedule_equals_host_schedule(lib, golden):
    g = golden
    EPR, GR = int(g["consts"][0]), int(g["consts"][4])
    for ci in (1, 3, 5):
        for win in (32, 128):
            cg = np.ascontiguousarray(g[f"gs_{ci}_{win}_0_cg"])
            ge, w, n = np.zeros((GR, 512), np.int32), np.zeros((GR, 512), np.int32), np.zeros(GR, np.int32)
            _lib.check(lib.mxk_gs_schedule_on_device(_p(cg), EPR, GR, win, 0, _p(ge), _p(w), _p(n), 512))
            for m in range(GR):
                assert n[m] == g[f"gs_{ci}_{win}_{m}_ge"].size
                assert np.array_equal(ge[m, : n[m]], g[f"gs_{ci}_{win}_{m}_ge"])
                assert np.array_equal(w[m, : n[m]], g[f"gs_{ci}_{win}_{m}_w"])
            # the hot-expert variant: device == host == the oracle's restatement
            for hot in (2, 3):
                _lib.check(lib.mxk_gs_schedule_on_device(_p(cg), EPR, GR, win, hot, _p(ge), _p(w), _p(n), 512))
                for m in range(GR):
                    hg, hw = np.zeros(512, np.int32), np.zeros(512, np.int32)
                    hn = lib.mxk_gs_schedule_member_hot(_p(cg), EPR, GR, win, m, hot, _p(hg), _p(hw), 512)
                    assert n[m] == hn and np.array_equal(ge[m, :hn], hg[:hn]) and np.array_equal(w[m, :hn], hw[:hn])


def test_hot_expert_schedule(lib):
    """Spreading limited to hot experts: 0 is the reference's schedule; otherwise every window of an
    expert with fewer windows than the limit stays with its owner, every window of the group lands on
    exactly one member, the product function agrees with the oracle's restatement, and the hottest
    member's cost does not grow against leaving everything with the owners."""
    from oracle import oracle as orc
    O = orc.lib()
    rng = np.random.default_rng(7)
    for gr, epr, win in ((4, 8, 128), (8, 32, 128), (2, 16, 32)):
        cg = (rng.zipf(1.3, gr * epr) * 20).clip(0, 3000).astype(np.int32)
        cost = lambda rows: (rows + 15) // 16                       # noqa: E731
        wins = lambda c: [min(win, c - w * win) for w in range((c + win - 1) // win)]   # noqa: E731
        own_cost = [sum(cost(r) for le in range(epr) for r in wins(int(cg[m * epr + le]))) for m in range(gr)]
        for hot in (0, 2, 3, 5):
            seen, loads = {}, []
            for m in range(gr):
                ge, w = np.zeros(8192, np.int32), np.zeros(8192, np.int32)
                n = lib.mxk_gs_schedule_member_hot(_p(cg), epr, gr, win, m, hot, _p(ge), _p(w), 8192)
                oge, ow = np.zeros(8192, np.int32), np.zeros(8192, np.int32)
                on = O.orc_gs_schedule_member_hot(cg, epr, gr, win, m, hot, oge, ow, 8192)
                assert n == on and np.array_equal(ge[:n], oge[:n]) and np.array_equal(w[:n], ow[:n])
                if hot == 0:
                    rge, rw = np.zeros(8192, np.int32), np.zeros(8192, np.int32)
                    rn = lib.mxk_gs_schedule_member(_p(cg), epr, gr, win, m, _p(rge), _p(rw), 8192)
                    assert rn == n and np.array_equal(rge[:n], ge[:n]) and np.array_equal(rw[:n], w[:n])
                load = 0
                for i in range(n):
                    key = (int(ge[i]), int(w[i]))
                    assert key not in seen
                    seen[key] = m
                    c = int(cg[ge[i]])
                    load += cost(min(win, c - int(w[i]) * win))
                    if hot > 0 and (c + win - 1) // win < hot:
                        assert int(ge[i]) // epr == m, "a cold expert's window left its owner"
                loads.append(load)
            assert len(seen) == int(sum((int(c) + win - 1) // win for c in cg))
            assert max(loads) <= max(own_cost)
    out = np.zeros(8, np.int32)
    assert lib.mxk_gs_schedule_member_hot(_p(np.zeros(32, np.int32)), 8, 4, 128, 0, -1, _p(out), _p(out), 8) == -1
