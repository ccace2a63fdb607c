"""Pins the CPU oracle against outputs of the reference itself.

Golden fixtures (tests/golden/*.npz) were produced by tests/golden/make_golden.py
from the reference's host C++ functions and Python quantisers.  Where the
compiled reference shim (oracle/_ref/libmoe_ref.so) is available it is also
called directly on fresh inputs.
"""
import os

import numpy as np
import pytest


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_e4m3_decode_table(orc, golden_dir):
    g = _load(golden_dir, "codec.npz")
    got = orc.e4m3_decode(np.arange(256, dtype=np.uint8))
    want = g["e4m3_decode"]
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(got)], want[~np.isnan(want)])
    assert got[0x7E] == 448.0 and got[0x38] == 1.0 and got[0x01] == 2.0 ** -9


def test_e4m3_quantize_sweep(orc, golden_dir):
    g = _load(golden_dir, "codec.npz")
    got = orc.e4m3_quantize(g["q_in"])
    assert np.array_equal(got, g["q_out"])


def test_e4m3_quantize_is_rne_of_decode(orc):
    """Every finite code point quantises to itself; midpoints go to the even code."""
    codes = np.array([b for b in range(256) if (b & 0x7F) != 0x7F], np.uint8)
    vals = orc.e4m3_decode(codes)
    back = orc.e4m3_quantize(vals)
    same = (back == codes) | ((vals == 0) & ((back & 0x7F) == 0))
    assert same.all()
    pos = np.array(sorted(set(vals[vals >= 0].tolist())), np.float32)
    mid = (pos[:-1].astype(np.float64) + pos[1:].astype(np.float64)) / 2
    qm = orc.e4m3_quantize(mid.astype(np.float32))
    assert (qm % 2 == 0).all()


def test_bf16_rne(orc, golden_dir):
    g = _load(golden_dir, "codec.npz")
    assert np.array_equal(orc.f32_to_bf16(g["bf16_in"]), g["bf16_out"])


def test_python_quantisers(orc, golden_dir):
    g = _load(golden_dir, "quant_py.npz")
    q, sf = orc.quant_rows_1x128(g["x"])
    assert np.array_equal(sf, g["xsf"])
    assert np.array_equal(q, g["xq"])
    wq, wsf = orc.quant_blocks_128x128(g["w"])
    assert np.array_equal(wsf, g["wsf"])
    assert np.array_equal(wq, g["wq"])
    back = orc.dequant_rows_1x128(g["xq"], g["xsf"])
    assert np.array_equal(back, g["back"])
    L = orc.lib()
    ce = np.array([L.orc_ue8m0_to_f32(L.orc_ue8m0_ceil(float(v))) for v in g["ceil_in"]], np.float32)
    assert np.array_equal(ce, g["ceil_out"])


def test_l1_l2_reduce_reference_mode(orc, golden_dir):
    """ref_l1 -> ref_quantize_fp8 -> ref_l2 -> ref_reduce of the reference on its own
    fixtures (WPROBE weights seeds 17/91, x byte pattern) at H=6144, I=2048."""
    g = _load(golden_dir, "numeric_ref_mode.npz")
    x = g["x"]
    H = x.shape[1]
    I = g["ffn_expect"].shape[1]
    EPR = 8
    e = int(g["expert"])
    w1 = orc.fill_weights(EPR * 2 * I, H, 17).reshape(EPR, 2 * I, H)[e]
    w2 = orc.fill_weights(EPR * H, I, 91).reshape(EPR, H, I)[e]
    h = orc.l1(x, None, w1, None)
    # same FP32 sequential order, only exp() may differ in the last ulp
    assert np.allclose(h, g["ffn_expect"], rtol=2e-6, atol=0)
    q, _ = orc.requant(g["ffn_expect"], scaled=False)
    assert np.array_equal(q, g["ffn_q"])
    out = orc.l2(g["ffn_q"], None, w2, None)
    assert np.array_equal(out, g["out_expect"])
    y = orc.reduce_all(g["comb"], g["tidx"], g["tw"], 2, int(g["E"]))
    assert np.array_equal(y, g["y"])


def test_make_routes_patterns(orc, golden_dir):
    g = _load(golden_dir, "routes.npz")
    for key in g.files:
        name, rank, R, tok, salt = key.split("_")
        pat = {"balanced": "balanced", "hot": "hot", "mixed": "mixed-invalid"}[name]
        # fixture generator is parameterised on the world; pick this rank's rows
        case_idx = orc.gen_reference_fixture(int(R), 8, 8, 128, 128, int(tok), pat, int(salt)).topk_idx
        assert np.array_equal(case_idx[int(rank), : int(tok)].reshape(-1), g[key]), key


def test_schedulers(orc, golden_dir):
    g = _load(golden_dir, "sched.npz")
    consts = g["consts"]
    EPR, GR, grid, nslice, ring = int(consts[0]), int(consts[4]), int(consts[6]), int(consts[7]), int(consts[8])
    L = orc.lib()
    for ci in range(6):
        for win in (32, 64, 128):
            for m in range(GR):
                cg = np.ascontiguousarray(g[f"gs_{ci}_{win}_{m}_cg"])
                ge = np.zeros(512, np.int32)
                w = np.zeros(512, np.int32)
                n = L.orc_gs_schedule_member(cg, EPR, GR, win, m, ge, w, 512)
                assert n == g[f"gs_{ci}_{win}_{m}_ge"].size
                assert np.array_equal(ge[:n], g[f"gs_{ci}_{win}_{m}_ge"])
                assert np.array_equal(w[:n], g[f"gs_{ci}_{win}_{m}_w"])
        counts = np.ascontiguousarray(g[f"win_{ci}_counts"])
        got = np.array([L.orc_select_win(counts, 256, cap, wmin, nslice, grid, ring)
                        for cap in (64, 96, 128) for wmin in (8, 32)], np.int32)
        assert np.array_equal(got, g[f"win_{ci}_out"])
        ci32 = counts.astype(np.int32)
        for grp in (0, 5):
            experts = np.arange(grp * 32, grp * 32 + 32, dtype=np.int32)
            st = np.zeros((32 * 64 * 4, 3), np.int32)
            mo = np.zeros(32 * 64 * 4, np.int32)
            ld = np.zeros(4, np.int64)
            n = L.orc_lpt_assign(ci32, experts, 32, 64, 4, 4, st.reshape(-1), mo, ld)
            assert np.array_equal(st[:n], g[f"lpt_{ci}_{grp}_tasks"])
            assert np.array_equal(mo[:n], g[f"lpt_{ci}_{grp}_member"])
            assert np.array_equal(ld, g[f"lpt_{ci}_{grp}_load"])


def test_against_compiled_reference(orc):
    """Direct call of the compiled reference functions on fresh seeded inputs."""
    R = orc.ref_lib()
    if R is None:
        pytest.skip("oracle/_ref/libmoe_ref.so not built (reference tree absent at build time)")
    H, I, EPR = R.ref_const(2), R.ref_const(3), R.ref_const(0)
    rng = np.random.default_rng(3)
    # random logical weights with a sprinkling of negative / large codes
    w1 = rng.integers(0, 0x7E, (2 * I, H)).astype(np.uint8) | (rng.integers(0, 2, (2 * I, H)).astype(np.uint8) << 7)
    w1 = (w1 & 0xBF).astype(np.uint8)          # keep magnitudes < 2 so sums stay tame
    x = (rng.integers(0, 0x40, (2, H)).astype(np.uint8) | (rng.integers(0, 2, (2, H)).astype(np.uint8) << 7))
    h_idx = np.arange(I)
    grow = (h_idx // 256) * 512 + h_idx % 256
    paired = np.empty_like(w1)
    paired[grow] = w1[:I]
    paired[grow + 256] = w1[I:]
    lane = np.zeros((EPR, 2 * I * H), np.uint8)
    R.ref_pack_lane(np.ascontiguousarray(paired), 2 * I, H, lane[1])
    want = np.zeros((2, I), np.float32)
    R.ref_l1_rows(x, lane.reshape(-1), 1, 2, want.reshape(-1), 4)
    got = orc.l1(x, None, w1, None)
    assert np.allclose(got, want, rtol=2e-6, atol=1e-30)
    # scale planes of all-127 (x1.0) change only the summation grouping
    got_s = orc.l1(x, np.full((2, H // 128), 127, np.uint8), w1, np.full((2 * I // 128, H // 128), 127, np.uint8))
    assert orc.rel_l2(got_s, want) < 1e-5
    # codec spot checks
    for v in (0.3, -17.0, 500.0, 1e-3):
        assert R.ref_e4m3_quantize(v) == orc.lib().orc_e4m3_quantize(v)


def test_recorded_route_corpus_replay(orc, golden_dir):
    """routes_from_counts (reference: test/mega_common.cuh:460-482) on the sampled launches of the
    real-decode corpus: the routes reproduce the recorded per-expert counts exactly (the
    reference's route_count_deviation == 0, :485-495), no token names an expert twice, and the
    prologue restatement then reports the same received counts on every owner rank."""
    g = _load(golden_dir, "tk_info.npz")
    R, EPR, topk = 8, 32, 8
    for counts in g["counts"]:
        tokens = int(counts.sum()) // (R * topk)
        routes = orc.routes_from_counts(counts, R, tokens, topk)
        assert routes.shape == (R, tokens, topk)
        assert np.array_equal(np.bincount(routes.reshape(-1), minlength=R * EPR), counts)
        srt = np.sort(routes, axis=2)
        assert not (srt[:, :, 1:] == srt[:, :, :-1]).any()
        case = orc.with_routes(orc.gen_case(R, EPR, topk, 128, 128, tokens, seed=3, scaled=False), routes)
        ref = orc.route_world(case)
        for r in range(R):
            assert np.array_equal(ref[r].prefix_tbl[:, R], counts[r * EPR:(r + 1) * EPR])
    with pytest.raises(ValueError):
        orc.routes_from_counts(g["counts"][0], R, 63, topk)
