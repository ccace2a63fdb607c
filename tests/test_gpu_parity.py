"""Parity of the CUDA path against the CPU oracle, called through the C ABI.

Tolerances (stated by the reference's own checker and the build target):
  * routing tables, dispatch layout, counts/offsets, pool bytes: bit-exact
    (reference: test/check.cu:183-195);
  * L1 output, decoded from FP8: |d| <= max(2e-3*scale, 7e-2*|want|) (test/check.cu:409);
  * L2 output (bf16 rows given the device's own FP8 hidden): rel 1e-2 / abs 1e-3
    (test/check.cu:433);
  * reduce given the device's own bf16 rows: bit-exact here (reference allows
    rel 1e-5 / abs 1e-6, test/check.cu:473);
  * end-to-end y: max relative L2 error per token <= 1e-2 against the oracle.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _stage_checks(world, ref, r, scaled):
    """Per-phase comparison on rank r, each phase fed with the device's own input."""
    case = world.case
    s = ref[r]
    rows = s.meta.shape[0]
    H, I, EPR = case.H, case.I, case.EPR
    # dispatch: pool bytes, scales and staged (src, token, k, weight)
    meta = world.table(r, "row_meta")[:rows]
    assert np.array_equal(meta[:, :3], s.meta)
    wbits = np.array([case.topk_w[m[0], m[1], m[2]] for m in s.meta], np.float32).view(np.int32)
    assert np.array_equal(meta[:, 3], wbits)
    pool = world.table(r, "pool")[:rows]
    assert np.array_equal(pool, s.pool)
    pool_sf = None
    if scaled:
        pool_sf = world.table(r, "pool_sf")[:rows, : H // 128]
        assert np.array_equal(pool_sf, s.pool_sf)
    ffn = world.table(r, "ffn")[:rows]
    ffn_sf = world.table(r, "ffn_sf")[:rows, : I // 128] if scaled else None
    for le in range(EPR):
        a, b = int(s.row_base[le]), int(s.row_base[le + 1])
        if a == b:
            continue
        e = r * EPR + le
        # L1: decoded device FP8 vs the oracle's pre-quantisation expectation
        want_h = s.h[a:b]
        got_h = orc.dequant_rows_1x128(np.ascontiguousarray(ffn[a:b]), None if not scaled else np.ascontiguousarray(ffn_sf[a:b]))
        if scaled:
            scale = np.repeat(orc.ue8m0_to_f32(np.ascontiguousarray(ffn_sf[a:b])), 128, axis=1)
            # per-row scale choice may differ by one step at an amax boundary: allow either
            assert (np.abs(ffn_sf[a:b].astype(int) - s.ffn_sf[a:b].astype(int)) <= 1).all()
        else:
            scale = np.ones_like(want_h)
        d = np.abs(got_h.astype(np.float64) - np.clip(want_h, -448 * scale, 448 * scale))
        lim = np.maximum(2e-3 * scale, 7e-2 * np.abs(want_h))
        assert (d <= lim).all(), f"L1 expert {e}: max excess {(d - lim).max()}"
        # L2 from the device's own hidden bytes
        want_o = orc.l2(np.ascontiguousarray(ffn[a:b]), None if not scaled else np.ascontiguousarray(ffn_sf[a:b]),
                        case.w2[e], None if not scaled else case.w2_sf[e])
        for g in range(a, b):
            src, tok, k = s.meta[g]
            got_row = orc.bf16_to_f32(world.table(src, "combine_rows").view(np.uint16)[k, tok])
            st = orc.check_close(got_row, want_o[g - a], 1e-2, 1e-3)
            assert st["bad"] == 0, f"L2 expert {e} row {g}: {st}"


def _reduce_check(world, r):
    case = world.case
    T = case.tokens[r]
    if T == 0:
        return
    comb = world.table(r, "combine_rows").view(np.uint16)
    want = orc.reduce_all(comb, case.topk_idx[r], case.topk_w[r], T, case.E)
    got32 = world.y32[r][:T].cpu().numpy()
    assert np.array_equal(got32, want), "reduce differs from the oracle on the device's own rows"
    got16 = world.y[r][:T].view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got16, orc.f32_to_bf16(want))


MODES = [1, 2]   # prologue protocol: 1 = pull (route scatter, barrier, owner pulls), 2 = push (sources store rows)


def _run_case(case, expert_window=128, full_stage_checks=True, e2e_tol=1e-2, cta_pair=None, dispatch_mode=0, ref=None):
    from gpu_world import World, assert_status_ok, check_tables
    ref = ref or orc.layer_world(case)
    w = World(case, expert_window=expert_window, dispatch_mode=dispatch_mode)
    try:
        w.run(cta_pair=cta_pair)
        assert_status_ok(w)
        check_tables(w, ref)
        for r in range(case.R):
            if full_stage_checks:
                _stage_checks(w, ref, r, case.scaled)
            _reduce_check(w, r)
            T = case.tokens[r]
            if T:
                got = w.y32[r][:T].cpu().numpy()
                err = orc.rel_l2(got, ref[r].y)
                assert err <= e2e_tol, f"rank {r}: end-to-end relative L2 {err}"
    finally:
        w.destroy()
    if case.R == 1:
        _run_fused(case, ref[0].y, expert_window, e2e_tol, cta_pair, dispatch_mode)


def _run_fused(case, want_y, expert_window, e2e_tol, cta_pair=None, dispatch_mode=0):
    """The same case through ONE launch of the whole layer (mxk_launch_full via fp8_mega_moe),
    twice on the same buffers: phases then overlap inside the persistent kernel."""
    import mini_mega_b200 as mm
    from gpu_world import dev_weights, load_inputs
    buf = mm.get_symm_buffer_for_mega_moe(None, case.E, case.cap, case.topk, case.H, case.I,
                                          expert_window=expert_window, dispatch_mode=dispatch_mode)
    try:
        load_inputs(case, [buf])
        l1, l2 = dev_weights(case, 0)
        T = case.tokens[0]
        for _ in range(3):
            y = torch.zeros((T, case.H), dtype=torch.bfloat16, device="cuda")
            mm.fp8_mega_moe(y, l1, l2, buf, cta_pair=cta_pair)
            torch.cuda.synchronize()
            st = buf.status()
            assert st.status == 0, f"device status {st.status} dbg {list(st.dbg)}"
            err = orc.rel_l2(y.float().cpu().numpy(), orc.bf16_to_f32(orc.f32_to_bf16(want_y)))
            assert err <= e2e_tol, f"fused launch: end-to-end relative L2 {err}"
    finally:
        buf.destroy()


@pytest.mark.parametrize("mode", MODES)
def test_toy_scaled(mode):
    """The CPU-runnable toy configuration: E=8, topk=2, H=512, I=256, T=32, world=1, UE8M0 block scales,
    top-k of router logits."""
    _run_case(orc.gen_case(1, 8, 2, 512, 256, 32, seed=1, routing="logits", scaled=True), dispatch_mode=mode)


@pytest.mark.parametrize("mode", MODES)
def test_toy_reference_mode(mode):
    """Same shape without scale planes: the reference kernel's own arithmetic (scale == 1)."""
    _run_case(orc.gen_case(1, 8, 2, 512, 256, 32, seed=2, routing="logits", scaled=False), dispatch_mode=mode)


@pytest.mark.parametrize("mode", MODES)
def test_multi_rank_world_scaled(mode):
    """4 ranks x 4 experts, ragged token counts including an empty rank."""
    _run_case(orc.gen_case(4, 4, 4, 1024, 512, [24, 0, 7, 33], seed=3, routing="uniform", scaled=True, cap=40),
              dispatch_mode=mode)


@pytest.mark.parametrize("mode", MODES)
def test_multi_window_skew(mode):
    """Zipf routing on few experts: several 128-row windows per expert, and a 64-row window run."""
    case = orc.gen_case(2, 2, 2, 512, 256, [150, 130], seed=4, routing="zipf", scaled=True)
    ref = orc.layer_world(case)
    _run_case(case, dispatch_mode=mode, ref=ref)
    _run_case(case, expert_window=64, dispatch_mode=mode, ref=ref)


@pytest.mark.parametrize("mode", MODES)
def test_invalid_ids(mode):
    """Negative expert ids are skipped everywhere (src/prologue.cuh:166-167, src/combine.cuh reduce)."""
    _run_case(orc.gen_case(2, 4, 4, 512, 256, [20, 12], seed=5, routing="uniform", scaled=True, invalid_frac=0.15),
              dispatch_mode=mode)


def test_reference_fixture_full_geometry():
    """The reference harness's own fixture at its frozen geometry (EPR=8, topk=8, H=6144,
    I=2048, balanced routes, WPROBE weights, byte-pattern x), R=1, 8 tokens."""
    _run_case(orc.gen_reference_fixture(1, 8, 8, 6144, 2048, 8, "balanced"))


def test_cta_pair_mode():
    """CTA-pair tiling (clusters of two CTAs, 256-row windows, 2-CTA MMA) forced on small cases:
    windows of fewer than 128 rows (the partner CTA has no rows), of 128..256 rows, and several
    windows per expert; with and without scale planes; pull- and push-mode prologue."""
    _run_case(orc.gen_case(1, 8, 2, 512, 256, 32, seed=13, routing="logits", scaled=True), cta_pair=2)
    _run_case(orc.gen_case(2, 2, 2, 512, 256, [300, 290], seed=14, routing="zipf", scaled=True), cta_pair=2, dispatch_mode=1)
    _run_case(orc.gen_case(1, 4, 2, 1024, 512, 400, seed=15, routing="uniform", scaled=False), cta_pair=2, dispatch_mode=2)


def test_pull_mode_many_rows_fused():
    """Pull-mode prologue with more than 4096 pool rows (one-pass route build, several windows per
    expert), phase-split against the oracle and then as ONE launch of the whole layer three times on
    the same buffers; single CTAs and CTA pairs."""
    case = orc.gen_case(1, 8, 4, 512, 256, 1100, seed=43, routing="zipf", scaled=True)
    ref = orc.layer_world(case)
    assert ref[0].meta.shape[0] >= 4096
    _run_case(case, dispatch_mode=1, cta_pair=1, ref=ref)
    _run_case(case, dispatch_mode=1, cta_pair=2, ref=ref, full_stage_checks=False)


def test_prefill_geometry_h7168():
    """The prefill-sized configuration's geometry (H=7168, I=2048: 56 K blocks = 14 scale groups per L1 task, scale
    rows of 56 live bytes in a stride of 64) on a small world: 8 experts, top-4, 600 tokens, so that the
    hottest expert fills more than two 128-row windows (and more than one 256-row window of a CTA
    pair).  Full stage checks with single CTAs and with CTA pairs, pull and push prologue."""
    case = orc.gen_case_bytes(1, 8, 4, 7168, 2048, 600, seed=41, routing="zipf")
    ref = orc.layer_world(case, threads=16)
    counts = np.bincount(case.topk_idx[0, :600].reshape(-1), minlength=8)
    assert counts.max() > 256
    for cta_pair, mode in ((1, 1), (2, 1), (1, 2), (2, 2)):
        _run_case(case, cta_pair=cta_pair, dispatch_mode=mode, ref=ref)


@pytest.mark.parametrize("mode", MODES)
def test_decode_world_full_width(mode):
    """The EP=8 decode shape as a multi-rank world at full width: 8 ranks x 4 experts, H=6144,
    I=2048, top-8, 16 tokens per rank (32 rows per expert on average).  Tables exact on every rank,
    stage checks, y within 1e-2."""
    case = orc.gen_case_bytes(8, 4, 8, 6144, 2048, 16, seed=42)
    _run_case(case, dispatch_mode=mode, ref=orc.layer_world(case, threads=16))


@pytest.mark.parametrize("group_ranks,skew_num,hot", [(4, -1, -1), (2, -1, -1), (4, 0, -1), (4, -1, 0), (2, 0, 2)])
def test_helper_groups_world(group_ranks, skew_num, hot):
    """Cross-rank helper scheduling (reference: MX_GROUP_SCHED, src/compute.cuh:700-835): a world of 4
    ranks with Zipf-skewed routing and 32-row windows, helper groups of 4 (one group) and of 2 (two
    interleaved groups), helpers forced on (-1) or decided by the reference's skew test (0 -> 2).
    Owner-side tables stay exact; every rank's window list equals the deterministic LPT of
    gs_schedule_member; every pool row holds the (source, token, k) and the bytes the oracle's model
    puts there, whether the rank owns the expert or helps with it; y within 1e-2.  `hot` -1 is the reference's
    schedule (every window may move), 0 the library's default (only experts with at least 3 windows are spread,
    the others stay with their owners), 2 a lower limit."""
    from gpu_world import World, assert_status_ok, check_tables
    case = orc.gen_case(4, 4, 4, 1024, 512, [60, 50, 40, 64], seed=61, routing="zipf", scaled=True)
    ref = orc.layer_world(case)
    want = orc.helper_world(case, ref, group_ranks, 32, 0 if skew_num < 0 else 2, hot_windows=0 if hot < 0 else (hot or 3))
    assert any(h["on"] for h in want)
    w = World(case, expert_window=32, dispatch_mode=2, group_ranks=group_ranks, group_skew_num=skew_num, group_hot_windows=hot)
    try:
        w.run()
        assert_status_ok(w)
        check_tables(w, ref)
        moved = 0
        for r in range(case.R):
            st = w.bufs[r].status()
            h = want[r]
            assert bool(st.helper_on) == h["on"], f"rank {r}: helper_on {st.helper_on}, expected {h['on']}"
            meta = w.table(r, "row_meta")
            rows = h["meta"].shape[0]
            assert st.total_rows == rows
            assert np.array_equal(meta[:rows, :3], h["meta"]), f"rank {r}: pool rows differ from the member's window list"
            pool = w.table(r, "pool")[:rows]
            assert np.array_equal(pool, case.x[h["meta"][:, 0], h["meta"][:, 1]])
            assert np.array_equal(w.table(r, "pool_sf")[:rows, : case.H // 128], case.x_sf[h["meta"][:, 0], h["meta"][:, 1]])
            if h["on"]:
                win = w.table(r, "windows")[: len(h["windows"])]
                assert st.n_windows == len(h["windows"])
                assert np.array_equal(win[:, [0, 3, 2]], np.array(h["windows"], np.int32).reshape(-1, 3))
                mm_ = w.bufs[r].group_members().index(r)
                moved += sum(1 for ge, _, _ in h["windows"] if ge // case.EPR != mm_)
            _reduce_check(w, r)
            T = case.tokens[r]
            err = orc.rel_l2(w.y32[r][:T].cpu().numpy(), ref[r].y)
            assert err <= 1e-2, f"rank {r}: end-to-end relative L2 {err}"
        assert moved > 0, "no window was computed by a helper: the case does not exercise the path"
    finally:
        w.destroy()
