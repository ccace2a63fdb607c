"""Protocol-level GPU tests: prologue tables on the reference's route patterns (including
over-capacity drops and invalid ids), bounded waits that expire without hanging, CUDA-graph
replay against eager results, and the split compute / reduce entry points."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("pattern", ["balanced", "hot", "mixed-invalid"])
def test_prelude_tables_on_reference_patterns(pattern, mode):
    """L0 check of the reference (test/check.cu:168-198): after the prologue alone, slot counts,
    source tables, received counts + checksum and prefix tables are exact on every rank —
    'hot' overflows the slot capacity (pairs dropped), 'mixed-invalid' carries ids of -1."""
    from gpu_world import World, check_tables
    R, EPR, topk, tokens = 2, 8, 8, 16
    case = orc.gen_reference_fixture(R, EPR, topk, 512, 256, tokens, pattern, salt=1)
    ref = orc.route_world(case)                 # slot capacity = max_tokens, like the reference
    w = World(case, dispatch_mode=mode)         # 1 = pull-mode prologue, 2 = push-mode prologue
    try:
        w.run(phases=(1, 2))                    # route for every rank, then set-up for every rank
        check_tables(w, ref)
        for r in range(R):
            st = w.bufs[r].status()
            assert st.status == 0
            rows = int(ref[r].prefix_tbl[:, R].sum())
            assert st.total_rows == rows
            want_windows = int(sum((int(c) + 127) // 128 for c in ref[r].prefix_tbl[:, R]))
            assert st.n_windows == want_windows
            # task list of this rank against the scheduler restatement
            win, tasks, n_l1 = orc.schedule(ref[r].prefix_tbl[:, R], ref[r].row_base, 128, 256 // 128, 512 // 256)
            assert st.n_tasks == tasks.shape[0] and st.n_l1_tasks == n_l1
            assert np.array_equal(w.table(r, "windows")[: win.shape[0], :3], win)
            assert np.array_equal(w.table(r, "tasks")[: tasks.shape[0]], tasks)
            # accepted-pair map: valid id and inside the slot capacity
            ps = w.table(r, "pair_state")[: tokens * topk]
            idx = case.topk_idx[r, :tokens].reshape(-1)
            seen = {}
            want = np.zeros_like(ps)
            for p, e in enumerate(idx):
                if 0 <= e < R * EPR:
                    seen[e] = seen.get(e, 0) + 1
                    want[p] = 1 if seen[e] <= case.cap else 0
            assert np.array_equal(ps, want)
    finally:
        w.destroy()


@pytest.mark.parametrize("mode", [1, 2])
def test_large_batch_route_tables(mode):
    """More pairs per rank than one scan step covers (the route build then works in one pass over
    the pairs: slice ranks, per-slice expert counts, grid barrier, exclusive sums), with a slot
    capacity below the per-expert load (drops) and invalid ids: every table still exact."""
    from gpu_world import World, check_tables
    case = orc.gen_case(2, 4, 8, 512, 256, [500, 410], seed=17, routing="uniform", scaled=True, invalid_frac=0.05)
    ref = orc.route_world(case, slot_cap=300)
    w = World(case, slot_capacity=300, dispatch_mode=mode)
    try:
        w.run(phases=(1, 2))
        check_tables(w, ref)
        for r in range(2):
            assert w.bufs[r].status().status == 0
            T = case.tokens[r]
            idx = case.topk_idx[r, :T].reshape(-1)
            seen, want = {}, np.zeros(T * 8, np.uint8)
            for p, e in enumerate(idx):
                if 0 <= e < 8:
                    seen[e] = seen.get(e, 0) + 1
                    want[p] = 1 if seen[e] <= 300 else 0
            assert np.array_equal(w.table(r, "pair_state")[: T * 8], want)
            assert (want == 0).sum() > 100   # the capacity really dropped pairs
    finally:
        w.destroy()


@pytest.mark.parametrize("mode", [1, 2])
def test_barrier_wait_expires_and_context_survives(mode):
    """A rank whose peer never arrives: the barrier wait runs out after max_spins*250 ns, the
    kernel records MXK_DEV_TIMEOUT_BARRIER and returns; nothing hangs or traps and the same
    process then runs a correct layer."""
    import mini_mega_b200 as mm
    from gpu_world import World
    from mini_mega_b200 import _lib
    case = orc.gen_case(2, 4, 2, 512, 256, [8, 8], seed=7, scaled=True)
    w = World(case, dispatch_mode=mode)
    try:
        lib = _lib.lib()
        a = w.args(0, max_spins=4000)   # 1 ms
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.mxk_launch_phases(C.byref(a), 1 | 2, st), "prelude of rank 0 only")
        torch.cuda.synchronize()
        s = w.bufs[0].status()
        assert s.status == 1 and s.dbg[0] >= 1, (s.status, list(s.dbg))
    finally:
        w.destroy()
    # context still usable
    small = orc.gen_case(1, 8, 2, 512, 256, 16, seed=8, scaled=True)
    buf = mm.get_symm_buffer_for_mega_moe(None, 8, 16, 2, 512, 256)
    try:
        from gpu_world import dev_weights, load_inputs
        load_inputs(small, [buf])
        l1, l2 = dev_weights(small, 0)
        y = torch.zeros((16, 512), dtype=torch.bfloat16, device="cuda")
        mm.fp8_mega_moe(y, l1, l2, buf)
        torch.cuda.synchronize()
        assert buf.status().status == 0
        assert orc.rel_l2(y.float().cpu().numpy(), orc.layer_world(small)[0].y) <= 1e-2
    finally:
        buf.destroy()


@pytest.mark.parametrize("mode", [1, 2])
def test_graph_replay_matches_eager(mode):
    """Reference graph check (test/check.cu:533-745): N layer launches captured in one CUDA graph
    with no host reset between nodes; every replay must reproduce the eager result (the
    launch counter and table parity live on the device)."""
    import mini_mega_b200 as mm
    from gpu_world import dev_weights, load_inputs
    case = orc.gen_case(1, 8, 4, 1024, 512, 48, seed=9, routing="uniform", scaled=True)
    buf = mm.get_symm_buffer_for_mega_moe(None, case.E, case.cap, case.topk, case.H, case.I, dispatch_mode=mode)
    try:
        load_inputs(case, [buf])
        l1, l2 = dev_weights(case, 0)
        T = case.tokens[0]
        y_eager = torch.zeros((T, case.H), dtype=torch.bfloat16, device="cuda")
        mm.fp8_mega_moe(y_eager, l1, l2, buf)
        torch.cuda.synchronize()
        assert orc.rel_l2(y_eager.float().cpu().numpy(), orc.layer_world(case)[0].y) <= 1e-2
        ys = [torch.zeros_like(y_eager) for _ in range(5)]
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                for y in ys:
                    mm.fp8_mega_moe(y, l1, l2, buf)
        for _ in range(3):
            for y in ys:
                y.zero_()
            g.replay()
            torch.cuda.synchronize()
            assert buf.status().status == 0
            for y in ys:
                assert torch.equal(y.view(torch.int16), y_eager.view(torch.int16))
        assert buf.status().launches == 1 + 3 * 5   # the eager layer plus three replays of five nodes
    finally:
        buf.destroy()


@pytest.mark.parametrize("mode", [1, 2])
def test_split_compute_then_reduce(mode):
    import mini_mega_b200 as mm
    from gpu_world import dev_weights, load_inputs
    case = orc.gen_case(1, 8, 2, 512, 256, 24, seed=10, routing="logits", scaled=True)
    buf = mm.get_symm_buffer_for_mega_moe(None, case.E, case.cap, case.topk, case.H, case.I, dispatch_mode=mode)
    try:
        load_inputs(case, [buf])
        l1, l2 = dev_weights(case, 0)
        y_full = torch.zeros((24, 512), dtype=torch.bfloat16, device="cuda")
        y_split = torch.zeros_like(y_full)
        mm.fp8_mega_moe(y_full, l1, l2, buf)
        mm.fp8_mega_moe_compute(l1, l2, buf, 24)
        mm.fp8_mega_moe_reduce(y_split, buf)
        torch.cuda.synchronize()
        assert buf.status().status == 0
        assert torch.equal(y_full.view(torch.int16), y_split.view(torch.int16))
    finally:
        buf.destroy()


def test_compute_without_reduce_then_full_layer():
    """A compute launch that is never followed by its reduce leaves arrival counts behind; the next
    layer must notice (the count table is not marked clean) and clear them before peers push."""
    import mini_mega_b200 as mm
    from gpu_world import dev_weights, load_inputs
    case = orc.gen_case(1, 8, 2, 512, 256, 24, seed=12, routing="logits", scaled=True)
    want = orc.layer_world(case)[0].y
    for mode in (1, 2):
        buf = mm.get_symm_buffer_for_mega_moe(None, case.E, case.cap, case.topk, case.H, case.I, dispatch_mode=mode)
        try:
            load_inputs(case, [buf])
            l1, l2 = dev_weights(case, 0)
            y = torch.zeros((24, 512), dtype=torch.bfloat16, device="cuda")
            mm.fp8_mega_moe(y, l1, l2, buf)
            mm.fp8_mega_moe_compute(l1, l2, buf, 24)      # rows pushed, counts raised, nobody reduces
            assert int(buf.table("combine_cnt").sum()) > 0
            y.zero_()
            mm.fp8_mega_moe(y, l1, l2, buf)
            torch.cuda.synchronize()
            assert buf.status().status == 0
            assert orc.rel_l2(y.float().cpu().numpy(), want) <= 1e-2
            assert int(buf.table("combine_cnt").sum()) == 0   # consumed counts are zeroed by the reduce
        finally:
            buf.destroy()


def test_ring_geometry_switches_between_launches():
    """Launches whose windows all have at most 32 rows stage 32 activation rows per ring slot and run
    five stages; any larger window brings the four-stage ring back.  The same buffers take small and
    large batches in turn, 8-bit and 4-bit weights, and every launch is checked against the oracle
    (the ring, its barriers and the tensor maps are per launch: nothing may carry over)."""
    import mini_mega_b200 as mm
    from gpu_world import dev_weights, load_inputs, to_e2m1_case
    small = orc.gen_case(1, 8, 2, 512, 256, 6, seed=31, routing="logits", scaled=True, cap=96)
    large = orc.gen_case(1, 8, 2, 512, 256, 96, seed=32, routing="zipf", scaled=True, cap=96)
    assert max(np.bincount(large.topk_idx[0][:96].ravel(), minlength=8)) > 32      # some window beyond the slim ring
    assert max(np.bincount(small.topk_idx[0][:6].ravel(), minlength=8)) <= 32
    for fmt in (0, 1):
        cases = [small, large]
        if fmt == 1:
            cases = [to_e2m1_case(orc.gen_case(1, 8, 2, 512, 256, 6, seed=31, routing="logits", scaled=True, cap=96), seed=33),
                     to_e2m1_case(orc.gen_case(1, 8, 2, 512, 256, 96, seed=32, routing="zipf", scaled=True, cap=96), seed=34)]
        wants = [orc.bf16_to_f32(orc.f32_to_bf16(orc.layer_world(c)[0].y)) for c in cases]
        buf = mm.get_symm_buffer_for_mega_moe(None, 8, 96, 2, 512, 256)
        try:
            for rep in range(3):
                for c, want in zip(cases, wants):
                    load_inputs(c, [buf])
                    l1, l2 = dev_weights(c, 0, weight_format=fmt)
                    T = c.tokens[0]
                    y = torch.zeros((T, 512), dtype=torch.bfloat16, device="cuda")
                    mm.fp8_mega_moe(y, l1, l2, buf, weight_format=fmt)
                    torch.cuda.synchronize()
                    st = buf.status()
                    assert st.status == 0, f"format {fmt} rep {rep} tokens {T}: device status {st.status} dbg {list(st.dbg)}"
                    err = orc.rel_l2(y.float().cpu().numpy(), want[:T])
                    assert err <= 1e-2, f"format {fmt} rep {rep} tokens {T}: relative L2 {err}"
        finally:
            buf.destroy()
