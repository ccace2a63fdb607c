"""4-bit (e2m1) weights through the CUDA library (reference: the MX_FP4_W build, src/common.cuh:99-134,
whose CPU checker expands the codes and reuses its 8-bit arithmetic, src/bench_check.cuh:405-421).
The oracle of the 4-bit layer is therefore the 8-bit oracle on the expanded bytes; in addition the
4-bit launch must give the very bits of an 8-bit launch on the expanded weights, since the tensor
core multiplies the same values."""
import ctypes as C

import numpy as np
import pytest
import torch

import mini_mega_b200 as mm
from mini_mega_b200 import _lib
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def test_fill_weights_e2m1_on_device():
    lib = _lib.lib()
    for rows, k, seed in ((33, 256, 17), (7, 1024, 91)):
        w = torch.zeros((rows, k // 2), dtype=torch.uint8, device="cuda")
        _lib.check(lib.mxk_fill_weights_e2m1(w.data_ptr(), rows, k, seed, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert np.array_equal(w.cpu().numpy(), orc.fill_weights_e2m1(rows, k, seed))
    assert lib.mxk_fill_weights_e2m1(None, 4, 4, 1, None) == -1
    assert lib.mxk_fill_weights_e2m1(C.c_void_p(256), 4, 5, 1, None) == -1     # odd k


def _run(case, dispatch_mode, cta_pair=None, tol=1e-2):
    from gpu_world import World, assert_status_ok, check_tables
    from test_gpu_parity import _reduce_check, _stage_checks
    ref = orc.layer_world(case)
    ys = {}
    for fmt in (1, 0):      # 4-bit launch, then the 8-bit launch on the expanded weights
        w = World(case, dispatch_mode=dispatch_mode, weight_format=fmt)
        try:
            w.run(cta_pair=cta_pair)
            assert_status_ok(w)
            check_tables(w, ref)
            for r in range(case.R):
                if fmt == 1:
                    _stage_checks(w, ref, r, case.scaled)
                    _reduce_check(w, r)
                T = case.tokens[r]
                if T:
                    got = w.y32[r][:T].cpu().numpy()
                    err = orc.rel_l2(got, ref[r].y)
                    assert err <= tol, f"format {fmt} rank {r}: end-to-end relative L2 {err}"
                    ys[(fmt, r)] = got
        finally:
            w.destroy()
    for r in range(case.R):
        if case.tokens[r]:
            assert np.array_equal(ys[(1, r)], ys[(0, r)]), f"rank {r}: 4-bit and expanded 8-bit launches differ"


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("scaled", [True, False])
def test_toy_layer_e2m1(mode, scaled):
    """The toy geometry (E=8, topk=2, H=512, I=256, 32 tokens) with 4-bit weights."""
    from gpu_world import to_e2m1_case
    case = to_e2m1_case(orc.gen_case(1, 8, 2, 512, 256, 32, seed=21, routing="logits", scaled=scaled), seed=21)
    _run(case, mode)


def test_multi_rank_world_e2m1():
    """4 ranks x 4 experts with ragged token counts: every rank's weights are 4-bit."""
    from gpu_world import to_e2m1_case
    case = to_e2m1_case(orc.gen_case(4, 4, 4, 1024, 512, [24, 0, 7, 33], seed=23, routing="uniform", scaled=True, cap=40), seed=23)
    _run(case, 0)


def test_cta_pair_windows_e2m1():
    """256-row windows on clusters of two CTAs: each CTA stages one 128-row half of the 4-bit weight tile."""
    from gpu_world import to_e2m1_case
    case = to_e2m1_case(orc.gen_case(1, 4, 2, 512, 256, 700, seed=25, routing="zipf", scaled=True), seed=25)
    _run(case, 0, cta_pair=2)


def test_helper_groups_with_e2m1_replicas():
    """Helper groups forced on in a world of 4 ranks: the group-replicated weights are 4-bit too."""
    from gpu_world import World, assert_status_ok, check_tables, to_e2m1_case
    case = to_e2m1_case(orc.gen_case(4, 4, 4, 1024, 512, [60, 50, 40, 64], seed=61, routing="zipf", scaled=True), seed=29)
    ref = orc.layer_world(case)
    w = World(case, expert_window=32, dispatch_mode=2, group_ranks=4, group_skew_num=-1, weight_format=1, group_hot_windows=-1)
    try:
        w.run()
        assert_status_ok(w)
        check_tables(w, ref)
        assert all(b.status().helper_on for b in w.bufs)
        for r in range(case.R):
            T = case.tokens[r]
            err = orc.rel_l2(w.y32[r][:T].cpu().numpy(), ref[r].y)
            assert err <= 1e-2, f"rank {r}: end-to-end relative L2 {err}"
    finally:
        w.destroy()


def test_fused_entry_point():
    """fp8_fp4_mega_moe (one launch of the whole layer) on an fp8xfp4 buffer, three times on the same buffers."""
    from gpu_world import dev_weights, load_inputs, to_e2m1_case
    case = to_e2m1_case(orc.gen_case(1, 8, 2, 512, 256, 48, seed=27, routing="zipf", scaled=True), seed=27)
    want = orc.bf16_to_f32(orc.f32_to_bf16(orc.layer_world(case)[0].y))
    buf = mm.get_symm_buffer_for_mega_moe(None, case.E, case.cap, case.topk, case.H, case.I, mma_type="fp8xfp4")
    try:
        load_inputs(case, [buf])
        l1, l2 = mm.transform_weights_for_mega_moe(*dev_weights(case, 0, weight_format=1), weight_format="e2m1")
        for _ in range(3):
            y = torch.zeros((case.tokens[0], case.H), dtype=torch.bfloat16, device="cuda")
            mm.fp8_fp4_mega_moe(y, l1, l2, buf)
            torch.cuda.synchronize()
            assert buf.status().status == 0
            assert orc.rel_l2(y.float().cpu().numpy(), want) <= 1e-2
        with pytest.raises(ValueError):
            mm.fp8_mega_moe(y, l1, l2, buf)          # 4-bit tensors given as 8-bit: shapes do not fit
    finally:
        buf.destroy()


def test_bad_weight_format_is_rejected():
    a = _lib.MxkLaunchArgs()
    a.R, a.rank, a.tokens = 1, 0, 4
    a.experts_per_rank, a.topk, a.hidden, a.intermediate, a.max_tokens = 8, 2, 512, 256, 32
    a.weight_format = 2
    assert _lib.lib().mxk_launch_full(C.byref(a), None) == -1
