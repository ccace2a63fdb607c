"""mxk_launch_full_static: the layer for hosts that are not allowed to allocate.

A serving process whose memory pool already owns the GPU, or a plugin inside a runtime
that forbids cudaMalloc after start-up, cannot hand the library freshly allocated rwk / unk
workspace blocks.  The static entry point keeps that workspace in an array inside the
library image.  Here it is called through the C ABI twice in a row (different inputs,
the array keeps the first call's leftovers) and must reproduce the regular entry point's
output bit for bit: both run the same kernels on the same inputs.

The file name sorts last so that a run that stops at the first failure has already run
every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(seed, tokens, geom=(8, 2, 512, 256, 32)):
    """One layer through the regular entry point and through the static one; returns the static
    workspace's launch counter after the call."""
    import mini_mega_b200 as mm
    from mini_mega_b200 import _lib
    from oracle import oracle as orc

    lib = _lib.lib()
    E, topk, H, I, cap = geom
    case = orc.gen_case(1, E, topk, H, I, tokens, seed=seed, routing="logits", scaled=True, cap=cap)
    buf = mm.get_symm_buffer_for_mega_moe(None, E, cap, topk, H, I)
    try:
        buf.x.view(torch.uint8).copy_(torch.from_numpy(case.x[0]))
        buf.x_sf.copy_(torch.from_numpy(case.x_sf[0]))
        buf.topk_idx.copy_(torch.from_numpy(case.topk_idx[0]))
        buf.topk_weights.copy_(torch.from_numpy(case.topk_w[0]))
        l1, l2 = mm.transform_weights_for_mega_moe(
            (torch.from_numpy(case.w1).cuda(), torch.from_numpy(case.w1_sf).cuda()),
            (torch.from_numpy(case.w2).cuda(), torch.from_numpy(case.w2_sf).cuda()))
        y_ref = torch.zeros((tokens, H), dtype=torch.bfloat16, device="cuda")
        y_new = torch.zeros_like(y_ref)
        y32_ref = torch.zeros((tokens, H), dtype=torch.float32, device="cuda")
        y32_new = torch.zeros_like(y32_ref)
        st = torch.cuda.current_stream().cuda_stream
        a = buf.launch_args(tokens, l1, l2, y_bf16=y_ref, y_f32=y32_ref)
        _lib.check(lib.mxk_launch_full(C.byref(a), st), "mxk_launch_full")
        b = buf.launch_args(tokens, l1, l2, y_bf16=y_new, y_f32=y32_new)
        b.rwk = b.unk = b.unk_peers = b.peer_bases = None   # the static entry point brings its own workspace
        _lib.check(lib.mxk_launch_full_static(C.byref(b), st), "mxk_launch_full_static")
        torch.cuda.synchronize()
        assert buf.status().status == 0
        sst = _lib.MxkStatus()
        _lib.check(lib.mxk_read_status_static(C.byref(sst)), "mxk_read_status_static")
        assert sst.status == 0, f"static workspace: device status {sst.status} dbg {list(sst.dbg)}"
        want = orc.layer_world(case)[0].y
        assert orc.rel_l2(y32_ref.cpu().numpy(), want) <= 1e-2       # the regular path is right ...
        assert torch.equal(y32_new, y32_ref)                          # ... and the static one is identical
        assert torch.equal(y_new.view(torch.int16), y_ref.view(torch.int16))
        return int(sst.launches)
    finally:
        buf.destroy()


def test_static_entry_matches_regular_entry_twice():
    n0 = _run_both(seed=31, tokens=32)
    n1 = _run_both(seed=32, tokens=19)   # second call: other inputs, fewer tokens, stale leftovers in the array
    assert n1 == n0 + 1                  # the launch counter keeps running from call to call


def test_static_entry_alternating_geometries():
    """Geometry A, then B (other top-k, capacity, widths: every table moves), then A again, each
    with its own routing: the launch counter sits at a geometry-independent place and keeps running,
    and a change of geometry clears the tables, so no call can take an earlier call's tagged words
    for current ones.  Every call must equal the regular entry point bit for bit."""
    A, B = (8, 2, 512, 256, 32), (4, 4, 1024, 512, 48)
    n = [_run_both(seed=33, tokens=32, geom=A), _run_both(seed=34, tokens=40, geom=B),
         _run_both(seed=35, tokens=27, geom=A), _run_both(seed=36, tokens=48, geom=B)]
    assert n == [n[0], n[0] + 1, n[0] + 2, n[0] + 3]


def test_static_entry_rejects_oversized_and_multi_rank():
    from mini_mega_b200 import _lib
    lib = _lib.lib()
    assert lib.mxk_static_scratch_bytes() == 32 << 20
    a = _lib.MxkLaunchArgs()
    a.R, a.rank, a.tokens = 1, 0, 16
    a.experts_per_rank, a.topk, a.hidden, a.intermediate, a.max_tokens = 256, 8, 6144, 2048, 4096
    dummy = torch.zeros(16, dtype=torch.uint8, device="cuda")
    a.self = dummy.data_ptr()
    assert lib.mxk_launch_full_static(C.byref(a), None) == -1
    assert b"static scratch holds" in lib.mxk_last_error()
    a.R = 2
    assert lib.mxk_launch_full_static(C.byref(a), None) == -1
    assert b"single-rank" in lib.mxk_last_error()
