"""The small entry points around the layer, through the C ABI: device-side test weights against
the oracle's generator (reference: fill_weights_lane / WPROBE_VAL, src/megakernel.cu:66-105),
the empty launch (launch_empty, :261-264), the resource dump (dump_kernel_resources, :270-282),
the host-side UE8M0 quantisers of mini_mega_b200.quant against the reference's own
(torch/mxmegakernel/utils/math.py, golden vectors in tests/golden/quant_py.npz)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_host_quantisers_match_reference_golden():
    from mini_mega_b200 import quant
    g = np.load(os.path.join(ROOT, "tests", "golden", "quant_py.npz"))
    q, e = quant.per_token_cast_to_fp8(torch.from_numpy(g["x"]))
    assert np.array_equal(e.numpy(), g["xsf"])
    assert np.array_equal(q.view(torch.uint8).numpy(), g["xq"])
    wq, we = quant.per_block_cast_to_fp8(torch.from_numpy(g["w"]))
    assert np.array_equal(we.numpy(), g["wsf"])
    assert np.array_equal(wq.view(torch.uint8).numpy(), g["wq"])
    back = quant.cast_back_from_fp8(torch.from_numpy(g["xq"]).view(torch.float8_e4m3fn), torch.from_numpy(g["xsf"]))
    assert np.array_equal(back.numpy(), g["back"])
    ce = quant.ue8m0_to_float(quant.ceil_to_ue8m0(torch.from_numpy(g["ceil_in"])))
    assert np.array_equal(ce.numpy(), g["ceil_out"])


@pytest.mark.gpu
def test_device_fill_weights_matches_oracle():
    from mini_mega_b200 import _lib
    from oracle import oracle as orc
    lib = _lib.lib()
    for rows, k, seed in ((2 * 256 * 3, 512, 17), (512 * 3, 256, 91), (7, 33, 5)):
        w = torch.zeros(rows * k, dtype=torch.uint8, device="cuda")
        _lib.check(lib.mxk_fill_weights(w.data_ptr(), rows, k, seed, torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert np.array_equal(w.cpu().numpy().reshape(rows, k), orc.fill_weights(rows, k, seed))
    assert lib.mxk_fill_weights(None, 4, 4, 1, None) == -1


@pytest.mark.gpu
def test_reference_fixture_with_device_generated_weights():
    """The reference harness fills its weights on the device (test/mega_common.cuh:229-241); the same
    through mxk_fill_weights, then the layer on those bytes against the oracle on its own."""
    import mini_mega_b200 as mm
    from gpu_world import load_inputs
    from mini_mega_b200 import _lib
    from oracle import oracle as orc
    case = orc.gen_reference_fixture(1, 8, 8, 512, 256, 16, "balanced")
    lib = _lib.lib()
    st = torch.cuda.current_stream().cuda_stream
    w1 = torch.zeros((8, 512, 512), dtype=torch.uint8, device="cuda")
    w2 = torch.zeros((8, 512, 256), dtype=torch.uint8, device="cuda")
    _lib.check(lib.mxk_fill_weights(w1.data_ptr(), 8 * 512, 512, 17, st))
    _lib.check(lib.mxk_fill_weights(w2.data_ptr(), 8 * 512, 256, 91, st))
    buf = mm.get_symm_buffer_for_mega_moe(None, 8, 16, 8, 512, 256)
    try:
        load_inputs(case, [buf])
        y = torch.zeros((16, 512), dtype=torch.bfloat16, device="cuda")
        mm.fp8_mega_moe(y, w1, w2, buf)
        torch.cuda.synchronize()
        assert buf.status().status == 0
        assert orc.rel_l2(y.float().cpu().numpy(), orc.layer_world(case)[0].y) <= 1e-2
    finally:
        buf.destroy()


@pytest.mark.gpu
def test_empty_launch_and_resource_dump(capfd):
    from mini_mega_b200 import _lib
    lib = _lib.lib()
    assert lib.mxk_launch_empty(148, 384, 0, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert lib.mxk_dump_kernel_resources() == 0
    out = capfd.readouterr().out
    assert "k_mega" in out and "regs=" in out
    assert lib.mxk_kernels_per_layer() == 1
    assert lib.mxk_ticks_count() == 16 and lib.mxk_rwk_ticks_off() > 0
