"""bf16 activations: the device quantiser (mxk_quantize_rows) against the oracle's restatement of
the reference quantiser per_token_cast_to_fp8(use_ue8m0=True, gran_k=128) — which is pinned to the
reference's own Python code by tests/golden/quant_py.npz — bit for bit, and the bf16xfp8 entry
point against the fp8 entry point fed with those bytes (identical output bits)."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu


def _bf16_rows(T, H, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((T, H)).astype(np.float32) * np.exp(rng.uniform(-6, 6, (T, 1))).astype(np.float32)
    x[0, :128] = 0.0                 # all-zero group: amax clamps to 1e-4
    if T > 2 and H >= 256:
        x[1, 128:256] *= 1e4         # large group
        x[2, 5] = 448.0 * 2.0 ** 3   # exactly representable maximum of its scale
    return torch.from_numpy(x).bfloat16()


@pytest.mark.parametrize("T,H", [(7, 512), (33, 6144), (1, 128)])
def test_quantize_rows_matches_reference_quantiser(T, H):
    from mini_mega_b200 import _lib
    lib = _lib.lib()
    xb = _bf16_rows(T, H, seed=T + H).cuda()
    q = torch.zeros((T, H), dtype=torch.uint8, device="cuda")
    sf = torch.zeros((T, H // 128), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.mxk_quantize_rows(xb.data_ptr(), T, H, q.data_ptr(), sf.data_ptr(), st), "mxk_quantize_rows")
    torch.cuda.synchronize()
    want_q, want_sf = orc.quant_rows_1x128(xb.float().cpu().numpy())
    assert np.array_equal(sf.cpu().numpy(), want_sf)
    assert np.array_equal(q.cpu().numpy(), want_q)
    # scale-free form: plain saturating round-to-nearest-even cast
    x2 = (xb.float() * 0 + torch.from_numpy(np.random.default_rng(1).uniform(-500, 500, (T, H)).astype(np.float32)).cuda()).bfloat16()
    _lib.check(lib.mxk_quantize_rows(x2.data_ptr(), T, H, q.data_ptr(), None, st), "mxk_quantize_rows")
    torch.cuda.synchronize()
    assert np.array_equal(q.cpu().numpy(), orc.e4m3_quantize(x2.float().cpu().numpy()))
    # argument checks fail loudly
    assert lib.mxk_quantize_rows(xb.data_ptr(), T, 100, q.data_ptr(), None, st) != 0


def test_bf16_entry_point_equals_fp8_entry_point():
    import mini_mega_b200 as mm
    from gpu_world import dev_weights
    case = orc.gen_case(1, 8, 2, 512, 256, 40, seed=21, routing="uniform", scaled=True)
    T = case.tokens[0]
    xb = _bf16_rows(T, case.H, seed=5)
    xq, xsf = orc.quant_rows_1x128(xb.float().numpy())
    l1, l2 = dev_weights(case, 0)
    ys = []
    for kind in ("fp8xfp8", "bf16xfp8"):
        buf = mm.get_symm_buffer_for_mega_moe(None, case.E, case.cap, case.topk, case.H, case.I, mma_type=kind)
        try:
            if kind == "fp8xfp8":
                buf.x.view(torch.uint8)[:T].copy_(torch.from_numpy(xq))
                buf.x_sf[:T].copy_(torch.from_numpy(xsf))
            else:
                assert buf.x.dtype == torch.bfloat16
                buf.x[:T].copy_(xb)
            buf.topk_idx[:T].copy_(torch.from_numpy(case.topk_idx[0, :T]))
            buf.topk_weights[:T].copy_(torch.from_numpy(case.topk_w[0, :T]))
            y = torch.zeros((T, case.H), dtype=torch.bfloat16, device="cuda")
            (mm.fp8_mega_moe if kind == "fp8xfp8" else mm.bf16_fp8_mega_moe)(y, l1, l2, buf)
            torch.cuda.synchronize()
            assert buf.status().status == 0
            ys.append(y)
        finally:
            buf.destroy()
    assert torch.equal(ys[0].view(torch.int16), ys[1].view(torch.int16))
    # and the result is the oracle's for those bytes
    c2 = orc.Case(case.R, case.EPR, case.topk, case.H, case.I, case.cap, case.tokens, True,
                  np.pad(xq, ((0, case.cap - T), (0, 0)))[None], np.pad(xsf, ((0, case.cap - T), (0, 0)), constant_values=127)[None],
                  case.topk_idx, case.topk_w, case.w1, case.w1_sf, case.w2, case.w2_sf, "bf16")
    want = orc.layer_world(c2)[0].y
    assert orc.rel_l2(ys[1].float().cpu().numpy(), want) <= 1e-2
