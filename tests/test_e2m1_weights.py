"""4-bit (e2m1) weights on the CPU: the code table, the packing and the Python quantisers against
vectors produced by the reference's own Python code (tests/golden/e2m1.npz, written by
tests/golden/make_golden.py from torch/mxmegakernel/utils/math.py:84-164), and the oracle's and
the library's restatements of the reference's fp4_code_to_fp8 (src/common.cuh:116-126)."""
import os

import numpy as np
import pytest
import torch

from mini_mega_b200 import _lib, quant
from oracle import oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def g():
    return np.load(os.path.join(ROOT, "tests", "golden", "e2m1.npz"))


def test_code_table(g):
    """Every code's value, as the E4M3 byte the tensor core multiplies with."""
    want = g["code_e4m3"]                       # 16 bytes from the reference's value table cast to E4M3
    assert list(want[:8]) == [0x00, 0x30, 0x38, 0x3C, 0x40, 0x44, 0x48, 0x4C]
    assert list(quant.E2M1_TO_E4M3) == list(want)
    L = orc.lib()
    assert [L.orc_e2m1_to_e4m3(c) for c in range(16)] == list(want)
    _lib.build()
    P = _lib.lib()
    assert [P.mxk_e2m1_to_e4m3(c) for c in range(16)] == list(want)
    # decoded through the oracle's E4M3 decoder the bytes are the e2m1 values themselves
    vals = orc.e4m3_decode(np.array(want, np.uint8))
    assert np.array_equal(vals[:8], np.array(quant.E2M1_MAGNITUDES, np.float32))
    assert np.array_equal(vals[8:], -vals[:8])


def test_python_quantisers_match_the_reference(g):
    x = torch.from_numpy(g["x"]).bfloat16()
    packed, e = quant.per_token_cast_to_fp4(x)
    assert np.array_equal(packed.numpy(), g["x_packed"])
    assert np.array_equal(e.numpy(), g["x_sf"])
    assert np.array_equal(quant.cast_back_from_fp4(packed, e).numpy(), g["x_back"])
    assert np.array_equal(quant.quantize_to_e2m1(torch.from_numpy(g["q_in"])).numpy(), g["q_codes"])
    codes = quant.unpack_e2m1(packed)
    assert torch.equal(quant.pack_e2m1(codes), packed)


def test_block_quantiser_and_expansion():
    """128x128 weight blocks: scale = power of two >= amax / 6; expansion through the oracle."""
    gen = torch.Generator().manual_seed(3)
    w = torch.randn((256, 384), generator=gen) * 0.02
    packed, e = quant.per_block_cast_to_fp4(w)
    assert packed.shape == (256, 192) and e.shape == (2, 3)
    bytes_ = orc.expand_e2m1(packed.numpy())
    assert np.array_equal(bytes_, quant.e2m1_to_e4m3(quant.unpack_e2m1(packed)).numpy())
    scale = np.repeat(np.repeat(orc.ue8m0_to_f32(e.numpy()), 128, 0), 128, 1)
    back = orc.e4m3_decode(bytes_) * scale
    # e2m1 has a relative step of at most 1/2 between neighbours: |error| <= scale * 1 (half of the 4 -> 6 gap)
    assert (np.abs(back - w.numpy()) <= scale * 1.0 + 1e-12).all()
    amax = np.abs(w.numpy()).reshape(2, 128, 3, 128).max(axis=(1, 3))
    s = orc.ue8m0_to_f32(e.numpy())
    assert (s * 6 >= amax).all() and (s * 3 < amax).all()


def test_fill_weights_e2m1_formula():
    w = orc.fill_weights_e2m1(5, 64, 17)
    codes = quant.unpack_e2m1(torch.from_numpy(w)).numpy()
    r, k = np.meshgrid(np.arange(5, dtype=np.uint32), np.arange(64, dtype=np.uint32), indexing="ij")
    assert np.array_equal(codes, (((np.uint32(17) + r * 131 + k * 7) >> 1) & 0xF).astype(np.uint8))
