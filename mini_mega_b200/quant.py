"""UE8M0 block quantisers for activations (1x128) and weights (128x128).

Same arithmetic as the reference's ``torch/mxmegakernel/utils/math.py`` (``ceil_to_ue8m0``
:13-16, ``per_token_cast_to_fp8`` :26-36, ``per_block_cast_to_fp8`` :62-72,
``cast_back_from_fp8`` :167-173) but returning the scale as its exponent byte, which
is what the kernels consume.  Pure torch, any device.
"""
from typing import Tuple

import torch


def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= |x| as a biased-exponent byte in [1, 254]."""
    bits = x.abs().float().contiguous().view(torch.int32)
    exp = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return exp.clamp(1, 254).to(torch.uint8)


def ue8m0_to_float(e: torch.Tensor) -> torch.Tensor:
    return (e.to(torch.int32) << 23).view(torch.float32)


def per_token_cast_to_fp8(x: torch.Tensor, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [m, n] (n % gran_k == 0) -> (float8_e4m3fn [m, n], uint8 exponents [m, n/gran_k])."""
    m, n = x.shape
    assert n % gran_k == 0
    v = x.float().view(m, n // gran_k, gran_k)
    amax = v.abs().amax(dim=2).clamp(1e-4)
    e = ceil_to_ue8m0(amax / 448.0)
    q = (v * (1.0 / ue8m0_to_float(e)).unsqueeze(2)).to(torch.float8_e4m3fn)
    return q.view(m, n), e


def per_block_cast_to_fp8(w: torch.Tensor, gran: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """w [m, n] (both % gran == 0) -> (float8_e4m3fn [m, n], uint8 exponents [m/gran, n/gran])."""
    m, n = w.shape
    assert m % gran == 0 and n % gran == 0
    v = w.float().view(m // gran, gran, n // gran, gran)
    amax = v.abs().amax(dim=(1, 3)).clamp(1e-4)
    e = ceil_to_ue8m0(amax / 448.0)
    q = (v * (1.0 / ue8m0_to_float(e))[:, None, :, None]).to(torch.float8_e4m3fn)
    return q.view(m, n), e


def cast_back_from_fp8(q: torch.Tensor, e: torch.Tensor, gran_k: int = 128) -> torch.Tensor:
    m, n = q.shape
    idx = torch.arange(n, device=q.device) // gran_k
    return q.float() * ue8m0_to_float(e)[:, idx]
