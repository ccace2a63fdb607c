"""UE8M0 block quantisers for activations (1x128) and weights (128x128).

Same arithmetic as the reference's ``torch/mxmegakernel/utils/math.py`` (``ceil_to_ue8m0``
:13-16, ``per_token_cast_to_fp8`` :26-36, ``per_block_cast_to_fp8`` :62-72,
``cast_back_from_fp8`` :167-173) but returning the scale as its exponent byte, which
is what the kernels consume.  The 4-bit (e2m1) helpers follow ``_quantize_to_fp4_e2m1``
:84-93, ``per_token_cast_to_fp4`` :96-122 and ``cast_back_from_fp4`` :152-164 with the same
packing (two codes per byte, the element of even index in the low nibble).  Pure torch, any device.
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


# ---- 4-bit (e2m1) weights -----------------------------------------------------------------
E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# the E4M3 byte of every e2m1 code (bit 3 = sign): what the tensor core multiplies with
E2M1_TO_E4M3 = tuple((0x80 if c & 8 else 0) | (0x00, 0x30, 0x38, 0x3C, 0x40, 0x44, 0x48, 0x4C)[c & 7] for c in range(16))


def quantize_to_e2m1(x: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 code of every element (uint8 in [0, 15]); a tie goes to the smaller magnitude,
    a value that rounds to zero loses its sign."""
    ax = x.abs()
    code = torch.zeros_like(x, dtype=torch.uint8)
    for boundary in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
        code += (ax > boundary).to(torch.uint8)
    return code | (((x < 0) & (code != 0)).to(torch.uint8) << 3)


def pack_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """[..., n] codes -> [..., n/2] bytes, element 2j in the low nibble of byte j."""
    assert codes.shape[-1] % 2 == 0
    c = codes.to(torch.uint8).reshape(*codes.shape[:-1], codes.shape[-1] // 2, 2)
    return ((c[..., 0] & 0xF) | ((c[..., 1] & 0xF) << 4)).contiguous()


def unpack_e2m1(packed: torch.Tensor) -> torch.Tensor:
    """[..., n/2] bytes -> [..., n] codes."""
    p = packed.view(torch.uint8) if packed.dtype != torch.uint8 else packed
    return torch.stack((p & 0xF, p >> 4), dim=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)


def e2m1_to_e4m3(codes: torch.Tensor) -> torch.Tensor:
    """The E4M3 bytes (uint8) the codes stand for."""
    return torch.tensor(E2M1_TO_E4M3, dtype=torch.uint8, device=codes.device)[codes.long()]


def per_token_cast_to_fp4(x: torch.Tensor, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [m, n] (n % gran_k == 0) -> (packed codes uint8 [m, n/2], uint8 exponents [m, n/gran_k]):
    scale = the power of two >= amax / 6 of every 1 x gran_k group."""
    m, n = x.shape
    assert n % gran_k == 0
    v = x.float().view(m, n // gran_k, gran_k)
    amax = v.abs().amax(dim=2).clamp_min(1e-4)
    e = ceil_to_ue8m0(amax / 6.0)
    codes = quantize_to_e2m1(v * (1.0 / ue8m0_to_float(e)).unsqueeze(2)).view(m, n)
    return pack_e2m1(codes), e


def per_block_cast_to_fp4(w: torch.Tensor, gran: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """w [m, n] (both % gran == 0) -> (packed codes uint8 [m, n/2], uint8 exponents [m/gran, n/gran]):
    the weight format of ``fp8_fp4_mega_moe`` (128 x 128 blocks share one scale, as for 8-bit weights)."""
    m, n = w.shape
    assert m % gran == 0 and n % gran == 0
    v = w.float().view(m // gran, gran, n // gran, gran)
    amax = v.abs().amax(dim=(1, 3)).clamp_min(1e-4)
    e = ceil_to_ue8m0(amax / 6.0)
    codes = quantize_to_e2m1(v * (1.0 / ue8m0_to_float(e))[:, None, :, None]).view(m, n)
    return pack_e2m1(codes), e


def cast_back_from_fp4(packed: torch.Tensor, e: torch.Tensor, gran_k: int = 128) -> torch.Tensor:
    """Inverse of per_token_cast_to_fp4: float32 [m, n]."""
    codes = unpack_e2m1(packed)
    mag = torch.tensor(E2M1_MAGNITUDES, dtype=torch.float32, device=codes.device)[(codes & 7).long()]
    val = torch.where((codes & 8) != 0, -mag, mag)
    idx = torch.arange(codes.shape[1], device=codes.device) // gran_k
    return val * ue8m0_to_float(e)[:, idx]
