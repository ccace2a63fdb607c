"""ctypes front-end of the CPU oracle (TEST INFRASTRUCTURE — never on the product path).

Only tests, the smoke entry and the benchmark's CPU-baseline leg import this
module.  It loads ``libmoe_oracle.so`` (this repository's restatement,
``moe_oracle.cpp``) and, when present, ``_ref/libmoe_ref.so`` (the reference's
own host functions compiled from its sources by ``oracle/Makefile``), and adds
numpy helpers: seeded input generators for the benchmark configurations and a
whole-world model of one MoE layer that returns every intermediate the CUDA
path materialises (routing tables, pool rows, FP8 hidden, bf16 rows, y).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C")
_i64p = np.ctypeslib.ndpointer(np.int64, flags="C")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C")


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference shim when the reference tree exists)."""
    so = os.path.join(_HERE, "libmoe_oracle.so")
    src = os.path.join(_HERE, "moe_oracle.cpp")
    stale = (not os.path.exists(so)) or os.path.getmtime(so) < os.path.getmtime(src)
    if force or stale or not os.path.exists(os.path.join(_HERE, "_ref", "libmoe_ref.so")):
        subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL)


def _opt(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    path = os.path.join(_HERE, "libmoe_oracle.so")
    if not os.path.exists(path):
        build()
    L = C.CDLL(path)
    L.orc_e4m3_decode.restype = C.c_float
    L.orc_e4m3_decode.argtypes = [C.c_uint8]
    L.orc_e4m3_quantize.restype = C.c_uint8
    L.orc_e4m3_quantize.argtypes = [C.c_float]
    L.orc_bf16_to_f32.restype = C.c_float
    L.orc_bf16_to_f32.argtypes = [C.c_uint16]
    L.orc_f32_to_bf16.restype = C.c_uint16
    L.orc_f32_to_bf16.argtypes = [C.c_float]
    L.orc_ue8m0_ceil.restype = C.c_uint8
    L.orc_ue8m0_ceil.argtypes = [C.c_float]
    L.orc_ue8m0_to_f32.restype = C.c_float
    L.orc_ue8m0_to_f32.argtypes = [C.c_uint8]
    L.orc_quant_rows_1x128.argtypes = [_f32p, C.c_int, C.c_int, _u8p, _u8p]
    L.orc_quant_blocks_128x128.argtypes = [_f32p, C.c_int, C.c_int, _u8p, _u8p]
    L.orc_dequant_rows_1x128.argtypes = [_u8p, C.c_void_p, C.c_int, C.c_int, _f32p]
    L.orc_route.argtypes = [_i64p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                            C.c_uint32, _i32p, _u32p, _u32p, _i32p]
    L.orc_pool_map.restype = C.c_int
    L.orc_pool_map.argtypes = [_i32p, _u32p, C.c_int, C.c_int, C.c_int, C.c_int, _i32p, _i32p]
    L.orc_schedule.restype = C.c_int
    L.orc_schedule.argtypes = [_i32p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, _i32p, _i32p,
                               C.POINTER(C.c_int), C.POINTER(C.c_int)]
    L.orc_gs_schedule_member.restype = C.c_int
    L.orc_gs_schedule_member.argtypes = [_i32p, C.c_int, C.c_int, C.c_int, C.c_int, _i32p, _i32p, C.c_int]
    L.orc_gs_schedule_member_hot.restype = C.c_int
    L.orc_gs_schedule_member_hot.argtypes = [_i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _i32p, _i32p, C.c_int]
    L.orc_lpt_assign.restype = C.c_int
    L.orc_lpt_assign.argtypes = [_i32p, _i32p, C.c_int, C.c_int, C.c_int, C.c_int, _i32p, _i32p,
                                 np.ctypeslib.ndpointer(np.int64, flags="C")]
    L.orc_select_win.restype = C.c_int
    L.orc_select_win.argtypes = [_u32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
    L.orc_fill_weights.argtypes = [_u8p, C.c_longlong, C.c_int, C.c_uint32]
    L.orc_fill_weights_e2m1.argtypes = [_u8p, C.c_longlong, C.c_int, C.c_uint32]
    L.orc_expand_e2m1.argtypes = [_u8p, C.c_longlong, C.c_int, _u8p]
    L.orc_e2m1_to_e4m3.argtypes = [C.c_uint8]
    L.orc_e2m1_to_e4m3.restype = C.c_uint8
    L.orc_l1.argtypes = [_u8p, C.c_void_p, _u8p, C.c_void_p, C.c_int, C.c_int, C.c_int, _f32p, C.c_int]
    L.orc_requant.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _u8p, C.c_void_p]
    L.orc_l2.argtypes = [_u8p, C.c_void_p, _u8p, C.c_void_p, C.c_int, C.c_int, C.c_int, _f32p, C.c_int]
    L.orc_reduce_all.argtypes = [_u16p, _i64p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                 _f32p, C.c_int]
    L.orc_f32_to_bf16_n.argtypes = [_f32p, C.c_longlong, _u16p]
    L.orc_e4m3_decode_n.argtypes = [_u8p, C.c_longlong, _f32p]
    L.orc_e4m3_quantize_n.argtypes = [_f32p, C.c_longlong, _u8p]
    _LIB = L
    return L


def ref_lib():
    """The reference's own host functions (None when the shim was never built)."""
    global _REF
    if _REF is not None:
        return _REF
    path = os.path.join(_HERE, "_ref", "libmoe_ref.so")
    if not os.path.exists(path):
        return None
    L = C.CDLL(path)
    L.ref_const.restype = C.c_int
    L.ref_const.argtypes = [C.c_int]
    L.ref_e4m3_decode.restype = C.c_float
    L.ref_e4m3_decode.argtypes = [C.c_uint8]
    L.ref_e4m3_quantize.restype = C.c_uint8
    L.ref_e4m3_quantize.argtypes = [C.c_float]
    L.ref_bf16_to_f32.restype = C.c_float
    L.ref_bf16_to_f32.argtypes = [C.c_uint16]
    L.ref_f32_to_bf16.restype = C.c_uint16
    L.ref_f32_to_bf16.argtypes = [C.c_float]
    L.ref_w_lane_get.restype = C.c_uint8
    L.ref_w_lane_get.argtypes = [_u8p, C.c_int, C.c_int, C.c_int]
    L.ref_pack_lane.argtypes = [_u8p, C.c_int, C.c_int, _u8p]
    L.ref_l1_rows.argtypes = [_u8p, _u8p, C.c_int, C.c_int, _f32p, C.c_int]
    L.ref_l2_rows.argtypes = [_u8p, _u8p, C.c_int, C.c_int, _f32p, C.c_int]
    L.ref_reduce_tokens.argtypes = [_u8p, _i64p, _f32p, C.c_int, C.c_int, C.c_int, _f32p, C.c_int]
    L.ref_quantize.argtypes = [_f32p, C.c_longlong, _u8p]
    L.ref_make_routes.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _i64p]
    L.ref_gs_schedule_member.restype = C.c_int
    L.ref_gs_schedule_member.argtypes = [_i32p, C.c_int, C.c_int, _i32p, _i32p, C.c_int]
    L.ref_select_win.restype = C.c_int
    L.ref_select_win.argtypes = [_u32p, C.c_int, C.c_int, C.c_int]
    L.ref_lpt_assign.restype = C.c_int
    L.ref_lpt_assign.argtypes = [_i32p, C.c_int, C.c_int, C.c_int, C.c_int, _i32p, _i32p,
                                 np.ctypeslib.ndpointer(np.int64, flags="C")]
    _REF = L
    return L


# ------------------------------------------------------------------ thin wrappers
def e4m3_decode(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, np.uint8)
    out = np.empty(b.shape, np.float32)
    lib().orc_e4m3_decode_n(b.reshape(-1), b.size, out.reshape(-1))
    return out


def e4m3_quantize(v: np.ndarray) -> np.ndarray:
    v = np.ascontiguousarray(v, np.float32)
    out = np.empty(v.shape, np.uint8)
    lib().orc_e4m3_quantize_n(v.reshape(-1), v.size, out.reshape(-1))
    return out


def f32_to_bf16(v: np.ndarray) -> np.ndarray:
    v = np.ascontiguousarray(v, np.float32)
    out = np.empty(v.shape, np.uint16)
    lib().orc_f32_to_bf16_n(v.reshape(-1), v.size, out.reshape(-1))
    return out


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def ue8m0_to_f32(e: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(e, np.uint8).astype(np.uint32) << 23).view(np.float32)


def quant_rows_1x128(x: np.ndarray):
    x = np.ascontiguousarray(x, np.float32)
    r, c = x.shape
    q = np.empty((r, c), np.uint8)
    sf = np.empty((r, c // 128), np.uint8)
    lib().orc_quant_rows_1x128(x, r, c, q, sf)
    return q, sf


def quant_blocks_128x128(w: np.ndarray):
    w = np.ascontiguousarray(w, np.float32)
    r, c = w.shape
    q = np.empty((r, c), np.uint8)
    sf = np.empty((r // 128, c // 128), np.uint8)
    lib().orc_quant_blocks_128x128(w, r, c, q, sf)
    return q, sf


def dequant_rows_1x128(q: np.ndarray, sf: Optional[np.ndarray]) -> np.ndarray:
    q = np.ascontiguousarray(q, np.uint8)
    out = np.empty(q.shape, np.float32)
    if sf is not None:
        sf = np.ascontiguousarray(sf, np.uint8)
    lib().orc_dequant_rows_1x128(q, _opt(sf), q.shape[0], q.shape[1], out)
    return out


def l1(x, x_sf, w1, w1_sf, threads=8) -> np.ndarray:
    """silu(x.W1[:I]^T) * (x.W1[I:]^T) for one expert, FP32, before re-quantisation."""
    x = np.ascontiguousarray(x, np.uint8)
    w1 = np.ascontiguousarray(w1, np.uint8)
    rows, H = x.shape
    I = w1.shape[0] // 2
    out = np.empty((rows, I), np.float32)
    if rows:
        xs = None if x_sf is None else np.ascontiguousarray(x_sf, np.uint8)
        ws = None if w1_sf is None else np.ascontiguousarray(w1_sf, np.uint8)
        lib().orc_l1(x, _opt(xs), w1, _opt(ws), rows, H, I, out, threads)
    return out


def requant(h, scaled: bool):
    h = np.ascontiguousarray(h, np.float32)
    rows, I = h.shape
    q = np.empty((rows, I), np.uint8)
    sf = np.empty((rows, I // 128), np.uint8) if scaled else None
    if rows:
        lib().orc_requant(h, rows, I, int(scaled), q, _opt(sf))
    return q, sf


def l2(a, a_sf, w2, w2_sf, threads=8) -> np.ndarray:
    a = np.ascontiguousarray(a, np.uint8)
    w2 = np.ascontiguousarray(w2, np.uint8)
    rows, I = a.shape
    H = w2.shape[0]
    out = np.empty((rows, H), np.float32)
    if rows:
        as_ = None if a_sf is None else np.ascontiguousarray(a_sf, np.uint8)
        ws = None if w2_sf is None else np.ascontiguousarray(w2_sf, np.uint8)
        lib().orc_l2(a, _opt(as_), w2, _opt(ws), rows, I, H, out, threads)
    return out


def reduce_all(combine_rows, topk_idx, weights, tokens, E, threads=8) -> np.ndarray:
    """combine_rows [topk][cap][H] uint16 (bf16 bits) -> y [tokens][H] float32."""
    combine_rows = np.ascontiguousarray(combine_rows, np.uint16)
    topk, cap, H = combine_rows.shape
    y = np.zeros((tokens, H), np.float32)
    if tokens:
        lib().orc_reduce_all(combine_rows, np.ascontiguousarray(topk_idx, np.int64),
                             np.ascontiguousarray(weights, np.float32), tokens, topk, E, cap, H,
                             y, threads)
    return y


def fill_weights(n_rows: int, k_cols: int, seed: int) -> np.ndarray:
    w = np.empty((n_rows, k_cols), np.uint8)
    lib().orc_fill_weights(w, n_rows, k_cols, seed)
    return w


def fill_weights_e2m1(n_rows: int, k_cols: int, seed: int) -> np.ndarray:
    """Packed e2m1 test weights [n_rows, k_cols / 2] (reference: WPROBE_FP4_CODE, src/common.cuh:127-131)."""
    w = np.empty((n_rows, k_cols // 2), np.uint8)
    lib().orc_fill_weights_e2m1(w, n_rows, k_cols, seed)
    return w


def expand_e2m1(packed: np.ndarray) -> np.ndarray:
    """Packed e2m1 codes [..., k / 2] -> the E4M3 bytes [..., k] they stand for (reference:
    fp4_code_to_fp8, src/common.cuh:116-126; w_lane_get of the 4-bit build, src/bench_check.cuh:405-421).
    The oracle of the 4-bit layer is the 8-bit oracle on these bytes."""
    p = np.ascontiguousarray(packed, np.uint8)
    rows = int(np.prod(p.shape[:-1])) if p.ndim > 1 else 1
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), np.uint8)
    lib().orc_expand_e2m1(p.reshape(rows, -1), rows, p.shape[-1] * 2, out.reshape(rows, -1))
    return out


def schedule(expert_rows, row_base, win_cap, nt1, nt2):
    expert_rows = np.ascontiguousarray(expert_rows, np.int32)
    row_base = np.ascontiguousarray(row_base, np.int32)
    EPR = expert_rows.size
    max_w = int(sum((int(c) + win_cap - 1) // win_cap for c in expert_rows)) + 1
    windows = np.zeros((max_w, 3), np.int32)
    tasks = np.zeros((max_w * (nt1 + nt2) + 1, 4), np.int32)
    nw, n1 = C.c_int(0), C.c_int(0)
    n = lib().orc_schedule(expert_rows, row_base, EPR, win_cap, nt1, nt2, windows, tasks,
                           C.byref(nw), C.byref(n1))
    return windows[: nw.value].copy(), tasks[:n].copy(), n1.value


# ------------------------------------------------------------------ input generators
@dataclass
class Case:
    """One seeded workload for a world of R ranks (whole-world arrays, host side)."""
    R: int
    EPR: int
    topk: int
    H: int
    I: int
    cap: int                      # max tokens per rank (buffer rows)
    tokens: List[int]             # valid tokens per rank
    scaled: bool
    x: np.ndarray                 # [R][cap][H] uint8 E4M3
    x_sf: Optional[np.ndarray]    # [R][cap][H/128] uint8 UE8M0
    topk_idx: np.ndarray          # [R][cap][topk] int64
    topk_w: np.ndarray            # [R][cap][topk] float32
    w1: np.ndarray                # [E][2I][H] uint8
    w1_sf: Optional[np.ndarray]   # [E][2I/128][H/128]
    w2: np.ndarray                # [E][H][I] uint8
    w2_sf: Optional[np.ndarray]   # [E][H/128][I/128]
    name: str = ""

    @property
    def E(self):
        return self.R * self.EPR


def _bf16_round(a: np.ndarray) -> np.ndarray:
    return bf16_to_f32(f32_to_bf16(a.astype(np.float32)))


def gen_routing(kind: str, rng, T: int, E: int, topk: int, perm=None) -> np.ndarray:
    """topk_idx [T][topk]: 'uniform' = distinct experts uniformly; 'zipf' = without
    replacement from Zipf(s=1.2) popularity over a seeded permutation; 'logits' =
    top-k of N(0,1) router logits (ties to the lower index)."""
    out = np.empty((T, topk), np.int64)
    if kind == "uniform":
        for t in range(T):
            out[t] = rng.choice(E, size=topk, replace=False)
    elif kind == "zipf":
        p = 1.0 / np.arange(1, E + 1) ** 1.2
        p /= p.sum()
        for t in range(T):
            out[t] = perm[rng.choice(E, size=topk, replace=False, p=p)]
    elif kind == "logits":
        lg = rng.standard_normal((T, E)).astype(np.float32)
        out[:] = np.argsort(-lg, axis=1, kind="stable")[:, :topk]
    else:
        raise ValueError(kind)
    return out


def gen_case(R, EPR, topk, H, I, tokens, seed=0, routing="uniform", scaled=True, cap=None,
             invalid_frac=0.0, name="") -> Case:
    """Seeded synthetic layer: x ~ N(0,1) in bf16 -> 1x128 UE8M0 E4M3; W1/W2 ~ N(0,0.02)
    -> 128x128 UE8M0 E4M3; router weights = softmax over the chosen k of N(0,1) logits.
    With scaled=False the tensors are raw casts (values kept inside E4M3 range), which
    is the reference kernel's own mode (scale == 1)."""
    rng = np.random.default_rng(seed)
    E = R * EPR
    if isinstance(tokens, int):
        tokens = [tokens] * R
    cap = cap or max(max(tokens), 1)
    x = np.zeros((R, cap, H), np.uint8)
    x_sf = np.full((R, cap, H // 128), 127, np.uint8) if scaled else None
    ti = np.zeros((R, cap, topk), np.int64)
    tw = np.zeros((R, cap, topk), np.float32)
    perm = rng.permutation(E)
    for r in range(R):
        T = tokens[r]
        if T == 0:
            continue
        xf = _bf16_round(rng.standard_normal((T, H)))
        if scaled:
            x[r, :T], x_sf[r, :T] = quant_rows_1x128(xf)
        else:
            x[r, :T] = e4m3_quantize(xf * 0.25)
        ti[r, :T] = gen_routing(routing, rng, T, E, topk, perm)
        if invalid_frac > 0:
            bad = rng.random((T, topk)) < invalid_frac
            ti[r, :T][bad] = -1
        lg = rng.standard_normal((T, topk)).astype(np.float32)
        ex = np.exp(lg - lg.max(axis=1, keepdims=True))
        tw[r, :T] = (ex / ex.sum(axis=1, keepdims=True)).astype(np.float32)
    w1 = np.empty((E, 2 * I, H), np.uint8)
    w2 = np.empty((E, H, I), np.uint8)
    w1_sf = np.empty((E, 2 * I // 128, H // 128), np.uint8) if scaled else None
    w2_sf = np.empty((E, H // 128, I // 128), np.uint8) if scaled else None
    for e in range(E):
        a = (rng.standard_normal((2 * I, H)) * 0.02).astype(np.float32)
        b = (rng.standard_normal((H, I)) * 0.02).astype(np.float32)
        if scaled:
            w1[e], w1_sf[e] = quant_blocks_128x128(a)
            w2[e], w2_sf[e] = quant_blocks_128x128(b)
        else:
            w1[e] = e4m3_quantize(a)
            w2[e] = e4m3_quantize(b)
    return Case(R, EPR, topk, H, I, cap, list(tokens), scaled, x, x_sf, ti, tw, w1, w1_sf, w2, w2_sf, name)


def gen_case_bytes(R, EPR, topk, H, I, tokens, seed=0, routing="uniform", cap=None, name="") -> Case:
    """Seeded synthetic layer drawn directly as E4M3 bytes + UE8M0 exponents (random sign and
    mantissa, exponent field 3..10, scale bytes near 2^-9 for weights and 2^-3 for activations):
    same shapes and value range as quantised N(0,0.02) weights / N(0,1) activations, without
    FP32 tensors or a quantisation pass, so that full-width worlds generate in seconds."""
    rng = np.random.default_rng(seed)
    E = R * EPR
    if isinstance(tokens, int):
        tokens = [tokens] * R
    cap = cap or max(max(tokens), 1)

    def fp8(shape):
        n = int(np.prod(shape))
        raw = rng.bit_generator.random_raw((2 * n + 7) // 8).view(np.uint8)   # raw 64-bit words: fastest source
        return ((raw[:n] & 0x87) | (((raw[n:] & 7) + 3) << 3)).reshape(shape)

    x = fp8((R, cap, H))
    x_sf = (rng.integers(0, 3, (R, cap, H // 128)) + 124).astype(np.uint8)
    ti = np.zeros((R, cap, topk), np.int64)
    tw = np.zeros((R, cap, topk), np.float32)
    perm = rng.permutation(E)
    for r in range(R):
        T = tokens[r]
        if T == 0:
            continue
        ti[r, :T] = gen_routing(routing, rng, T, E, topk, perm)
        lg = rng.standard_normal((T, topk)).astype(np.float32)
        ex = np.exp(lg - lg.max(axis=1, keepdims=True))
        tw[r, :T] = (ex / ex.sum(axis=1, keepdims=True)).astype(np.float32)
    # one random block per weight kind; expert e holds it rotated by a prime multiple of e bytes
    # (distinct per expert, and a full-width world of 1.2 GB generates in a few seconds)
    b1, b2 = fp8((2 * I * H,)), fp8((H * I,))
    w1 = np.empty((E, 2 * I, H), np.uint8)
    w2 = np.empty((E, H, I), np.uint8)
    for e in range(E):
        w1[e] = np.roll(b1, e * 7919).reshape(2 * I, H)
        w2[e] = np.roll(b2, e * 4099).reshape(H, I)
    w1_sf = (rng.integers(0, 3, (E, 2 * I // 128, H // 128)) + 118).astype(np.uint8)
    w2_sf = (rng.integers(0, 3, (E, H // 128, I // 128)) + 118).astype(np.uint8)
    return Case(R, EPR, topk, H, I, cap, list(tokens), True, x, x_sf, ti, tw, w1, w1_sf, w2, w2_sf, name)


def routes_from_counts(per_expert, R: int, tokens: int, topk: int) -> np.ndarray:
    """Routes [R][tokens][topk] that reproduce recorded per-expert received-pair counts
    (the replay of the reference's real-serving TK_INFO corpora, test/mega_common.cuh:460-482):
    walking the global experts in order, the j-th pair overall goes to source rank j % R,
    q = j / R, token q % tokens, top-k position q / tokens.  Raises if the counts do not
    fill R*tokens*topk pairs or a token would name an expert twice."""
    per_expert = np.asarray(per_expert, np.int64)
    total = int(per_expert.sum())
    if total != R * tokens * topk:
        raise ValueError(f"counts hold {total} pairs, the world has {R * tokens * topk}")
    ge = np.repeat(np.arange(per_expert.size, dtype=np.int64), per_expert)   # expert of pair j
    j = np.arange(total)
    src, q = j % R, j // R
    out = np.zeros((R, tokens, topk), np.int64)
    out[src, q % tokens, q // tokens] = ge
    srt = np.sort(out, axis=2)
    if (srt[:, :, 1:] == srt[:, :, :-1]).any():
        raise ValueError("a token names an expert twice")
    return out


def with_routes(case: Case, routes: np.ndarray) -> Case:
    """The same case with its top-k expert ids replaced by `routes` [R][tokens][topk]."""
    ti = case.topk_idx.copy()
    for r in range(case.R):
        ti[r, : case.tokens[r]] = routes[r, : case.tokens[r]]
    return Case(case.R, case.EPR, case.topk, case.H, case.I, case.cap, list(case.tokens), case.scaled, case.x,
                case.x_sf, ti, case.topk_w, case.w1, case.w1_sf, case.w2, case.w2_sf, case.name)


def gen_reference_fixture(R, EPR, topk, H, I, tokens, pattern="balanced", salt=0, cap=None) -> Case:
    """The reference harness's deterministic fixtures with run-time geometry:
    x byte (rank*37 + t*7 + c*3) & 0x3f and top-k weight 1 + 0.25*rank + 0.01*(i%7)
    (test/mega_common.cuh:167-178); weights WPROBE_VAL with seeds 17 / 91
    (src/megakernel.h:46-47, test/mega_common.cuh:229-241), every rank holding the
    same bytes; routes balanced / hot / mixed-invalid (src/bench_check.cuh:42-69)."""
    E = R * EPR
    cap = cap or tokens
    x = np.zeros((R, cap, H), np.uint8)
    ti = np.zeros((R, cap, topk), np.int64)
    tw = np.zeros((R, cap, topk), np.float32)
    t_ = np.arange(cap)[:, None]
    c_ = np.arange(H)[None, :]
    for r in range(R):
        x[r] = ((r * 37 + t_ * 7 + c_ * 3) & 0x3F).astype(np.uint8)
        i = np.arange(cap * topk)
        tw[r] = (np.float32(1.0) + np.float32(r) * np.float32(0.25)
                 + (i % 7).astype(np.float32) * np.float32(0.01)).reshape(cap, topk)
        n = tokens * topk
        idx = np.arange(n)
        if pattern == "balanced":
            v = (idx + r * EPR + salt) % E
        elif pattern == "hot":
            v = np.where(idx % 4 != 3, 0, 1 + (idx // 4 + r * 3 + salt) % (E - 1))
        elif pattern == "mixed-invalid":
            s = (0x9E3779B97F4A7C15 ^ ((r + 1) * 0x1234567)) & 0xFFFFFFFFFFFFFFFF
            s ^= (salt * 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
            v = np.empty(n, np.int64)
            for j in range(n):
                s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
                v[j] = -1 if ((s >> 33) % 100) < 10 else (s >> 20) % E
        else:
            raise ValueError(pattern)
        ti[r, :tokens] = np.asarray(v, np.int64).reshape(tokens, topk)
    w1_one = fill_weights(EPR * 2 * I, H, 17).reshape(EPR, 2 * I, H)
    w2_one = fill_weights(EPR * H, I, 91).reshape(EPR, H, I)
    w1 = np.concatenate([w1_one] * R, axis=0)
    w2 = np.concatenate([w2_one] * R, axis=0)
    return Case(R, EPR, topk, H, I, cap, [tokens] * R, False, x, None, ti, tw, w1, None, w2, None,
                f"ref-{pattern}")


# ------------------------------------------------------------------ whole-world model
@dataclass
class RankState:
    route_slot_counts: np.ndarray     # [E] int32 (as source rank)
    src_index_table: np.ndarray       # [EPR][R][slot_cap] uint32 (as owner)
    recv_counts: np.ndarray           # [R][recv_stride] uint32 (as owner)
    prefix_tbl: np.ndarray            # [EPR][R+1] int32
    row_base: np.ndarray              # [EPR+1] int32
    meta: np.ndarray                  # [rows][3] (src, token, k)
    pool: np.ndarray = None           # [rows][H] uint8
    pool_sf: np.ndarray = None
    h: np.ndarray = None              # [rows][I] float32 (pre-quant)
    ffn: np.ndarray = None            # [rows][I] uint8
    ffn_sf: np.ndarray = None
    out: np.ndarray = None            # [rows][H] float32 (pre-bf16)
    combine_rows: np.ndarray = None   # [topk][cap][H] uint16 (as source rank)
    y: np.ndarray = None              # [tokens][H] float32


def route_world(case: Case, slot_cap: Optional[int] = None, recv_stride: int = 0,
                epoch: int = 1) -> List[RankState]:
    R, EPR, topk = case.R, case.EPR, case.topk
    E = R * EPR
    slot_cap = slot_cap or case.cap
    recv_stride = recv_stride or ((EPR + 1 + 3) & ~3)
    rsc = np.zeros((R, E), np.int32)
    tbl = np.zeros((R, EPR, R, slot_cap), np.uint32)
    recv = np.zeros((R, R, recv_stride), np.uint32)
    pfx = np.zeros((R, EPR, R + 1), np.int32)
    lib().orc_route(np.ascontiguousarray(case.topk_idx), np.asarray(case.tokens, np.int32), R, EPR,
                    topk, case.cap, slot_cap, recv_stride, epoch, rsc, tbl, recv, pfx)
    out = []
    for r in range(R):
        rows = int(pfx[r, :, R].sum())
        row_base = np.zeros(EPR + 1, np.int32)
        meta = np.zeros((max(rows, 1), 3), np.int32)
        n = lib().orc_pool_map(np.ascontiguousarray(pfx[r]), np.ascontiguousarray(tbl[r]), R, EPR,
                               topk, slot_cap, row_base, meta)
        assert n == rows
        out.append(RankState(rsc[r].copy(), tbl[r].copy(), recv[r].copy(), pfx[r].copy(), row_base,
                             meta[:rows].copy()))
    return out


def layer_world(case: Case, slot_cap: Optional[int] = None, threads: int = 8,
                only_rank: Optional[int] = None) -> List[RankState]:
    """Run the whole layer on the CPU for every rank of the world.

    y_r[t] = sum_k w_k * bf16( requant(SwiGLU(x W1_e^T)) W2_e^T ), k ascending, FP32.
    With ``only_rank`` the expert-side compute is done for that owner rank only
    (the other ranks keep routing tables but no numerics, and no y is produced).
    """
    R, EPR, topk, H, I = case.R, case.EPR, case.topk, case.H, case.I
    st = route_world(case, slot_cap)
    comb = [np.zeros((topk, case.cap, H), np.uint16) for _ in range(R)]
    for r in range(R):
        if only_rank is not None and r != only_rank:
            continue
        s = st[r]
        rows = s.meta.shape[0]
        s.pool = np.zeros((rows, H), np.uint8)
        s.pool_sf = np.zeros((rows, H // 128), np.uint8) if case.scaled else None
        for g in range(rows):
            src, tok, _ = s.meta[g]
            s.pool[g] = case.x[src, tok]
            if case.scaled:
                s.pool_sf[g] = case.x_sf[src, tok]
        s.h = np.zeros((rows, I), np.float32)
        s.ffn = np.zeros((rows, I), np.uint8)
        s.ffn_sf = np.zeros((rows, I // 128), np.uint8) if case.scaled else None
        s.out = np.zeros((rows, H), np.float32)
        for le in range(EPR):
            a, b = int(s.row_base[le]), int(s.row_base[le + 1])
            if a == b:
                continue
            e = r * EPR + le
            s.h[a:b] = l1(s.pool[a:b], None if not case.scaled else s.pool_sf[a:b], case.w1[e],
                          None if not case.scaled else case.w1_sf[e], threads)
            q, sf = requant(s.h[a:b], case.scaled)
            s.ffn[a:b] = q
            if case.scaled:
                s.ffn_sf[a:b] = sf
            s.out[a:b] = l2(q, sf, case.w2[e], None if not case.scaled else case.w2_sf[e], threads)
        ob = f32_to_bf16(s.out)
        for g in range(rows):
            src, tok, k = s.meta[g]
            comb[src][k, tok] = ob[g]
    for r in range(R):
        st[r].combine_rows = comb[r]
        if only_rank is None:
            st[r].y = reduce_all(comb[r], case.topk_idx[r], case.topk_w[r], case.tokens[r],
                                 R * EPR, threads)
    return st


def helper_world(case: Case, states: List[RankState], group_ranks: int, win_cap: int, skew_num: int = 2,
                 max_windows: int = 512, hot_windows: int = 0):
    """Cross-rank helper scheduling of the reference (src/compute.cuh:700-835, src/group_sched.cuh):
    ranks form interleaved groups (group = rank % n_groups, member = rank // n_groups); when a
    group's load is skewed (max * n_experts > skew_num * sum; skew_num 0 = always) its (expert,
    window) units are spread over the members by gs_schedule_member, and a member computes the
    windows it was given — its own and other members' — in the order of its list, the rows of a
    window keeping the owner's pool order.  Returns per rank a dict: on (bool), windows
    [(ge, w, rows)], meta [rows][3] (src, token, k) in the rank's pool order; ranks of groups that
    are not skewed keep the owner layout (on = False, meta = the owner's).
    hot_windows > 0 (the CUDA path's default is 3): only experts with at least that many windows are
    spread, the others stay with their owners; a group without a hot expert is left alone."""
    R, EPR = case.R, case.EPR
    n_groups = R // group_ranks
    out = [None] * R
    for g in range(n_groups):
        members = [g + m * n_groups for m in range(group_ranks)]
        tot = np.zeros(group_ranks * EPR, np.int32)
        for m, r in enumerate(members):
            tot[m * EPR:(m + 1) * EPR] = states[r].prefix_tbl[:, R]
        skewed = int(tot.max()) * tot.size > skew_num * int(tot.sum())
        # a member's list holds at most max_windows entries (reference kGsMemberCap); the CUDA path keeps
        # the owner layout when the whole group has more windows than that
        skewed = skewed and int(sum((int(c) + win_cap - 1) // win_cap for c in tot)) <= max_windows
        skewed = skewed and (hot_windows <= 0 or (int(tot.max()) + win_cap - 1) // win_cap >= hot_windows)
        for m, r in enumerate(members):
            if not skewed:
                out[r] = {"on": False, "windows": [], "meta": states[r].meta.copy()}
                continue
            ge = np.zeros(max_windows, np.int32)
            w = np.zeros(max_windows, np.int32)
            n = lib().orc_gs_schedule_member_hot(tot, EPR, group_ranks, win_cap, m, max(hot_windows, 0), ge, w, max_windows)
            if n > max_windows:
                raise ValueError("member window list exceeds its capacity")
            wins, meta = [], []
            for i in range(n):
                owner = members[int(ge[i]) // EPR]
                le = int(ge[i]) % EPR
                rows = min(win_cap, int(tot[ge[i]]) - int(w[i]) * win_cap)
                a0 = int(states[owner].row_base[le]) + int(w[i]) * win_cap
                wins.append((int(ge[i]), int(w[i]), rows))
                meta.append(states[owner].meta[a0:a0 + rows])
            out[r] = {"on": True, "windows": wins,
                      "meta": np.concatenate(meta) if meta else np.zeros((0, 3), np.int32)}
    return out


def rel_l2(got: np.ndarray, want: np.ndarray) -> float:
    """max over rows of ||got-want||_2 / ||want||_2 (rows with zero norm compare absolutely)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    if got.size == 0:
        return 0.0
    num = np.sqrt(((got - want) ** 2).sum(axis=-1))
    den = np.sqrt((want ** 2).sum(axis=-1))
    return float(np.max(num / np.maximum(den, 1e-20)))


def check_close(got, want, rel_tol, abs_tol) -> Dict[str, float]:
    """The reference's element test |got-want| <= max(abs_tol, rel_tol*|want|)
    (src/bench_check.cuh:522-547); returns counts and maxima."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    d = np.abs(got - want)
    both_nan = np.isnan(got) & np.isnan(want)
    one_nan = np.isnan(got) ^ np.isnan(want)
    d = np.where(both_nan, 0.0, d)
    bad = (d > np.maximum(abs_tol, rel_tol * np.abs(want))) | one_nan
    return {"n": int(d.size), "bad": int(bad.sum()), "max_abs": float(np.nanmax(d)) if d.size else 0.0}
