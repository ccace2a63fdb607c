"""Generate the golden fixtures under tests/golden/ from the REFERENCE itself.

Run in a container that has the reference checkout (its path is the first argument):

    python tests/golden/make_golden.py /path/to/reference [--only-tk-info | --only-e2m1]

Three sources are used, none copied into this repository:
  * the reference's host-side C++ functions, compiled from its sources into
    oracle/_ref/libmoe_ref.so by oracle/Makefile (E4M3/bf16 codecs, ref_l1,
    ref_l2, ref_reduce, make_routes, gs_schedule_member, select_win, lpt_assign);
  * the reference's Python quantisers, imported by file path from
    torch/mxmegakernel/utils/math.py (ceil_to_ue8m0, per_token_cast_to_fp8,
    per_block_cast_to_fp8, cast_back_from_fp8; for e2m1.npz _quantize_to_fp4_e2m1,
    per_token_cast_to_fp4, cast_back_from_fp4, _dequantize_from_fp4_e2m1).
  * the reference's recorded route corpus test/76.real_decode/dataset.tk_info, of
    which four launches' per-expert counts are kept (tk_info.npz).
The fixtures are small .npz files; tests/test_oracle_golden.py checks the
oracle against them on any machine.
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import oracle as orc  # noqa: E402


def make_tk_info(ref_root):
    """A sample of the reference's real-decode route corpus (test/76.real_decode/dataset.tk_info:
    per launch, the pairs each of 32 ranks x 8 experts received in live serving): the most
    skewed, the median and the least skewed of the 4096-pair launches, and the most skewed
    launch with fewer pairs.  Stored as counts per global expert [launches][256]."""
    import collections
    import re
    launches = collections.OrderedDict()
    with open(os.path.join(ref_root, "test", "76.real_decode", "dataset.tk_info"), errors="ignore") as fh:
        for line in fh:
            m = re.match(r"\[TK_INFO\] rank=(\d+) launch=(\d+) n=(\d+) : (.*)", line.strip())
            if m:
                launches.setdefault(int(m.group(2)), {})[int(m.group(1))] = [int(v) for v in m.group(4).split()]
    full = {k: np.array([d[r] for r in range(32)], np.int32).reshape(-1) for k, d in launches.items()
            if len(d) == 32 and all(len(v) == 8 for v in d.values())}
    skew = lambda c: c.max() / c.mean()
    big = sorted((k for k, c in full.items() if c.sum() == 4096), key=lambda k: skew(full[k]))
    small = sorted((k for k, c in full.items() if c.sum() < 4096 and c.sum() % 64 == 0 and c.sum() >= 2048),
                   key=lambda k: skew(full[k]))
    pick = [big[-1], big[len(big) // 2], big[0], small[-1]]
    np.savez_compressed(os.path.join(HERE, "tk_info.npz"), launch=np.array(pick, np.int32),
                        counts=np.stack([full[k] for k in pick]))
    print("tk_info launches", pick, "pairs", [int(full[k].sum()) for k in pick],
          "max/mean", [round(float(skew(full[k])), 1) for k in pick])


def _ref_math(ref_root):
    spec = importlib.util.spec_from_file_location(
        "ref_math", os.path.join(ref_root, "torch", "mxmegakernel", "utils", "math.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def make_e2m1(m):
    """4-bit (e2m1) codes: the reference's Python quantiser, packing and value table
    (torch/mxmegakernel/utils/math.py:84-164)."""
    import torch
    g4 = torch.Generator().manual_seed(5)
    x4 = torch.randn((6, 384), generator=g4).bfloat16()
    x4[1, 128:256] = 0            # all-zero group -> amax clamp
    x4[2, :128] *= 300.0
    p4, sf4 = m.per_token_cast_to_fp4(x4, use_ue8m0=True, gran_k=128)
    back4 = m.cast_back_from_fp4(p4, sf4, 128)
    q_in = torch.tensor([0.0, 0.25, 0.2500001, -0.25, 0.75, 0.76, 1.25, 1.3, 1.75, 1.8, 2.5, 2.6, 3.5, 3.6, 5.0, 5.1,
                         6.0, 100.0, -0.1, -0.3, -6.0, -7.0], dtype=torch.float32)
    q_codes = m._quantize_to_fp4_e2m1(q_in).view(torch.uint8)
    codes = torch.arange(16, dtype=torch.int8)
    code_e4m3 = m._dequantize_from_fp4_e2m1(codes).to(torch.float8_e4m3fn).view(torch.uint8)
    code_e4m3[8] = 0x80           # the value table folds -0 into +0; the kernel keeps the sign bit of the code
    np.savez_compressed(
        os.path.join(HERE, "e2m1.npz"),
        x=x4.float().numpy(), x_packed=p4.view(torch.uint8).numpy(),
        x_sf=(sf4.contiguous().view(torch.int32) >> 23).to(torch.uint8).numpy(), x_back=back4.numpy(),
        q_in=q_in.numpy(), q_codes=q_codes.numpy(), code_e4m3=code_e4m3.numpy())


def main():
    ref_root = next((a for a in sys.argv[1:] if not a.startswith("--")), os.environ.get("REF", ""))
    if not os.path.isdir(os.path.join(ref_root, "src")):
        sys.exit("usage: make_golden.py /path/to/reference [--only-tk-info | --only-e2m1]  (or REF=/path/to/reference)")
    if "--only-e2m1" in sys.argv:
        make_e2m1(_ref_math(ref_root))
        return
    if "--only-tk-info" in sys.argv:
        make_tk_info(ref_root)
        return
    make_tk_info(ref_root)
    orc.build()
    R = orc.ref_lib()
    assert R is not None, "oracle/_ref/libmoe_ref.so missing: run make -C oracle with the reference present"
    H, I, EPR, TOPK = R.ref_const(2), R.ref_const(3), R.ref_const(0), R.ref_const(1)

    # ---- codecs: all 256 E4M3 bytes, a float sweep for the quantiser, bf16 ----
    dec = np.array([R.ref_e4m3_decode(b) for b in range(256)], np.float32)
    rng = np.random.default_rng(7)
    sweep = np.concatenate([
        np.linspace(-500, 500, 2001).astype(np.float32),
        (rng.standard_normal(4000) * np.exp(rng.uniform(-8, 6, 4000))).astype(np.float32),
        dec[np.isfinite(dec)],
        np.array([0.0, -0.0, 1.0 / 1024, 3.0 / 1024, 0.0146484375, 447.9, 448.0, 464.0, 1e9,
                  np.inf, -np.inf, np.nan], np.float32)])
    enc = np.array([R.ref_e4m3_quantize(float(v)) for v in sweep], np.uint8)
    bfin = np.concatenate([(rng.standard_normal(4000) * np.exp(rng.uniform(-20, 20, 4000))).astype(np.float32),
                           np.array([1.00390625, 1.01171875, 3.3895314e38, np.inf], np.float32)])
    bf = np.array([R.ref_f32_to_bf16(float(v)) for v in bfin], np.uint16)
    np.savez_compressed(os.path.join(HERE, "codec.npz"), e4m3_decode=dec, q_in=sweep, q_out=enc,
                        bf16_in=bfin, bf16_out=bf)

    # ---- numerics at the reference's frozen geometry: 3 rows of local expert 2 ----
    expert, rows = 2, 3
    w1_log = orc.fill_weights(EPR * 2 * I, H, 17).reshape(EPR, 2 * I, H)
    w2_log = orc.fill_weights(EPR * H, I, 91).reshape(EPR, H, I)
    # reference lane order; the L1 rows are the reference's gate/up pairing at
    # width 256 (src/bench_check.cuh:444-445): packed row (h/256)*512 + h%256 is
    # the gate of hidden column h and +256 its up row.
    h_idx = np.arange(I)
    grow = (h_idx // 256) * 512 + h_idx % 256
    w1_pairing = np.empty((2 * I, H), np.uint8)
    w1_pairing[grow] = w1_log[expert, :I]
    w1_pairing[grow + 256] = w1_log[expert, I:]
    w1_lane = np.zeros((EPR, 2 * I * H), np.uint8)
    w2_lane = np.zeros((EPR, H * I), np.uint8)
    R.ref_pack_lane(np.ascontiguousarray(w1_pairing), 2 * I, H, w1_lane[expert])
    R.ref_pack_lane(np.ascontiguousarray(w2_log[expert]), H, I, w2_lane[expert])
    x = ((5 * 37 + np.arange(rows)[:, None] * 7 + np.arange(H)[None, :] * 3) & 0x3F).astype(np.uint8)
    ffn_expect = np.zeros((rows, I), np.float32)
    R.ref_l1_rows(x, w1_lane.reshape(-1), expert, rows, ffn_expect.reshape(-1), 8)
    ffn_q = np.zeros((rows, I), np.uint8)
    R.ref_quantize(ffn_expect.reshape(-1), rows * I, ffn_q.reshape(-1))
    out_expect = np.zeros((rows, H), np.float32)
    R.ref_l2_rows(ffn_q, w2_lane.reshape(-1), expert, rows, out_expect.reshape(-1), 8)
    # reduce: 2 tokens, cap 2, bf16 rows from a seeded normal, one invalid k
    cap, tokens, E = 2, 2, 4 * EPR
    comb = orc.f32_to_bf16(rng.standard_normal((TOPK, cap, H)).astype(np.float32))
    tidx = rng.integers(0, E, (cap, TOPK)).astype(np.int64)
    tidx[1, 3] = -1
    tw = rng.random((cap, TOPK)).astype(np.float32)
    y = np.zeros((tokens, H), np.float32)
    R.ref_reduce_tokens(comb.view(np.uint8).reshape(-1), tidx, tw, tokens, E, cap, y.reshape(-1), 2)
    np.savez_compressed(os.path.join(HERE, "numeric_ref_mode.npz"), expert=expert, x=x,
                        ffn_expect=ffn_expect, ffn_q=ffn_q, out_expect=out_expect,
                        comb=comb, tidx=tidx, tw=tw, y=y, E=E)

    # ---- route patterns, schedulers ----
    routes = {}
    for pat, name in ((0, "balanced"), (1, "hot"), (2, "mixed")):
        for (rank, Rr, tok, salt) in ((0, 2, 16, 0), (1, 2, 16, 3), (3, 8, 24, 1)):
            out = np.zeros(tok * TOPK, np.int64)
            R.ref_make_routes(pat, rank, Rr, tok, salt, out)
            routes[f"{name}_{rank}_{Rr}_{tok}_{salt}"] = out
    np.savez_compressed(os.path.join(HERE, "routes.npz"), **routes)

    sched = {}
    GE, GR = R.ref_const(5), R.ref_const(4)
    for ci in range(6):
        r2 = np.random.default_rng(100 + ci)
        if ci % 2 == 0:
            cg = r2.integers(0, 40, GE).astype(np.int32)
        else:
            cg = (r2.zipf(1.6, GE) * 6).clip(0, 512).astype(np.int32)
        for win in (32, 64, 128):
            for m in range(GR):
                ge = np.zeros(512, np.int32)
                w = np.zeros(512, np.int32)
                n = R.ref_gs_schedule_member(cg, win, m, ge, w, 512)
                sched[f"gs_{ci}_{win}_{m}_cg"] = cg
                sched[f"gs_{ci}_{win}_{m}_ge"] = ge[:n].copy()
                sched[f"gs_{ci}_{win}_{m}_w"] = w[:n].copy()
        counts = (r2.integers(0, 60, 256) if ci % 2 == 0 else (r2.zipf(1.5, 256) * 4).clip(0, 512)).astype(np.uint32)
        sched[f"win_{ci}_counts"] = counts
        sched[f"win_{ci}_out"] = np.array(
            [R.ref_select_win(counts, 256, cap_hint, wmin) for cap_hint in (64, 96, 128) for wmin in (8, 32)], np.int32)
        ci32 = counts.astype(np.int32)
        for g in (0, 5):
            st = np.zeros((32 * 64 * 4, 3), np.int32)
            mo = np.zeros(32 * 64 * 4, np.int32)
            ld = np.zeros(4, np.int64)
            n = R.ref_lpt_assign(ci32, 64, 4, g, 4, st.reshape(-1), mo, ld)
            sched[f"lpt_{ci}_{g}_tasks"] = st[:n].copy()
            sched[f"lpt_{ci}_{g}_member"] = mo[:n].copy()
            sched[f"lpt_{ci}_{g}_load"] = ld.copy()
    sched["consts"] = np.array([R.ref_const(i) for i in range(10)], np.int32)
    np.savez_compressed(os.path.join(HERE, "sched.npz"), **sched)

    # ---- Python quantisers (torch) ----
    import torch
    m = _ref_math(ref_root)
    g = torch.Generator().manual_seed(11)
    xt = torch.randn((5, 384), generator=g).bfloat16()
    xt[2, 128:256] = 0          # all-zero group -> amax clamp 1e-4
    xt[3, :128] *= 1000.0
    xq, xsf = m.per_token_cast_to_fp8(xt, use_ue8m0=True, gran_k=128)
    wt = torch.randn((256, 384), generator=g) * 0.02
    wq, wsf = m.per_block_cast_to_fp8(wt, use_ue8m0=True, gran_k=128)
    back = m.cast_back_from_fp8(xq, xsf, 128)
    cin = torch.tensor([1e-4 / 448, 0.5, 0.75, 1.0, 1.0000001, 3.9, 4.0, 1e-30, 1e30, 2.0 ** -126], dtype=torch.float32)
    cout = m.ceil_to_ue8m0(cin)
    np.savez_compressed(
        os.path.join(HERE, "quant_py.npz"),
        x=xt.float().numpy(), xq=xq.view(torch.uint8).numpy(),
        xsf=(xsf.view(torch.int32) >> 23).to(torch.uint8).numpy(),
        w=wt.numpy(), wq=wq.view(torch.uint8).numpy(),
        wsf=(wsf.contiguous().view(torch.int32) >> 23).to(torch.uint8).numpy(),
        back=back.numpy(), ceil_in=cin.numpy(), ceil_out=cout.numpy())
    make_e2m1(m)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
