"""Parity at the baseline's full geometry (E=256, topk=8, H=6144, I=2048, UE8M0 block scales).

The CPU oracle cannot evaluate a whole full-size layer in seconds, so these tests combine
  * an oracle comparison on a bounded sample (the tokens are routed inside a subset of the
    256 experts so that only those experts' weights have to be evaluated on the CPU), and
  * size-independent properties of the layer: exact linearity in the top-k weights and
    invariance under a permutation of the tokens.
Weights are generated on the device (seeded) and only the sampled experts are copied back.
"""
import numpy as np
import pytest
import torch

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

E, TOPK, H, I = 256, 8, 6144, 2048


def _device_weights(seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)

    def fp8(shape):
        r = torch.randint(0, 256, shape, generator=g, device="cuda", dtype=torch.uint8)
        ex = torch.randint(3, 11, shape, generator=g, device="cuda", dtype=torch.uint8)
        return (r & 0x87) | (ex << 3)   # sign, mantissa random; exponent field 3..10; never NaN

    w1 = torch.cat([fp8((32, 2 * I, H)) for _ in range(E // 32)])
    w2 = torch.cat([fp8((32, H, I)) for _ in range(E // 32)])
    s1 = (torch.randint(0, 3, (E, 2 * I // 128, H // 128), generator=g, device="cuda", dtype=torch.uint8) + 118)
    s2 = (torch.randint(0, 3, (E, H // 128, I // 128), generator=g, device="cuda", dtype=torch.uint8) + 118)
    return w1, s1, w2, s2


def _inputs(T, experts_pool, seed):
    rng = np.random.default_rng(seed)
    x = ((rng.integers(0, 256, (T, H)) & 0x87) | (rng.integers(3, 11, (T, H)) << 3)).astype(np.uint8)
    x_sf = (rng.integers(0, 3, (T, H // 128)) + 124).astype(np.uint8)
    idx = np.stack([rng.choice(experts_pool, TOPK, replace=False) for _ in range(T)]).astype(np.int64)
    lg = rng.standard_normal((T, TOPK)).astype(np.float32)
    w = np.exp(lg - lg.max(1, keepdims=True))
    w = (w / w.sum(1, keepdims=True)).astype(np.float32)
    return x, x_sf, idx, w


def _run(buf, l1, l2, x, x_sf, idx, w):
    import mini_mega_b200 as mm
    T = x.shape[0]
    buf.x.view(torch.uint8)[:T].copy_(torch.from_numpy(x))
    buf.x_sf[:T].copy_(torch.from_numpy(x_sf))
    buf.topk_idx[:T].copy_(torch.from_numpy(idx))
    buf.topk_weights[:T].copy_(torch.from_numpy(w))
    y = torch.zeros((T, H), dtype=torch.bfloat16, device="cuda")
    mm.fp8_mega_moe(y, l1, l2, buf)
    torch.cuda.synchronize()
    st = buf.status()
    assert st.status == 0, f"device status {st.status} dbg {list(st.dbg)}"
    return y


def test_full_geometry_sample_and_properties():
    import mini_mega_b200 as mm
    w1, s1, w2, s2 = _device_weights(5)
    l1, l2 = mm.transform_weights_for_mega_moe((w1, s1), (w2, s2))
    T = 24
    pool = np.array([3, 17, 40, 77, 101, 130, 155, 170, 199, 200, 231, 255])   # 12 of the 256 experts
    x, x_sf, idx, w = _inputs(T, pool, seed=6)
    buf = mm.get_symm_buffer_for_mega_moe(None, E, 64, TOPK, H, I)
    try:
        y = _run(buf, l1, l2, x, x_sf, idx, w)
        # ---- oracle on the sample: only the 12 routed experts are evaluated on the CPU
        want = np.zeros((T, H), np.float32)
        # k-ascending accumulation exactly as the reduce does
        per_pair = {}
        for e in pool:
            hit = np.argwhere(idx == e)
            if hit.size == 0:
                continue
            rows = hit[:, 0]
            h = orc.l1(x[rows], x_sf[rows], w1[e].cpu().numpy(), s1[e].cpu().numpy())
            q, sf = orc.requant(h, True)
            out = orc.bf16_to_f32(orc.f32_to_bf16(orc.l2(q, sf, w2[e].cpu().numpy(), s2[e].cpu().numpy())))
            for (t, k), o in zip(hit, out):
                per_pair[(int(t), int(k))] = o
        for t in range(T):
            acc = np.zeros(H, np.float32)
            for k in range(TOPK):
                acc = acc + per_pair[(t, k)] * np.float32(w[t, k])
            want[t] = acc
        err = orc.rel_l2(y.float().cpu().numpy(), want)
        assert err <= 1e-2, f"full-geometry sample: relative L2 {err}"

        # ---- linearity: doubling every top-k weight doubles y exactly (powers of two are exact)
        y2 = _run(buf, l1, l2, x, x_sf, idx, (w * np.float32(2.0)).astype(np.float32))
        assert torch.equal((y.float() * 2).bfloat16().view(torch.int16), y2.view(torch.int16))

        # ---- permutation of the tokens permutes y (rows are computed independently of their slot)
        perm = np.random.default_rng(7).permutation(T)
        yp = _run(buf, l1, l2, x[perm], x_sf[perm], idx[perm], w[perm])
        assert torch.equal(yp.view(torch.int16), y[torch.from_numpy(perm).cuda()].view(torch.int16))
    finally:
        buf.destroy()


@pytest.mark.parametrize("cta_pair", [1, 2])
def test_skewed_routing_full_width(cta_pair):
    """Zipf(1.2)-skewed routing (the hottest expert gets many windows) at full H / I on a world of
    32 experts: end-to-end against the oracle on sampled tokens, with single-CTA windows of
    128 rows and with CTA-pair windows of 256 rows."""
    import mini_mega_b200 as mm
    case_E, T = 32, 160
    rng = np.random.default_rng(11)
    g = torch.Generator(device="cuda")
    g.manual_seed(12)
    r = torch.randint(0, 256, (case_E, 2 * I, H), generator=g, device="cuda", dtype=torch.uint8)
    ex = torch.randint(3, 11, (case_E, 2 * I, H), generator=g, device="cuda", dtype=torch.uint8)
    w1 = (r & 0x87) | (ex << 3)
    r = torch.randint(0, 256, (case_E, H, I), generator=g, device="cuda", dtype=torch.uint8)
    ex = torch.randint(3, 11, (case_E, H, I), generator=g, device="cuda", dtype=torch.uint8)
    w2 = (r & 0x87) | (ex << 3)
    s1 = torch.full((case_E, 2 * I // 128, H // 128), 119, dtype=torch.uint8, device="cuda")
    s2 = torch.full((case_E, H // 128, I // 128), 119, dtype=torch.uint8, device="cuda")
    l1, l2 = mm.transform_weights_for_mega_moe((w1, s1), (w2, s2))
    p = 1.0 / np.arange(1, case_E + 1) ** 1.2
    p /= p.sum()
    perm = rng.permutation(case_E)
    idx = np.stack([perm[rng.choice(case_E, 4, replace=False, p=p)] for _ in range(T)]).astype(np.int64)
    x = ((rng.integers(0, 256, (T, H)) & 0x87) | (rng.integers(3, 11, (T, H)) << 3)).astype(np.uint8)
    x_sf = (rng.integers(0, 3, (T, H // 128)) + 124).astype(np.uint8)
    w = rng.random((T, 4)).astype(np.float32)
    buf = mm.get_symm_buffer_for_mega_moe(None, case_E, T, 4, H, I)
    try:
        buf.x.view(torch.uint8)[:T].copy_(torch.from_numpy(x))
        buf.x_sf[:T].copy_(torch.from_numpy(x_sf))
        buf.topk_idx[:T].copy_(torch.from_numpy(idx))
        buf.topk_weights[:T].copy_(torch.from_numpy(w))
        y = torch.zeros((T, H), dtype=torch.bfloat16, device="cuda")
        mm.fp8_mega_moe(y, l1, l2, buf, cta_pair=cta_pair)
        torch.cuda.synchronize()
        st = buf.status()
        assert st.status == 0, f"device status {st.status} dbg {list(st.dbg)}"
        counts = np.bincount(idx.reshape(-1), minlength=case_E)
        assert counts.max() > 128, "the hottest expert should need more than one window"
        win = 128 * cta_pair
        assert st.n_windows == int(sum((c + win - 1) // win for c in counts))
        # oracle on 24 sampled tokens (all their experts)
        sample = rng.choice(T, 24, replace=False)
        want = np.zeros((len(sample), H), np.float32)
        cache = {}
        for si, t in enumerate(sample):
            acc = np.zeros(H, np.float32)
            for k in range(4):
                e = int(idx[t, k])
                if e not in cache:
                    cache[e] = (w1[e].cpu().numpy(), s1[e].cpu().numpy(), w2[e].cpu().numpy(), s2[e].cpu().numpy())
                a1, b1, a2, b2 = cache[e]
                h = orc.l1(x[t:t + 1], x_sf[t:t + 1], a1, b1)
                q, sf = orc.requant(h, True)
                o = orc.bf16_to_f32(orc.f32_to_bf16(orc.l2(q, sf, a2, b2)))[0]
                acc = acc + o * np.float32(w[t, k])
            want[si] = acc
        err = orc.rel_l2(y.float().cpu().numpy()[sample], want)
        assert err <= 1e-2, f"skewed routing: relative L2 {err}"
    finally:
        buf.destroy()
