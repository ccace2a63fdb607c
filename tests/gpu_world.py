"""Test helper: drive an oracle ``Case`` through the CUDA library on ONE GPU.

A world of R ranks lives in one process (``SymmBuffer.local_world``); the ranks'
kernels are issued phase by phase through ``mxk_launch_phases`` so that no kernel
ever waits for one that has not been launched.  Everything goes through the C ABI.
"""
import ctypes as C

import numpy as np
import torch

import mini_mega_b200 as mm
from mini_mega_b200 import _lib

PHASES = (1, 2, 4, 8, 16)  # route, setup, dispatch, gemm, reduce


def dev_weights(case, r, device="cuda", weight_format=0):
    """This rank's expert weights on the device, in the form fp8_mega_moe takes (weight_format 1:
    the packed e2m1 codes ``case.w1_packed / w2_packed`` that ``case.w1 / w2`` are the expansion of)."""
    EPR = case.EPR
    sl = slice(r * EPR, (r + 1) * EPR)
    src1, src2 = (case.w1_packed, case.w2_packed) if weight_format == 1 else (case.w1, case.w2)
    w1 = torch.from_numpy(np.ascontiguousarray(src1[sl])).to(device)
    w2 = torch.from_numpy(np.ascontiguousarray(src2[sl])).to(device)
    if not case.scaled:
        return w1, w2
    s1 = torch.from_numpy(np.ascontiguousarray(case.w1_sf[sl])).to(device)
    s2 = torch.from_numpy(np.ascontiguousarray(case.w2_sf[sl])).to(device)
    return (w1, s1), (w2, s2)


def to_e2m1_case(case, seed=0):
    """Turn an oracle case into its 4-bit twin: random e2m1 codes for every weight, kept packed in
    ``w1_packed / w2_packed`` for the device, while ``w1 / w2`` become the E4M3 bytes the codes stand
    for, so that the 8-bit oracle is the oracle of the 4-bit layer.  Scale planes are kept."""
    from oracle import oracle as orc
    rng = np.random.default_rng(seed + 4)
    E, H, I = case.E, case.H, case.I
    case.w1_packed = rng.integers(0, 256, (E, 2 * I, H // 2), dtype=np.uint8)
    case.w2_packed = rng.integers(0, 256, (E, H, I // 2), dtype=np.uint8)
    if case.scaled:
        # the planes were chosen for bytes that reach 448; codes reach 6: 2^6 keeps the products' range
        case.w1_sf = (case.w1_sf + 6).astype(np.uint8)
        case.w2_sf = (case.w2_sf + 6).astype(np.uint8)
    else:
        # no scales to absorb the range: keep to the codes of 0 and +-0.5 so that nothing saturates
        case.w1_packed &= 0x99
        case.w2_packed &= 0x99
    case.w1 = orc.expand_e2m1(case.w1_packed)
    case.w2 = orc.expand_e2m1(case.w2_packed)
    return case


def load_inputs(case, bufs):
    for r, b in enumerate(bufs):
        b.x.view(torch.uint8).copy_(torch.from_numpy(case.x[r]))
        if case.scaled:
            b.x_sf.copy_(torch.from_numpy(case.x_sf[r]))
        b.topk_idx.copy_(torch.from_numpy(case.topk_idx[r]))
        b.topk_weights.copy_(torch.from_numpy(case.topk_w[r]))


class World:
    def __init__(self, case, slot_capacity=0, expert_window=128, dispatch_mode=0, group_ranks=0, group_skew_num=0,
                 weight_format=0, group_hot_windows=0):
        self.case = case
        self.weight_format = weight_format
        self.bufs = mm.SymmBuffer.local_world(case.R, case.E, case.cap, case.topk, case.H, case.I,
                                              slot_capacity=slot_capacity, expert_window=expert_window,
                                              dispatch_mode=dispatch_mode, group_ranks=group_ranks,
                                              group_skew_num=group_skew_num, group_hot_windows=group_hot_windows)
        self.weights = [dev_weights(case, r, weight_format=weight_format) for r in range(case.R)]
        # helper groups: every member holds the weights of all its group's experts, in member order
        self.group_weights = [None] * case.R
        if group_ranks > 1:
            for r, b in enumerate(self.bufs):
                ws = [self.weights[m] for m in b.group_members()]
                if case.scaled:
                    self.group_weights[r] = tuple((torch.cat([w[i][0] for w in ws]).contiguous(),
                                                   torch.cat([w[i][1] for w in ws]).contiguous()) for i in range(2))
                else:
                    self.group_weights[r] = tuple(torch.cat([w[i] for w in ws]).contiguous() for i in range(2))
        self.y = [torch.zeros((max(case.tokens[r], 1), case.H), dtype=torch.bfloat16, device="cuda")
                  for r in range(case.R)]
        self.y32 = [torch.zeros((max(case.tokens[r], 1), case.H), dtype=torch.float32, device="cuda")
                    for r in range(case.R)]
        load_inputs(case, self.bufs)

    def args(self, r, **kw):
        l1, l2 = self.weights[r]
        return self.bufs[r].launch_args(self.case.tokens[r], l1, l2, y_bf16=self.y[r], y_f32=self.y32[r],
                                        group_weights=self.group_weights[r], weight_format=self.weight_format, **kw)

    def run(self, phases=PHASES, **kw):
        lib = _lib.lib()
        st = torch.cuda.current_stream().cuda_stream
        for ph in phases:
            for r in range(self.case.R):
                if ph == 16 and self.case.tokens[r] == 0:
                    continue
                a = self.args(r, **kw)
                _lib.check(lib.mxk_launch_phases(C.byref(a), ph, st), f"phase {ph} rank {r}")
        torch.cuda.synchronize()

    def table(self, r, name):
        return self.bufs[r].table(name).cpu().numpy()

    def destroy(self):
        for b in self.bufs:
            b.destroy()


def assert_status_ok(world):
    for r, b in enumerate(world.bufs):
        st = b.status()
        assert st.status == 0, f"rank {r}: device status {st.status} dbg {list(st.dbg)}"


def check_tables(world, ref_states, slot_cap=None):
    """Routing, dispatch layout and per-expert counts/offsets: bit-exact."""
    case = world.case
    R, EPR = case.R, case.EPR
    par = 1  # first launch on fresh buffers runs at epoch 1
    for r in range(R):
        s = ref_states[r]
        assert np.array_equal(world.table(r, "route_slot_counts"), s.route_slot_counts), f"route_slot_counts r{r}"
        tbl = world.table(r, "src_index_table")[par].astype(np.uint32)
        assert np.array_equal(tbl, s.src_index_table), f"src_index_table r{r}"
        recv = world.table(r, "expert_recv_counts")[par].astype(np.uint32)
        assert np.array_equal(recv[:, : EPR + 1], s.recv_counts[:, : EPR + 1]), f"expert_recv_counts r{r}"
        assert np.array_equal(world.table(r, "prefix_tbl"), s.prefix_tbl), f"prefix_tbl r{r}"
        assert np.array_equal(world.table(r, "expert_row_base"), s.row_base), f"expert_row_base r{r}"
