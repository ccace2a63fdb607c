"""Worker of the multi-process tests (one process per rank).

mode "gpu":  real expert-parallel layer over NCCL-bootstrapped IPC buffers, one GPU per rank, once
             with the pull-mode and once with the push-mode prologue: three launches on the same
             buffers with different inputs (exercises the epoch-parity tables, counter reset and
             ragged / empty ranks), integer tables exact, y checked against the oracle; then five
             layers captured in one CUDA graph and replayed three times on every rank (no host
             reset in between: stale flags or tags across ranks would show), each node's y equal
             to the eager result bit for bit (reference: test/check.cu:533-745).
mode "gloo": CPU ranks: each rank derives its own routing share, ranks exchange them like the
             device scatter does, and the assembled tables must equal the whole-world oracle.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import oracle as orc  # noqa: E402


def cases(R):
    return [
        orc.gen_case(R, 4, 4, 1024, 512, [24 + 3 * r for r in range(R)], seed=21, routing="uniform", scaled=True, cap=48),
        orc.gen_case(R, 4, 4, 1024, 512, [0 if r == R - 1 else 9 + r for r in range(R)], seed=22, routing="zipf",
                     scaled=True, cap=48),
        orc.gen_case(R, 4, 4, 1024, 512, [48] * R, seed=23, routing="uniform", scaled=True, cap=48, invalid_frac=0.1),
    ]


def run_gpu():
    import mini_mega_b200 as mm
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    group = dist.group.WORLD
    worst = 0.0
    all_cases = cases(world)
    refs = [orc.layer_world(c) for c in all_cases]
    for mode in (1, 2):
        buf = None
        launches = 0
        for ci, case in enumerate(all_cases):
            if buf is None:
                buf = mm.get_symm_buffer_for_mega_moe(group, case.E, case.cap, case.topk, case.H, case.I,
                                                      dispatch_mode=mode)
            T = case.tokens[rank]
            buf.x.view(torch.uint8).copy_(torch.from_numpy(case.x[rank]))
            buf.x_sf.copy_(torch.from_numpy(case.x_sf[rank]))
            buf.topk_idx.copy_(torch.from_numpy(case.topk_idx[rank]))
            buf.topk_weights.copy_(torch.from_numpy(case.topk_w[rank]))
            sl = slice(rank * case.EPR, (rank + 1) * case.EPR)
            l1, l2 = mm.transform_weights_for_mega_moe(
                (torch.from_numpy(case.w1[sl]).cuda(), torch.from_numpy(case.w1_sf[sl]).cuda()),
                (torch.from_numpy(case.w2[sl]).cuda(), torch.from_numpy(case.w2_sf[sl]).cuda()))
            y = torch.zeros((T, case.H), dtype=torch.bfloat16, device="cuda")
            torch.cuda.synchronize()
            dist.barrier()
            mm.fp8_mega_moe(y, l1, l2, buf)
            launches += 1
            torch.cuda.synchronize()
            st = buf.status()
            assert st.status == 0, f"rank {rank} mode {mode} case {ci}: device status {st.status} dbg {list(st.dbg)}"
            ref = refs[ci]
            # integer tables of this rank: bit-exact
            par = int(st.launches & 1)
            s = ref[rank]
            assert np.array_equal(buf.table("route_slot_counts").cpu().numpy(), s.route_slot_counts)
            assert np.array_equal(buf.table("prefix_tbl").cpu().numpy(), s.prefix_tbl)
            tbl = buf.table("src_index_table")[par].cpu().numpy().astype(np.uint32)
            for le in range(case.EPR):     # rows are defined up to their count; later slots keep older launches
                for src in range(world):
                    n = int(s.prefix_tbl[le, src + 1] - s.prefix_tbl[le, src])
                    assert np.array_equal(tbl[le, src, :n], s.src_index_table[le, src, :n]), (mode, ci, le, src)
            rows = s.meta.shape[0]
            assert np.array_equal(buf.table("row_meta")[:rows, :3].cpu().numpy(), s.meta)
            assert np.array_equal(buf.table("pool")[:rows].cpu().numpy(), s.pool)
            if T:
                err = orc.rel_l2(y.float().cpu().numpy(), ref[rank].y)
                worst = max(worst, err)
                assert err <= 1e-2, f"rank {rank} mode {mode} case {ci}: relative L2 {err}"
            dist.barrier()
        # graph of five layers on the last case's inputs, replayed three times
        y_eager = y.clone()
        ys = [torch.zeros_like(y_eager) for _ in range(5)]
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for yy in ys:
                    mm.fp8_mega_moe(yy, l1, l2, buf)
        for rep in range(3):
            for yy in ys:
                yy.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            g.replay()
            torch.cuda.synchronize()
            st = buf.status()
            assert st.status == 0, f"rank {rank} mode {mode} replay {rep}: device status {st.status} dbg {list(st.dbg)}"
            for ni, yy in enumerate(ys):
                assert torch.equal(yy.view(torch.int16), y_eager.view(torch.int16)), (mode, rep, ni)
        assert buf.status().launches == launches + 15
        dist.barrier()
        del g
        buf.destroy()
    # many rows per rank with the pull-mode prologue (one-pass route build, thousands of rows pulled
    # over NVLink, CTA pairs chosen by load)
    big = orc.gen_case(world, 4, 4, 1024, 512, [1100] * world, seed=24, routing="uniform", scaled=True, cap=1100)
    big_ref = orc.layer_world(big)
    buf = mm.get_symm_buffer_for_mega_moe(group, big.E, big.cap, big.topk, big.H, big.I, dispatch_mode=1)
    buf.x.view(torch.uint8).copy_(torch.from_numpy(big.x[rank]))
    buf.x_sf.copy_(torch.from_numpy(big.x_sf[rank]))
    buf.topk_idx.copy_(torch.from_numpy(big.topk_idx[rank]))
    buf.topk_weights.copy_(torch.from_numpy(big.topk_w[rank]))
    sl = slice(rank * big.EPR, (rank + 1) * big.EPR)
    l1, l2 = mm.transform_weights_for_mega_moe(
        (torch.from_numpy(big.w1[sl]).cuda(), torch.from_numpy(big.w1_sf[sl]).cuda()),
        (torch.from_numpy(big.w2[sl]).cuda(), torch.from_numpy(big.w2_sf[sl]).cuda()))
    y = torch.zeros((1100, big.H), dtype=torch.bfloat16, device="cuda")
    for rep in range(2):
        y.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        mm.fp8_mega_moe(y, l1, l2, buf)
        torch.cuda.synchronize()
        st = buf.status()
        assert st.status == 0, f"rank {rank} large pull-mode layer: device status {st.status} dbg {list(st.dbg)}"
        s_ = big_ref[rank]
        rows = s_.meta.shape[0]
        assert rows >= 4096 and st.total_rows == rows
        assert np.array_equal(buf.table("row_meta")[:rows, :3].cpu().numpy(), s_.meta)
        assert np.array_equal(buf.table("pool")[:rows].cpu().numpy(), s_.pool)
        err = orc.rel_l2(y.float().cpu().numpy(), s_.y)
        worst = max(worst, err)
        assert err <= 1e-2, f"rank {rank} large pull-mode layer: relative L2 {err}"
        dist.barrier()
    buf.destroy()
    # cross-rank helper scheduling over real peer memory: one helper group spanning the world, helpers
    # forced on; a member computes windows of the other rank's experts from its weight replica, pulling
    # the rows from the source rank's input block; tables of the owner stay exact, pool rows follow the
    # member's window list, y within tolerance; two launches on the same buffers
    if world <= 16:
        buf = None
        for ci in (0, 1):
            case = all_cases[ci]
            if buf is None:
                buf = mm.get_symm_buffer_for_mega_moe(group, case.E, case.cap, case.topk, case.H, case.I, dispatch_mode=2,
                                                      expert_window=32, group_ranks=world, group_skew_num=-1,
                                                      group_hot_windows=2 if ci == 0 else 0)
            T = case.tokens[rank]
            buf.x.view(torch.uint8).copy_(torch.from_numpy(case.x[rank]))
            buf.x_sf.copy_(torch.from_numpy(case.x_sf[rank]))
            buf.topk_idx.copy_(torch.from_numpy(case.topk_idx[rank]))
            buf.topk_weights.copy_(torch.from_numpy(case.topk_w[rank]))
            sl = slice(rank * case.EPR, (rank + 1) * case.EPR)
            l1, l2 = mm.transform_weights_for_mega_moe(
                (torch.from_numpy(case.w1[sl]).cuda(), torch.from_numpy(case.w1_sf[sl]).cuda()),
                (torch.from_numpy(case.w2[sl]).cuda(), torch.from_numpy(case.w2_sf[sl]).cuda()))
            gw = mm.gather_group_weights(buf, l1, l2)
            assert torch.equal(gw[0][0].cpu(), torch.from_numpy(case.w1)) and torch.equal(gw[1][1].cpu(), torch.from_numpy(case.w2_sf))
            y = torch.zeros((T, case.H), dtype=torch.bfloat16, device="cuda")
            torch.cuda.synchronize()
            dist.barrier()
            mm.fp8_mega_moe(y, l1, l2, buf, group_weights=gw)
            torch.cuda.synchronize()
            st = buf.status()
            assert st.status == 0, f"rank {rank} helpers case {ci}: device status {st.status} dbg {list(st.dbg)}"
            ref = refs[ci]
            want = orc.helper_world(case, ref, world, 32, 0, hot_windows=buf.group_hot_windows or 3)[rank]
            assert bool(st.helper_on) == want["on"]
            rows = want["meta"].shape[0]
            assert st.total_rows == rows
            assert np.array_equal(buf.table("prefix_tbl").cpu().numpy(), ref[rank].prefix_tbl)
            assert np.array_equal(buf.table("row_meta")[:rows, :3].cpu().numpy(), want["meta"])
            assert np.array_equal(buf.table("pool")[:rows].cpu().numpy(), case.x[want["meta"][:, 0], want["meta"][:, 1]])
            if T:
                err = orc.rel_l2(y.float().cpu().numpy(), ref[rank].y)
                worst = max(worst, err)
                assert err <= 1e-2, f"rank {rank} helpers case {ci}: relative L2 {err}"
            dist.barrier()
        buf.destroy()
    print(f"MP_OK rank={rank} worst_rel_l2={worst:.3e}", flush=True)
    dist.destroy_process_group()


def run_gloo():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    case = cases(world)[0]
    want = orc.route_world(case)
    # this rank's routing share: counts per global expert and the ordered pair list per expert
    E, EPR, topk, cap = case.E, case.EPR, case.topk, case.cap
    idx = case.topk_idx[rank, : case.tokens[rank]].reshape(-1)
    counts = np.zeros(E, np.int64)
    rows = [[] for _ in range(E)]
    for p, e in enumerate(idx):
        if 0 <= e < E and counts[e] < cap:
            rows[e].append(p)
            counts[e] += 1
    assert np.array_equal(counts.astype(np.int32), want[rank].route_slot_counts)
    # "scatter": every rank publishes its rows; owners assemble [le][src][slot] and the prefix table
    gathered = [None] * world
    dist.all_gather_object(gathered, rows)
    tbl = np.zeros((EPR, world, cap), np.uint32)
    prefix = np.zeros((EPR, world + 1), np.int32)
    for le in range(EPR):
        c = 0
        for src in range(world):
            r_ = gathered[src][rank * EPR + le]
            tbl[le, src, : len(r_)] = r_
            prefix[le, src] = c
            c += len(r_)
        prefix[le, world] = c
    assert np.array_equal(tbl, want[rank].src_index_table)
    assert np.array_equal(prefix, want[rank].prefix_tbl)
    total = torch.tensor([int(prefix[:, world].sum())])
    dist.all_reduce(total)
    assert int(total) == int(sum((case.topk_idx[r, : case.tokens[r]] >= 0).sum() for r in range(world)))
    print(f"MP_OK rank={rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    {"gpu": run_gpu, "gloo": run_gloo}[sys.argv[1]]()
