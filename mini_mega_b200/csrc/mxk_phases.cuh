// ============================================================================
// mxk_phases.cuh — the non-GEMM phases of the MoE layer as CTA-cooperative
// device functions of the persistent kernel (k_mega in mxk_kernels.cu).  Every
// function is called by ALL threads of a CTA; block size is read at run time.
//
//   route_phase     per-rank route build: deterministic slot per (token,k) pair,
//                   scatter of pair indices into the owner ranks' tables, count
//                   publish as epoch-tagged words (they double as the cross-rank
//                   barrier); the last CTA then writes the row checksums and
//                   advances the launch counter
//                   (reference: route_build_body / publish_counts_body /
//                    xbar_route_ready_body, src/prologue.cuh:126-256, src/flags.cuh:284-377)
//   setup_phase     CTA 0: barrier wait, prefix table, windows, cost-ordered task
//                   list; the other CTAs wait for its "set-up done" flag
//                   (reference: task_setup_body, src/prologue.cuh:269-498)
//   dispatch_phase  EP dispatch: one warp per pool row pulls the routed FP8 row
//                   and its 1x128 scales from the source rank's symmetric buffer
//                   (reference: r19_pull_flags, src/compute_big.cuh:1691-1946)
//   reduce_phase    top-k weighted sum at the source rank
//                   (reference: reduce_tile_body, src/combine.cuh:488-656)
//
// Small batches run the PUSH-mode prologue instead of route scatter / barrier / pull
// (three dependent trips over NVLink): push_phase stores every token's routing, weights,
// scales and E4M3 row into the staging area of the ranks that own its experts; push_tables
// lets EVERY CTA derive the world's routing tables from those words in shared memory (no
// leader CTA, no flag); push_dispatch copies the rows from the staging area into the pool.
// The tables that result are the same, bit for bit, as the pull-mode ones.
// ============================================================================
#pragma once

// Slots are handed out in ascending pair index idx = token*topk + k, so every
// table row (and with it the pool row order) is deterministic; the reference
// uses a shared-memory atomicAdd and accepts any order (src/prologue.cuh:164-180).
constexpr int kRoutePer = 8;

// Cross-rank words of the prologue are EPOCH-TAGGED 64-bit values {payload (low), epoch (high)}
// written with one 8-byte store: a consumer polls the word itself until the tag is this launch's
// epoch, so neither the producer nor the consumer needs a system-scope fence or a separate
// flag on the critical path (the reference orders payload -> fence -> flag and adds a checksum
// word against torn rows, src/flags.cuh:4, src/prologue.cuh:248-255,339-340).
__device__ __forceinline__ uint64_t tagged(uint32_t payload, long long epoch) {
    return ((uint64_t)(uint32_t)epoch << 32) | payload;
}

// Slots are handed out in ascending pair index idx = token*topk + k, so every table row (and
// with it the pool row order) is deterministic; the reference uses a shared-memory atomicAdd
// and accepts any order (src/prologue.cuh:164-180).
// The route build can be run by the whole CTA or by a team of its warps (the epilogue warps of the
// GEMM phase, while they wait for the first accumulators): thread numbering and the barrier are
// the team's.
struct Team {
    int tid, nthr, bar;   // bar 0 = the CTA barrier, else a named barrier of `nthr` threads
    __device__ __forceinline__ void sync() const {
        if (bar == 0) __syncthreads();
        else asm volatile("bar.sync %0, %1;" ::"r"(bar), "r"(nthr) : "memory");
    }
};

// Arrival counters of the rows peers push to this rank (combine_cnt) must be zero before any
// peer can push for this launch.  The reduce phase zeroes every count it has consumed and the
// last CTA to leave it records the launch in cnt_clean_epoch; when the previous launch did that
// (the normal case) nothing has to be cleared here.  Otherwise — a compute launch without a
// reduce, a reduce that gave up — the whole grid clears the table and meets at a barrier before
// anything of this launch leaves the rank: a peer can push only after it has seen this rank's
// routing, and that is published behind the barrier.
__device__ void ensure_counts_clean(const KArgs& a, DevFlags* f, long long epoch, uint32_t clean_epoch) {
    if (clean_epoch == (uint32_t)(epoch - 1)) return;   // uniform over the grid
    const int tid = threadIdx.x, nthr = blockDim.x;
    unsigned* cnt = reinterpret_cast<unsigned*>(a.unk + a.L.combine_cnt_off);
#pragma unroll 1
    for (int i = blockIdx.x * nthr + tid; i < a.topk * a.cap; i += gridDim.x * nthr) cnt[i] = 0;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        atomicAdd(&f->clear_blocks_done, 1u);
        const unsigned want = gridDim.x;
        if (!spin_until([&] { return ld_acquire_gpu(&f->clear_blocks_done) >= want; }, a.local_wait_ns, nullptr))
            raise_status(f, MXK_DEV_TIMEOUT_PIPE, 2);
    }
    __syncthreads();
}

// Route build for LARGE batches in one pass over the pairs (the per-expert scan of route_phase
// below costs every CTA a full pass per expert it owns).  CTA c takes the c-th slice of this
// rank's pairs, ranks every pair among the earlier pairs of its slice with the same expert and
// counts the slice's pairs per expert; the slice counts go to a [grid][E] table in global memory,
// the grid meets at a barrier, and the exclusive sum over the earlier slices turns a pair's rank
// into its slot — the same ascending-pair-index order as the per-expert scan.  `s_i` is scratch
// of 2 * slice + 2 * E ints.  Returns false when the shapes do not fit (the caller then scans).
__device__ bool route_onepass(const KArgs& a, DevFlags* f, long long epoch, int* s_i, int scratch_ints,
                              const bool local_only) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int par = (int)(epoch & 1);
    const int np = a.tokens * a.topk, E = a.E, G = (int)gridDim.x, c = (int)blockIdx.x;
    const int S = (np + G - 1) / G;
    if (E > 2048 || G > a.L.route_scratch_ctas || 2 * S + 2 * E > scratch_ints) return false;   // uniform over the grid
    int* s_id = s_i;            // [S] expert of the slice's pair, -1 = invalid
    int* s_rank = s_id + S;     // [S] earlier pairs of the slice with the same expert
    int* s_hist = s_rank + S;   // [E] pairs of the slice per expert
    int* s_base = s_hist + E;   // [E] pairs of the earlier slices per expert
    const int p0 = min(np, c * S), n = min(np, p0 + S) - p0;
    const int64_t* ti = a.topk_idx;
    uint8_t* pair_state = a.rwk + a.L.pair_state_off;
    int* rsc = reinterpret_cast<int*>(a.rwk + a.L.route_slot_counts_off);
    int* g_cnt = reinterpret_cast<int*>(a.rwk + a.L.route_scratch_off);   // [G][E]
#pragma unroll 1
    for (int e = tid; e < E; e += nthr) s_hist[e] = 0;
#pragma unroll 1
    for (int i = tid; i < n; i += nthr) {
        const int64_t v = ti[p0 + i];
        s_id[i] = (uint64_t)v < (uint64_t)E ? (int)v : -1;   // invalid ids take no slot (src/prologue.cuh:166-167)
    }
    __syncthreads();
#pragma unroll 1
    for (int i = tid; i < n; i += nthr) {
        const int id = s_id[i];
        int r = 0;
        if (id >= 0) {
#pragma unroll 8
            for (int j = 0; j < i; ++j) r += s_id[j] == id ? 1 : 0;
            atomicAdd(&s_hist[id], 1);
        }
        s_rank[i] = r;
    }
    __syncthreads();
#pragma unroll 1
    for (int e = tid; e < E; e += nthr) g_cnt[(size_t)c * E + e] = s_hist[e];
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        atomicAdd(&f->route_sync, 1u);
        const unsigned want = (unsigned)G;
        if (!spin_until([&] { return ld_acquire_gpu(&f->route_sync) >= want; }, a.local_wait_ns, nullptr))
            raise_status(f, MXK_DEV_TIMEOUT_PIPE, 2);
    }
    __syncthreads();
    // pairs of the earlier slices per expert (coalesced over the experts); the experts this CTA
    // owns (e = c, c + G, ...) also get their totals, their count is published from here
#pragma unroll 1
    for (int e = tid; e < E; e += nthr) {
        int before = 0, total = 0;
#pragma unroll 1
        for (int c0 = 0; c0 < G; c0 += 16) {   // sixteen loads in flight, then the sums
            int v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = c0 + j < G ? ld_relaxed_gpu(g_cnt + (size_t)(c0 + j) * E + e) : 0;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                before += c0 + j < c ? v[j] : 0;
                total += v[j];
            }
        }
        s_base[e] = before;
        if (e % G == c) {
            const int cnt = total < a.slot_cap ? total : a.slot_cap;
            rsc[e] = cnt;
            if (!local_only) {
                uint64_t* recv = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(a.unk_peers[a.fEPR.div(e)]) +
                                                             a.L.expert_recv_counts_off) +
                                 ((size_t)par * a.R + a.rank) * a.L.recv_stride;
                st_relaxed_sys_u64(recv + a.fEPR.mod(e), tagged((uint32_t)cnt, epoch));
            }
        }
    }
    __syncthreads();
#pragma unroll 1
    for (int i = tid; i < n; i += nthr) {
        const int id = s_id[i], p = p0 + i;
        bool ok = false;
        if (id >= 0) {
            const int slot = s_base[id] + s_rank[i];
            ok = slot < a.slot_cap;   // over capacity: dropped (src/prologue.cuh:171-174)
            if (ok && !local_only) {
                uint64_t* tbl = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(a.unk_peers[a.fEPR.div(id)]) +
                                                            a.L.src_index_table_off) +
                                (((size_t)par * a.EPR + a.fEPR.mod(id)) * a.R + a.rank) * (size_t)a.slot_cap;
                st_relaxed_sys_u64(tbl + slot, tagged((uint32_t)p, epoch));
            }
        }
        pair_state[p] = ok ? 1 : 0;
    }
    return true;
}

// `local_only` (push mode): only this rank's own tables are written — route_slot_counts and the
// accepted-pair map; nothing is scattered to the owner ranks, they derive their tables from the
// pushed routing words.
__device__ void route_phase(const KArgs& a, DevFlags* f, long long epoch, int* s_wtot /*[kRoutePer * warps]*/,
                            int* s_big, int s_big_ints /* large scratch for the one-pass variant */, const bool local_only,
                            const Team team) {
    const int tid = team.tid, lane = tid & 31, warp = tid >> 5;
    const int nthr = team.nthr, nwarps = nthr >> 5;
    const int par = (int)(epoch & 1);
    const int np = a.tokens * a.topk;
    const int64_t* ti = a.topk_idx;
    uint8_t* pair_state = a.rwk + a.L.pair_state_off;
    int* rsc = reinterpret_cast<int*>(a.rwk + a.L.route_slot_counts_off);

    // many pairs: one pass over this rank's pairs instead of one scan per expert
    const bool onepass = team.bar == 0 && np > kRoutePer * nthr && route_onepass(a, f, epoch, s_big, s_big_ints, local_only);
#pragma unroll 1
    for (int e = blockIdx.x; e < a.E && !onepass; e += gridDim.x) {
        const int dst = a.fEPR.div(e), le = a.fEPR.mod(e);
        uint8_t* peer_unk = reinterpret_cast<uint8_t*>(a.unk_peers[dst]);
        uint64_t* tbl = reinterpret_cast<uint64_t*>(peer_unk + a.L.src_index_table_off) +
                        (((size_t)par * a.EPR + le) * a.R + a.rank) * (size_t)a.slot_cap;
        int base = 0;
        // kRoutePer sub-chunks of blockDim pairs per iteration: the index loads of all sub-chunks
        // are in flight together, then slots are handed out sub-chunk by sub-chunk (ascending idx)
#pragma unroll 1
        for (int p0 = 0; p0 < np; p0 += nthr * kRoutePer) {
            bool hit[kRoutePer];
            unsigned bal[kRoutePer];
            int64_t v[kRoutePer];
#pragma unroll
            for (int j = 0; j < kRoutePer; ++j) {
                const int p = p0 + j * nthr + tid;
                v[j] = p < np ? ti[p] : (int64_t)-2;
            }
#pragma unroll
            for (int j = 0; j < kRoutePer; ++j) {
                hit[j] = v[j] == (int64_t)e;
                bal[j] = __ballot_sync(0xFFFFFFFFu, hit[j]);
                if (lane == 0) s_wtot[j * nwarps + warp] = __popc(bal[j]);
            }
            team.sync();
#pragma unroll
            for (int j = 0; j < kRoutePer; ++j) {
                int wpre = 0, tot = 0;
#pragma unroll 1
                for (int w = 0; w < nwarps; ++w) {
                    const int c = s_wtot[j * nwarps + w];
                    wpre += (w < warp) ? c : 0;
                    tot += c;
                }
                if (hit[j]) {
                    const int p = p0 + j * nthr + tid;
                    const int slot = base + wpre + __popc(bal[j] & ((1u << lane) - 1u));
                    const bool ok = slot < a.slot_cap;  // over capacity: dropped (src/prologue.cuh:171-174)
                    if (ok && !local_only) st_relaxed_sys_u64(tbl + slot, tagged((uint32_t)p, epoch));
                    pair_state[p] = ok ? 1 : 0;
                }
                base += tot;
            }
            team.sync();
        }
        if (tid == 0) {
            const int c = base < a.slot_cap ? base : a.slot_cap;
            rsc[e] = c;
            if (!local_only) {
                uint64_t* recv = reinterpret_cast<uint64_t*>(peer_unk + a.L.expert_recv_counts_off) +
                                 ((size_t)par * a.R + a.rank) * a.L.recv_stride;
                st_relaxed_sys_u64(recv + le, tagged((uint32_t)c, epoch));
            }
        }
    }
    // The launch bookkeeping below belongs to the LAST CTA: CTA 0 goes straight on to poll the
    // counts and build the tables, which is the critical path of the prologue.
    const bool closer = blockIdx.x == gridDim.x - 1;
    if (closer && !onepass)  // invalid expert ids (negative / >= E) take no slot (src/prologue.cuh:166-167)
#pragma unroll 1
        for (int p = tid; p < np; p += nthr)
            if ((uint64_t)ti[p] >= (uint64_t)a.E) pair_state[p] = 0;

    // Everything below is off the critical path (the counts are already on their way): make
    // this CTA's local tables visible, arrive, and let the last CTA close the launch bookkeeping.
    __threadfence();
    team.sync();
    if (tid == 0) atomicAdd(&f->route_blocks_done, 1u);
    if (!closer) return;

    if (tid == 0) {
        const unsigned want = gridDim.x;
        if (!spin_until([&] { return ld_acquire_gpu(&f->route_blocks_done) >= want; }, a.local_wait_ns, nullptr))
            raise_status(f, MXK_DEV_TIMEOUT_PIPE, 2);
    }
    team.sync();
    // Row checksum word ~(sum + 1) at index EPR of each row sent (src/prologue.cuh:248-255), kept
    // for layout parity with the reference; nothing here waits on it.
#pragma unroll 1
    for (int d = tid; d < a.R && !local_only; d += nthr) {
        uint32_t csum = 0;
#pragma unroll 1
        for (int le = 0; le < a.EPR; ++le) csum += (uint32_t)ld_relaxed_gpu(rsc + d * a.EPR + le);
        uint64_t* recv = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(a.unk_peers[d]) +
                                                     a.L.expert_recv_counts_off) +
                         ((size_t)par * a.R + a.rank) * a.L.recv_stride;
        st_relaxed_sys_u64(recv + a.EPR, tagged(~(csum + 1u), epoch));
    }
    if (tid == 0) {
        f->route_blocks_done = 0;
        f->clear_blocks_done = 0;  // every CTA is past the clear barrier, if there was one
        f->route_sync = 0;         // and past the barrier of the one-pass route
        // a rank without tokens receives no rows and runs no reduce: its (all-zero) table stays clean
        if (a.tokens == 0) f->cnt_clean_epoch = (uint32_t)epoch;
        __threadfence();           // the reduce phase takes the counter as "every CTA's route tables are written"
        f->current_time = epoch;   // every CTA has read the old value before arriving above
    }
    team.sync();
}

// From the per-(local expert, source rank) counts s_cnt[EPR][R] of this launch: the prefix table
// (written to `prefix`, [EPR][R+1], shared or global memory), rows per expert, the experts ranked
// by descending row count (ties by index: the hottest experts' windows are claimed first so the
// dynamic queue ends on the cheap ones — LPT order), the first window of every sorted position and
// the first pool row of every expert (reference: task_setup_body, src/prologue.cuh:423-452).
// Called by all threads of a CTA; the results are valid after it returns.
__device__ void build_tables(const KArgs& a, const int* s_cnt, int* prefix, int* s_tot /*[EPR]*/,
                             int* s_order /*[EPR]*/, int* s_first /*[EPR+1]*/, int* s_base /*[EPR+1]*/) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int EPR = a.EPR, R = a.R;
#pragma unroll 1
    for (int le = tid; le < EPR; le += nthr) {
        int c = 0;
#pragma unroll 1
        for (int r = 0; r < R; ++r) {
            prefix[le * (R + 1) + r] = c;
            c += s_cnt[le * R + r];
        }
        prefix[le * (R + 1) + R] = c;
        s_tot[le] = c;
    }
    __syncthreads();
#pragma unroll 1
    for (int le = tid; le < EPR; le += nthr) {
        const int c = s_tot[le];
        int rk = 0;
#pragma unroll 1
        for (int j = 0; j < EPR; ++j) {
            const int cj = s_tot[j];
            rk += (cj > c || (cj == c && j < le)) ? 1 : 0;
        }
        s_order[rk] = le;
    }
    __syncthreads();
    if (tid < 32) {
        // exclusive scans by warp 0: pool rows in expert-index order, windows in sorted order
        const int lane = tid;
        int carry_rows = 0, carry_win = 0;
#pragma unroll 1
        for (int b = 0; b < EPR; b += 32) {
            const int i = b + lane;
            const int c = i < EPR ? s_tot[i] : 0;
            const int cs = i < EPR ? s_tot[s_order[i]] : 0;
            const int w = cs > 0 ? (cs + a.win_cap - 1) / a.win_cap : 0;
            int ic = c, iw = w;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int uc = __shfl_up_sync(0xFFFFFFFFu, ic, d), uw = __shfl_up_sync(0xFFFFFFFFu, iw, d);
                if (lane >= d) { ic += uc; iw += uw; }
            }
            if (i < EPR) { s_base[i] = carry_rows + ic - c; s_first[i] = carry_win + iw - w; }
            carry_rows += __shfl_sync(0xFFFFFFFFu, ic, 31);
            carry_win += __shfl_sync(0xFFFFFFFFu, iw, 31);
        }
        if (lane == 0) { s_base[EPR] = carry_rows; s_first[EPR] = carry_win; }
    }
    __syncthreads();
}

__device__ __forceinline__ bool tables_overflow(const KArgs& a, int n_windows, int total_rows) {
    const int nt1 = a.I / 128, nt2 = a.H / kBlockN;
    return n_windows > a.L.max_windows || (long long)n_windows * (nt1 + nt2) > a.L.max_tasks || total_rows > a.L.pool_rows;
}

// CTA 0 writes the tables of this launch to global memory (row bases, windows, the task list — L1
// tasks then L2 tasks, each (expert, n-tile, window) with windows fastest so that concurrent CTAs
// share a weight tile in L2), clears the gate counters, and publishes the set-up flag.
struct PushTabs;
__device__ void publish_helper_lists(const KArgs& a, const PushTabs* T);
__device__ void helper_counts(const PushTabs* T, int* n_windows, int* n_l1, int* rows);
__device__ void publish_tables(const KArgs& a, DevFlags* f, long long epoch, const int* s_tot, const int* s_order,
                               const int* s_first, const int* s_base, const PushTabs* helper = nullptr) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int EPR = a.EPR;
    const int par = (int)(epoch & 1);
    const bool ts = a.ticks != 0 && tid == 0;
    int* row_base = reinterpret_cast<int*>(a.rwk + a.L.expert_row_base_off);
    int* first_win = reinterpret_cast<int*>(a.rwk + a.L.expert_first_win_off);
#pragma unroll 1
    for (int le = tid; le <= EPR; le += nthr) row_base[le] = s_base[le];
#pragma unroll 1
    for (int p = tid; p < EPR; p += nthr) first_win[s_order[p]] = s_first[p];

    int n_windows = s_first[EPR];
    const int total_rows = s_base[EPR];
    const int nt1 = a.I / 128, nt2 = a.H / kBlockN;
    const bool overflow = tables_overflow(a, n_windows, total_rows);
    if (overflow) n_windows = 0;
    int4* windows = reinterpret_cast<int4*>(a.rwk + a.L.windows_off);
    int4* tasks = reinterpret_cast<int4*>(a.rwk + a.L.tasks_off);
    uint32_t* l1_done = reinterpret_cast<uint32_t*>(a.rwk + a.L.l1_done_off);
    uint32_t* pool_ready = reinterpret_cast<uint32_t*>(a.rwk + a.L.pool_ready_off);
    // The gate counters exist once per launch parity.  This launch's copy was cleared while the
    // previous launch ran (push mode counts rows into it without waiting for this CTA); the other
    // copy, last used by the previous launch, is cleared here for the next one.
    {
        const int prev_windows = min(max(ld_relaxed_gpu(&f->n_windows), 0), a.L.max_windows);
        uint32_t* l1_o = l1_done + (size_t)(par ^ 1) * a.L.max_windows;
        uint32_t* pr_o = pool_ready + (size_t)(par ^ 1) * a.L.max_windows;
#pragma unroll 1
        for (int i = tid; i < prev_windows; i += nthr) { l1_o[i] = 0; pr_o[i] = 0; }
    }
    __syncthreads();   // n_windows of the previous launch was read by every thread above
    l1_done += (size_t)par * a.L.max_windows;
    pool_ready += (size_t)par * a.L.max_windows;
    int n_l1 = n_windows * nt1;
    if (helper) {
        // cross-rank helper scheduling: the lists are this member's windows, not the owner layout
        publish_helper_lists(a, helper);
    } else if (!overflow) {
        // one warp per expert (sorted position p), lanes over its windows and tasks
        const int lane = tid & 31, wid = tid >> 5, nwarps = nthr >> 5;
#pragma unroll 1
        for (int p = wid; p < EPR; p += nwarps) {
            const int e = s_order[p], c = s_tot[e];
            const int fw = s_first[p], nw = s_first[p + 1] - fw;
            if (nw == 0) break;  // sorted: every later expert is empty too
#pragma unroll 1
            for (int w = lane; w < nw; w += 32) {
                const int rows = min(a.win_cap, c - w * a.win_cap);
                windows[fw + w] = make_int4(e, s_base[e] + w * a.win_cap, rows, 0);
                if (!a.push) { l1_done[fw + w] = 0; pool_ready[fw + w] = 0; }
            }
#pragma unroll 1
            for (int i = lane; i < nt1 * nw; i += 32) {
                const int nt = i / nw, w = i % nw;
                tasks[fw * nt1 + i] = make_int4(0, fw + w, nt, min(a.win_cap, c - w * a.win_cap));
            }
#pragma unroll 1
            for (int i = lane; i < nt2 * nw; i += 32) {
                const int nt = i / nw, w = i % nw;
                tasks[n_l1 + fw * nt2 + i] = make_int4(1, fw + w, nt, min(a.win_cap, c - w * a.win_cap));
            }
        }
    }
    if (ts) f->dbg_ts[4] = gtimer_ns();
    if (tid == 0) {
        if (overflow) raise_status(f, MXK_DEV_BAD_TABLE, 3);
        int rows_out = overflow ? 0 : total_rows;
        if (helper) helper_counts(helper, &n_windows, &n_l1, &rows_out);
        f->helper_on = helper ? 1 : 0;
        f->n_windows = n_windows;
        f->n_l1_tasks = n_l1;
        f->n_tasks = n_windows * (nt1 + nt2);
        f->total_rows = rows_out;
        f->task_ctr[par ^ 1] = 0;   // the next launch's claim counter
    }
    __threadfence();
    __syncthreads();
    if (ts) f->dbg_ts[5] = gtimer_ns();
    if (tid == 0) st_release_gpu(&f->setup_epoch, (uint32_t)epoch);
    if (ts) f->dbg_ts[6] = gtimer_ns();
}

// Pull mode, CTA 0: wait for every source rank's counts (this IS the cross-rank barrier), build
// and publish the tables; `s_i` is scratch shared memory of 4*EPR + 2 + EPR*R ints.
__device__ void setup_phase_leader(const KArgs& a, DevFlags* f, long long epoch, int* s_i) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int EPR = a.EPR, R = a.R;
    int* s_tot = s_i;                  // [EPR]
    int* s_order = s_tot + EPR;        // [EPR] expert at sorted position p
    int* s_first = s_order + EPR;      // [EPR+1] first window of position p
    int* s_base = s_first + EPR + 1;   // [EPR+1] first pool row of expert le
    const int par = (int)(epoch & 1);

    // Cross-rank barrier = every (source rank, local expert) count word carries this epoch.
    int* s_cnt = s_base + EPR + 1;     // [EPR][R]
    const uint64_t* recv = reinterpret_cast<const uint64_t*>(a.unk + a.L.expert_recv_counts_off) +
                           (size_t)par * R * a.L.recv_stride;
#pragma unroll 1
    for (int i = tid; i < EPR * R; i += nthr) {
        const int le = i / R, r = i % R;
        const uint64_t* wp = recv + (size_t)r * a.L.recv_stride + le;
        uint64_t w = 0;
        const bool ok = spin_until([&] { w = ld_relaxed_sys_u64(wp); return (uint32_t)(w >> 32) == (uint32_t)epoch; },
                                   a.remote_wait_ns, nullptr);
        if (!ok) { raise_status(f, MXK_DEV_TIMEOUT_BARRIER, 0); w = 0; }
        s_cnt[i] = (int)(uint32_t)w;
    }
    __syncthreads();
    const bool ts = a.ticks != 0 && tid == 0;
    if (ts) f->dbg_ts[0] = gtimer_ns();
    build_tables(a, s_cnt, reinterpret_cast<int*>(a.rwk + a.L.prefix_tbl_off), s_tot, s_order, s_first, s_base);
    if (ts) f->dbg_ts[3] = gtimer_ns();
    publish_tables(a, f, epoch, s_tot, s_order, s_first, s_base);
}

// Every other CTA waits until CTA 0 has published the tables of this epoch.
__device__ bool setup_phase_wait(const KArgs& a, DevFlags* f, long long epoch, int* s_flag) {
    if (threadIdx.x == 0) {
        // relaxed polls with a short back-off (148 CTAs watch this word while CTA 0 works),
        // one acquire fence once it flips
        const bool ok = spin_until([&] { if (ld_relaxed_gpu(&f->setup_epoch) == (uint32_t)epoch) return true; __nanosleep(200); return false; },
                                   a.remote_wait_ns + a.local_wait_ns, nullptr);
        fence_acq_rel_gpu();
        if (!ok) raise_status(f, MXK_DEV_TIMEOUT_BARRIER, 1);
        *s_flag = ok ? 1 : 0;
    }
    __syncthreads();
    return *s_flag != 0;
}

// One warp per pool row: locate (expert, source rank, slot), read the pair index
// the source wrote, then pull the row's H bytes and H/128 scale bytes from the
// source rank's symmetric buffer with 16-byte loads over NVLink; finally count
// the row into its window's pool_ready counter (the TMA producer of the GEMM
// phase waits on it).
__device__ void dispatch_phase(const KArgs& a, DevFlags* f, long long epoch, int* s_tab) {
    const int lane = threadIdx.x & 31;
    const int nwarps_cta = blockDim.x >> 5;
    const int gwarp = blockIdx.x * nwarps_cta + (threadIdx.x >> 5);
    const int nwarps = gridDim.x * nwarps_cta;
    const int total = ld_relaxed_gpu(&f->total_rows);
    const int par = (int)(epoch & 1);
    const int R = a.R, EPR = a.EPR, H = a.H;
    const uint64_t* tbl = reinterpret_cast<const uint64_t*>(a.unk + a.L.src_index_table_off) +
                          (size_t)par * EPR * R * a.slot_cap;
    uint8_t* pool = a.rwk + a.L.pool_off;
    uint8_t* pool_sf = a.rwk + a.L.pool_sf_off;
    int4* meta = reinterpret_cast<int4*>(a.rwk + a.L.row_meta_off);
    uint32_t* pool_ready = reinterpret_cast<uint32_t*>(a.rwk + a.L.pool_ready_off) + (size_t)par * a.L.max_windows;
    const int kb = H / 128;
    if (blockIdx.x * nwarps_cta >= total) return;  // no row for this CTA (uniform per CTA)

    // Row-lookup tables of this launch, copied once per CTA into shared memory: the per-row
    // searches would otherwise be chains of dependent global loads.
    int* row_base = s_tab;                  // [EPR+1]
    int* first_win = row_base + EPR + 1;    // [EPR]
    int* prefix = first_win + EPR;          // [EPR][R+1]
    {
        const int* g_base = reinterpret_cast<const int*>(a.rwk + a.L.expert_row_base_off);
        const int* g_fw = reinterpret_cast<const int*>(a.rwk + a.L.expert_first_win_off);
        const int* g_pf = reinterpret_cast<const int*>(a.rwk + a.L.prefix_tbl_off);
#pragma unroll 1
        for (int i = threadIdx.x; i <= EPR; i += blockDim.x) row_base[i] = ld_relaxed_gpu(g_base + i);
#pragma unroll 1
        for (int i = threadIdx.x; i < EPR; i += blockDim.x) first_win[i] = ld_relaxed_gpu(g_fw + i);
#pragma unroll 1
        for (int i = threadIdx.x; i < EPR * (R + 1); i += blockDim.x) prefix[i] = ld_relaxed_gpu(g_pf + i);
        __syncthreads();
    }

#pragma unroll 1
    for (int g = gwarp; g < total; g += nwarps) {
        int lo = 0, hi = EPR;  // largest le with row_base[le] <= g
#pragma unroll 1
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (row_base[mid] <= g) lo = mid; else hi = mid;
        }
        const int le = lo;
        const int gl = g - row_base[le];
        const int* pf = prefix + le * (R + 1);
        int slo = 0, shi = R;  // largest src with pf[src] <= gl (src/compute_big.cuh:1760-1769)
#pragma unroll 1
        while (shi - slo > 1) {
            const int mid = (slo + shi) >> 1;
            if (pf[mid] <= gl) slo = mid; else shi = mid;
        }
        const int src = slo, slot = gl - pf[src];
        // the pair index the source rank wrote for this slot (epoch-tagged: poll until it is this launch's)
        uint64_t tw = 0;
        {
            const uint64_t* tp = tbl + ((size_t)le * R + src) * a.slot_cap + slot;
            if (!spin_until([&] { tw = ld_relaxed_sys_u64(tp); return (uint32_t)(tw >> 32) == (uint32_t)epoch; },
                            a.remote_wait_ns, nullptr)) {
                if (lane == 0) raise_status(f, MXK_DEV_TIMEOUT_BARRIER, 2);
                tw = 0;
            }
        }
        uint32_t idx = (uint32_t)tw;
        if (idx >= (uint32_t)(a.cap * a.topk)) {   // not a pair index of this geometry: never form an address from it
            if (lane == 0) raise_status(f, MXK_DEV_BAD_TABLE, 3);
            idx = 0;
        }
        const int token = a.ftopk.div((int)idx), k = (int)idx - token * a.topk;
        const uint8_t* peer = a.peer_bases[src];
        const uint4* srow = reinterpret_cast<const uint4*>(peer + a.x_off + (size_t)token * H);
        uint4* drow = reinterpret_cast<uint4*>(pool + (size_t)g * H);
        const int n16 = H / 16;
        uint32_t wbits = 0;
        if (lane == 0)  // issued first so that it travels with the row
            wbits = ld_relaxed_sys(reinterpret_cast<const uint32_t*>(peer + a.weights_off) + (size_t)token * a.topk + k);
        // the row's scale bytes too (up to 64 K blocks): requested before the row so that the whole
        // row costs ONE round trip to the source rank
        uint8_t sfb[2] = {127, 127};
        if (a.scaled) {
            const uint8_t* ssf = peer + a.x_sf_off + (size_t)token * kb;
            if (lane < kb) sfb[0] = ld_relaxed_sys_u8(ssf + lane);
            if (lane + 32 < kb) sfb[1] = ld_relaxed_sys_u8(ssf + lane + 32);
        }
        // up to 16 loads in flight per lane before the first store (the strong loads are not
        // reordered by the compiler, so issue order is what hides the NVLink round trip)
#pragma unroll 1
        for (int i0 = lane; i0 < n16; i0 += 32 * 16) {
            uint4 v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (i0 + 32 * j < n16) v[j] = ld_relaxed_sys_v4(srow + i0 + 32 * j);
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (i0 + 32 * j < n16) drow[i0 + 32 * j] = v[j];
        }
        if (a.scaled) {
            const uint8_t* ssf = peer + a.x_sf_off + (size_t)token * kb;
#pragma unroll 1
            for (int i = lane; i < a.L.sf_stride_h; i += 32)
                pool_sf[(size_t)g * a.L.sf_stride_h + i] =
                    i < 64 ? sfb[i >> 5] : (i < kb ? ld_relaxed_sys_u8(ssf + i) : (uint8_t)127);
        }
        if (lane == 0) meta[g] = make_int4(src, token, k, (int)wbits);
        // the row is complete: every lane makes its stores visible at GPU scope and to TMA
        // (a release by lane 0 alone does not cover the other lanes' stores), then count the row
        __threadfence();
        fence_proxy_async_global();
        __syncwarp();
        if (lane == 0) red_release_gpu_add(pool_ready + first_win[le] + a.fwin.div(gl), 1u);
    }
}

// ============================================================ push-mode prologue
// Staging area `xin` in unk, per launch parity and source rank: 16 header words (word 0 = token
// count of the source in this launch) followed by one row per token:
//   [topk routing words][topk weight words][sfw scale words][H/4 row words]
// Every word is {payload u32, epoch u32}, stored with 8-byte (or 2 x 8-byte) stores: the reader
// polls the word itself until the tag is this launch's epoch, so the data needs neither a fence
// nor a flag.  Routing and weight words go to every rank, scale and row words only to the ranks
// that own one of the token's experts.  Two parities are enough for the same reason as in the
// pull-mode tables: no rank can finish launch N+1 before every rank has pushed for N+1.
constexpr int kPushMaxEPR = 256;       // local experts whose tables fit the control block
constexpr int kPushMaxR = 64;
constexpr int kSlimRows = 32;         // activation rows staged per ring slot when every window is that small
constexpr int kPushMaxPairs = 16384;   // routing words of the whole world kept in shared memory per CTA
constexpr int kPushAutoPairsPerRank = 2048;  // dispatch_mode 0 pushes up to this many routed pairs per rank (max_tokens * topk)
constexpr int kPushAutoPairsPerRankWorld = 1024;  // ... in a world of several ranks, where the tagged rows cross NVLink
constexpr int kHelperHotWindows = 3;         // helper groups spread the windows of experts with at least this many windows
constexpr int kPushMaxCnt = 4096;      // EPR * (R + 1)

constexpr int kHelperMaxWin = 512;     // windows one member may be handed (reference: kGsMemberCap, src/group_sched.cuh:150-154)

struct PushTabs {   // tables of this launch, in the control block of shared memory for the whole kernel
    int n_tasks, n_l1, n_windows, total_rows;
    int parts;                    // warps that share the copy of one pool row (each counts into pool_ready)
    int helper;                   // 1: cross-rank helper scheduling is on, the tables are this member's window list
    int slim;                     // 1: no window of this launch has more than kSlimRows rows (see gemm_phase)
    union {
        struct {                          // owner layout: this rank computes exactly its own experts
            int tot[kPushMaxEPR];         // rows of local expert le
            int order[kPushMaxEPR];       // expert at sorted position p (descending rows)
            int first[kPushMaxEPR + 1];   // first window of sorted position p
            int base[kPushMaxEPR + 1];    // first pool row of local expert le
        };
        struct {                          // helper layout: window i of this member's list
            int gw[kHelperMaxWin];        // (group expert ge << 16) | window w of that expert
            int rr[kHelperMaxWin];        // (first pool row << 10) | rows
        };
    };
};

struct PushScratch {   // carved from the operand-tile region, which is idle until the GEMM phase
    int* wid;      // [kPushMaxPairs] routing word of world pair i (expert id or -1), sources in rank order
    int* cnt;      // [GE][R] pairs per (group expert, source); GE = EPR without helper groups
    int* prefix;   // [GE][R+1]
    int* fw_e;     // [EPR] first window of local expert le
    int* tok;      // [R] tokens of source r in this launch
    int* sb;       // [R+1] first world pair of source r
    int* flag;     // [1] every source arrived in time
    int* tot;      // [EPR] owner-layout tables of this rank's own experts (published by CTA 0; the
    int* order;    // [EPR]  copy in PushTabs is what the GEMM phase uses unless helpers are on)
    int* first;    // [EPR+1]
    int* base;     // [EPR+1]
    int* totg;     // [GE] rows per group expert
    int* gws;      // [GE+1] first entry of group expert ge in widx
    int* widx;     // [group windows] index of (ge, w) in this member's list, -1 = another member's
    int* scan;     // [17] warp totals of the compaction below, then the length of `mine`
    unsigned short* mine;   // [kPushMaxPairs] the world pairs whose expert belongs to this rank's group, ascending
};
constexpr int kPushMaxGroupWin = 4096;   // windows of a whole helper group (lookup table entries)
__device__ __forceinline__ PushScratch push_scratch(uint8_t* tiles) {
    PushScratch sc;
    sc.wid = reinterpret_cast<int*>(tiles);
    sc.cnt = sc.wid + kPushMaxPairs;
    sc.prefix = sc.cnt + kPushMaxCnt;
    sc.fw_e = sc.prefix + kPushMaxCnt + kPushMaxEPR;
    sc.tok = sc.fw_e + kPushMaxEPR;
    sc.sb = sc.tok + kPushMaxR;
    sc.flag = sc.sb + kPushMaxR + 1;
    sc.tot = sc.flag + 1;
    sc.order = sc.tot + kPushMaxEPR;
    sc.first = sc.order + kPushMaxEPR;
    sc.base = sc.first + kPushMaxEPR + 1;
    sc.totg = sc.base + kPushMaxEPR + 1;
    sc.gws = sc.totg + kPushMaxCnt;
    sc.widx = sc.gws + kPushMaxCnt + 1;
    sc.scan = sc.widx + kPushMaxGroupWin;
    sc.mine = reinterpret_cast<unsigned short*>(sc.scan + 20);
    return sc;
}
static_assert(kPushMaxPairs <= 65536, "pair indices fit 16 bits");
static_assert((kPushMaxPairs + kPushMaxPairs / 2 + 4 * kPushMaxCnt + 8 * kPushMaxEPR + 2 * kPushMaxR + kPushMaxGroupWin + 48) * 4 <= 192 * 1024,
              "push-mode scratch fits the operand-tile region (4 stages of 48 KB)");
__device__ __forceinline__ int xin_sf_words(int H) { return (((H / 128) + 3) / 4 + 1) & ~1; }   // even: rows stay 16-byte aligned
__device__ __forceinline__ uint64_t* xin_block(const KArgs& a, void* unk_base, int par, int src) {
    return reinterpret_cast<uint64_t*>(static_cast<uint8_t*>(unk_base) + a.L.xin_off) +
           ((size_t)par * a.R + src) * (size_t)a.L.xin_src_words;
}
// largest r with sb[r] <= i (sources without tokens share their successor's start)
__device__ __forceinline__ int push_src_of(const int* sb, int R, int i) {
    int lo = 0, hi = R;
#pragma unroll 1
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (sb[mid] <= i) lo = mid; else hi = mid;
    }
    return lo;
}

// Source side: store this rank's tokens into the owners' staging areas.  Work unit = (token,
// destination rank), spread over the grid.  `s_ids` is scratch for tokens*topk ints.
// Every global load of a unit (row, weights, scales, peer pointer) is issued before anything
// waits, and for the CTA's first unit even before the routing words are in shared memory: the
// whole phase costs one memory round trip plus the stores.
__device__ void push_phase(const KArgs& a, DevFlags* f, long long epoch, int* s_ids) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int par = (int)(epoch & 1), R = a.R, topk = a.topk, H = a.H;
    const int np = a.tokens * topk;
    const int sfw = xin_sf_words(H), kb = H / 128, row_words = a.L.xin_row_words, n16 = H / 8;
    const uint32_t* wts = reinterpret_cast<const uint32_t*>(a.self + a.weights_off);
    const uint8_t* xsf = a.self + a.x_sf_off;
    constexpr int kMaxPer = 3;   // 16-byte units of a row per thread: H <= 8192 -> 1024 units over 384 threads
    struct Unit { uint2 x[kMaxPer]; uint32_t w, sf; void* peer; };
    auto load_unit = [&](int u, Unit& un) {
        const int t = a.fR.div(u);
        const uint2* xs = reinterpret_cast<const uint2*>(a.self + a.x_off + (size_t)t * H);
#pragma unroll
        for (int j = 0; j < kMaxPer; ++j)
            if (tid + j * nthr < n16) un.x[j] = xs[tid + j * nthr];
        un.w = (tid >= topk && tid < 2 * topk) ? wts[(size_t)t * topk + tid - topk] : 0u;
        un.sf = 0;
        if (a.scaled && tid >= 128 && tid < 128 + sfw) {   // four scale bytes per word, 127 (x1.0) beyond H/128
            const int i = tid - 128;
#pragma unroll 1
            for (int j = 0; j < 4; ++j) {
                const int b = 4 * i + j;
                un.sf |= (uint32_t)(b < kb ? xsf[(size_t)t * kb + b] : (uint8_t)127) << (8 * j);
            }
        }
        un.peer = a.unk_peers[a.fR.mod(u + t)];
    };
    const int n_units = a.tokens * R;
    Unit un;
    if ((int)blockIdx.x < n_units) load_unit(blockIdx.x, un);
    void* hdr_peer = (blockIdx.x == gridDim.x - 1 && tid < R) ? a.unk_peers[tid] : nullptr;
#pragma unroll 1
    for (int p = tid; p < np; p += nthr) {   // invalid ids (negative / >= E) travel as -1 (src/prologue.cuh:166-167)
        const int64_t v = a.topk_idx[p];
        s_ids[p] = (uint64_t)v < (uint64_t)a.E ? (int)v : -1;
    }
    if (hdr_peer)   // header: how many rows the destination has to expect from this rank
        st_relaxed_sys_u64(xin_block(a, hdr_peer, par, a.rank), tagged((uint32_t)a.tokens, epoch));
    __syncthreads();
#pragma unroll 1
    for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
        const int t = a.fR.div(u), d = a.fR.mod(u + t);
        bool routed = false;
#pragma unroll 1
        for (int k = 0; k < topk; ++k) {
            const int e = s_ids[t * topk + k];
            routed |= e >= 0 && a.fEPR.div(e) == d;
        }
        uint64_t* row = xin_block(a, un.peer, par, a.rank) + 16 + (size_t)t * row_words;
        if (tid < topk) st_relaxed_sys_u64(row + tid, tagged((uint32_t)s_ids[t * topk + tid], epoch));
        else if (tid < 2 * topk) st_relaxed_sys_u64(row + tid, tagged(un.w, epoch));
        if (routed) {
            if (a.scaled && tid >= 128 && tid < 128 + sfw) st_relaxed_sys_u64(row + 2 * topk + tid - 128, tagged(un.sf, epoch));
            uint64_t* xd = row + 2 * topk + sfw;
#pragma unroll
            for (int j = 0; j < kMaxPer; ++j) {
                const int i = tid + j * nthr;
                if (i < n16) st_relaxed_sys_v2_u64(xd + 2 * i, tagged(un.x[j].x, epoch), tagged(un.x[j].y, epoch));
            }
        }
        if (u + (int)gridDim.x < n_units) load_unit(u + gridDim.x, un);
    }
}

__device__ void helper_counts(const PushTabs* T, int* n_windows, int* n_l1, int* rows) {
    *n_windows = T->n_windows; *n_l1 = T->n_l1; *rows = T->total_rows;
}
// Helper layout: window i = (ge, first pool row, rows, w), tasks window-major (kind, i, n-tile, rows).
__device__ void publish_helper_lists(const KArgs& a, const PushTabs* T) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int nt1 = a.I / 128, nt2 = a.H / kBlockN;
    int4* windows = reinterpret_cast<int4*>(a.rwk + a.L.windows_off);
    int4* tasks = reinterpret_cast<int4*>(a.rwk + a.L.tasks_off);
#pragma unroll 1
    for (int i = tid; i < T->n_windows; i += nthr)
        windows[i] = make_int4(T->gw[i] >> 16, T->rr[i] >> 10, T->rr[i] & 1023, T->gw[i] & 0xFFFF);
#pragma unroll 1
    for (int t = tid; t < T->n_tasks; t += nthr) {
        const int kind = t >= T->n_l1 ? 1 : 0, nt = kind ? nt2 : nt1, tt = kind ? t - T->n_l1 : t;
        tasks[t] = make_int4(kind, tt / nt, tt % nt, T->rr[tt / nt] & 1023);
    }
}

// The member's window list of the helper group, by ONE WARP: the assignment of
// sched_member_windows (descending cost, (ge, w) ascending, least-loaded member, ties to the owner
// then the lowest member) with the members' loads held one per lane, so that a window costs a few
// shuffles instead of a loop over the members.  Every lane returns the same counts.
__device__ void helper_member_list(const int* totg, int GE, const FastDiv fEPR, int G, int win_cap, int member, int hot_windows,
                                   PushTabs* T) {
    const int lane = threadIdx.x & 31;
    int load = 0, n = 0, rowcur = 0;
    const int full_cost = sched_window_cost(win_cap);
    if (hot_windows > 0 && lane < G) {   // lane m: the work of member m's own experts that stays with it
        const int EPR = GE / G;
#pragma unroll 1
        for (int le = 0; le < EPR; ++le) {
            const int c = max(totg[lane * EPR + le], 0);
            if (c == 0 || sched_expert_hot(c, win_cap, hot_windows)) continue;
            load += (c / win_cap) * full_cost + (c % win_cap ? sched_window_cost(c % win_cap) : 0);
        }
    }
#pragma unroll 1
    for (int level = full_cost; level >= 1; --level) {
#pragma unroll 1
        for (int ge0 = 0; ge0 < GE; ge0 += 32) {
            const int ge = ge0 + lane;
            const int c = ge < GE ? max(totg[ge], 0) : 0;
            const int n_full = c / win_cap, tail = c % win_cap;
            int w_lo = 0, w_hi = 0;
            if (level == full_cost) w_hi = n_full;
            if (tail != 0 && sched_window_cost(tail) == level) {
                if (w_hi == 0) w_lo = n_full;
                w_hi = n_full + 1;
            }
            // hot-expert schedule: a cold expert of ANOTHER member changes nothing here (its windows stay with
            // that member, whose load already counts them), so only hot experts and this member's own are walked
            const bool relevant = hot_windows <= 0 || sched_expert_hot(c, win_cap, hot_windows) || fEPR.div(ge) == member;
            unsigned mask = __ballot_sync(0xFFFFFFFFu, w_hi > w_lo && relevant);
#pragma unroll 1
            while (mask) {
                const int l = __ffs(mask) - 1;
                mask &= mask - 1;
                const int g_e = ge0 + l, owner = fEPR.div(g_e);
                const int lo = __shfl_sync(0xFFFFFFFFu, w_lo, l), hi = __shfl_sync(0xFFFFFFFFu, w_hi, l);
                const int ctot = __shfl_sync(0xFFFFFFFFu, c, l);
                const bool hot = sched_expert_hot(ctot, win_cap, hot_windows);
#pragma unroll 1
                for (int w = lo; w < hi; ++w) {
                    int best = owner;
                    if (hot) {
                        const int mine = lane < G ? load : 0x7FFFFFFF;
                        int mn = mine;
#pragma unroll
                        for (int d = 16; d > 0; d >>= 1) mn = min(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, d));
                        const unsigned tie = __ballot_sync(0xFFFFFFFFu, mine == mn);
                        best = ((tie >> owner) & 1u) ? owner : __ffs(tie) - 1;
                        if (lane == best) load += level;
                    }
                    if (best == member) {
                        const int rows = min(win_cap, ctot - w * win_cap);
                        if (lane == 0 && n < kHelperMaxWin) {
                            T->gw[n] = (g_e << 16) | w;
                            T->rr[n] = (rowcur << 10) | rows;
                        }
                        ++n;
                        rowcur += rows;
                    }
                }
            }
        }
    }
    if (lane == 0) { T->n_windows = n; T->total_rows = rowcur; }
}

// Owner side, EVERY CTA: wait for all sources' routing words of this launch (this is the
// cross-rank barrier), count the pairs per (group expert, source) and build the tables in shared
// memory: the owner-layout tables of this rank's own experts always (scratch; CTA 0 publishes
// them), and what the GEMM phase runs on — the same tables, or, when helper groups are configured
// and the group's load is skewed, this member's window list.  Without helper groups the "group" is
// the rank itself.  Returns false when a source did not arrive in time or the tables overflow.
__device__ bool push_tables(const KArgs& a, DevFlags* f, long long epoch, const PushScratch& sc, PushTabs* T) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int par = (int)(epoch & 1), R = a.R, topk = a.topk, EPR = a.EPR;
    const int G = a.group_ranks, GE = G * EPR, n_groups = R / G, my_group = a.rank % n_groups, mm = a.rank / n_groups;
    const uint32_t ep = (uint32_t)epoch;
    const uint64_t* mine = xin_block(a, a.unk, par, 0);
    const size_t src_words = (size_t)a.L.xin_src_words;
    const int row_words = a.L.xin_row_words;
    if (tid == 0) *sc.flag = 1;
#pragma unroll 1
    for (int i = tid; i < GE * R; i += nthr) sc.cnt[i] = 0;
#pragma unroll 1
    for (int r = tid; r < R; r += nthr) {
        const uint64_t* hp = mine + r * src_words;
        uint64_t w = 0;
        if (!spin_until([&] { w = ld_relaxed_sys_u64(hp); return (uint32_t)(w >> 32) == ep; }, a.remote_wait_ns, nullptr)) {
            if (blockIdx.x == 0) raise_status(f, MXK_DEV_TIMEOUT_BARRIER, 0);
            *sc.flag = 0;
            w = 0;
        }
        sc.tok[r] = min((int)(uint32_t)w, a.cap);
    }
    __syncthreads();
#pragma unroll 1
    for (int r = tid; r <= R; r += nthr) {   // first world pair of source r
        int c = 0;
#pragma unroll 1
        for (int q = 0; q < r; ++q) c += sc.tok[q];
        sc.sb[r] = c * topk;
    }
    __syncthreads();
    const int W = sc.sb[R];   // <= R * cap * topk <= kPushMaxPairs
#pragma unroll 1
    for (int i0 = tid; i0 < W; i0 += nthr * 4) {   // four polls in flight per thread
        const uint64_t* ptr[4];
        uint64_t w[4];
        int src[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = i0 + j * nthr;
            if (i < W) {
                src[j] = push_src_of(sc.sb, R, i);
                const int q = i - sc.sb[src[j]];
                const int qt = a.ftopk.div(q);
                ptr[j] = mine + src[j] * src_words + 16 + (size_t)qt * row_words + (q - qt * topk);
                w[j] = ld_relaxed_sys_u64(ptr[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = i0 + j * nthr;
            if (i >= W) continue;
            uint64_t t = w[j];
            const uint64_t* tp = ptr[j];
            if ((uint32_t)(t >> 32) != ep &&
                !spin_until([&] { t = ld_relaxed_sys_u64(tp); return (uint32_t)(t >> 32) == ep; }, a.remote_wait_ns, nullptr)) {
                if (blockIdx.x == 0) raise_status(f, MXK_DEV_TIMEOUT_BARRIER, 0);
                *sc.flag = 0;
                t = 0xFFFFFFFFull;
            }
            const int e = (int)(uint32_t)t;
            sc.wid[i] = e;
            if (e >= 0) {
                const int owner = a.fEPR.div(e);
                if (owner < R && a.fng.mod(owner) == my_group)
                    atomicAdd(&sc.cnt[(a.fng.div(owner) * EPR + (e - owner * EPR)) * R + src[j]], 1);
            }
        }
    }
    __syncthreads();
    {
        // The dispatch gives one warp to every (pair of this rank's group, row part).  Walking the whole
        // world's pairs for that leaves the warps with an uneven number of real items (on 8 ranks seven
        // pairs in eight belong to other ranks, and a warp that draws two or three of the eighth kind
        // runs them one after the other); a compact list gives every warp at most one more than any
        // other.  Every CTA must build the SAME list: thread t compacts the contiguous slice
        // [t*c, (t+1)*c) and a block-wide exclusive sum places it, so the list is the ascending order.
        auto is_mine = [&](int e) -> bool {
            if (e < 0) return false;
            const int owner = a.fEPR.div(e);
            return owner < R && a.fng.mod(owner) == my_group;
        };
        const int c = (W + nthr - 1) / nthr, lo = min(tid * c, W), hi = min(lo + c, W);
        int n = 0;
#pragma unroll 1
        for (int i = lo; i < hi; ++i) n += is_mine(sc.wid[i]) ? 1 : 0;
        int incl = n;   // inclusive sum inside the warp
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if ((tid & 31) >= d) incl += v;
        }
        if ((tid & 31) == 31) sc.scan[tid >> 5] = incl;
        __syncthreads();
        int base = incl - n;
#pragma unroll 1
        for (int w = 0; w < (tid >> 5); ++w) base += sc.scan[w];
#pragma unroll 1
        for (int i = lo; i < hi; ++i)
            if (is_mine(sc.wid[i])) sc.mine[base++] = (unsigned short)i;
        if (tid == nthr - 1) sc.scan[16] = base;   // the last thread ends at the total
        __syncthreads();
    }
    const bool ts = a.ticks != 0 && tid == 0 && blockIdx.x == 0;
    if (ts) f->dbg_ts[0] = gtimer_ns();
    // pairs beyond the slot capacity of a (source, expert) row are dropped (src/prologue.cuh:171-174)
#pragma unroll 1
    for (int i = tid; i < GE * R; i += nthr) sc.cnt[i] = min(sc.cnt[i], a.slot_cap);
    __syncthreads();
#pragma unroll 1
    for (int ge = tid; ge < GE && G > 1; ge += nthr) {   // prefix rows and totals of the whole group
        int c = 0;
#pragma unroll 1
        for (int r = 0; r < R; ++r) {
            sc.prefix[ge * (R + 1) + r] = c;
            c += sc.cnt[ge * R + r];
        }
        sc.prefix[ge * (R + 1) + R] = c;
        sc.totg[ge] = c;
    }
    build_tables(a, sc.cnt + mm * EPR * R, sc.prefix + mm * EPR * (R + 1), sc.tot, sc.order, sc.first, sc.base);
    if (ts) f->dbg_ts[3] = gtimer_ns();
    const int nt1 = a.I / 128, nt2 = a.H / kBlockN;
    // helpers on? (the same answer on every member of the group: it depends on the group's totals only)
    if (tid == 0) {
        int helper = 0;
        if (G > 1) {
            long long mx = 0, sum = 0, nwin = 0;
#pragma unroll 1
            for (int ge = 0; ge < GE; ++ge) {
                const long long c = sc.totg[ge];
                mx = c > mx ? c : mx;
                sum += c;
                nwin += sched_window_count((int)c, a.win_cap);
            }
            // with hot-only spreading there must be a hot expert, or nothing would move
            helper = mx * GE > (long long)a.skew_num * sum && nwin <= kHelperMaxWin && nwin <= kPushMaxGroupWin &&
                     sched_expert_hot((int)mx, a.win_cap, a.hot_windows);
        }
        T->helper = helper;
    }
    __syncthreads();
    bool overflow;
    if (T->helper) {
        if (tid < 32) helper_member_list(sc.totg, GE, a.fEPR, G, a.win_cap, mm, a.hot_windows, T);
        if (tid == 32) {   // first lookup entry of every group expert
            int c = 0;
#pragma unroll 1
            for (int ge = 0; ge < GE; ++ge) { sc.gws[ge] = c; c += sched_window_count(sc.totg[ge], a.win_cap); }
            sc.gws[GE] = c;
        }
        __syncthreads();
#pragma unroll 1
        for (int i = tid; i < sc.gws[GE]; i += nthr) sc.widx[i] = -1;
        __syncthreads();
#pragma unroll 1
        for (int i = tid; i < T->n_windows; i += nthr) sc.widx[sc.gws[T->gw[i] >> 16] + (T->gw[i] & 0xFFFF)] = i;
        overflow = tables_overflow(a, T->n_windows, T->total_rows);
        if (tid == 0) {
            if (overflow) { T->n_windows = 0; T->total_rows = 0; }
            T->n_l1 = T->n_windows * nt1;
            T->n_tasks = T->n_windows * (nt1 + nt2);
        }
    } else {
#pragma unroll 1
        for (int i = tid; i < EPR; i += nthr) { T->tot[i] = sc.tot[i]; T->order[i] = sc.order[i]; }
#pragma unroll 1
        for (int i = tid; i <= EPR; i += nthr) { T->first[i] = sc.first[i]; T->base[i] = sc.base[i]; }
        const int n_windows = sc.first[EPR], total_rows = sc.base[EPR];
        overflow = tables_overflow(a, n_windows, total_rows);
        if (tid == 0) {
            T->n_windows = overflow ? 0 : n_windows;
            T->n_l1 = overflow ? 0 : n_windows * nt1;
            T->n_tasks = overflow ? 0 : n_windows * (nt1 + nt2);
            T->total_rows = overflow ? 0 : total_rows;
        }
#pragma unroll 1
        for (int p = tid; p < EPR; p += nthr) sc.fw_e[sc.order[p]] = sc.first[p];
    }
    if (tid == 0) {
        // a pool row is copied by `parts` warps when there are warps to spare, so that the copy of a
        // row costs one round trip to the staging area instead of several
        const int nwarps = (int)gridDim.x * (nthr >> 5);
        const int n_items = sc.scan[16];
        T->parts = n_items <= nwarps ? 4 : (n_items <= 2 * nwarps ? 2 : 1);
        // the largest window of the launch: the hottest expert's rows, capped by the window size
        int mx = 0;
        if (T->helper) {
#pragma unroll 1
            for (int ge = 0; ge < GE; ++ge) mx = max(mx, sc.totg[ge]);
        } else {
            mx = sc.tot[sc.order[0]];
        }
        T->slim = min(mx, a.win_cap) <= kSlimRows ? 1 : 0;
    }
    __syncthreads();
    return *sc.flag != 0 && !overflow;
}

// CTA 0, after its share of the dispatch: the tables of this launch in global memory, in the
// pull-mode formats (prefix table, received counts + checksum word, row bases, windows, tasks,
// status header).  Nothing in the kernel waits for them.
__device__ void push_publish(const KArgs& a, DevFlags* f, long long epoch, const PushScratch& sc, const PushTabs* T) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int par = (int)(epoch & 1), R = a.R, EPR = a.EPR;
    const int mm = a.rank / (R / a.group_ranks);
    const int* cnt = sc.cnt + mm * EPR * R;                 // this rank's own experts inside the group tables
    const int* prefix = sc.prefix + mm * EPR * (R + 1);
    int* g_prefix = reinterpret_cast<int*>(a.rwk + a.L.prefix_tbl_off);
#pragma unroll 1
    for (int i = tid; i < EPR * (R + 1); i += nthr) g_prefix[i] = prefix[i];
    uint64_t* recv = reinterpret_cast<uint64_t*>(a.unk + a.L.expert_recv_counts_off) + (size_t)par * R * a.L.recv_stride;
#pragma unroll 1
    for (int i = tid; i < EPR * R; i += nthr) {
        const int le = i / R, r = i % R;
        recv[(size_t)r * a.L.recv_stride + le] = tagged((uint32_t)cnt[i], epoch);
    }
#pragma unroll 1
    for (int r = tid; r < R; r += nthr) {   // the reference's checksum word of a count row (src/prologue.cuh:248-255)
        uint32_t csum = 0;
#pragma unroll 1
        for (int le = 0; le < EPR; ++le) csum += (uint32_t)cnt[le * R + r];
        recv[(size_t)r * a.L.recv_stride + EPR] = tagged(~(csum + 1u), epoch);
    }
    publish_tables(a, f, epoch, sc.tot, sc.order, sc.first, sc.base, T->helper ? T : nullptr);
}

// Owner / helper side: one WARP per (world pair whose row this rank computes, part of its row).
// The pair's slot inside the (expert, source) row is the number of earlier pairs of the same
// source with the same expert — the ascending-pair-index order of the pull-mode route — which
// fixes its place among the expert's rows; the warp then copies its part of the row into the
// pool: from the staging area when the expert is this rank's own (tags stripped), from the
// source rank's input block when it computes the window for another member of its helper group
// (that member received the pushed row, not this one).  Part 0 also stores the scale bytes and
// the staged (source, token, k, weight).  Every part counts itself into the window's pool_ready.
// `do_tables`: also write the pair index into src_index_table (same words a pull-mode source writes).
__device__ void push_dispatch(const KArgs& a, DevFlags* f, long long epoch, const PushScratch& sc, const PushTabs* T,
                              const bool do_tables, const bool do_rows) {
    const int lane = threadIdx.x & 31;
    const int nwarps_cta = blockDim.x >> 5;
    const int nwarps = gridDim.x * nwarps_cta;
    // CTA 0 publishes the tables afterwards: it takes the last items, the last CTA the first ones
    const int gwarp = ((int)gridDim.x - 1 - (int)blockIdx.x) * nwarps_cta + (threadIdx.x >> 5);
    const int par = (int)(epoch & 1), R = a.R, topk = a.topk, EPR = a.EPR, H = a.H;
    const int n_groups = R / a.group_ranks, my_group = a.rank % n_groups;
    const uint32_t ep = (uint32_t)epoch;
    const int P = T->parts;
    const bool helper = T->helper != 0;
    const uint64_t* mine = xin_block(a, a.unk, par, 0);
    const size_t src_words = (size_t)a.L.xin_src_words;
    const int row_words = a.L.xin_row_words, sfw = xin_sf_words(H), kb = H / 128, sfw_real = (kb + 3) / 4;
    uint64_t* tbl = reinterpret_cast<uint64_t*>(a.unk + a.L.src_index_table_off) + (size_t)par * EPR * R * a.slot_cap;
    uint8_t* pool = a.rwk + a.L.pool_off;
    uint8_t* pool_sf = a.rwk + a.L.pool_sf_off;
    int4* meta = reinterpret_cast<int4*>(a.rwk + a.L.row_meta_off);
    uint32_t* pool_ready = reinterpret_cast<uint32_t*>(a.rwk + a.L.pool_ready_off) + (size_t)par * a.L.max_windows;
    const int pshift = P == 4 ? 2 : (P == 2 ? 1 : 0);
    const int n16 = H / 8, per_part = n16 >> pshift;   // 8-byte row units; H % 256 == 0: per_part is a multiple of 8
    const int n_mine = sc.scan[16];
#pragma unroll 1
    for (int it = gwarp; it < n_mine * P; it += nwarps) {
        const int i = sc.mine[it >> pshift], part = it & (P - 1);   // parts are a power of two
        const int e = sc.wid[i];
        if (e < 0) continue;                         // (every `continue` here is uniform over the warp)
        const int owner = a.fEPR.div(e);
        if (owner >= R || a.fng.mod(owner) != my_group) continue;
        const bool own = owner == a.rank;
        if (!own && !helper) continue;
        const int le = e - owner * EPR, ge = a.fng.div(owner) * EPR + le;
        const int src = push_src_of(sc.sb, R, i);
        const int p = i - sc.sb[src];
        const int token = a.ftopk.div(p), k = p - token * topk;
        const uint64_t* row = mine + src * src_words + 16 + (size_t)token * row_words;
        const uint64_t* xs = row + 2 * topk + sfw;
        const uint8_t* peer = a.peer_bases[src];     // the source's input block, for rows of other members' experts
        const uint2* px = reinterpret_cast<const uint2*>(peer + a.x_off + (size_t)token * H);
        const int u_lo = part * per_part, u_hi = u_lo + per_part;
        const bool lead = do_rows && part == 0;
        // this part's row words first (up to eight loads in flight per lane): they do not depend on
        // the slot, which is counted while they travel
        ulonglong2 v[8];
        uint64_t wword = 0, sfword = 0;
        if (own) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (do_rows && u_lo + lane + 32 * j < u_hi) v[j] = ld_relaxed_sys_v2_u64(xs + 2 * (u_lo + lane + 32 * j));
            if (lead && lane == 0) wword = ld_relaxed_sys_u64(row + topk + k);
            if (lead && a.scaled && lane < sfw_real) sfword = ld_relaxed_sys_u64(row + 2 * topk + lane);
        }
        int c = 0;
#pragma unroll 4
        for (int j = lane; j < p; j += 32) c += sc.wid[sc.sb[src] + j] == e ? 1 : 0;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, d);
        const int slot = c;
        if (slot >= a.slot_cap) continue;           // over capacity: dropped
        const int gl = sc.prefix[ge * (R + 1) + src] + slot;
        if (own && do_tables && part == 0 && lane == 0) tbl[((size_t)le * R + src) * a.slot_cap + slot] = tagged((uint32_t)p, epoch);
        int g, ready_idx;
        if (helper) {
            const int gw_ = a.fwin.div(gl);
            const int li = sc.widx[sc.gws[ge] + gw_];
            if (li < 0) continue;                   // another member computes this window
            g = (T->rr[li] >> 10) + (gl - gw_ * a.win_cap);
            ready_idx = li;
        } else {
            g = T->base[le] + gl;
            ready_idx = sc.fw_e[le] + a.fwin.div(gl);
        }
        if (!do_rows) continue;
        bool ok = true;
        uint2* drow = reinterpret_cast<uint2*>(pool + (size_t)g * H);
        if (own) {
            auto settle = [&](const uint64_t* wp, uint64_t w) -> uint32_t {   // the word, polled until it is this launch's
                if ((uint32_t)(w >> 32) != ep &&
                    !spin_until([&] { w = ld_relaxed_sys_u64(wp); return (uint32_t)(w >> 32) == ep; }, a.remote_wait_ns, nullptr))
                    ok = false;
                return (uint32_t)w;
            };
#pragma unroll 1
            for (int u0 = u_lo + lane; u0 < u_hi; u0 += 32 * 8) {
                if (u0 != u_lo + lane) {   // rows wider than 8 x 32 units per part: further batches
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (u0 + 32 * j < u_hi) v[j] = ld_relaxed_sys_v2_u64(xs + 2 * (u0 + 32 * j));
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int u = u0 + 32 * j;
                    if (u >= u_hi) continue;
                    ulonglong2 t = v[j];
                    if (((uint32_t)(t.x >> 32) != ep || (uint32_t)(t.y >> 32) != ep) &&
                        !spin_until([&] { t = ld_relaxed_sys_v2_u64(xs + 2 * u);
                                          return (uint32_t)(t.x >> 32) == ep && (uint32_t)(t.y >> 32) == ep; },
                                    a.remote_wait_ns, nullptr))
                        ok = false;
                    drow[u] = make_uint2((uint32_t)t.x, (uint32_t)t.y);
                }
            }
            if (lead) {
                if (a.scaled) {
                    uint32_t* dsf = reinterpret_cast<uint32_t*>(pool_sf + (size_t)g * a.L.sf_stride_h);
                    if (lane < a.L.sf_stride_h / 4)   // sf_stride_h <= 64 bytes: one word per lane
                        dsf[lane] = lane < sfw_real ? settle(row + 2 * topk + lane, sfword) : 0x7F7F7F7Fu;
                }
                if (lane == 0) meta[g] = make_int4(src, token, k, (int)settle(row + topk + k, wword));
            }
        } else {
            // a window of another member's expert: the row comes from the source rank's input block
            // (the inputs of a launch stay put until the source's own reduce is done, and that waits
            // for this row's result)
#pragma unroll 1
            for (int u0 = u_lo + lane; u0 < u_hi; u0 += 32 * 8) {
                uint2 q[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (u0 + 32 * j < u_hi) q[j] = ld_relaxed_sys_v2_u32(px + u0 + 32 * j);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (u0 + 32 * j < u_hi) drow[u0 + 32 * j] = q[j];
            }
            if (lead) {
                if (a.scaled) {
                    const uint8_t* ssf = peer + a.x_sf_off + (size_t)token * kb;
#pragma unroll 1
                    for (int b = lane; b < a.L.sf_stride_h; b += 32)
                        pool_sf[(size_t)g * a.L.sf_stride_h + b] = b < kb ? ld_relaxed_sys_u8(ssf + b) : (uint8_t)127;
                }
                if (lane == 0)
                    meta[g] = make_int4(src, token, k, (int)ld_relaxed_sys(reinterpret_cast<const uint32_t*>(peer + a.weights_off) +
                                                                           (size_t)token * topk + k));
            }
        }
        if (!__all_sync(0xFFFFFFFFu, ok ? 1 : 0) && lane == 0) raise_status(f, MXK_DEV_TIMEOUT_BARRIER, 2);
        // this part of the row is complete: every lane makes its stores visible at GPU scope and to
        // TMA, then the part is counted
        __threadfence();
        fence_proxy_async_global();
        __syncwarp();
        if (lane == 0) red_release_gpu_add(pool_ready + ready_idx, 1u);
    }
}

// y[t] = sum over k (ascending, FP32, product then sum) of w_k * bf16 row_k
// (reference: src/combine.cuh:601-627, src/bench_check.cuh:484-499).
//
// Every arrival count a token has waited for is zeroed once it is complete (all `need` adds of this
// launch have landed by then, and peers push again only after this rank's next launch has
// published its routing); the last CTA to finish records the launch in cnt_clean_epoch, which lets
// the next launch skip the clear of the table (ensure_counts_clean).
__device__ void reduce_tokens(const KArgs& a, DevFlags* f, int* s_ok /*[64]*/, float* s_w /*[64]*/);
__device__ void reduce_phase(const KArgs& a, DevFlags* f, long long epoch, int* s_ok, float* s_w) {
    // the accepted-pair map is written by the route build of every CTA; the launch counter moves
    // once all of them have arrived (long ago, normally)
    if (threadIdx.x == 0 &&
        !spin_until([&] { return ld_acquire_gpu_s64(&f->current_time) >= epoch; }, a.local_wait_ns, nullptr))
        raise_status(f, MXK_DEV_TIMEOUT_PIPE, 2);
    __syncthreads();
    reduce_tokens(a, f, s_ok, s_w);
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();   // this CTA's zeroed counts before its arrival
        if (atomicAdd(&f->reduce_blocks_done, 1u) == gridDim.x - 1) {
            f->reduce_blocks_done = 0;
            __threadfence();
            if (ld_relaxed_gpu(&f->status) == 0) f->cnt_clean_epoch = (uint32_t)epoch;
        }
    }
}
__device__ void reduce_tokens(const KArgs& a, DevFlags* f, int* s_ok /*[64]*/, float* s_w /*[64]*/) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int H = a.H, topk = a.topk;
    const uint8_t* pair_state = a.rwk + a.L.pair_state_off;
    uint32_t* cnt = reinterpret_cast<uint32_t*>(a.unk + a.L.combine_cnt_off);
    const uint16_t* rows = reinterpret_cast<const uint16_t*>(a.unk + a.L.combine_rows_off);
    const float* tw = reinterpret_cast<const float*>(a.self + a.weights_off);
    const uint32_t need = (uint32_t)(H / kBlockN) * 2u;
    if (a.tokens > 2 * (int)gridDim.x && topk <= 32) {
        // Many tokens per CTA: one WARP per token, so that the wait for a token's rows and the
        // latency of its loads overlap across the warps of the CTA (a CTA-wide token would put
        // a poll, a fence and two barriers between any two tokens).  Same arithmetic order.
        const int lane = tid & 31, warp = tid >> 5, nw = nthr >> 5;
#pragma unroll 1
        for (int t = blockIdx.x * nw + warp; t < a.tokens; t += (int)gridDim.x * nw) {
            int ok = 0;
            float w_mine = 0.0f;
            if (lane < topk) {
                ok = ld_relaxed_gpu_u8(pair_state + t * topk + lane);
                if (ok && !a.skip_combine) {
                    uint32_t* c = cnt + (size_t)lane * a.cap + t;
                    if (!spin_until([&] { return ld_relaxed_sys(c) >= need; }, a.remote_wait_ns, nullptr)) {
                        raise_status(f, MXK_DEV_TIMEOUT_REDUCE, 4);
                        ok = 0;
                    } else {
                        // acquire: the counted row segments are visible (the pushers release their rows
                        // with a fence before the relaxed adds); then the count is consumed
                        (void)(a.R > 1 ? ld_acquire_sys(c) : ld_acquire_gpu(c));
                        *c = 0;
                    }
                }
                w_mine = tw[(size_t)t * topk + lane];
            }
            __syncwarp();  // the other lanes' loads are ordered after the polling lanes' acquires
            const unsigned okmask = __ballot_sync(0xFFFFFFFFu, ok != 0);
            // two column groups per pass: up to 16 row segments of 16 B in flight per lane
            // (H/8 is a multiple of 32, so the second group's validity is uniform over the warp)
#pragma unroll 1
            for (int c0 = lane; c0 < H / 8; c0 += 64) {
                const bool two = c0 + 32 < H / 8;
                float acc[2][8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[0][j] = acc[1][j] = 0.0f;
#pragma unroll 1
                for (int k0 = 0; k0 < topk; k0 += 8) {
                    uint4 v[2][8];
                    float wk[8];
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        wk[kk] = __shfl_sync(0xFFFFFFFFu, w_mine, (k0 + kk) & 31);
                        if (k0 + kk < topk && ((okmask >> (k0 + kk)) & 1u)) {
                            const uint4* row = reinterpret_cast<const uint4*>(rows + ((size_t)(k0 + kk) * a.cap + t) * H);
                            v[0][kk] = ld_relaxed_sys_v4(row + c0);
                            if (two) v[1][kk] = ld_relaxed_sys_v4(row + c0 + 32);
                        }
                    }
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk) {
                        if (k0 + kk >= topk || !((okmask >> (k0 + kk)) & 1u)) continue;
                        const float w = wk[kk];
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            if (g == 1 && !two) break;
                            const uint32_t u[4] = {v[g][kk].x, v[g][kk].y, v[g][kk].z, v[g][kk].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                acc[g][2 * j] = __fadd_rn(acc[g][2 * j], __fmul_rn(__uint_as_float(u[j] << 16), w));
                                acc[g][2 * j + 1] = __fadd_rn(acc[g][2 * j + 1], __fmul_rn(__uint_as_float(u[j] & 0xFFFF0000u), w));
                            }
                        }
                    }
                }
#pragma unroll
                for (int g = 0; g < 2; ++g) {
                    if (g == 1 && !two) break;
                    const int c8 = c0 + 32 * g;
                    if (a.y) {
                        float4* o = reinterpret_cast<float4*>(a.y + (size_t)t * H + c8 * 8);
                        o[0] = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
                        o[1] = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
                    }
                    if (a.y_bf16) {
                        uint4 o;
                        o.x = pack_bf16x2(acc[g][0], acc[g][1]); o.y = pack_bf16x2(acc[g][2], acc[g][3]);
                        o.z = pack_bf16x2(acc[g][4], acc[g][5]); o.w = pack_bf16x2(acc[g][6], acc[g][7]);
                        *reinterpret_cast<uint4*>(a.y_bf16 + (size_t)t * H + c8 * 8) = o;
                    }
                }
            }
        }
        return;
    }
#pragma unroll 1
    for (int t = blockIdx.x; t < a.tokens; t += gridDim.x) {
        if (tid < topk) {
            int ok = ld_relaxed_gpu_u8(pair_state + t * topk + tid);
            if (ok && !a.skip_combine) {
                uint32_t* c = cnt + (size_t)tid * a.cap + t;
                if (!spin_until([&] { return ld_relaxed_sys(c) >= need; }, a.remote_wait_ns, nullptr)) {
                    raise_status(f, MXK_DEV_TIMEOUT_REDUCE, 4);
                    ok = 0;
                } else {
                    (void)(a.R > 1 ? ld_acquire_sys(c) : ld_acquire_gpu(c));   // acquire: the counted row segments are visible
                    *c = 0;
                }
            }
            s_ok[tid] = ok;
            s_w[tid] = tw[(size_t)t * topk + tid];
        }
        __syncthreads();
#pragma unroll 1
        for (int c8 = tid; c8 < H / 8; c8 += nthr) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll 1
            for (int k0 = 0; k0 < topk; k0 += 8) {
                uint4 v[8];  // up to 8 rows in flight, then summed in k order
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)
                    if (k0 + kk < topk && s_ok[k0 + kk])
                        v[kk] = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(rows + ((size_t)(k0 + kk) * a.cap + t) * H) + c8);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    if (k0 + kk >= topk || !s_ok[k0 + kk]) continue;
                    const float w = s_w[k0 + kk];
                    const uint32_t u[4] = {v[kk].x, v[kk].y, v[kk].z, v[kk].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc[2 * j] = __fadd_rn(acc[2 * j], __fmul_rn(__uint_as_float(u[j] << 16), w));
                        acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __fmul_rn(__uint_as_float(u[j] & 0xFFFF0000u), w));
                    }
                }
            }
            if (a.y) {
                float4* o = reinterpret_cast<float4*>(a.y + (size_t)t * H + c8 * 8);
                o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
                o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
            }
            if (a.y_bf16) {
                uint4 o;
                o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
                o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
                *reinterpret_cast<uint4*>(a.y_bf16 + (size_t)t * H + c8 * 8) = o;
            }
        }
        __syncthreads();
    }
}
