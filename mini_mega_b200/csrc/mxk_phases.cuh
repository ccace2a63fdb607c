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
__device__ void route_phase(const KArgs& a, DevFlags* f, long long epoch, int* s_wtot /*[kRoutePer * warps]*/) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nthr = blockDim.x, nwarps = nthr >> 5;
    const int par = (int)(epoch & 1);
    const int np = a.tokens * a.topk;
    const int64_t* ti = a.topk_idx;
    uint8_t* pair_state = a.rwk + a.L.pair_state_off;
    int* rsc = reinterpret_cast<int*>(a.rwk + a.L.route_slot_counts_off);

    // Arrival counters of the rows peers will push to this rank in this launch.  Cleared before
    // any count of this launch leaves the CTA: a peer can push only after it has seen ALL counts
    // of this rank, and the previous launch's reduce has consumed the old values.
    unsigned* cnt = reinterpret_cast<unsigned*>(a.unk + a.L.combine_cnt_off);
    for (int i = blockIdx.x * nthr + tid; i < a.topk * a.cap; i += gridDim.x * nthr) cnt[i] = 0;
    __threadfence();
    __syncthreads();

    for (int e = blockIdx.x; e < a.E; e += gridDim.x) {
        const int dst = e / a.EPR, le = e % a.EPR;
        uint8_t* peer_unk = reinterpret_cast<uint8_t*>(a.unk_peers[dst]);
        uint64_t* tbl = reinterpret_cast<uint64_t*>(peer_unk + a.L.src_index_table_off) +
                        (((size_t)par * a.EPR + le) * a.R + a.rank) * (size_t)a.slot_cap;
        int base = 0;
        // kRoutePer sub-chunks of blockDim pairs per iteration: the index loads of all sub-chunks
        // are in flight together, then slots are handed out sub-chunk by sub-chunk (ascending idx)
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
            __syncthreads();
#pragma unroll
            for (int j = 0; j < kRoutePer; ++j) {
                int wpre = 0, tot = 0;
                for (int w = 0; w < nwarps; ++w) {
                    const int c = s_wtot[j * nwarps + w];
                    wpre += (w < warp) ? c : 0;
                    tot += c;
                }
                if (hit[j]) {
                    const int p = p0 + j * nthr + tid;
                    const int slot = base + wpre + __popc(bal[j] & ((1u << lane) - 1u));
                    const bool ok = slot < a.slot_cap;  // over capacity: dropped (src/prologue.cuh:171-174)
                    if (ok) st_relaxed_sys_u64(tbl + slot, tagged((uint32_t)p, epoch));
                    pair_state[p] = ok ? 1 : 0;
                }
                base += tot;
            }
            __syncthreads();
        }
        if (tid == 0) {
            const int c = base < a.slot_cap ? base : a.slot_cap;
            rsc[e] = c;
            uint64_t* recv = reinterpret_cast<uint64_t*>(peer_unk + a.L.expert_recv_counts_off) +
                             ((size_t)par * a.R + a.rank) * a.L.recv_stride;
            st_relaxed_sys_u64(recv + le, tagged((uint32_t)c, epoch));
        }
    }
    // The launch bookkeeping below belongs to the LAST CTA: CTA 0 goes straight on to poll the
    // counts and build the tables, which is the critical path of the prologue.
    const bool closer = blockIdx.x == gridDim.x - 1;
    if (closer)  // invalid expert ids (negative / >= E) take no slot (src/prologue.cuh:166-167)
        for (int p = tid; p < np; p += nthr)
            if ((uint64_t)ti[p] >= (uint64_t)a.E) pair_state[p] = 0;

    // Everything below is off the critical path (the counts are already on their way): make
    // this CTA's local tables visible, arrive, and let the last CTA close the launch bookkeeping.
    __threadfence();
    __syncthreads();
    if (tid == 0) atomicAdd(&f->route_blocks_done, 1u);
    if (!closer) return;

    if (tid == 0) {
        const unsigned want = gridDim.x;
        if (!spin_until([&] { return ld_acquire_gpu(&f->route_blocks_done) >= want; }, a.local_wait_ns, nullptr))
            raise_status(f, MXK_DEV_TIMEOUT_PIPE, 2);
    }
    __syncthreads();
    // Row checksum word ~(sum + 1) at index EPR of each row sent (src/prologue.cuh:248-255), kept
    // for layout parity with the reference; nothing here waits on it.
    for (int d = tid; d < a.R; d += nthr) {
        uint32_t csum = 0;
        for (int le = 0; le < a.EPR; ++le) csum += (uint32_t)ld_relaxed_gpu(rsc + d * a.EPR + le);
        uint64_t* recv = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(a.unk_peers[d]) +
                                                     a.L.expert_recv_counts_off) +
                         ((size_t)par * a.R + a.rank) * a.L.recv_stride;
        st_relaxed_sys_u64(recv + a.EPR, tagged(~(csum + 1u), epoch));
    }
    if (tid == 0) {
        f->route_blocks_done = 0;
        f->current_time = epoch;  // every CTA has read the old value before arriving above
    }
    __syncthreads();
}

// CTA 0 builds the tables; `s_i` is scratch shared memory of 4*EPR + 2 + EPR*R ints.
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

    int* prefix = reinterpret_cast<int*>(a.rwk + a.L.prefix_tbl_off);
    for (int le = tid; le < EPR; le += nthr) {
        int c = 0;
        for (int r = 0; r < R; ++r) {
            prefix[le * (R + 1) + r] = c;
            c += s_cnt[le * R + r];
        }
        prefix[le * (R + 1) + R] = c;
        s_tot[le] = c;
    }
    __syncthreads();
    if (ts) f->dbg_ts[1] = gtimer_ns();
    // Experts by descending row count, ties by index: the hottest experts' windows
    // are claimed first so the dynamic queue ends on the cheap ones (LPT order).
    for (int le = tid; le < EPR; le += nthr) {
        const int c = s_tot[le];
        int rk = 0;
        for (int j = 0; j < EPR; ++j) {
            const int cj = s_tot[j];
            rk += (cj > c || (cj == c && j < le)) ? 1 : 0;
        }
        s_order[rk] = le;
    }
    __syncthreads();
    if (ts) f->dbg_ts[2] = gtimer_ns();
    if (tid < 32) {
        // exclusive scans by warp 0: pool rows in expert-index order, windows in sorted order
        const int lane = tid;
        int carry_rows = 0, carry_win = 0;
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
    if (ts) f->dbg_ts[3] = gtimer_ns();
    int* row_base = reinterpret_cast<int*>(a.rwk + a.L.expert_row_base_off);
    int* first_win = reinterpret_cast<int*>(a.rwk + a.L.expert_first_win_off);
    for (int le = tid; le <= EPR; le += nthr) row_base[le] = s_base[le];
    for (int p = tid; p < EPR; p += nthr) first_win[s_order[p]] = s_first[p];

    int n_windows = s_first[EPR];
    const int total_rows = s_base[EPR];
    const int nt1 = a.I / 128, nt2 = a.H / kBlockN;
    bool overflow = false;
    if (n_windows > a.L.max_windows || (long long)n_windows * (nt1 + nt2) > a.L.max_tasks ||
        total_rows > a.L.pool_rows) {
        overflow = true;
        n_windows = 0;
    }
    int4* windows = reinterpret_cast<int4*>(a.rwk + a.L.windows_off);
    int4* tasks = reinterpret_cast<int4*>(a.rwk + a.L.tasks_off);
    uint32_t* l1_done = reinterpret_cast<uint32_t*>(a.rwk + a.L.l1_done_off);
    uint32_t* pool_ready = reinterpret_cast<uint32_t*>(a.rwk + a.L.pool_ready_off);
    const int n_l1 = n_windows * nt1;
    if (!overflow) {
        // one warp per expert (sorted position p), lanes over its windows and tasks
        const int lane = tid & 31, wid = tid >> 5, nwarps = nthr >> 5;
        for (int p = wid; p < EPR; p += nwarps) {
            const int e = s_order[p], c = s_tot[e];
            const int fw = s_first[p], nw = s_first[p + 1] - fw;
            if (nw == 0) break;  // sorted: every later expert is empty too
            for (int w = lane; w < nw; w += 32) {
                const int rows = min(a.win_cap, c - w * a.win_cap);
                windows[fw + w] = make_int4(e, s_base[e] + w * a.win_cap, rows, 0);
                l1_done[fw + w] = 0;
                pool_ready[fw + w] = 0;
            }
            for (int i = lane; i < nt1 * nw; i += 32) {
                const int nt = i / nw, w = i % nw;
                tasks[fw * nt1 + i] = make_int4(0, fw + w, nt, min(a.win_cap, c - w * a.win_cap));
            }
            for (int i = lane; i < nt2 * nw; i += 32) {
                const int nt = i / nw, w = i % nw;
                tasks[n_l1 + fw * nt2 + i] = make_int4(1, fw + w, nt, min(a.win_cap, c - w * a.win_cap));
            }
        }
    }
    if (ts) f->dbg_ts[4] = gtimer_ns();
    if (tid == 0) {
        if (overflow) raise_status(f, MXK_DEV_BAD_TABLE, 3);
        f->n_windows = n_windows;
        f->n_l1_tasks = n_l1;
        f->n_tasks = n_windows * (nt1 + nt2);
        f->total_rows = overflow ? 0 : total_rows;
        f->task_counter = a.pair ? gridDim.x >> 1 : gridDim.x;  // first task of a CTA (pair) is its index
    }
    __threadfence();
    __syncthreads();
    if (ts) f->dbg_ts[5] = gtimer_ns();
    if (tid == 0) st_release_gpu(&f->setup_epoch, (uint32_t)epoch);
    if (ts) f->dbg_ts[6] = gtimer_ns();
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
    uint32_t* pool_ready = reinterpret_cast<uint32_t*>(a.rwk + a.L.pool_ready_off);
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
        for (int i = threadIdx.x; i <= EPR; i += blockDim.x) row_base[i] = ld_relaxed_gpu(g_base + i);
        for (int i = threadIdx.x; i < EPR; i += blockDim.x) first_win[i] = ld_relaxed_gpu(g_fw + i);
        for (int i = threadIdx.x; i < EPR * (R + 1); i += blockDim.x) prefix[i] = ld_relaxed_gpu(g_pf + i);
        __syncthreads();
    }

    for (int g = gwarp; g < total; g += nwarps) {
        int lo = 0, hi = EPR;  // largest le with row_base[le] <= g
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (row_base[mid] <= g) lo = mid; else hi = mid;
        }
        const int le = lo;
        const int gl = g - row_base[le];
        const int* pf = prefix + le * (R + 1);
        int slo = 0, shi = R;  // largest src with pf[src] <= gl (src/compute_big.cuh:1760-1769)
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
        const uint32_t idx = (uint32_t)tw;
        const int token = (int)(idx / (uint32_t)a.topk), k = (int)(idx % (uint32_t)a.topk);
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
        if (lane == 0) red_release_gpu_add(pool_ready + first_win[le] + gl / a.win_cap, 1u);
    }
}

// y[t] = sum over k (ascending, FP32, product then sum) of w_k * bf16 row_k
// (reference: src/combine.cuh:601-627, src/bench_check.cuh:484-499).
__device__ void reduce_phase(const KArgs& a, DevFlags* f, int* s_ok /*[64]*/, float* s_w /*[64]*/) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int H = a.H, topk = a.topk;
    const uint8_t* pair_state = a.rwk + a.L.pair_state_off;
    const uint32_t* cnt = reinterpret_cast<const uint32_t*>(a.unk + a.L.combine_cnt_off);
    const uint16_t* rows = reinterpret_cast<const uint16_t*>(a.unk + a.L.combine_rows_off);
    const float* tw = reinterpret_cast<const float*>(a.self + a.weights_off);
    const uint32_t need = (uint32_t)(H / kBlockN) * 2u;
    if (a.tokens > 2 * (int)gridDim.x && topk <= 32) {
        // Many tokens per CTA: one WARP per token, so that the wait for a token's rows and the
        // latency of its loads overlap across the warps of the CTA (a CTA-wide token would put
        // a poll, a fence and two barriers between any two tokens).  Same arithmetic order.
        const int lane = tid & 31, warp = tid >> 5, nw = nthr >> 5;
        for (int t = blockIdx.x * nw + warp; t < a.tokens; t += (int)gridDim.x * nw) {
            int ok = 0;
            float w_mine = 0.0f;
            if (lane < topk) {
                ok = ld_relaxed_gpu_u8(pair_state + t * topk + lane);
                if (ok && !a.skip_combine) {
                    const uint32_t* c = cnt + (size_t)lane * a.cap + t;
                    if (!spin_until([&] { return ld_relaxed_sys(c) >= need; }, a.remote_wait_ns, nullptr)) {
                        raise_status(f, MXK_DEV_TIMEOUT_REDUCE, 4);
                        ok = 0;
                    }
                    fence_world(a.R > 1);  // acquire: the counted row segments are visible
                }
                w_mine = tw[(size_t)t * topk + lane];
            }
            __syncwarp();  // the other lanes' loads are ordered after the polling lanes' acquires
            const unsigned okmask = __ballot_sync(0xFFFFFFFFu, ok != 0);
            // two column groups per pass: up to 16 row segments of 16 B in flight per lane
            // (H/8 is a multiple of 32, so the second group's validity is uniform over the warp)
            for (int c0 = lane; c0 < H / 8; c0 += 64) {
                const bool two = c0 + 32 < H / 8;
                float acc[2][8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[0][j] = acc[1][j] = 0.0f;
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
    for (int t = blockIdx.x; t < a.tokens; t += gridDim.x) {
        if (tid < topk) {
            int ok = ld_relaxed_gpu_u8(pair_state + t * topk + tid);
            if (ok && !a.skip_combine) {
                const uint32_t* c = cnt + (size_t)tid * a.cap + t;
                if (!spin_until([&] { return ld_relaxed_sys(c) >= need; }, a.remote_wait_ns, nullptr)) {
                    raise_status(f, MXK_DEV_TIMEOUT_REDUCE, 4);
                    ok = 0;
                }
                fence_world(a.R > 1);  // acquire: the counted row segments are visible
            }
            s_ok[tid] = ok;
            s_w[tid] = tw[(size_t)t * topk + tid];
        }
        __syncthreads();
        for (int c8 = tid; c8 < H / 8; c8 += nthr) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
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
