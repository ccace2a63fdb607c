// ============================================================================
// mxk_gemm.cuh — persistent grouped GEMM of the MoE layer on tcgen05.
// Included by mxk_kernels.cu after KArgs / DevFlags are defined.
//
// One CTA per SM pulls (window, n-tile) tasks from a global queue:
//   L1 task: D[128 rows, 256] = X_window . [W1 gate rows | W1 up rows]^T over K = H,
//            epilogue SwiGLU -> per-row 1x128 UE8M0 requantisation -> ffn (E4M3)
//   L2 task: D[128 rows, 256] = ffn_window . W2[256 rows]^T over K = I,
//            epilogue bf16 -> rows pushed to the source rank's combine_rows
// (reference: task loop src/compute.cuh:1050-1236, L1 family
//  src/compute_big.cuh:320-515,888-1161, L2 family :1231-1679, fused combine push
//  src/combine.cuh:347-372; there the MMA is a register-fragment warp MMA and the
//  four N/K slices of a window synchronise through flags.)
//
// The whole K extent accumulates in tensor memory with the block-scaled MMA
// (kind::mxf8f6f4): the UE8M0 scale of each 128-wide K block — 1x128 per
// activation row, 128x128 per weight block — is staged as a TMEM scale tile, so
// the epilogue runs once per task.
//
// Warp roles (384 threads):
//   warp 0      task scheduler + TMA producer (operand tiles, 4-stage ring)
//   warp 1      MMA issuer (one lane), owns the TMEM allocation
//   warps 2-3   scale-tile builders (even / odd tasks): global scale planes -> shared
//               tiles -> tensor memory (tcgen05.cp)
//   warps 4-11  epilogue: warp w reads TMEM lanes 32*(w%4).., column half (w-4)/4
// ============================================================================
#pragma once

constexpr int kStages = 4;
constexpr int kABytes = kBlockM * kBlockK;           // 16 KB activation tile
constexpr int kBBytes = kBlockN * kBlockK;           // 32 KB weight tile (two 128-row halves)
constexpr int kStageBytes = kABytes + kBBytes;       // 48 KB
// CTA-pair mode (cta_group::2): each CTA of a cluster of two stages its own 128 activation rows
// and ONE 128-row half of the weight tile; the pair's MMA (M = 256, N = 256) reads both halves.
// Per 128-row block of M each SM then moves 32 KB instead of 48 KB through shared memory.
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = 2 * kABytes;         // 32 KB
constexpr int kSlimStages = 5;                       // single CTAs, windows of at most kSlimRows rows: 5 x (4 KB + 32 KB)
constexpr int kMaxStages = kPairStages;
static_assert(kSlimStages * (kSlimRows * kBlockK + kBBytes) <= kStages * kStageBytes && kSlimStages <= kMaxStages, "slim ring fits the tile region");
static_assert(kPairStages * kPairStageBytes == kStages * kStageBytes, "both modes use the same tile region");
constexpr int kTaskRing = 4;
constexpr int kGemmThreads = 384;
constexpr int kEpiWarps = 8;
constexpr int kFirstEpiWarp = 4;
constexpr int kTmemCols = 512;
constexpr int kTmemSfCol = 256;       // scale tiles live behind the 256 accumulator columns: ring slot s at
                                      // columns 256 + 16*s (12 used: activation rows, weight halves 0 and 1)
constexpr int kSfRing = 8;            // shared-memory scale-tile slots (one per 4 K blocks)
constexpr int kSfSlotBytes = 3 * 512; // A rows, weight half 0, weight half 1
constexpr int kPrefetchBytesPerCta = 704 * 1024;  // L2 prefetch during the prologue: 148 CTAs x 704 KB = 104 MB
constexpr int kPubDepth = 8;          // combine-row arrival counts a thread may hold back before one fence releases them
constexpr int kControlBytes = 20480;  // barriers, task ring, exchange words, count queues, push-mode tables
constexpr int kGemmSmem = kStages * kStageBytes + 1024 /*align*/ + kSfRing * kSfSlotBytes + kControlBytes;

// Wait-time accounting (reference: clock64 phase stamps in local_flags.pre_ticks,
// src/kernel.cuh:52-124): each role sums the cycles it spent blocked and adds them to
// DevFlags::ticks at exit.  Slots: 0 producer/empty stage, 1 producer/L1->L2 gate, 2 MMA/full
// stage, 3 MMA/accumulator drain, 4 MMA/scale tile, 5 epilogue/accumulators ready,
// 6 CTA lifetime, 7 producer/task ring, 8 epilogue busy (drain to stores issued),
// 15 epilogue accumulator drain (part of 8).
#define MXK_TIMED(slot_var, expr) ([&] { if (!timed) return (expr); const long long t0_ = clock64(); const bool r_ = (expr); slot_var += clock64() - t0_; return r_; }())

struct GemmSmem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t sf_full[kSfRing];    // scale tiles of a group copied into tensor memory (commit of the copies)
    uint64_t sf_empty[kSfRing];   // the group's MMAs retired: shared slot and TMEM columns reusable
    uint64_t sf_peer[kSfRing];    // pair mode, leader only: the partner CTA has written its shared tile
    uint64_t tmem_full;
    uint64_t tmem_empty;
    uint64_t task_full[kTaskRing];
    uint64_t task_empty[kTaskRing];
    int4 task[kTaskRing];
    unsigned long long xch[2][2][128];  // amax exchange between the two column halves
    uint32_t pubq[kPubDepth][kEpiWarps * 32];   // per epilogue thread: queued arrival counts, (rank << 24) | (k * cap + token)
    uint32_t tmem_base;
    int abort_flag;
    PushTabs tabs;                // push mode: this launch's tables, built by every CTA for itself
};

static_assert(sizeof(GemmSmem) <= kControlBytes, "control block must fit the space reserved behind the tile rings");
static_assert(kGemmSmem + 2048 <= 227 * 1024, "dynamic + static shared memory of the kernel within the 227 KB of a CTA");

// Push mode: task `t` of the queue and window `w`, computed from the tables in shared memory
// (pull mode reads the same records from the lists CTA 0 wrote to global memory).  Task order:
// L1 tasks then L2 tasks; per sorted expert position p its windows x n-tiles, windows fastest.
__device__ __forceinline__ int tabs_pos_of_window(const PushTabs* T, int EPR, int w) {
    int lo = 0, hi = EPR;   // largest p with first[p] <= w (empty experts sit at the end)
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (T->first[mid] <= w) lo = mid; else hi = mid;
    }
    return lo;
}
// The expert index of a window addresses the weight arrays: with helper groups configured these
// are the group's replicated arrays (ge = member * EPR + local expert), else this rank's own.
__device__ __forceinline__ int4 tabs_window(const PushTabs* T, const KArgs& a, int w) {
    if (T->helper) return make_int4(T->gw[w] >> 16, T->rr[w] >> 10, T->rr[w] & 1023, 0);
    const int p = tabs_pos_of_window(T, a.EPR, w);
    const int e = T->order[p], wl = w - T->first[p];
    return make_int4(a.ge_base + e, T->base[e] + wl * a.win_cap, min(a.win_cap, T->tot[e] - wl * a.win_cap), 0);
}
__device__ __forceinline__ int4 tabs_task(const PushTabs* T, const KArgs& a, int t) {
    const int kind = t >= T->n_l1 ? 1 : 0;
    const int nt = kind ? a.H / kBlockN : a.I / 128;
    const int tt = kind ? t - T->n_l1 : t;
    if (T->helper)   // the member's window list: window-major, n-tile minor
        return make_int4(kind, tt / nt, tt % nt, T->rr[tt / nt] & 1023);
    const int p = tabs_pos_of_window(T, a.EPR, tt / nt);
    const int fw = T->first[p], nw = T->first[p + 1] - fw;
    const int i = tt - fw * nt;
    const int w = i % nw;
    return make_int4(kind, fw + w, i / nw, min(a.win_cap, T->tot[T->order[p]] - w * a.win_cap));
}

// Barrier initialisation (one thread) — part of the kernel prologue.
// In pair mode the barriers the MMA issuer waits on (scale tile ready, accumulators drained) and
// the task-ring release live in the leader CTA and count the arrivals of both CTAs.
__device__ void gemm_init_barriers(GemmSmem* S, const bool pair) {
    const uint32_t ctas = pair ? 2u : 1u;
    for (int s = 0; s < kMaxStages; ++s) { mbar_init(&S->full[s], 1); mbar_init(&S->empty[s], 1); }
    for (int s = 0; s < kSfRing; ++s) { mbar_init(&S->sf_full[s], 1); mbar_init(&S->sf_empty[s], 1); mbar_init(&S->sf_peer[s], 1); }
    mbar_init(&S->tmem_full, 1);
    mbar_init(&S->tmem_empty, kEpiWarps * ctas);
    for (int s = 0; s < kTaskRing; ++s) { mbar_init(&S->task_full[s], 1); mbar_init(&S->task_empty[s], (3 + kEpiWarps) * ctas); }
    S->abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
}

// The GEMM phase of the persistent kernel; called by all threads of the CTA after the
// set-up tables of this launch are visible.  Returns when every role has left its loop.
template <bool kPair>
__device__ void gemm_phase(const KArgs& a, DevFlags* f, const long long epoch, const PushTabs* tabs,
                           unsigned long long* trace, int* deferred_route_smem, uint8_t* tiles, uint8_t* sf_tiles, GemmSmem* S,
                           const uint32_t tmem_base, const CUtensorMap* tm_pool_p, const CUtensorMap* tm_ffn_p,
                           const CUtensorMap* tm_w1_p, const CUtensorMap* tm_w2_p, const CUtensorMap* tm_pool_slim_p,
                           const CUtensorMap* tm_ffn_slim_p) {
    const CUtensorMap& tm_pool = *tm_pool_p;
    const CUtensorMap& tm_ffn = *tm_ffn_p;
    const CUtensorMap& tm_w1 = *tm_w1_p;
    const CUtensorMap& tm_w2 = *tm_w2_p;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &S->abort_flag;
    const uint64_t wait_ns = a.local_wait_ns;
    const bool timed = a.ticks != 0;
    const long long t_start = clock64();

    const int par = (int)(epoch & 1);
    // pull mode: written by the set-up phase of this same kernel (CTA 0); push mode: own tables
    (void)tabs;   // = &S->tabs in push mode; addressed through S below, so that no extra pointer stays live in the hot loops
    const int n_tasks = a.push ? S->tabs.n_tasks : ld_relaxed_gpu(&f->n_tasks);
    const int4* tasks = reinterpret_cast<const int4*>(a.rwk + a.L.tasks_off);
    const int4* windows = reinterpret_cast<const int4*>(a.rwk + a.L.windows_off);
    auto get_task = [&](int t) -> int4 { return a.push ? tabs_task(&S->tabs, a, t) : ld_relaxed_gpu_v4(tasks + t); };
    auto get_window = [&](int w) -> int4 { return a.push ? tabs_window(&S->tabs, a, w) : ld_relaxed_gpu_v4(windows + w); };
    uint32_t* l1_done = reinterpret_cast<uint32_t*>(a.rwk + a.L.l1_done_off) + (size_t)par * a.L.max_windows;
    const uint32_t* pool_ready = reinterpret_cast<const uint32_t*>(a.rwk + a.L.pool_ready_off) + (size_t)par * a.L.max_windows;
    const int kb1 = a.H / kBlockK, kb2 = a.I / kBlockK;
    const int nt1 = a.I / 128;
    const uint32_t l1_need = (uint32_t)nt1 * kEpiWarps * (kPair ? 2u : 1u);   // arrivals that complete a window's ffn rows
    const uint32_t row_parts = a.push ? (uint32_t)S->tabs.parts : 1u;             // pool_ready arrivals per dispatched row
    // Pair mode: CTA `crank` of the cluster owns rows [128*crank, 128*crank+128) of a 256-row
    // window and weight half `crank`; rank 0 (the leader) claims tasks and issues the MMAs.
    const uint32_t crank = kPair ? cluster_ctarank() : 0u;
    const bool leader = crank == 0;
    const int n_units = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;   // CTAs or CTA pairs pulling tasks
    const int unit_id = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    // Ring geometry.  Pairs: 6 stages of 32 KB.  Single CTAs: 4 stages of 48 KB (128 activation rows +
    // 256 weight rows) — or, when no window of the launch has more than kSlimRows rows (decode: a few
    // rows per expert), 5 stages of 36 KB with only kSlimRows activation rows staged per slot.  The MMA
    // still reads 128 rows from the slot's start; rows kSlimRows.. are then the first bytes of the same
    // slot's weight tile, they produce accumulator rows nobody reads.  The gain is the fifth stage: a
    // quarter more weight bytes in flight per CTA, which is what a latency-bound stream (packed 4-bit
    // weights: 16 KB of traffic per 32 KB tile) is short of.
    const bool slim = !kPair && a.push && a.slim_ok && S->tabs.slim != 0;
    const uint32_t a_bytes = kPair ? (uint32_t)kABytes : (slim ? (uint32_t)(kSlimRows * kBlockK) : (uint32_t)kABytes);
    const uint32_t kNStages = kPair ? (uint32_t)kPairStages : (slim ? (uint32_t)kSlimStages : (uint32_t)kStages);
    const uint32_t kStageB = kPair ? (uint32_t)kPairStageBytes : a_bytes + (uint32_t)kBBytes;
    // barrier helpers: in pair mode consumers release ring slots / scale tiles / accumulators on
    // the leader's barriers (cluster address of rank 0; for the leader that is its own barrier)
    auto wait_bar = [&](uint64_t* bar, uint32_t parity) -> bool {
        if constexpr (kPair) return mbar_wait_cluster(bar, parity, wait_ns, abort_flag);
        else return mbar_wait(bar, parity, wait_ns, abort_flag);
    };
    auto arrive_leader = [&](uint64_t* bar) {
        if constexpr (kPair) mbar_arrive_cluster(mapa_u32(smem_u32(bar), 0));
        else mbar_arrive(bar);
    };

    if (warp == 0) {
        // ------------------------------------------------ scheduler + TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tm_pool); tma_prefetch_desc(&tm_ffn);
            tma_prefetch_desc(&tm_w1); tma_prefetch_desc(&tm_w2);
            uint32_t stage = 0, phase = 0;
            long long w_empty = 0, w_gate = 0, w_ring = 0;
            const uint64_t stream_policy = l2_policy_evict_first();
            // Claim the task of iteration `i` and publish it in the ring.  With many tasks per
            // CTA the next task is published one iteration early, so that the scale-tile builder
            // can work ahead across the task boundary; with few tasks per CTA (decode) claiming
            // late keeps the tail of the dynamic queue balanced.
            const bool lookahead = n_tasks > 8 * n_units;
            bool ring_dead = false;
            auto claim_publish = [&](uint32_t i) -> int4 {
                const uint32_t slot = i % kTaskRing;
                if constexpr (kPair) {
                    if (!leader) {
                        // the partner's producer consumes the leader's ring entries like any other role
                        if (!MXK_TIMED(w_ring, wait_bar(&S->task_full[slot], (i / kTaskRing) & 1))) {
                            ring_dead = true;
                            return make_int4(-1, 0, 0, 0);
                        }
                        const int4 tk = S->task[slot];
                        arrive_leader(&S->task_empty[slot]);
                        return tk;
                    }
                }
                if (!MXK_TIMED(w_ring, wait_bar(&S->task_empty[slot], ((i / kTaskRing) & 1) ^ 1))) {
                    ring_dead = true;
                    return make_int4(-1, 0, 0, 0);
                }
                const int t = i == 0 ? unit_id : n_units + (int)atomicAdd(&f->task_ctr[par], 1u);
                const int4 tk = t < n_tasks ? get_task(t) : make_int4(-1, 0, 0, 0);
                S->task[slot] = tk;
                mbar_arrive(&S->task_full[slot]);
                if constexpr (kPair) {
                    st_cluster_v4(mapa_u32(smem_u32(&S->task[slot]), 1), tk);
                    mbar_arrive_cluster(mapa_u32(smem_u32(&S->task_full[slot]), 1));  // release: after the store
                }
                return tk;
            };
            // The window record and the gate counter of a task are two dependent global round
            // trips; with the look-ahead they are requested for the NEXT task while this task's
            // loads are being issued, so that a task starts without them on its critical path.
            auto gate_passed = [&](const int4& tk, const int4& wn) -> bool {   // one acquire load
                return tk.x == 1 ? ld_acquire_gpu(l1_done + tk.y) >= l1_need
                                 : ld_acquire_gpu(pool_ready + tk.y) >= (uint32_t)wn.z * row_parts;
            };
            int4 pending = claim_publish(0);
            int4 pending_win = make_int4(0, 0, 0, 0);
            bool pending_win_valid = false, pending_gate = false;
            for (uint32_t it = 0;; ++it) {
                if (ring_dead) { raise_status(f, MXK_DEV_TIMEOUT_PIPE, 3); *abort_flag = 1; break; }
                const int4 task = pending;
                if (task.x < 0) break;
                const int4 win = pending_win_valid ? pending_win : get_window(task.y);
                const bool gate_ok = pending_win_valid && pending_gate;
                pending_win_valid = false;
                if (lookahead) pending = claim_publish(it + 1);
                const int e = win.x, row0 = win.y + 128 * (int)crank;
                const bool is_l2 = task.x == 1;
                const CUtensorMap* ma = slim ? (is_l2 ? tm_ffn_slim_p : tm_pool_slim_p) : (is_l2 ? &tm_ffn : &tm_pool);
                const CUtensorMap* mb = is_l2 ? &tm_w2 : &tm_w1;
                const int nkb = is_l2 ? kb2 : kb1;
                const int brow0 = is_l2 ? e * a.H + task.z * kBlockN : e * 2 * a.I + task.z * 128;
                const int brow1 = is_l2 ? brow0 + 128 : brow0 + a.I;
                // weight tiles of K block kb into ring stage st (the stage's byte count is announced with them)
                // a 128-row weight tile counts on the barrier with the bytes read from memory: half of its
                // 16 KB in shared memory when the weights are packed 4-bit codes
                const uint32_t b_half_tx = a.w_fp4 ? kABytes / 2 : kABytes;
                auto load_b = [&](int kb, uint32_t st) {
                    uint8_t* sa = tiles + st * kStageB;
                    if constexpr (kPair) {
                        // both CTAs' bytes complete on the leader's barrier: 2 x (A 16 KB + weight half 16 KB)
                        if (leader) mbar_expect_tx(&S->full[st], 2 * (kABytes + b_half_tx));
                        tma_load_2d_pair_hint(sa + kABytes, mb, kb * kBlockK, leader ? brow0 : brow1, mapa_u32(smem_u32(&S->full[st]), 0), stream_policy);
                    } else {
                        mbar_expect_tx(&S->full[st], a_bytes + 2 * b_half_tx);
                        tma_load_2d_hint(sa + a_bytes, mb, kb * kBlockK, brow0, &S->full[st], stream_policy);
                        tma_load_2d_hint(sa + a_bytes + kABytes, mb, kb * kBlockK, brow1, &S->full[st], stream_policy);
                    }
                };
                // L2: every L1 tile of this window must have landed in ffn; L1: every row of this
                // window must have been pulled into the pool.  The weight tiles do not depend on that:
                // while the gate is still closed they are requested into whatever stages are free, so
                // that HBM streams during the wait (the first task of a layer waits for the dispatch).
                int pre = 0;
                if (!gate_ok) {
                    uint32_t st2 = stage, ph2 = phase;
                    while (pre < nkb && pre < (int)kNStages && mbar_try_wait(&S->empty[st2], ph2 ^ 1)) {
                        load_b(pre, st2);
                        ++pre;
                        if (++st2 == kNStages) { st2 = 0; ph2 ^= 1; }
                    }
                    if (!MXK_TIMED(w_gate, spin_until([&] { return gate_passed(task, win); }, wait_ns, abort_flag))) {
                        raise_status(f, MXK_DEV_TIMEOUT_GATE, 4); *abort_flag = 1; break;
                    }
                }
                if (trace && it == 0) trace[8] = gtimer_ns();
                fence_proxy_async_global();  // pool / ffn rows were written with ordinary stores
                if (trace && it == 0) trace[9] = gtimer_ns();   // first activation tile requested next
                bool dead = false;
                for (int kb = 0; kb < nkb; ++kb) {
                    if (lookahead && pending.x >= 0) {
                        // request the next task's window record with the first stage, read its gate
                        // two stages later (the record has arrived by then): each is one round trip
                        // taken out of the slack of the stage ring instead of the next task's start
                        if (kb == 0) { pending_win = get_window(pending.y); pending_win_valid = true; pending_gate = false; }
                        else if (kb == 2) pending_gate = gate_passed(pending, pending_win);
                    }
                    if (kb >= pre) {
                        if (!MXK_TIMED(w_empty, mbar_wait(&S->empty[stage], phase ^ 1, wait_ns, abort_flag))) { dead = true; break; }
                        load_b(kb, stage);
                    }
                    uint8_t* sa = tiles + stage * kStageB;
                    if constexpr (kPair) tma_load_2d_pair(sa, ma, kb * kBlockK, row0, mapa_u32(smem_u32(&S->full[stage]), 0));
                    else tma_load_2d(sa, ma, kb * kBlockK, row0, &S->full[stage]);
                    if (++stage == kNStages) { stage = 0; phase ^= 1; }
                }
                if (dead) { raise_status(f, MXK_DEV_TIMEOUT_PIPE, 5); *abort_flag = 1; break; }
                if (!lookahead) pending = claim_publish(it + 1);
            }
            atomicAdd(&f->ticks[0], (unsigned long long)w_empty);
            atomicAdd(&f->ticks[1], (unsigned long long)w_gate);
            atomicAdd(&f->ticks[7], (unsigned long long)w_ring);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0 && leader) {
            uint32_t stage = 0, phase = 0, sfg = 0;
            long long w_full = 0, w_drain = 0, w_sf = 0;
            bool stage_ready = false;   // full[stage] already seen complete by the early poll
            bool sf_ready = false;      // likewise sf_full of the next group
            const uint64_t tile_desc0 = umma_smem_desc_sw128(smem_u32(tiles));
            const uint32_t idesc0 = umma_idesc_mx_e4m3(kPair ? 2 * kBlockM : kBlockM, kBlockN, 0, 0) |
                                    (a.w_fp4 ? kUmmaBFormatE2M1 : 0u);
            for (uint32_t it = 0;; ++it) {
                const uint32_t slot = it % kTaskRing;
                if (!mbar_wait(&S->task_full[slot], (it / kTaskRing) & 1, wait_ns, abort_flag)) {
                    raise_status(f, MXK_DEV_TIMEOUT_PIPE, 3); *abort_flag = 1; break;
                }
                const int4 task = S->task[slot];
                mbar_arrive(&S->task_empty[slot]);
                if (task.x < 0) break;
                const int nkb = task.x == 1 ? kb2 : kb1;
                // the epilogue must have drained the previous task's accumulators
                bool dead = !MXK_TIMED(w_drain, wait_bar(&S->tmem_empty, (it & 1) ^ 1));
                // One K block is 512 tensor-pipe cycles; a barrier poll, a commit or a tensor-memory
                // copy each cost this thread on the order of 100 cycles, so the issue path must stay
                // short or the pipe runs dry: descriptors by addition, scale ids as constants, the
                // next stage and the next scale group polled under the MMAs already queued, and the
                // scale-tile copies issued by the builder warps instead of here.
                uint32_t acc = 0;
                if (trace && it == 0 && !dead) {
                    // time line: when the first operand tile of the layer has landed (kept out of the issue
                    // loop below, where even a never-taken test per K block cost 3 % of a prefill-sized layer)
                    if (MXK_TIMED(w_full, mbar_wait(&S->full[stage], phase, wait_ns, abort_flag))) { stage_ready = true; trace[10] = gtimer_ns(); }
                    else dead = true;
                }
                for (int kb0 = 0; kb0 < nkb && !dead; kb0 += 4) {
                    // a new group of four K blocks: its scale tiles were copied into TMEM slot
                    // sf_slot by a builder warp
                    const uint32_t sf_slot = sfg % kSfRing;
                    if (!sf_ready && !MXK_TIMED(w_sf, wait_bar(&S->sf_full[sf_slot], (sfg / kSfRing) & 1))) { dead = true; break; }
                    sf_ready = false;
                    const uint32_t tsf = tmem_base + kTmemSfCol + sf_slot * 16;
                    const uint32_t nsf_slot = (sfg + 1) % kSfRing, nsf_parity = ((sfg + 1) / kSfRing) & 1;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (kb0 + i >= nkb) break;
                        if (!stage_ready && !MXK_TIMED(w_full, mbar_wait(&S->full[stage], phase, wait_ns, abort_flag))) { dead = true; break; }
                        tc_fence_after();
                        const uint64_t adesc = tile_desc0 + (uint64_t)(stage * (kStageB >> 4));
                        const uint64_t bdesc = adesc + (uint64_t)(a_bytes >> 4);
                        const uint32_t idesc = idesc0 | ((uint32_t)i << 4) | ((uint32_t)i << 29);   // scale byte i of the group
                        uint32_t nstage = stage + 1, nphase = phase;
                        if (nstage == kNStages) { nstage = 0; nphase ^= 1; }
                        if constexpr (kPair) {
                            umma_mxf8_pair(tmem_base, adesc, bdesc, idesc, tsf, tsf + 4, acc);
                            umma_mxf8_pair(tmem_base, adesc + 2, bdesc + 2, idesc, tsf, tsf + 4, 1u);
                            stage_ready = mbar_try_wait(&S->full[nstage], nphase);   // poll the next stage under the MMAs
                            if (i == 2) sf_ready = mbar_try_wait_cluster(&S->sf_full[nsf_slot], nsf_parity);
                            umma_mxf8_pair(tmem_base, adesc + 4, bdesc + 4, idesc, tsf, tsf + 4, 1u);
                            umma_mxf8_pair(tmem_base, adesc + 6, bdesc + 6, idesc, tsf, tsf + 4, 1u);
                            // one commit releases the stage in both CTAs: both producers move on
                            umma_commit_pair_both(smem_u32(&S->empty[stage]));
                        } else {
                            umma_mxf8(tmem_base, adesc, bdesc, idesc, tsf, tsf + 4, acc);
                            umma_mxf8(tmem_base, adesc + 2, bdesc + 2, idesc, tsf, tsf + 4, 1u);
                            stage_ready = mbar_try_wait(&S->full[nstage], nphase);   // poll the next stage under the MMAs
                            if (i == 2) sf_ready = mbar_try_wait(&S->sf_full[nsf_slot], nsf_parity);  // and the next group's scales
                            umma_mxf8(tmem_base, adesc + 4, bdesc + 4, idesc, tsf, tsf + 4, 1u);
                            umma_mxf8(tmem_base, adesc + 6, bdesc + 6, idesc, tsf, tsf + 4, 1u);
                            umma_commit(&S->empty[stage]);  // stage reusable once these MMAs retire
                        }
                        acc = 1u;
                        stage = nstage; phase = nphase;
                    }
                    if (dead) break;
                    if constexpr (kPair) {
                        umma_commit_pair_both(smem_u32(&S->sf_empty[sf_slot]));
                    } else {
                        umma_commit(&S->sf_empty[sf_slot]);
                    }
                    ++sfg;
                }
                if (dead) { raise_status(f, MXK_DEV_TIMEOUT_PIPE, 6); *abort_flag = 1; break; }
                if constexpr (kPair) {
                    umma_commit_pair_both(smem_u32(&S->tmem_full));
                } else {
                    umma_commit(&S->tmem_full);  // accumulators complete
                }
            }
            atomicAdd(&f->ticks[2], (unsigned long long)w_full);
            atomicAdd(&f->ticks[3], (unsigned long long)w_drain);
            atomicAdd(&f->ticks[4], (unsigned long long)w_sf);
        }
    } else if (warp == 2 || warp == 3) {
        // ------------------------------------------------------ scale-tile builders
        // Two warps share the work by TASK: warp 2 builds the scale tiles of the even-numbered ring
        // entries, warp 3 those of the odd ones.  Preparing a task is a chain of dependent global
        // round trips (window record, gate counter, scale rows) that takes about as long as the MMAs
        // of a short task; with alternating tasks each warp works one task ahead of the MMA issuer
        // instead of in lock-step with it.  Both warps read every ring entry to keep the group count.
        const uint32_t my_parity = (uint32_t)(warp - 2);
        // Slot layout (what UTCCP 32x128b.warpx4 expects): tile byte 16*l + 4*j + i is the
        // scale of row l + 32*j for K block i of the group.  The two weight tiles repeat one
        // 4-byte word (a 128x128 block has one scale per K block).
        const uint8_t* pool_sf = a.rwk + a.L.pool_sf_off;
        const uint8_t* ffn_sf = a.rwk + a.L.ffn_sf_off;
        uint32_t sfg = 0;
        for (uint32_t it = 0;; ++it) {
            const uint32_t slot = it % kTaskRing;
            bool ok = true;
            if (lane == 0) ok = wait_bar(&S->task_full[slot], (it / kTaskRing) & 1);
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            if (!ok) { if (lane == 0) { raise_status(f, MXK_DEV_TIMEOUT_PIPE, 3); *abort_flag = 1; } break; }
            const int4 task = S->task[slot];
            __syncwarp();
            if (lane == 0) arrive_leader(&S->task_empty[slot]);
            if (task.x < 0) break;
            const bool is_l2 = task.x == 1;
            const int nkb = is_l2 ? kb2 : kb1;
            const int ngroups = (nkb + 3) >> 2;
            if ((it & 1u) != my_parity) { sfg += (uint32_t)ngroups; continue; }   // the other warp's task
            const int4 win = get_window(task.y);
            const int e = win.x, row0 = win.y + 128 * (int)crank, rows = task.w - 128 * (int)crank;
            const uint8_t* asf = nullptr;   // activation scale rows of this window
            int asf_stride = 0;
            const uint8_t* wsf0 = nullptr;
            const uint8_t* wsf1 = nullptr;
            if (a.scaled) {
                if (is_l2) {
                    // ffn scales are written by L1 epilogues of this same kernel
                    // every lane acquires for itself: its own scale loads below must be ordered
                    // after the counter, and a warp shuffle gives no memory ordering
                    bool ready = spin_until([&] { return ld_acquire_gpu(l1_done + task.y) >= l1_need; }, wait_ns, abort_flag);
                    ready = __all_sync(0xFFFFFFFFu, ready ? 1 : 0) != 0;
                    if (!ready) { if (lane == 0) { raise_status(f, MXK_DEV_TIMEOUT_GATE, 4); *abort_flag = 1; } break; }
                    asf = ffn_sf + (size_t)row0 * a.L.sf_stride_i;
                    asf_stride = a.L.sf_stride_i;
                    wsf0 = a.w2_sf + ((size_t)e * (a.H / 128) + task.z * 2) * nkb;
                    wsf1 = wsf0 + nkb;
                } else {
                    // pool scales are written by the dispatch phase of this same kernel
                    bool ready = true;
                    const uint32_t need_rows = (uint32_t)win.z * row_parts;
                    ready = spin_until([&] { return ld_acquire_gpu(pool_ready + task.y) >= need_rows; }, wait_ns, abort_flag);
                    ready = __all_sync(0xFFFFFFFFu, ready ? 1 : 0) != 0;
                    if (!ready) { if (lane == 0) { raise_status(f, MXK_DEV_TIMEOUT_GATE, 4); *abort_flag = 1; } break; }
                    asf = pool_sf + (size_t)row0 * a.L.sf_stride_h;
                    asf_stride = a.L.sf_stride_h;
                    wsf0 = a.w1_sf + ((size_t)e * (2 * a.I / 128) + task.z) * nkb;
                    wsf1 = wsf0 + (size_t)nt1 * nkb;
                }
            }
            // Per group of four K blocks: 4 activation words per lane (rows l, l+32, l+64, l+96)
            // and one word per weight half.  The loads of group g+1 are issued before the wait
            // for group g's slot, so their latency hides behind the ring.
            const bool wsf_words = a.scaled && (nkb & 3) == 0 &&
                                   ((reinterpret_cast<uintptr_t>(wsf0) | reinterpret_cast<uintptr_t>(wsf1)) & 3) == 0;
            auto load_group = [&](int g, uint32_t (&wa)[4], uint32_t& w0, uint32_t& w1) {
                wa[0] = wa[1] = wa[2] = wa[3] = 0x7F7F7F7Fu;
                w0 = w1 = 0x7F7F7F7Fu;
                if (!a.scaled || g >= ngroups) return;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int r = lane + 32 * j;
                    if (r < rows) wa[j] = ld_relaxed_gpu(reinterpret_cast<const uint32_t*>(asf + (size_t)r * asf_stride) + g);
                }
                if (wsf_words) {   // the four K blocks' weight scales are one aligned word per half
                    w0 = __ldg(reinterpret_cast<const uint32_t*>(wsf0) + g);
                    w1 = __ldg(reinterpret_cast<const uint32_t*>(wsf1) + g);
                    return;
                }
                w0 = 0; w1 = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int kb = g * 4 + i;
                    const uint32_t b0 = kb < nkb ? __ldg(wsf0 + kb) : 127u;
                    const uint32_t b1 = kb < nkb ? __ldg(wsf1 + kb) : 127u;
                    w0 |= b0 << (8 * i);
                    w1 |= b1 << (8 * i);
                }
            };
            uint32_t wa[4], w0, w1;
            load_group(0, wa, w0, w1);
            bool dead = false;
            for (int g = 0; g < ngroups; ++g, ++sfg) {
                uint32_t na[4], n0, n1;
                load_group(g + 1, na, n0, n1);
                const uint32_t sslot = sfg % kSfRing;
                bool free_ = true;
                if (lane == 0) free_ = mbar_wait(&S->sf_empty[sslot], ((sfg / kSfRing) & 1) ^ 1, wait_ns, abort_flag);
                free_ = __shfl_sync(0xFFFFFFFFu, free_ ? 1 : 0, 0) != 0;
                if (!free_) { dead = true; break; }
                uint4* dst = reinterpret_cast<uint4*>(sf_tiles + sslot * kSfSlotBytes);
                dst[lane] = make_uint4(wa[0], wa[1], wa[2], wa[3]);
                dst[32 + lane] = make_uint4(w0, w0, w0, w0);
                dst[64 + lane] = make_uint4(w1, w1, w1, w1);
                fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor-core copy
                __syncwarp();
                if (lane == 0) {
                    // copy the three tiles into the slot's TMEM columns; the commit reports them done
                    const uint32_t tsf = tmem_base + kTmemSfCol + sslot * 16;
                    const uint64_t sfdesc = umma_smem_desc_sf(smem_u32(dst));
                    if constexpr (kPair) {
                        if (leader) {  // one copy serves both CTAs: the partner's tile must be in place
                            if (wait_bar(&S->sf_peer[sslot], (sfg / kSfRing) & 1)) {
                                tc_fence_after();
                                utccp_32x128b_warpx4_pair(tsf, sfdesc);
                                utccp_32x128b_warpx4_pair(tsf + 4, sfdesc + (512 >> 4));
                                utccp_32x128b_warpx4_pair(tsf + 8, sfdesc + (1024 >> 4));
                                umma_commit_pair(smem_u32(&S->sf_full[sslot]));
                            } else {
                                free_ = false;
                            }
                        } else {
                            arrive_leader(&S->sf_peer[sslot]);
                        }
                    } else {
                        tc_fence_after();          // after the wait on sf_empty: the slot's last readers retired
                        utccp_32x128b_warpx4(tsf, sfdesc);                    // activation rows
                        utccp_32x128b_warpx4(tsf + 4, sfdesc + (512 >> 4));   // weight rows 0..127
                        utccp_32x128b_warpx4(tsf + 8, sfdesc + (1024 >> 4));  // weight rows 128..255
                        umma_commit(&S->sf_full[sslot]);
                    }
                }
                if constexpr (kPair) {
                    free_ = __shfl_sync(0xFFFFFFFFu, free_ ? 1 : 0, 0) != 0;
                    if (!free_) { dead = true; break; }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) wa[j] = na[j];
                w0 = n0; w1 = n1;
            }
            if (dead) { if (lane == 0) { raise_status(f, MXK_DEV_TIMEOUT_PIPE, 5); *abort_flag = 1; } break; }
        }
    } else if (warp >= kFirstEpiWarp) {
        // ------------------------------------------------------------- epilogue
        const int q = warp & 3, half = (warp - kFirstEpiWarp) >> 2;
        const int r = q * 32 + lane;  // row inside the window
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        uint8_t* ffn = a.rwk + a.L.ffn_off;
        uint8_t* ffn_sf = a.rwk + a.L.ffn_sf_off;
        const int4* meta = reinterpret_cast<const int4*>(a.rwk + a.L.row_meta_off);
        long long w_acc = 0, t_busy = 0, t_drain = 0, t_pub = 0;
        // Push mode, fused launch: this rank's own route bookkeeping (slot counts, accepted-pair map,
        // launch counter), done here by the eight epilogue warps while the first accumulators fill.
        if (deferred_route_smem)
            route_phase(a, f, epoch, deferred_route_smem, nullptr, 0, true,
                        Team{(int)threadIdx.x - kFirstEpiWarp * 32, kEpiWarps * 32, 1});
        // Publishing a task's output (release of l1_done / combine_cnt) has to wait until the
        // task's stores are performed.  It is deferred past the drain of the NEXT task's
        // accumulators when those are already complete, so that the store latency hides
        // behind work instead of holding the tensor memory; it is never held across a wait
        // (an L2 task of this very CTA may be gated on it).
        //
        // The arrival counts of pushed combine rows (L2 tasks) are batched on top of that: a fence
        // that makes a thread's row segments visible to another GPU costs several microseconds
        // whatever it has to wait for, more than the MMAs of an L2 task, so a thread queues up to
        // kPubDepth counts and releases them with ONE fence followed by relaxed adds — when the
        // queue is full (after a drain, before the next stores are issued) or the task queue ends.
        // Holding them back cannot stall this kernel: only the reduce phase waits for them.
        int pend_l1 = 0;             // an L1 window share (l1_done) awaits its publish
        uint32_t* pend_ptr = nullptr;
        int pub_n = 0;               // queued row counts of this thread
        const int tq = (int)threadIdx.x - kFirstEpiWarp * 32;
        auto flush_l1 = [&] {
            if (!pend_l1) return;
            const long long t_p0 = timed ? clock64() : 0;
            // every lane makes its own stores visible at GPU scope (and to the TMA reads of
            // the L2 tasks) before lane 0 counts the warp's share as done
            __threadfence();
            fence_proxy_async_global();
            __syncwarp();
            if (lane == 0) red_release_gpu_add(pend_ptr, 1u);
            pend_l1 = 0;
            if (timed) t_pub += clock64() - t_p0;
        };
        auto flush_rows = [&] {
            if (pub_n == 0) return;
            const long long t_p0 = timed ? clock64() : 0;
            fence_world(a.R > 1);   // every row segment this thread has stored is visible before the counts
            for (int i = 0; i < pub_n; ++i) {
                const uint32_t en = S->pubq[i][tq];
                uint32_t* cnt = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(a.unk_peers[en >> 24]) + a.L.combine_cnt_off) +
                                (en & 0xFFFFFFu);
                if (a.R > 1) red_relaxed_sys_add(cnt, 1u); else red_relaxed_gpu_add(cnt, 1u);
            }
            pub_n = 0;
            if (timed) t_pub += clock64() - t_p0;
        };
        auto flush_publish = [&] { flush_l1(); flush_rows(); };
        for (uint32_t it = 0;; ++it) {
            const uint32_t slot = it % kTaskRing;
            bool ok = true;
            if (lane == 0) ok = wait_bar(&S->task_full[slot], (it / kTaskRing) & 1);
            ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
            if (!ok) { if (lane == 0) { raise_status(f, MXK_DEV_TIMEOUT_PIPE, 3); *abort_flag = 1; } break; }
            const int4 task = S->task[slot];
            __syncwarp();
            if (lane == 0) arrive_leader(&S->task_empty[slot]);
            if (task.x < 0) { flush_publish(); break; }
            const int4 win = get_window(task.y);
            const int row0 = win.y + 128 * (int)crank, rows = task.w - 128 * (int)crank;
            const bool is_l2 = task.x == 1;
            const bool warp_active = q * 32 < rows;
            const bool row_valid = r < rows;

            bool got = false;
            if (lane == 0) got = mbar_try_wait(&S->tmem_full, it & 1);
            got = __shfl_sync(0xFFFFFFFFu, got ? 1 : 0, 0) != 0;
            if (!got) {   // about to block: publish the L1 share first (an L2 task may be gated on it);
                          // queued row counts stay queued until eight are together or the queue ends
                flush_l1();
                if (lane == 0) got = MXK_TIMED(w_acc, mbar_wait(&S->tmem_full, it & 1, wait_ns, abort_flag));
                got = __shfl_sync(0xFFFFFFFFu, got ? 1 : 0, 0) != 0;
            }
            const long long t_busy0 = clock64();
            if (!got) { if (lane == 0) { raise_status(f, MXK_DEV_TIMEOUT_PIPE, 6); *abort_flag = 1; } break; }
            tc_fence_after();
            // drain this warp's share of the accumulators into registers, then release TMEM
            uint32_t vg[64], vu[64];
            if (warp_active) {
                const uint32_t t0 = lane_addr + half * 64;
                tmem_ld64(t0, vg);
                tmem_ld64(t0 + 128, vu);
                tmem_wait_ld();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_leader(&S->tmem_empty);
            if (timed) t_drain += clock64() - t_busy0;
            flush_l1();        // the previous task's stores have had the drain to complete
            if (pub_n == kPubDepth) flush_rows();

            if (!is_l2) {
                // ---- SwiGLU + per-row 1x128 requantisation to E4M3 -> ffn
                if (warp_active) {
                    float amax = 0.0f;
#pragma unroll
                    for (int j = 0; j < 64; ++j) {
                        const float g = __uint_as_float(vg[j]);
                        const float hv = (g / (1.0f + expf(-g))) * __uint_as_float(vu[j]);  // silu(g)*u (src/compute.cuh:242-244)
                        vg[j] = __float_as_uint(hv);
                        amax = fmaxf(amax, fabsf(hv));
                    }
                    float inv = 1.0f;
                    uint32_t ex = 127;
                    if (a.scaled) {
                        // the other column half of this row lives in warp +-4: swap partial maxima
                        const uint32_t tag = it + 1;
                        volatile unsigned long long* mine = &S->xch[it & 1][half][r];
                        volatile unsigned long long* theirs = &S->xch[it & 1][half ^ 1][r];
                        *mine = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(amax);
                        unsigned long long o = 0;
                        const bool gotx = spin_until([&] { o = *theirs; return (uint32_t)(o >> 32) == tag; }, wait_ns, abort_flag);
                        if (!gotx) { raise_status(f, MXK_DEV_TIMEOUT_PIPE, 5); *abort_flag = 1; }
                        amax = fmaxf(amax, __uint_as_float((uint32_t)o));
                        const float s = fmaxf(amax, 1e-4f) / 448.0f;  // per_token_cast_to_fp8, utils/math.py:33-35
                        const uint32_t bits = __float_as_uint(s);
                        ex = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) ? 1u : 0u);
                        ex = min(254u, max(1u, ex));
                        inv = __uint_as_float((254u - ex) << 23);
                    }
                    if (row_valid) {
                        uint4* dst = reinterpret_cast<uint4*>(ffn + (size_t)(row0 + r) * a.I + task.z * 128 + half * 64);
                        uint4 prev = make_uint4(0, 0, 0, 0);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint4 o;
                            o.x = pack_e4m3x4(__uint_as_float(vg[c * 16 + 0]) * inv, __uint_as_float(vg[c * 16 + 1]) * inv,
                                              __uint_as_float(vg[c * 16 + 2]) * inv, __uint_as_float(vg[c * 16 + 3]) * inv);
                            o.y = pack_e4m3x4(__uint_as_float(vg[c * 16 + 4]) * inv, __uint_as_float(vg[c * 16 + 5]) * inv,
                                              __uint_as_float(vg[c * 16 + 6]) * inv, __uint_as_float(vg[c * 16 + 7]) * inv);
                            o.z = pack_e4m3x4(__uint_as_float(vg[c * 16 + 8]) * inv, __uint_as_float(vg[c * 16 + 9]) * inv,
                                              __uint_as_float(vg[c * 16 + 10]) * inv, __uint_as_float(vg[c * 16 + 11]) * inv);
                            o.w = pack_e4m3x4(__uint_as_float(vg[c * 16 + 12]) * inv, __uint_as_float(vg[c * 16 + 13]) * inv,
                                              __uint_as_float(vg[c * 16 + 14]) * inv, __uint_as_float(vg[c * 16 + 15]) * inv);
                            if (c & 1) st_global_v8(dst + c - 1, prev, o); else prev = o;   // 32-byte stores
                        }
                        if (a.scaled && half == 0) ffn_sf[(size_t)(row0 + r) * a.L.sf_stride_i + task.z] = (uint8_t)ex;
                    }
                }
                pend_l1 = 1;
                pend_ptr = l1_done + task.y;
            } else {
                // ---- bf16 rows pushed to the source rank + per-pair arrival count
                if (row_valid && !a.skip_combine) {
                    const int4 m = ld_relaxed_gpu_v4(meta + row0 + r);  // src, token, k, weight
                    uint8_t* peer_unk = reinterpret_cast<uint8_t*>(a.unk_peers[m.x]);
                    uint16_t* crow = reinterpret_cast<uint16_t*>(peer_unk + a.L.combine_rows_off) +
                                     ((size_t)m.z * a.cap + m.y) * a.H + task.z * kBlockN + half * 64;
                    uint4* d0 = reinterpret_cast<uint4*>(crow);
                    uint4* d1 = reinterpret_cast<uint4*>(crow + 128);
                    auto pack8 = [](const uint32_t* v) {
                        uint4 o;
                        o.x = pack_bf16x2(__uint_as_float(v[0]), __uint_as_float(v[1]));
                        o.y = pack_bf16x2(__uint_as_float(v[2]), __uint_as_float(v[3]));
                        o.z = pack_bf16x2(__uint_as_float(v[4]), __uint_as_float(v[5]));
                        o.w = pack_bf16x2(__uint_as_float(v[6]), __uint_as_float(v[7]));
                        return o;
                    };
#pragma unroll
                    for (int c = 0; c < 8; c += 2) {   // 32-byte stores: one full sector each
                        st_global_v8(d0 + c, pack8(&vg[c * 8]), pack8(&vg[c * 8 + 8]));
                        st_global_v8(d1 + c, pack8(&vu[c * 8]), pack8(&vu[c * 8 + 8]));
                    }
                    S->pubq[pub_n++][tq] = ((uint32_t)m.x << 24) | (uint32_t)(m.z * a.cap + m.y);
                }
            }
            t_busy += clock64() - t_busy0;
        }
        if (warp == kFirstEpiWarp && lane == 0) {
            atomicAdd(&f->ticks[5], (unsigned long long)w_acc);
            atomicAdd(&f->ticks[8], (unsigned long long)t_busy);
            atomicAdd(&f->ticks[15], (unsigned long long)t_drain);
            atomicAdd(&f->ticks[14], (unsigned long long)t_pub);
        }
    }
    if (threadIdx.x == 0) atomicAdd(&f->ticks[6], (unsigned long long)(clock64() - t_start));

}
