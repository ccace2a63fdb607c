// ============================================================================
// mxk_kernels.cu — B200 (sm_100a) FP8xFP8 MoE layer: device kernels and the C
// ABI declared in include/mxk_b200.h.
//
// One layer = ONE launch of the persistent kernel k_mega (one CTA per SM), which runs
// the phases route -> set-up -> dispatch -> grouped GEMMs (+ combine push) -> reduce
// (mxk_phases.cuh, mxk_gemm.cuh).  mxk_launch_phases can run any subset of phases per
// launch; the single-GPU tests of a multi-rank world use that to interleave the ranks.
// ============================================================================
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/mxk_b200.h"
#include "mxk_device.cuh"
#include "mxk_sched.cuh"

namespace {

using namespace mxk;

// ------------------------------------------------------------------ constants
constexpr int kBlockM = 128;          // rows of a window = UMMA M
constexpr int kBlockK = 128;          // bytes of K per pipeline stage = scale block
constexpr int kBlockN = 256;          // weight rows per task = UMMA N (two 128-row halves)
constexpr uint64_t kDefaultLocalWaitNs = 2000000000ull;    // 2 s
constexpr uint64_t kDefaultRemoteWaitNs = 20000000000ull;  // 20 s

struct DevFlags {  // head of rwk (flags_off)
    long long current_time;      // completed prologues; the running launch is +1
    unsigned route_blocks_done;
    unsigned clear_blocks_done;  // arrivals at the grid barrier behind a full clear of combine_cnt
    unsigned route_sync;         // arrivals at the grid barrier of the one-pass route
    unsigned pad0_;
    unsigned task_ctr[2];        // claimed tasks beyond the first per CTA, by launch parity (the
                                 // copy of the other parity is reset for the next launch)
    int n_tasks, n_l1_tasks, n_windows, total_rows;
    int helper_on;               // the last launch ran the member's window list of the helper group
    int status;
    int dbg[8];
    unsigned long long ticks[16];
    unsigned long long dbg_ts[8];  // set-up leader time stamps (diagnostic, MXK_TICKS=1)
    unsigned setup_epoch;        // epoch whose tables CTA 0 has published; every CTA polls it
    unsigned pad2_[31];          // while CTA 0 writes the fields above
    unsigned reduce_blocks_done; // CTAs that have finished the reduce phase of this launch
    unsigned cnt_clean_epoch;    // launch whose reduce has consumed AND zeroed every arrival count
    unsigned long long trace[64];  // MxkStatus.trace
};
static_assert(sizeof(DevFlags) <= 1024, "status header must fit its 1 KB slot");
static_assert(offsetof(DevFlags, ticks) % 8 == 0 && offsetof(DevFlags, trace) % 8 == 0, "64-bit fields aligned");

struct KArgs {
    int R, rank, EPR, E, topk, H, I, cap, slot_cap, tokens, win_cap;
    int gemm_grid, skip_combine, scaled, ticks, pair;
    int push;                    // push-mode prologue (see push_phase)
    int group_ranks;             // members of a helper group (1 = none); helper scheduling needs push mode
    int skew_num;                // helpers on when max * n_experts > skew_num * sum over the group's experts
    int hot_windows;             // helpers take windows only of experts with at least this many windows (0 = of all)
    int ge_base;                 // this rank's first expert inside the weight arrays (member * EPR with group weights)
    int w_experts;               // experts in the weight arrays w1 / w2 (EPR, or group_ranks * EPR)
    int prefetch_bytes;          // bytes of W1 every CTA asks into L2 while the prologue runs
    int w_fp4;                   // weights are e2m1 codes, two per byte; TMA unpacks them to one code per byte
    int slim_ok;                 // launches whose windows are all small may use the five-stage ring (MXK_SLIM=0: never)
    FastDiv fR, fEPR, ftopk, fng, fwin;   // division by R, EPR, topk, R / group_ranks, win_cap
    unsigned long long local_wait_ns, remote_wait_ns;
    uint8_t* rwk;
    uint8_t* unk;
    void* const* unk_peers;
    const uint8_t* self;
    uint8_t* const* peer_bases;
    const int64_t* topk_idx;
    const uint8_t* w1;
    const uint8_t* w2;
    const uint8_t* w1_sf;
    const uint8_t* w2_sf;
    long long x_off, x_sf_off, weights_off;
    float* y;
    uint16_t* y_bf16;
    MxkLayout L;
};

__device__ __forceinline__ DevFlags* flags_of(const KArgs& a) {
    return reinterpret_cast<DevFlags*>(a.rwk + a.L.flags_off);
}
__device__ __forceinline__ void raise_status(DevFlags* f, int code, int dbg_slot) {
    atomicAdd(&f->dbg[dbg_slot], 1);
    atomicCAS(&f->status, 0, code);
}

#include "mxk_phases.cuh"
#include "mxk_gemm.cuh"

// ============================================================== k_mega ========
// The persistent kernel: one CTA per SM runs the phases selected by phase_mask in
// layer order.  CTAs wait on each other (route arrival, set-up flag, L1->L2 and
// pool counters), so the grid never exceeds the SM count and every CTA is resident.
template <bool kPair>
__device__ __forceinline__ void mega_body(const KArgs& a, const int phase_mask, const CUtensorMap& tm_pool,
                                          const CUtensorMap& tm_ffn, const CUtensorMap& tm_pool_slim,
                                          const CUtensorMap& tm_ffn_slim, const CUtensorMap& tm_w1,
                                          const CUtensorMap& tm_w2) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sf_tiles = tiles + kStages * kStageBytes;
    GemmSmem* S = reinterpret_cast<GemmSmem*>(sf_tiles + kSfRing * kSfSlotBytes);
    __shared__ int s_small[kRoutePer * 32];
    __shared__ float s_w[64];
    DevFlags* f = flags_of(a);
    const int warp = threadIdx.x >> 5;
    const bool do_gemm = (phase_mask & MXK_PHASE_GEMM) != 0;

    // Time line of the first and the last CTA (MxkStatus.trace), MXK_TICKS=1 only.
    unsigned long long* trace = nullptr;
    if (a.ticks != 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) trace = f->trace + (blockIdx.x == 0 ? 0 : 32);
    const bool stamp = a.ticks != 0 && threadIdx.x == 0;
    const uint64_t t0 = stamp ? gtimer_ns() : 0;
    if (trace && threadIdx.x == 0) trace[0] = t0;

    // the launch counter is advanced by the last CTA at the end of the route phase, after every
    // CTA has arrived there — i.e. after this read
    const long long epoch = ld_relaxed_gpu(&f->current_time) + ((phase_mask & MXK_PHASE_ROUTE) ? 1 : 0);
    const uint32_t clean_epoch = ld_relaxed_gpu(&f->cnt_clean_epoch);   // see ensure_counts_clean

    if (do_gemm) {
        if (threadIdx.x == 0) gemm_init_barriers(S, kPair);
        for (int i = threadIdx.x; i < 2 * 2 * 128; i += blockDim.x) (&S->xch[0][0][0])[i] = 0ull;
        if (warp == 1) {
            if constexpr (kPair) { tmem_alloc_pair(&S->tmem_base, kTmemCols); tmem_relinquish_pair(); }
            else { tmem_alloc(&S->tmem_base, kTmemCols); tmem_relinquish(); }
        }
        tc_fence_before();
    }
    // pair mode: the partner's barriers must be initialised before anything arrives on them
    if constexpr (kPair) cluster_sync_all(); else __syncthreads();
    uint32_t tmem_base = 0;
    if (do_gemm) {
        tc_fence_after();
        tmem_base = S->tmem_base;
    }
    if (trace && threadIdx.x == 0) trace[1] = gtimer_ns();

    // Phase stamps in ns since this CTA started (MxkStatus.ticks 9..13: end of route, set-up,
    // dispatch, GEMM, reduce; CTA 0 for the first two, maximum over CTAs for the rest).
    if (stamp && blockIdx.x == 0 && (phase_mask & MXK_PHASE_SETUP))
        for (int i = 0; i < 16; ++i) f->ticks[i] = 0;  // other CTAs add to them only after the set-up flag

    // While routing, barrier and dispatch run, HBM would sit idle: pull a slice of the expert
    // weights into L2 now (any W1 tile of a non-empty expert is needed later in this layer; the
    // streaming loads are evict-first, so these lines survive until their task comes up).
    if (do_gemm && (phase_mask & MXK_PHASE_ROUTE) && warp == 1) {
        // issued by all lanes of one warp (a lane per K block), so that the warp reaches the
        // route phase's first barrier without delay
        const int nt1 = a.I / 128, nkb = a.H / kBlockK;
        const int per_cta = min(nkb, a.prefetch_bytes / (2 * kABytes));
        for (int tile = blockIdx.x; tile < a.EPR * nt1 && tile < (int)gridDim.x; tile += gridDim.x) {
            const int e = tile / nt1, nt = tile % nt1;
            const int row0 = (a.ge_base + e) * 2 * a.I + nt * 128;   // this rank's own experts inside the weight arrays
            for (int kb = (int)(threadIdx.x & 31); kb < per_cta; kb += 32) {
                tma_prefetch_l2_2d(&tm_w1, kb * kBlockK, row0);
                tma_prefetch_l2_2d(&tm_w1, kb * kBlockK, row0 + a.I);
            }
        }
    }

    const PushScratch sc = push_scratch(tiles);   // push mode: the tile region is scratch until the GEMM phase
    const Team cta_team{(int)threadIdx.x, (int)blockDim.x, 0};
    // Push mode keeps only this rank's own bookkeeping in the route build (slot counts, accepted-pair
    // map, launch counter); nothing before the reduce phase needs it, so in a fused launch the
    // epilogue warps do it while they wait for the first accumulators (gemm_phase).
    const bool defer_route = a.push && do_gemm && (phase_mask & MXK_PHASE_ROUTE);
    if (phase_mask & MXK_PHASE_ROUTE) {
        ensure_counts_clean(a, f, epoch, clean_epoch);
        if (a.push) {
            push_phase(a, f, epoch, sc.wid);
            if (trace && threadIdx.x == 0) trace[2] = gtimer_ns();
            __syncthreads();   // the scratch is reused below
            if (!defer_route) route_phase(a, f, epoch, s_small, reinterpret_cast<int*>(tiles), kStages * kStageBytes / 4, true, cta_team);
        } else {
            route_phase(a, f, epoch, s_small, reinterpret_cast<int*>(tiles), kStages * kStageBytes / 4, false, cta_team);
        }
    }
    if (stamp && blockIdx.x == 0) f->ticks[9] = gtimer_ns() - t0;
    if (trace && threadIdx.x == 0) trace[3] = gtimer_ns();

    bool tables_ok = true;
    const PushTabs* tabs = nullptr;
    if (a.push) {
        if (phase_mask & (MXK_PHASE_SETUP | MXK_PHASE_DISPATCH | MXK_PHASE_GEMM)) {
            const bool setup = (phase_mask & MXK_PHASE_SETUP) != 0, disp = (phase_mask & MXK_PHASE_DISPATCH) != 0;
            tables_ok = push_tables(a, f, epoch, sc, &S->tabs);
            tabs = &S->tabs;
            if (trace && threadIdx.x == 0) trace[5] = gtimer_ns();
            if (a.ticks == 2) {   // diagnostic (MXK_TICKS=2): the same tables once more, to tell cold-start cost from work
                tables_ok = push_tables(a, f, epoch, sc, &S->tabs);
                if (trace && threadIdx.x == 0) trace[13] = gtimer_ns();
            }
            if (stamp && blockIdx.x == 0) f->ticks[10] = gtimer_ns() - t0;
            if (tables_ok && (setup || disp)) push_dispatch(a, f, epoch, sc, tabs, setup, disp);
            if (trace && threadIdx.x == 0) trace[6] = gtimer_ns();
            if (setup && blockIdx.x == 0) push_publish(a, f, epoch, sc, tabs);   // raises the status itself on overflow
            fence_proxy_async_smem();   // the scratch becomes TMA destination next
            __syncthreads();
        }
    } else {
        if (phase_mask & MXK_PHASE_SETUP) {
            // the tile region is idle until the GEMM phase: CTA 0 borrows it as scratch
            if (blockIdx.x == 0) setup_phase_leader(a, f, epoch, reinterpret_cast<int*>(tiles));
            else tables_ok = setup_phase_wait(a, f, epoch, s_small);
            __syncthreads();
        }
        if (stamp && blockIdx.x == 0) f->ticks[10] = gtimer_ns() - t0;
        if (trace && threadIdx.x == 0) trace[6] = gtimer_ns();
        if ((phase_mask & MXK_PHASE_DISPATCH) && tables_ok) {
            dispatch_phase(a, f, epoch, reinterpret_cast<int*>(tiles));  // tile region still idle: scratch
            fence_proxy_async_smem();
            __syncthreads();
        }
    }
    if (stamp) atomicMax(&f->ticks[11], (unsigned long long)(gtimer_ns() - t0));
    if (trace && threadIdx.x == 0) trace[7] = gtimer_ns();

    if (do_gemm) {
        if (tables_ok)
            gemm_phase<kPair>(a, f, epoch, tabs, trace, defer_route ? s_small : nullptr, tiles, sf_tiles, S, tmem_base, &tm_pool,
                              &tm_ffn, &tm_w1, &tm_w2, &tm_pool_slim, &tm_ffn_slim);
        else if (defer_route)   // no GEMM phase after all (tables failed): the launch bookkeeping still has to happen
            route_phase(a, f, epoch, s_small, nullptr, 0, true, cta_team);
        if (S->abort_flag) __nanosleep(200000);  // let copies / MMAs in flight drain
        tc_fence_before();
        // pair mode: neither CTA may free tensor memory or leave while its partner can still
        // arrive on its barriers or its MMAs still write both halves
        if constexpr (kPair) cluster_sync_all(); else __syncthreads();
        if (warp == 1) {
            __syncwarp();
            if constexpr (kPair) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
        }
    }
    if (stamp) atomicMax(&f->ticks[12], (unsigned long long)(gtimer_ns() - t0));
    if (trace && threadIdx.x == 0) trace[11] = gtimer_ns();

    if (phase_mask & MXK_PHASE_REDUCE) reduce_phase(a, f, epoch, s_small, s_w);
    if (stamp) atomicMax(&f->ticks[13], (unsigned long long)(gtimer_ns() - t0));
    if (trace && threadIdx.x == 0) trace[12] = gtimer_ns();
}

__global__ void __launch_bounds__(kGemmThreads, 1)
k_mega(const KArgs a, const int phase_mask, const __grid_constant__ CUtensorMap tm_pool,
       const __grid_constant__ CUtensorMap tm_ffn, const __grid_constant__ CUtensorMap tm_w1,
       const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_pool_slim,
       const __grid_constant__ CUtensorMap tm_ffn_slim) {
    mega_body<false>(a, phase_mask, tm_pool, tm_ffn, tm_pool_slim, tm_ffn_slim, tm_w1, tm_w2);
}

// The same layer with the GEMM phase on CTA pairs (clusters of two, 2-CTA tcgen05 MMA with
// M = 256): for windows of up to 256 rows, i.e. the compute-bound regime.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
k_mega_pair(const KArgs a, const int phase_mask, const __grid_constant__ CUtensorMap tm_pool,
            const __grid_constant__ CUtensorMap tm_ffn, const __grid_constant__ CUtensorMap tm_w1,
            const __grid_constant__ CUtensorMap tm_w2) {
    mega_body<true>(a, phase_mask, tm_pool, tm_ffn, tm_pool, tm_ffn, tm_w1, tm_w2);   // pairs never stage slim slots
}

__global__ void k_empty() {}

// The cross-rank window scheduler on the device: thread m computes member m's list (the same pure
// function the host entry point calls; reference check.cu:287-315 re-runs it on the host to find
// which windows a rank computes, which doubles as a host/device determinism test).
__global__ void k_sched_members(const int* rows_of_ge, int EPR, int group_ranks, int win_cap, int hot_windows, int* out_ge,
                                int* out_w, int* out_n, int cap) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= group_ranks) return;
    out_n[m] = sched_member_windows(rows_of_ge, EPR, group_ranks, win_cap, m, out_ge + (size_t)m * cap, out_w + (size_t)m * cap, cap,
                                    hot_windows);
}

// bf16 rows -> E4M3 + one UE8M0 scale per 128 columns, the reference's activation quantiser
// (per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=128), torch/mxmegakernel/utils/math.py:26-36:
// amax of the group clamped to 1e-4, sf = 2^ceil(log2(amax/448)), q = RNE(x / sf)); with
// sf == nullptr a plain saturating RNE cast, which is what the reference kernel's bf16
// prefold does (src/prologue.cuh:105-122).  One warp per 128-column group, 4 values per lane.
__global__ void k_quant_rows(const uint16_t* __restrict__ x, int tokens, int H, uint8_t* __restrict__ q,
                             uint8_t* __restrict__ sf) {
    const int groups = H / 128;
    const long long n = (long long)tokens * groups;
    const int lane = threadIdx.x & 31;
    const long long w0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nw = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long g = w0; g < n; g += nw) {
        const long long t = g / groups;
        const int c = (int)(g % groups);
        const uint2 raw = *reinterpret_cast<const uint2*>(x + t * H + c * 128 + lane * 4);
        const float v[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
                            __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u)};
        float inv = 1.0f;
        if (sf) {
            float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, d));
            const float s = fmaxf(amax, 1e-4f) / 448.0f;
            const uint32_t bits = __float_as_uint(s);
            uint32_t ex = ((bits >> 23) & 0xFF) + ((bits & 0x7FFFFF) ? 1u : 0u);   // ceil to a power of two
            ex = min(254u, max(1u, ex));
            inv = __uint_as_float((254u - ex) << 23);
            if (lane == 0) sf[t * groups + c] = (uint8_t)ex;
        }
        *reinterpret_cast<uint32_t*>(q + t * H + c * 128 + lane * 4) =
            pack_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
    }
}

__global__ void k_fill_weights(uint8_t* w, long long n_rows, int k_cols, uint32_t seed) {
    const long long n = n_rows * k_cols;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / k_cols), k = (uint32_t)(i % k_cols);
        w[i] = (uint8_t)((seed + row * 131u + k * 7u) & 0x3f);
    }
}

// Packed e2m1 test weights: code ((seed + 131*row + 7*k) >> 1) & 0xf at logical (row, k), two codes
// per byte (even k in the low nibble), row-major.
__global__ void k_fill_weights_e2m1(uint8_t* w, long long n_rows, int k_cols, uint32_t seed) {
    const int kb = k_cols / 2;
    const long long n = n_rows * kb;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / kb), k = 2u * (uint32_t)(i % kb);
        const uint32_t lo = ((seed + row * 131u + k * 7u) >> 1) & 0xfu, hi = ((seed + row * 131u + (k + 1) * 7u) >> 1) & 0xfu;
        w[i] = (uint8_t)(lo | (hi << 4));
    }
}

// =============================================================== host side ====
thread_local std::string g_err;
int fail(int code, const std::string& msg) {
    g_err = msg;
    return code;
}
int cuda_fail(cudaError_t e, const char* what) {
    g_err = std::string(what) + ": " + cudaGetErrorString(e);
    return (int)e;
}

int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

int check_geom(const MxkGeom* g) {
    if (!g) return fail(MXK_ERR_BAD_ARG, "null geometry");
    if (g->R < 1 || g->R > 1024 || g->rank < 0 || g->rank >= g->R) return fail(MXK_ERR_BAD_ARG, "bad R/rank");
    if (g->experts_per_rank < 1 || g->experts_per_rank > 1024) return fail(MXK_ERR_BAD_ARG, "experts_per_rank must be in [1,1024]");
    if (g->topk < 1 || g->topk > 64) return fail(MXK_ERR_BAD_ARG, "topk must be in [1,64]");
    if (g->hidden < 256 || g->hidden % 256 || g->hidden > 8192) return fail(MXK_ERR_BAD_ARG, "hidden must be a multiple of 256 in [256, 8192]");
    if (g->intermediate < 128 || g->intermediate % 128 || g->intermediate > 8192) return fail(MXK_ERR_BAD_ARG, "intermediate must be a multiple of 128 in [128, 8192]");
    if (g->max_tokens < 1) return fail(MXK_ERR_BAD_ARG, "max_tokens must be positive");
    if (g->slot_capacity < 0) return fail(MXK_ERR_BAD_ARG, "slot_capacity must be >= 0");
    return 0;
}

int compute_layout(const MxkGeom* g, MxkLayout* L) {
    if (int rc = check_geom(g)) return rc;
    if (!L) return fail(MXK_ERR_BAD_ARG, "null layout");
    std::memset(L, 0, sizeof(*L));
    const int64_t R = g->R, EPR = g->experts_per_rank, E = R * EPR, topk = g->topk, H = g->hidden, I = g->intermediate;
    const int64_t cap = g->max_tokens, slot = g->slot_capacity ? g->slot_capacity : g->max_tokens;
    int64_t o = 0;
    auto take = [&](int64_t bytes) { const int64_t at = o; o = align_up(o + bytes, 256); return at; };
    // sym
    L->x_off = take(cap * H);
    L->x_sf_off = take(cap * (H / 128));
    L->topk_idx_off = take(cap * topk * 8);
    L->topk_weights_off = take(cap * topk * 4);
    L->sym_bytes = o;
    // unk
    o = 0;
    L->recv_stride = (int32_t)align_up(EPR + 1, 64);
    L->src_index_table_off = take(2 * EPR * R * slot * 8);
    L->expert_recv_counts_off = take(2 * R * (int64_t)L->recv_stride * 8);
    L->combine_rows_off = take(topk * cap * H * 2);
    L->combine_cnt_off = take(topk * cap * 4);
    // push-mode staging area, only for geometries whose world routing fits a CTA's shared memory
    L->push_eligible = (R <= kPushMaxR && EPR <= kPushMaxEPR && R * cap * topk <= kPushMaxPairs &&
                        EPR * (R + 1) <= kPushMaxCnt) ? 1 : 0;
    L->push_auto = (L->push_eligible && (int64_t)cap * topk <= (R > 1 ? kPushAutoPairsPerRankWorld : kPushAutoPairsPerRank)) ? 1 : 0;
    {
        const int64_t sfw = (((H / 128) + 3) / 4 + 1) & ~(int64_t)1;
        L->xin_row_words = (int32_t)(2 * topk + sfw + H / 4);
        L->xin_src_words = 16 + cap * (int64_t)L->xin_row_words;
        L->xin_off = take(L->push_eligible ? 2 * R * L->xin_src_words * 8 : 0);
    }
    L->unk_bytes = o;
    // rwk
    o = 0;
    L->pool_rows = R * cap * topk;
    L->max_windows = (int32_t)(EPR + L->pool_rows / 8);
    const int64_t tasks_per_window = I / 128 + H / 256;
    // windows of fewer than 128 rows exist only for the tail of an expert or when
    // win_cap < 128; the task table is sized for win_cap >= 32 plus one tail each
    int64_t max_tasks = (EPR + L->pool_rows / 32) * tasks_per_window;
    if (max_tasks > 0x7FFFFFF0ll) max_tasks = 0x7FFFFFF0ll;
    L->max_tasks = (int32_t)max_tasks;
    L->sf_stride_h = (int32_t)align_up(H / 128, 16);
    L->sf_stride_i = (int32_t)align_up(I / 128, 16);
    L->flags_off = take(1024);
    L->route_slot_counts_off = take(E * 4);
    L->pair_state_off = take(cap * topk);
    L->route_scratch_ctas = 256;   // per-slice expert counts of the one-pass route build, [CTAs][E]
    L->route_scratch_off = take((int64_t)L->route_scratch_ctas * E * 4);
    L->prefix_tbl_off = take(EPR * (R + 1) * 4);
    L->expert_row_base_off = take((EPR + 1) * 4);
    L->windows_off = take((int64_t)L->max_windows * 16);
    L->tasks_off = take((int64_t)L->max_tasks * 16);
    L->l1_done_off = take(2 * (int64_t)L->max_windows * 4);
    L->pool_ready_off = take(2 * (int64_t)L->max_windows * 4);
    L->expert_first_win_off = take(EPR * 4);
    L->row_meta_off = take(L->pool_rows * 16);
    L->pool_off = take((L->pool_rows + 128) * H);
    L->pool_sf_off = take(L->pool_rows * L->sf_stride_h);
    L->ffn_off = take((L->pool_rows + 128) * I);
    L->ffn_sf_off = take(L->pool_rows * L->sf_stride_i);
    L->rwk_bytes = o;
    return 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// uint8 [rows][k] row-major, tile `box_rows` rows x 128 bytes, 128-byte swizzle.
int make_map(CUtensorMap* m, const void* base, int64_t rows, int64_t k, int box_rows = 128) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail(MXK_ERR_NO_DRIVER, "cuTensorMapEncodeTiled not available from the CUDA driver");
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k};
    const cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MXK_ERR_TENSOR_MAP, "cuTensorMapEncodeTiled failed, CUresult " + std::to_string((int)r));
    return 0;
}

// e2m1 codes [rows][k], two per byte in memory (row pitch k / 2 bytes); a tile of 128 rows x 128 codes
// arrives in shared memory as 128 x 128 BYTES, one code per byte position in the padded form the
// block-scaled MMA reads (every 16 codes: 8 bytes of data, 8 bytes of gap), 128-byte swizzle.
// The driver asks for: base 32-byte aligned, k a multiple of 128, pitch a multiple of 32 bytes,
// an inner box of exactly 128 codes.
int make_map_e2m1(CUtensorMap* m, const void* base, int64_t rows, int64_t k) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail(MXK_ERR_NO_DRIVER, "cuTensorMapEncodeTiled not available from the CUDA driver");
    if ((reinterpret_cast<uintptr_t>(base) & 31) || k % 128)
        return fail(MXK_ERR_BAD_ARG, "e2m1 weights must be 32-byte aligned with k a multiple of 128");
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)(k / 2)};
    const cuuint32_t box[2] = {128, 128};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MXK_ERR_TENSOR_MAP, "cuTensorMapEncodeTiled (e2m1) failed, CUresult " + std::to_string((int)r));
    return 0;
}

// Wait-time accounting and phase stamps: MXK_TICKS=1 in the environment, or mxk_set_ticks().
int g_ticks_override = -1;
int ticks_enabled() {
    static const int ticks_env = [] { const char* e = std::getenv("MXK_TICKS"); return e && e[0] >= '1' && e[0] <= '2' ? e[0] - '0' : 0; }();
    return g_ticks_override >= 0 ? g_ticks_override : ticks_env;
}

struct DeviceInfo { int sm_count = 0; int cc = 0; bool ok = false; };
int device_info(DeviceInfo* out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    static thread_local int cached_dev = -1;
    static thread_local DeviceInfo cached;
    if (cached_dev != dev) {
        int major = 0, minor = 0, sms = 0;
        if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cached.sm_count = sms;
        cached.cc = major * 10 + minor;
        cached.ok = true;
        cached_dev = dev;
    }
    *out = cached;
    return 0;
}

int build_kargs(const MxkLaunchArgs* la, KArgs* k) {
    if (!la) return fail(MXK_ERR_BAD_ARG, "null launch args");
    MxkGeom g{};
    g.R = la->R; g.rank = la->rank;
    // zero geometry fields select the reference's frozen scene (src/common.cuh:18-24)
    g.experts_per_rank = la->experts_per_rank ? la->experts_per_rank : 8;
    g.topk = la->topk ? la->topk : 8;
    g.hidden = la->hidden ? la->hidden : 6144;
    g.intermediate = la->intermediate ? la->intermediate : 2048;
    g.max_tokens = la->max_tokens ? la->max_tokens : (la->slot_capacity ? la->slot_capacity : 512);
    g.slot_capacity = la->slot_capacity;
    std::memset(k, 0, sizeof(*k));
    if (int rc = compute_layout(&g, &k->L)) return rc;
    if (!la->rwk || !la->unk || !la->unk_peers || !la->self || !la->peer_bases)
        return fail(MXK_ERR_BAD_ARG, "rwk / unk / unk_peers / self / peer_bases must be non-null");
    if (la->tokens < 0 || la->tokens > g.max_tokens) return fail(MXK_ERR_BAD_ARG, "tokens outside [0, max_tokens]");
    if (la->in_bf16) return fail(MXK_ERR_BAD_ARG, "in_bf16 input is not supported");
    if (la->skip_prologue) return fail(MXK_ERR_BAD_ARG, "skip_prologue is not supported");
    int win = la->win_cap ? la->win_cap : 128;
    // same rule as the reference binding: window in [8,128], multiple of 8 (torch/csrc/apis/mega.hpp:230-233)
    if (win < 8 || win > 128 || win % 8) return fail(MXK_ERR_BAD_ARG, "win_cap must be a multiple of 8 in [8,128]");
    if ((int64_t)g.topk * g.max_tokens > 0xFFFFFF || g.R > 255)
        return fail(MXK_ERR_BAD_ARG, "topk * max_tokens must fit 24 bits and R 8 bits (arrival-count queue entries)");
    if ((la->w1_sf == nullptr) != (la->w2_sf == nullptr)) return fail(MXK_ERR_BAD_ARG, "w1_sf and w2_sf must both be set or both be null");
    // set-up and dispatch borrow the operand-tile region of shared memory for their tables
    if ((4ll * g.experts_per_rank + 2 + (int64_t)g.experts_per_rank * (g.R + 1)) * 4 > (int64_t)kStages * kStageBytes)
        return fail(MXK_ERR_BAD_ARG, "experts_per_rank * (R + 1) tables exceed the shared-memory scratch of the prologue");
    if (la->dispatch_mode < 0 || la->dispatch_mode > 2) return fail(MXK_ERR_BAD_ARG, "dispatch_mode must be 0, 1 or 2");
    if (la->dispatch_mode == 2 && !k->L.push_eligible)
        return fail(MXK_ERR_BAD_ARG, "dispatch_mode = 2 (push) needs R <= 64, experts_per_rank <= 256 and R * max_tokens * topk <= 16384");
    const bool want_helpers = la->group_ranks > 1 && la->group_weights_ready;
    k->push = la->dispatch_mode == 2 || (la->dispatch_mode == 0 && (k->L.push_auto || (want_helpers && k->L.push_eligible)));
    // cross-rank helper scheduling: group-replicated weights, push-mode prologue only
    k->group_ranks = 1; k->skew_num = 2; k->hot_windows = 0; k->ge_base = 0; k->w_experts = g.experts_per_rank;
    const uint8_t *w1 = la->w1, *w2 = la->w2, *w1_sf = la->w1_sf, *w2_sf = la->w2_sf;
    if (la->group_ranks < 0) return fail(MXK_ERR_BAD_ARG, "group_ranks must be >= 0");
    if (la->group_ranks > 1 && la->group_weights_ready) {
        const int G = la->group_ranks;
        if (G > kSchedMaxGroupRanks || g.R % G) return fail(MXK_ERR_BAD_ARG, "group_ranks must divide R and be at most 16");
        if (!k->push) return fail(MXK_ERR_BAD_ARG, "helper groups need the push-mode prologue (dispatch_mode 2 or an eligible geometry)");
        if ((int64_t)G * g.experts_per_rank * (g.R + 1) > kPushMaxCnt)
            return fail(MXK_ERR_BAD_ARG, "group_ranks * experts_per_rank * (R + 1) exceeds the shared-memory tables of the prologue");
        if (!la->w1_group || !la->w2_group) return fail(MXK_ERR_BAD_ARG, "w1_group / w2_group must be non-null with group_weights_ready");
        if ((la->w1_sf_group == nullptr) != (la->w2_sf_group == nullptr) || (la->w1_sf_group == nullptr) != (la->w1_sf == nullptr))
            return fail(MXK_ERR_BAD_ARG, "group scale planes must be given exactly when w1_sf / w2_sf are");
        k->group_ranks = G;
        k->skew_num = la->group_skew_num == 0 ? 2 : (la->group_skew_num < 0 ? 0 : la->group_skew_num);
        k->hot_windows = la->group_hot_windows == 0 ? kHelperHotWindows : (la->group_hot_windows < 0 ? 0 : la->group_hot_windows);
        k->ge_base = (g.rank / (g.R / G)) * g.experts_per_rank;
        k->w_experts = G * g.experts_per_rank;
        w1 = la->w1_group; w2 = la->w2_group; w1_sf = la->w1_sf_group; w2_sf = la->w2_sf_group;
    }
    if (la->weight_format != MXK_WEIGHTS_E4M3 && la->weight_format != MXK_WEIGHTS_E2M1)
        return fail(MXK_ERR_BAD_ARG, "weight_format must be MXK_WEIGHTS_E4M3 or MXK_WEIGHTS_E2M1");
    k->w_fp4 = la->weight_format == MXK_WEIGHTS_E2M1;
    {
        static const int slim_env = [] { const char* e = std::getenv("MXK_SLIM"); return e ? std::atoi(e) : 1; }();
        k->slim_ok = slim_env != 0;
    }
    k->R = g.R; k->rank = g.rank; k->EPR = g.experts_per_rank; k->E = g.R * g.experts_per_rank;
    k->topk = g.topk; k->H = g.hidden; k->I = g.intermediate; k->cap = g.max_tokens;
    k->slot_cap = g.slot_capacity ? g.slot_capacity : g.max_tokens;
    k->tokens = la->tokens; k->win_cap = win;
    k->skip_combine = la->skip_combine; k->scaled = la->w1_sf != nullptr;
    k->ticks = ticks_enabled();  // the kernel accounts its wait cycles and stamps its phases (MxkStatus.ticks / trace)
    {
        // MXK_MAX_SPINS: bound of every device wait (units of 250 ns) for launches that leave max_spins at 0
        static const int spins_env = [] { const char* e = std::getenv("MXK_MAX_SPINS"); return e ? std::atoi(e) : 0; }();
        const int spins = la->max_spins > 0 ? la->max_spins : spins_env;
        k->local_wait_ns = spins > 0 ? (unsigned long long)spins * 250ull : kDefaultLocalWaitNs;
        k->remote_wait_ns = spins > 0 ? (unsigned long long)spins * 250ull : kDefaultRemoteWaitNs;
    }
    k->rwk = static_cast<uint8_t*>(la->rwk); k->unk = static_cast<uint8_t*>(la->unk);
    k->unk_peers = la->unk_peers; k->self = la->self; k->peer_bases = la->peer_bases;
    k->topk_idx = la->topk_idx ? la->topk_idx : reinterpret_cast<const int64_t*>(la->self + la->topk_idx_off);
    k->w1 = w1; k->w2 = w2; k->w1_sf = w1_sf; k->w2_sf = w2_sf;
    k->x_off = la->x_off; k->x_sf_off = la->x_sf_off; k->weights_off = la->weights_off;
    k->y = la->y; k->y_bf16 = la->y_bf16;
    DeviceInfo di;
    if (int rc = device_info(&di)) return rc;
    if (di.cc / 10 != 10) return fail(MXK_ERR_DEVICE, "this library runs on sm_100 (B200) only, device is sm_" + std::to_string(di.cc));
    int grid = la->grid > 0 ? la->grid : di.sm_count;
    if (grid > di.sm_count) grid = di.sm_count;  // CTAs wait on each other: all must be resident
    // CTA-pair tiling pays once windows fill up (compute-bound regime); with few rows per
    // expert a 256-row window would only halve the number of CTAs streaming weights
    int pair = la->cta_pair;
    if (pair < 0 || pair > 2) return fail(MXK_ERR_BAD_ARG, "cta_pair must be 0, 1 or 2");
    if (pair == 0) pair = (win == 128 && grid >= 2 && (int64_t)la->tokens * g.topk >= 256ll * g.experts_per_rank) ? 2 : 1;
    if (pair == 2) {
        if (win != 128) return fail(MXK_ERR_BAD_ARG, "cta_pair = 2 needs win_cap = 128");
        if (grid < 2) return fail(MXK_ERR_BAD_ARG, "cta_pair = 2 needs a grid of at least 2 CTAs");
        grid &= ~1;
        k->pair = 1;
        k->win_cap = 256;   // rows per window of a CTA pair
    }
    k->gemm_grid = grid;
    {
        // MXK_PREFETCH_KB overrides the L2 prefetch per CTA (tuning knob; 0 switches it off)
        static const int pf_env = [] { const char* e = std::getenv("MXK_PREFETCH_KB"); return e ? std::atoi(e) * 1024 : -1; }();
        // The push-mode prologue is short and made of dependent memory round trips; a bulk prefetch
        // issued beside it lengthens every one of them (measured: first operand tile at 24.4 us with
        // 704 KB per CTA against 20.9 us without, GEMM phase unchanged).  With large batches the pull-mode
        // prologue is itself memory traffic (route build, row copies) and loses more to the prefetch than
        // the GEMM phase gains (prefill-sized quarter: layer 392 us with it, 389 us without).  Only the
        // pull-mode prologue of a small batch, three round trips with the memory system idle, prefetches.
        const bool small_batch = (int64_t)k->cap * k->topk <= kPushAutoPairsPerRank;
        k->prefetch_bytes = pf_env >= 0 ? pf_env : ((k->push || !small_batch) ? 0 : kPrefetchBytesPerCta);
    }
    k->fR = FastDiv::make((uint32_t)k->R); k->fEPR = FastDiv::make((uint32_t)k->EPR); k->ftopk = FastDiv::make((uint32_t)k->topk);
    k->fng = FastDiv::make((uint32_t)(k->R / k->group_ranks)); k->fwin = FastDiv::make((uint32_t)k->win_cap);
    return 0;
}

constexpr int kPhaseAll = MXK_PHASE_ROUTE | MXK_PHASE_SETUP | MXK_PHASE_DISPATCH | MXK_PHASE_GEMM | MXK_PHASE_REDUCE;

// One launch of the persistent kernel running the phases in `mask`.
int launch_mega(const KArgs& k, int mask, cudaStream_t st) {
    mask &= kPhaseAll;
    if ((mask & MXK_PHASE_REDUCE) && !k.y && !k.y_bf16) return fail(MXK_ERR_BAD_ARG, "y or y_bf16 must be non-null");
    if ((mask & MXK_PHASE_REDUCE) && k.tokens == 0) mask &= ~MXK_PHASE_REDUCE;  // nothing to reduce on this rank
    if (mask == 0) return 0;
    // The four tensor maps depend only on (workspace, weights, geometry): a serving loop launches the
    // same ones every layer, so the last few sets are kept per thread instead of being re-encoded.
    struct MapSet { const void* rwk; const void* w1; const void* w2; int64_t rows; int H, I, EPR, fp4; CUtensorMap m[6]; };
    static thread_local MapSet cache[4];
    static thread_local int cache_n = 0, cache_next = 0;
    CUtensorMap zero_maps[6];
    const CUtensorMap* maps = zero_maps;
    if (mask & MXK_PHASE_GEMM) {
        if (!k.w1 || !k.w2) return fail(MXK_ERR_BAD_ARG, "w1 / w2 must be non-null");
        const MapSet* hit = nullptr;
        for (int i = 0; i < cache_n; ++i) {
            const MapSet& c = cache[i];
            if (c.rwk == k.rwk && c.w1 == k.w1 && c.w2 == k.w2 && c.rows == k.L.pool_rows && c.H == k.H && c.I == k.I && c.EPR == k.w_experts && c.fp4 == k.w_fp4) {
                hit = &c;
                break;
            }
        }
        if (!hit) {
            MapSet n;
            std::memset(&n, 0, sizeof(n));
            n.rwk = k.rwk; n.w1 = k.w1; n.w2 = k.w2; n.rows = k.L.pool_rows; n.H = k.H; n.I = k.I; n.EPR = k.w_experts; n.fp4 = k.w_fp4;
            if (int rc = make_map(&n.m[0], k.rwk + k.L.pool_off, k.L.pool_rows + 128, k.H)) return rc;
            if (int rc = make_map(&n.m[1], k.rwk + k.L.ffn_off, k.L.pool_rows + 128, k.I)) return rc;
            if (k.w_fp4) {
                if (int rc = make_map_e2m1(&n.m[2], k.w1, (int64_t)k.w_experts * 2 * k.I, k.H)) return rc;
                if (int rc = make_map_e2m1(&n.m[3], k.w2, (int64_t)k.w_experts * k.H, k.I)) return rc;
            } else {
                if (int rc = make_map(&n.m[2], k.w1, (int64_t)k.w_experts * 2 * k.I, k.H)) return rc;
                if (int rc = make_map(&n.m[3], k.w2, (int64_t)k.w_experts * k.H, k.I)) return rc;
            }
            // the same activation tensors with kSlimRows-row boxes (launches whose windows are all that small)
            if (int rc = make_map(&n.m[4], k.rwk + k.L.pool_off, k.L.pool_rows + 128, k.H, kSlimRows)) return rc;
            if (int rc = make_map(&n.m[5], k.rwk + k.L.ffn_off, k.L.pool_rows + 128, k.I, kSlimRows)) return rc;
            cache[cache_next] = n;
            hit = &cache[cache_next];
            cache_next = (cache_next + 1) % 4;
            if (cache_n < 4) ++cache_n;
        }
        maps = hit->m;
    } else {
        std::memset(zero_maps, 0, sizeof(zero_maps));
    }
    const CUtensorMap &tm_pool = maps[0], &tm_ffn = maps[1], &tm_w1 = maps[2], &tm_w2 = maps[3], &tm_pool_slim = maps[4], &tm_ffn_slim = maps[5];
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(k_mega, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(k_mega)");
        e = cudaFuncSetAttribute(k_mega_pair, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(k_mega_pair)");
        attr_dev = dev;
    }
    if (k.pair) {
        // every CTA pair must be resident at once (CTAs wait on each other): ask the runtime how
        // many clusters of two fit and never launch more
        static thread_local int max_pairs = 0, pairs_dev = -1;
        if (pairs_dev != dev) {
            cudaLaunchConfig_t cfg;
            std::memset(&cfg, 0, sizeof(cfg));
            cfg.gridDim = dim3(2, 1, 1); cfg.blockDim = dim3(kGemmThreads, 1, 1); cfg.dynamicSmemBytes = kGemmSmem;
            cudaLaunchAttribute at;
            at.id = cudaLaunchAttributeClusterDimension;
            at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
            cfg.attrs = &at; cfg.numAttrs = 1;
            int n = 0;
            cudaError_t e = cudaOccupancyMaxActiveClusters(&n, k_mega_pair, &cfg);
            if (e != cudaSuccess) return cuda_fail(e, "cudaOccupancyMaxActiveClusters(k_mega_pair)");
            if (n < 1) return fail(MXK_ERR_DEVICE, "no CTA pair of k_mega_pair fits on this device");
            max_pairs = n; pairs_dev = dev;
        }
        KArgs kk = k;
        if (kk.gemm_grid > 2 * max_pairs) kk.gemm_grid = 2 * max_pairs;
        k_mega_pair<<<kk.gemm_grid, kGemmThreads, kGemmSmem, st>>>(kk, mask, tm_pool, tm_ffn, tm_w1, tm_w2);
    }
    else
        k_mega<<<k.gemm_grid, kGemmThreads, kGemmSmem, st>>>(k, mask, tm_pool, tm_ffn, tm_w1, tm_w2, tm_pool_slim, tm_ffn_slim);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : cuda_fail(e, k.pair ? "launch k_mega_pair" : "launch k_mega");
}

// ------------------------------------------------------------ static scratch
// Workspace for mxk_launch_full_static: lives in the module image, so it exists on every
// GPU that loads this library from load until exit and never goes through an allocator.
constexpr size_t kStaticScratchBytes = 32u << 20;  // 32 MiB
constexpr size_t kStaticPtrBytes = 256;            // two pointer tables of one entry each
constexpr int kStaticMaxDevices = 64;
static __device__ __align__(256) uint8_t g_static_scratch[kStaticScratchBytes];

__global__ void k_static_ptrs(void** sym_table, void** unk_table, void* sym, void* unk) {
    sym_table[0] = sym;
    unk_table[0] = unk;
}

// Device address of g_static_scratch on the current device.  In host code the array's
// name is only a stand-in, so the address is asked from the runtime once per device.
int static_scratch_base(uint8_t** out, int* dev_out) {
    static uint8_t* base[kStaticMaxDevices] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= kStaticMaxDevices) return fail(MXK_ERR_BAD_ARG, "device index beyond the static scratch table");
    if (!base[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
        base[dev] = static_cast<uint8_t*>(p);
    }
    *out = base[dev];
    *dev_out = dev;
    return 0;
}

}  // namespace

// ================================================================== C ABI =====
extern "C" {

const char* mxk_last_error(void) { return g_err.c_str(); }
int mxk_version(void) { return 100; }

int mxk_compute_layout(const MxkGeom* g, MxkLayout* out) { return compute_layout(g, out); }
int64_t mxk_sym_bytes(const MxkGeom* g) { MxkLayout L; return compute_layout(g, &L) ? -1 : L.sym_bytes; }
int64_t mxk_rwk_bytes(const MxkGeom* g) { MxkLayout L; return compute_layout(g, &L) ? -1 : L.rwk_bytes; }
int64_t mxk_unk_bytes(const MxkGeom* g) { MxkLayout L; return compute_layout(g, &L) ? -1 : L.unk_bytes; }

int mxk_launch_prelude(const MxkLaunchArgs* a, void* stream) {
    KArgs k;
    if (int rc = build_kargs(a, &k)) return rc;
    return launch_mega(k, MXK_PHASE_ROUTE | MXK_PHASE_SETUP, static_cast<cudaStream_t>(stream));
}
int mxk_launch_compute(const MxkLaunchArgs* a, void* stream) {
    KArgs k;
    if (int rc = build_kargs(a, &k)) return rc;
    return launch_mega(k, kPhaseAll & ~MXK_PHASE_REDUCE, static_cast<cudaStream_t>(stream));
}
int mxk_launch_reduce(const MxkLaunchArgs* a, void* stream) {
    KArgs k;
    if (int rc = build_kargs(a, &k)) return rc;
    if (!k.y && !k.y_bf16) return fail(MXK_ERR_BAD_ARG, "y or y_bf16 must be non-null");
    return launch_mega(k, MXK_PHASE_REDUCE, static_cast<cudaStream_t>(stream));
}
int mxk_launch_full(const MxkLaunchArgs* a, void* stream) {
    KArgs k;
    if (int rc = build_kargs(a, &k)) return rc;
    if (!k.y && !k.y_bf16) return fail(MXK_ERR_BAD_ARG, "y or y_bf16 must be non-null");
    return launch_mega(k, kPhaseAll, static_cast<cudaStream_t>(stream));
}
int mxk_kernels_per_layer(void) { return 1; }

int mxk_launch_full_static(const MxkLaunchArgs* a, void* stream) {
    if (!a) return fail(MXK_ERR_BAD_ARG, "null launch args");
    if (a->R != 1 || a->rank != 0) return fail(MXK_ERR_BAD_ARG, "mxk_launch_full_static serves a single-rank world only (R=1)");
    if (!a->self) return fail(MXK_ERR_BAD_ARG, "self (the input block) must be non-null");
    MxkGeom g{};
    g.R = 1; g.rank = 0;
    g.experts_per_rank = a->experts_per_rank ? a->experts_per_rank : 8;
    g.topk = a->topk ? a->topk : 8;
    g.hidden = a->hidden ? a->hidden : 6144;
    g.intermediate = a->intermediate ? a->intermediate : 2048;
    g.max_tokens = a->max_tokens ? a->max_tokens : (a->slot_capacity ? a->slot_capacity : 512);
    g.slot_capacity = a->slot_capacity;
    MxkLayout L;
    if (int rc = compute_layout(&g, &L)) return rc;
    const size_t need = kStaticPtrBytes + (size_t)L.unk_bytes + (size_t)L.rwk_bytes;
    if (need > kStaticScratchBytes)
        return fail(MXK_ERR_BAD_ARG, "workspace of this geometry needs " + std::to_string(need) +
                                         " bytes, the static scratch holds " + std::to_string(kStaticScratchBytes));
    uint8_t* base = nullptr;
    int dev = 0;
    if (int rc = static_scratch_base(&base, &dev)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Layout of the array: the two pointer tables, then rwk, then unk.  rwk comes first so that its
    // status header — whose first word is the launch counter — sits at the same address whatever
    // the geometry: the counter is zero when the module is loaded and must keep running from call
    // to call, because the prologue's words are tagged with it and a counter that started over
    // would make an earlier call's words look current.
    static_assert(offsetof(DevFlags, current_time) == 0 && sizeof(long long) == 8, "launch counter leads the header");
    uint8_t* rwk = base + kStaticPtrBytes;
    uint8_t* unk = rwk + L.rwk_bytes;
    // The array keeps whatever the previous call left.  Calls of one geometry continue on it like
    // launches on an ordinary workspace.  A call with ANOTHER geometry finds the tables of the old
    // one at different offsets, so everything behind the launch counter is cleared first (the
    // memset runs on the caller's stream, before this call's kernel and after the previous one).
    static MxkGeom last_geom[kStaticMaxDevices] = {};
    cudaError_t e;
    if (std::memcmp(&last_geom[dev], &g, sizeof(g)) != 0) {
        e = cudaMemsetAsync(rwk + 8, 0, need - kStaticPtrBytes - 8, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(static workspace)");
        last_geom[dev] = g;
    } else {
        // a device-side failure of an earlier call must not be reported for this one
        static_assert(offsetof(DevFlags, dbg) == offsetof(DevFlags, status) + sizeof(int), "status word, then the expiry counters");
        e = cudaMemsetAsync(rwk + offsetof(DevFlags, status), 0, sizeof(int) * 9, st);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(status words)");
    }
    void** sym_table = reinterpret_cast<void**>(base);
    void** unk_table = reinterpret_cast<void**>(base + 128);
    k_static_ptrs<<<1, 1, 0, st>>>(sym_table, unk_table, const_cast<uint8_t*>(a->self), unk);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "launch static pointer set-up");
    MxkLaunchArgs b = *a;
    b.rwk = rwk;
    b.unk = unk;
    b.unk_peers = reinterpret_cast<void* const*>(unk_table);
    b.peer_bases = reinterpret_cast<uint8_t* const*>(sym_table);
    KArgs k;
    if (int rc = build_kargs(&b, &k)) return rc;
    if (!k.y && !k.y_bf16) return fail(MXK_ERR_BAD_ARG, "y or y_bf16 must be non-null");
    return launch_mega(k, kPhaseAll, st);
}
int mxk_read_status_static(MxkStatus* out) {
    uint8_t* base = nullptr;
    int dev = 0;
    if (int rc = static_scratch_base(&base, &dev)) return rc;
    return mxk_read_status(base + kStaticPtrBytes, out);
}
int64_t mxk_static_scratch_bytes(void) { return (int64_t)kStaticScratchBytes; }

int mxk_launch_phases(const MxkLaunchArgs* a, int phase_mask, void* stream) {
    KArgs k;
    if (int rc = build_kargs(a, &k)) return rc;
    return launch_mega(k, phase_mask, static_cast<cudaStream_t>(stream));
}

int mxk_launch_empty(int grid, int threads, int64_t smem, void* stream) {
    if (grid < 1 || threads < 1 || threads > 1024 || smem < 0 || smem > 48 * 1024)
        return fail(MXK_ERR_BAD_ARG, "bad empty-launch geometry");
    k_empty<<<grid, threads, (size_t)smem, static_cast<cudaStream_t>(stream)>>>();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : cuda_fail(e, "launch empty");
}

int mxk_fill_weights(uint8_t* w, int64_t n_rows, int32_t k_cols, uint32_t seed, void* stream) {
    if (!w || n_rows < 0 || k_cols < 1) return fail(MXK_ERR_BAD_ARG, "bad fill_weights arguments");
    if (n_rows == 0) return 0;
    k_fill_weights<<<1024, 256, 0, static_cast<cudaStream_t>(stream)>>>(w, n_rows, k_cols, seed);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : cuda_fail(e, "launch fill_weights");
}

int mxk_fill_weights_e2m1(uint8_t* w, int64_t n_rows, int32_t k_cols, uint32_t seed, void* stream) {
    if (!w || n_rows < 0 || k_cols < 2 || k_cols % 2) return fail(MXK_ERR_BAD_ARG, "bad fill_weights_e2m1 arguments");
    if (n_rows == 0) return 0;
    k_fill_weights_e2m1<<<1024, 256, 0, static_cast<cudaStream_t>(stream)>>>(w, n_rows, k_cols, seed);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : cuda_fail(e, "launch fill_weights_e2m1");
}

uint8_t mxk_e2m1_to_e4m3(uint8_t code) {
    // e2m1: sign, 2 exponent bits (bias 1), 1 mantissa bit; exponent 0 is the subnormal pair {0, 0.5}
    const uint8_t sign = (code & 8u) ? 0x80u : 0u, e = (code >> 1) & 3u, m = code & 1u;
    const uint8_t mag = e == 0 ? (m ? 0x30u : 0u) : (uint8_t)(((e + 6u) << 3) | (m << 2));
    return sign | mag;
}

int mxk_quantize_rows(const void* x_bf16, int32_t tokens, int32_t hidden, void* x_fp8, void* x_sf, void* stream) {
    if (!x_bf16 || !x_fp8 || tokens < 0 || hidden < 128 || hidden % 128)
        return fail(MXK_ERR_BAD_ARG, "quantize_rows: null pointer, negative tokens or hidden not a multiple of 128");
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 7) || (reinterpret_cast<uintptr_t>(x_fp8) & 3))
        return fail(MXK_ERR_BAD_ARG, "quantize_rows: x_bf16 must be 8-byte and x_fp8 4-byte aligned");
    if (tokens == 0) return 0;
    const long long warps = (long long)tokens * (hidden / 128);
    const int blocks = (int)std::min<long long>((warps + 7) / 8, 148 * 8);
    k_quant_rows<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(x_bf16), tokens, hidden, static_cast<uint8_t*>(x_fp8), static_cast<uint8_t*>(x_sf));
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : cuda_fail(e, "launch k_quant_rows");
}

int mxk_dump_kernel_resources(void) {
    struct { const char* name; const void* fn; } ks[] = {
        {"k_mega", (const void*)k_mega}, {"k_mega_pair", (const void*)k_mega_pair},
        {"k_quant_rows", (const void*)k_quant_rows}, {"k_fill_weights", (const void*)k_fill_weights}};
    for (auto& k : ks) {
        cudaFuncAttributes at;
        cudaError_t e = cudaFuncGetAttributes(&at, k.fn);
        if (e != cudaSuccess) return cuda_fail(e, "cudaFuncGetAttributes");
        std::printf("[RES] %-10s regs=%d local=%zu static_smem=%zu max_threads=%d\n", k.name, at.numRegs,
                    at.localSizeBytes, at.sharedSizeBytes, at.maxThreadsPerBlock);
    }
    std::printf("[RES] k_mega dynamic smem=%d threads=%d\n", kGemmSmem, kGemmThreads);
    return 0;
}

int mxk_read_status(const void* rwk, MxkStatus* out) {
    if (!rwk || !out) return fail(MXK_ERR_BAD_ARG, "null argument");
    DevFlags f;
    cudaError_t e = cudaMemcpy(&f, rwk, sizeof(f), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(status)");
    out->launches = f.current_time;
    out->status = f.status;
    out->n_tasks = f.n_tasks; out->n_l1_tasks = f.n_l1_tasks; out->n_windows = f.n_windows; out->total_rows = f.total_rows;
    out->helper_on = f.helper_on;
    for (int i = 0; i < 8; ++i) out->dbg[i] = f.dbg[i];
    for (int i = 0; i < 16; ++i) out->ticks[i] = f.ticks[i];
    for (int i = 0; i < 64; ++i) out->trace[i] = f.trace[i];
    return 0;
}

// Byte offset of the per-layer wait / phase counters (MxkStatus.ticks) inside rwk and their
// number, for hosts that copy them back themselves (reference: pre_ticks readers,
// torch/csrc/flags_bridge.cu:44-51).
// ---- skew-aware schedulers (pure functions of mxk_sched.cuh) -----------------------------
int mxk_group_ranks(void) { return 4; }   // ranks per helper group the reference builds with (kGroupRanks)
static int sched_args_ok(const int32_t* rows_of_ge, int EPR, int group_ranks, int win_cap) {
    if (!rows_of_ge || EPR < 1 || group_ranks < 1 || group_ranks > kSchedMaxGroupRanks || win_cap < 1)
        return fail(MXK_ERR_BAD_ARG, "scheduler: null counts, EPR < 1, window < 1 or group size outside [1,16]");
    return 0;
}
int mxk_gs_schedule_member(const int32_t* rows_of_ge, int EPR, int group_ranks, int win_cap, int member,
                           int32_t* out_ge, int32_t* out_w, int cap) {
    if (sched_args_ok(rows_of_ge, EPR, group_ranks, win_cap)) return MXK_ERR_BAD_ARG;
    if (member < 0 || member >= group_ranks || cap < 0 || (cap > 0 && (!out_ge || !out_w)))
        return fail(MXK_ERR_BAD_ARG, "scheduler: member outside the group or null output");
    return sched_member_windows(rows_of_ge, EPR, group_ranks, win_cap, member, out_ge, out_w, cap);
}
int mxk_gs_schedule_member_hot(const int32_t* rows_of_ge, int EPR, int group_ranks, int win_cap, int member, int hot_windows,
                               int32_t* out_ge, int32_t* out_w, int cap) {
    if (sched_args_ok(rows_of_ge, EPR, group_ranks, win_cap)) return MXK_ERR_BAD_ARG;
    if (member < 0 || member >= group_ranks || cap < 0 || hot_windows < 0 || (cap > 0 && (!out_ge || !out_w)))
        return fail(MXK_ERR_BAD_ARG, "scheduler: member outside the group, negative hot_windows or null output");
    return sched_member_windows(rows_of_ge, EPR, group_ranks, win_cap, member, out_ge, out_w, cap, hot_windows);
}
int mxk_gs_group_skewed(const int32_t* rows_of_ge, int n_experts, int skew_num) {
    if (!rows_of_ge || n_experts < 1) return fail(MXK_ERR_BAD_ARG, "scheduler: null counts");
    return sched_group_skewed(rows_of_ge, n_experts, skew_num) ? 1 : 0;
}
int mxk_lpt_assign(const int32_t* counts, const int32_t* experts, int n_experts, int win_cap, int n_slice, int n_members,
                   int32_t* tasks, int32_t* member_of, int64_t* load, int cap) {
    if (!counts || !experts || !tasks || !member_of || !load || n_experts < 1 || win_cap < 1 || n_slice < 1 || n_members < 1 || cap < 0)
        return fail(MXK_ERR_BAD_ARG, "lpt_assign: null pointer or non-positive size");
    static_assert(sizeof(long long) == sizeof(int64_t), "64-bit loads");
    return sched_lpt_assign(counts, experts, n_experts, win_cap, n_slice, n_members, tasks, member_of,
                            reinterpret_cast<long long*>(load), cap);
}
int mxk_gs_schedule_on_device(const int32_t* rows_of_ge, int EPR, int group_ranks, int win_cap, int hot_windows,
                              int32_t* out_ge, int32_t* out_w, int32_t* out_n, int cap) {
    if (sched_args_ok(rows_of_ge, EPR, group_ranks, win_cap)) return MXK_ERR_BAD_ARG;
    if (!out_ge || !out_w || !out_n || cap < 1 || hot_windows < 0) return fail(MXK_ERR_BAD_ARG, "scheduler: null output");
    const size_t n_in = (size_t)EPR * group_ranks * 4, n_out = (size_t)group_ranks * cap * 4;
    int *d_in = nullptr, *d_ge = nullptr, *d_w = nullptr, *d_n = nullptr;
    cudaError_t e = cudaMalloc(&d_in, n_in);
    if (e == cudaSuccess) e = cudaMalloc(&d_ge, n_out);
    if (e == cudaSuccess) e = cudaMalloc(&d_w, n_out);
    if (e == cudaSuccess) e = cudaMalloc(&d_n, (size_t)group_ranks * 4);
    if (e == cudaSuccess) e = cudaMemcpy(d_in, rows_of_ge, n_in, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) {
        k_sched_members<<<1, 32>>>(d_in, EPR, group_ranks, win_cap, hot_windows, d_ge, d_w, d_n, cap);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpy(out_ge, d_ge, n_out, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(out_w, d_w, n_out, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(out_n, d_n, (size_t)group_ranks * 4, cudaMemcpyDeviceToHost);
    cudaFree(d_in); cudaFree(d_ge); cudaFree(d_w); cudaFree(d_n);
    return e == cudaSuccess ? 0 : cuda_fail(e, "scheduler on device");
}

int mxk_set_ticks(int on) {
    const int before = ticks_enabled();
    g_ticks_override = on < 0 ? -1 : (on > 2 ? 1 : on);
    return before;
}
int64_t mxk_rwk_ticks_off(void) { return (int64_t)offsetof(DevFlags, ticks); }   // flags_off is 0 in every layout
int64_t mxk_ticks_count(void) { return 16; }

// Window chooser, restated from the reference's cost model with its own
// calibration table (src/win_select.cuh:45-128): argmin over {32,48,64,96,128}
// of waves(win) * t_task(win) with 4 slices per window on a 28-block grid, a
// skew floor of ceil(max/8) and a 96 cap when max*E > 3*sum.
int mxk_select_win(const uint32_t* counts, int E, int cap_hint, int win_min) {
    static const int cand[5] = {32, 48, 64, 96, 128};
    static const long long tq[5] = {10375, 8251, 8904, 10051, 9792};
    uint32_t mx = 0;
    unsigned long long total = 0;
    for (int e = 0; e < E; ++e) { if (counts[e] > mx) mx = counts[e]; total += counts[e]; }
    int floor_w = win_min, cap = cap_hint;
    if (E > 0 && (unsigned long long)mx * E > 3ull * total) {
        const int need = (int)((mx + 7u) / 8u);
        if (need > floor_w) floor_w = need;
        if (floor_w <= 96 && cap > 96) cap = 96;
    }
    int best = -1;
    unsigned long long bc = 0;
    for (int i = 0; i < 5; ++i) {
        if (cand[i] < floor_w || cand[i] > cap) continue;
        unsigned long long W = 0;
        for (int e = 0; e < E; ++e) W += (counts[e] + (uint32_t)cand[i] - 1u) / (uint32_t)cand[i];
        const unsigned long long c = ((W * 4ull + 27ull) / 28ull) * (unsigned long long)tq[i];
        if (best < 0 || c < bc) { best = cand[i]; bc = c; }
    }
    return best < 0 ? cap : best;
}

int mxk_symm_alloc(void** ptr, int64_t bytes) {
    if (!ptr || bytes <= 0) return fail(MXK_ERR_BAD_ARG, "bad symm_alloc arguments");
    cudaError_t e = cudaMalloc(ptr, (size_t)bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc");
    e = cudaMemset(*ptr, 0, (size_t)bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemset");
    e = cudaDeviceSynchronize();
    return e == cudaSuccess ? 0 : cuda_fail(e, "cudaDeviceSynchronize");
}
int mxk_symm_free(void* ptr) {
    cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? 0 : cuda_fail(e, "cudaFree");
}
int mxk_ipc_export(void* ptr, uint8_t handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) return cuda_fail(e, "cudaIpcGetMemHandle");
    std::memcpy(handle, &h, 64);
    return 0;
}
int mxk_ipc_import(const uint8_t handle[64], void** ptr) {
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, 64);
    cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    return e == cudaSuccess ? 0 : cuda_fail(e, "cudaIpcOpenMemHandle");
}
int mxk_ipc_close(void* ptr) {
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? 0 : cuda_fail(e, "cudaIpcCloseMemHandle");
}

}  // extern "C"
