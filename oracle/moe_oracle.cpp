// ============================================================================
// moe_oracle.cpp — CPU restatement of the FP8xFP8 MoE layer (TEST INFRASTRUCTURE).
//
// This file is the checker for the CUDA path, never the product: only tests,
// the smoke entry and the benchmark's cpu_baseline leg may load it.  Every
// function cites the reference file:line whose behaviour it restates.  The
// reference freezes geometry at compile time (src/common.cuh:18-24); here every
// dimension is a run-time argument and the expert weights are addressed in
// their LOGICAL row-major form ([2I][H] gate rows then up rows, [H][I]) instead
// of the reference's MetaX lane-tiled bytes (src/bench_check.cuh:268-272).
//
// Parity status:
//   * reference mode (no scale planes): pinned against the reference's own host
//     functions compiled from its sources (oracle/_ref, see oracle/Makefile) and
//     against golden vectors made by the reference's Python quantisers.
//   * scaled mode (UE8M0 1x128 / 128x128): the reference kernel has no scale
//     path, so the GEMM-with-scales restatement is "parity unpinned"; only its
//     quantisers/dequantisers are pinned (torch/mxmegakernel/utils/math.py).
// ============================================================================
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

#define ORC_API extern "C" __attribute__((visibility("default")))

// ------------------------------------------------------------------ codecs --
// E4M3 (OCP FP8): sign, 4-bit exponent (bias 7), 3-bit mantissa; 0x7F/0xFF NaN,
// no infinity, largest finite 448.  Follows src/bench_check.cuh:326-352.
static float g_e4m3[256];
static struct E4m3Init {
    E4m3Init() {
        for (int i = 0; i < 256; ++i) {
            const int sign = (i >> 7) & 1, ex = (i >> 3) & 0xF, man = i & 7;
            float v;
            if (ex == 0xF && man == 7) v = std::numeric_limits<float>::quiet_NaN();
            else if (ex == 0) v = std::ldexp((float)man / 8.0f, -6);
            else v = std::ldexp(1.0f + (float)man / 8.0f, ex - 7);
            g_e4m3[i] = sign ? -v : v;
        }
    }
} g_e4m3_init;

ORC_API float orc_e4m3_decode(uint8_t b) { return g_e4m3[b]; }

// float -> E4M3, round-to-nearest-even, saturating to +-448, NaN -> 0x7F.
// Follows src/bench_check.cuh:362-380.
ORC_API uint8_t orc_e4m3_quantize(float v) {
    if (std::isnan(v)) return 0x7Fu;
    const uint32_t sign = std::signbit(v) ? 0x80u : 0u;
    const float a = std::fabs(v);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7Eu);
    if (a < 1.0f / 64.0f) {  // subnormal range, step 2^-9
        const int q = (int)std::nearbyint(a * 512.0f);
        return (uint8_t)(sign | (uint32_t)q);
    }
    int e2 = 0;
    const float mant = std::frexp(a, &e2) * 2.0f;  // [1,2)
    int q = (int)std::nearbyint(mant * 8.0f);      // [8,16]
    int enc = (e2 - 1) + 7;
    if (q == 16) { q = 8; ++enc; }
    if (enc > 15) return (uint8_t)(sign | 0x7Eu);
    return (uint8_t)(sign | ((uint32_t)enc << 3) | (uint32_t)(q - 8));
}

// bf16 <-> f32 (src/bench_check.cuh:384-400).
ORC_API float orc_bf16_to_f32(uint16_t h) {
    const uint32_t u = (uint32_t)h << 16;
    float v;
    std::memcpy(&v, &u, 4);
    return v;
}
ORC_API uint16_t orc_f32_to_bf16(float v) {
    uint32_t u;
    std::memcpy(&u, &v, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return (uint16_t)(u >> 16);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

// UE8M0: an unsigned power-of-two scale stored as its biased exponent byte.
// ceil_to_ue8m0 (torch/mxmegakernel/utils/math.py:13-16): exponent field plus
// one when any mantissa bit is set, clamped to [1,254].
ORC_API uint8_t orc_ue8m0_ceil(float x) {
    uint32_t bits;
    const float ax = std::fabs(x);
    std::memcpy(&bits, &ax, 4);
    int ex = (int)((bits >> 23) & 0xFF) + ((bits & 0x7FFFFFu) ? 1 : 0);
    ex = std::min(254, std::max(1, ex));
    return (uint8_t)ex;
}
ORC_API float orc_ue8m0_to_f32(uint8_t e) {
    const uint32_t u = (uint32_t)e << 23;  // unpack_ue8m0_from_int, math.py:140-141
    float v;
    std::memcpy(&v, &u, 4);
    return v;
}

// --------------------------------------------------------------- quantisers --
// per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=128), math.py:26-36:
// amax over each 1x128 group clamped to 1e-4, sf = ceil_pow2(amax/448),
// q = e4m3(x * (1/sf)).  cols must be a multiple of 128 here.
ORC_API void orc_quant_rows_1x128(const float* x, int rows, int cols, uint8_t* q,
                                  uint8_t* sf) {
    const int nb = cols / 128;
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < nb; ++b) {
            const float* p = x + (size_t)r * cols + (size_t)b * 128;
            float amax = 0.0f;
            for (int i = 0; i < 128; ++i) amax = std::max(amax, std::fabs(p[i]));
            amax = std::max(amax, 1e-4f);
            const uint8_t e = orc_ue8m0_ceil(amax / 448.0f);
            const float inv = 1.0f / orc_ue8m0_to_f32(e);
            sf[(size_t)r * nb + b] = e;
            for (int i = 0; i < 128; ++i)
                q[(size_t)r * cols + (size_t)b * 128 + i] = orc_e4m3_quantize(p[i] * inv);
        }
}

// per_block_cast_to_fp8(w, use_ue8m0=True, gran_k=128), math.py:62-72:
// one scale per 128x128 block.  rows and cols must be multiples of 128 here.
ORC_API void orc_quant_blocks_128x128(const float* w, int rows, int cols,
                                      uint8_t* q, uint8_t* sf) {
    const int rb = rows / 128, cb = cols / 128;
    for (int br = 0; br < rb; ++br)
        for (int bc = 0; bc < cb; ++bc) {
            float amax = 0.0f;
            for (int i = 0; i < 128; ++i)
                for (int j = 0; j < 128; ++j)
                    amax = std::max(amax, std::fabs(w[(size_t)(br * 128 + i) * cols + bc * 128 + j]));
            amax = std::max(amax, 1e-4f);
            const uint8_t e = orc_ue8m0_ceil(amax / 448.0f);
            const float inv = 1.0f / orc_ue8m0_to_f32(e);
            sf[(size_t)br * cb + bc] = e;
            for (int i = 0; i < 128; ++i)
                for (int j = 0; j < 128; ++j) {
                    const size_t o = (size_t)(br * 128 + i) * cols + bc * 128 + j;
                    q[o] = orc_e4m3_quantize(w[o] * inv);
                }
        }
}

// cast_back_from_fp8 (math.py:167-173): q * sf[group].
ORC_API void orc_dequant_rows_1x128(const uint8_t* q, const uint8_t* sf, int rows,
                                    int cols, float* out) {
    const int nb = cols / 128;
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c)
            out[(size_t)r * cols + c] =
                g_e4m3[q[(size_t)r * cols + c]] *
                (sf ? orc_ue8m0_to_f32(sf[(size_t)r * nb + c / 128]) : 1.0f);
}

// ----------------------------------------------------------------- routing --
// Whole-world model of the prologue, one call for all R ranks.
//   topk_idx [R][t_stride][topk] int64; tokens[r] valid rows on rank r.
// Outputs (all caller-zeroed):
//   route_slot_counts [R][E]                    src/prologue.cuh:221-224
//   src_index_table   [R owner][EPR][R src][slot_cap]   src/prologue.cuh:164-180
//   recv_counts       [R owner][R src][recv_stride]; word EPR of each row holds
//                     ~(sum + epoch)             src/prologue.cuh:241-255
//   prefix_tbl        [R owner][EPR][R+1]        src/prologue.cuh:423-432
// Slot order: ascending pair index idx = token*topk + k.  The reference assigns
// slots with a shared-memory atomicAdd, so any permutation is legal there
// (src/bench_check.cuh:109-131); ascending order is the deterministic member of
// that set and is what the CUDA path emits.
ORC_API void orc_route(const int64_t* topk_idx, const int* tokens, int R, int EPR,
                       int topk, int t_stride, int slot_cap, int recv_stride,
                       uint32_t epoch, int32_t* route_slot_counts,
                       uint32_t* src_index_table, uint32_t* recv_counts,
                       int32_t* prefix_tbl) {
    const int E = R * EPR;
    for (int src = 0; src < R; ++src) {
        std::vector<int> slots(E, 0);
        const int64_t* ti = topk_idx + (size_t)src * t_stride * topk;
        const int np = tokens[src] * topk;
        for (int idx = 0; idx < np; ++idx) {
            const int64_t raw = ti[idx];
            if ((uint64_t)raw >= (uint64_t)E) continue;  // invalid ids skipped (:166-167)
            const int e = (int)raw;
            const int slot = slots[e]++;
            if (slot >= slot_cap) continue;  // over capacity: dropped (:171-174)
            const int dst = e / EPR, le = e % EPR;
            src_index_table[(((size_t)dst * EPR + le) * R + src) * slot_cap + slot] = (uint32_t)idx;
        }
        for (int e = 0; e < E; ++e) {
            const int c = std::min(slots[e], slot_cap);
            route_slot_counts[(size_t)src * E + e] = c;
            recv_counts[((size_t)(e / EPR) * R + src) * recv_stride + (e % EPR)] = (uint32_t)c;
        }
        for (int d = 0; d < R; ++d) {
            uint32_t csum = 0;
            for (int le = 0; le < EPR; ++le)
                csum += (uint32_t)route_slot_counts[(size_t)src * E + d * EPR + le];
            recv_counts[((size_t)d * R + src) * recv_stride + EPR] = ~(csum + epoch);
        }
    }
    for (int owner = 0; owner < R; ++owner)
        for (int le = 0; le < EPR; ++le) {
            int c = 0;
            int32_t* row = prefix_tbl + ((size_t)owner * EPR + le) * (R + 1);
            for (int r = 0; r < R; ++r) {
                row[r] = c;
                c += (int)recv_counts[((size_t)owner * R + r) * recv_stride + le];
            }
            row[R] = c;
        }
}

// Pool row -> source mapping on one owner rank (src/compute_big.cuh:1760-1769,
// staged meta :1833-1840).  Rows of local expert le occupy
// [row_base[le], row_base[le+1]) in le order; row g of the expert comes from
// src = max{r : prefix[le][r] <= g}, slot = g - prefix[le][src],
// idx = table[le][src][slot], token = idx / topk, k = idx % topk.
// meta [rows][3] = (src, token, k).  Returns the total row count.
ORC_API int orc_pool_map(const int32_t* prefix_tbl, const uint32_t* src_tbl, int R,
                         int EPR, int topk, int slot_cap, int32_t* row_base,
                         int32_t* meta) {
    int base = 0;
    for (int le = 0; le < EPR; ++le) {
        const int32_t* pf = prefix_tbl + (size_t)le * (R + 1);
        row_base[le] = base;
        for (int g = 0; g < pf[R]; ++g) {
            int src = 0;
            while (src + 1 < R && pf[src + 1] <= g) ++src;
            const int slot = g - pf[src];
            const uint32_t idx = src_tbl[((size_t)le * R + src) * slot_cap + slot];
            int32_t* m = meta + (size_t)(base + g) * 3;
            m[0] = src;
            m[1] = (int)(idx / (uint32_t)topk);
            m[2] = (int)(idx % (uint32_t)topk);
        }
        base += pf[R];
    }
    row_base[EPR] = base;
    return base;
}

// ---------------------------------------------------------------- scheduler --
// Tile scheduler of the CUDA path (no counterpart with this exact shape in the
// reference; it plays the role of the (expert, window, slice) enumeration of
// src/compute.cuh:896-903,1120-1133 with the cost ordering of R19_BLOCK_LPT,
// src/compute.cuh:932-983).  Experts are visited by descending row count,
// ties by ascending index; each expert is cut in windows of win_cap rows.
// L1 tasks come first, then L2 tasks, each ordered (expert, n-tile, window).
//   tasks[n][4] = (kind 0|1, window id, n-tile, rows in window)
//   windows[w][3] = (local expert, first pool row, rows)
// Returns the task count; *n_windows and *n_l1 are filled.
ORC_API int orc_schedule(const int32_t* expert_rows, const int32_t* row_base,
                         int EPR, int win_cap, int nt1, int nt2, int32_t* windows,
                         int32_t* tasks, int* n_windows, int* n_l1) {
    std::vector<int> order(EPR);
    for (int i = 0; i < EPR; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(),
                     [&](int a, int b) { return expert_rows[a] > expert_rows[b]; });
    int nw = 0;
    std::vector<int> first_win(EPR), num_win(EPR);
    for (int p = 0; p < EPR; ++p) {
        const int e = order[p], c = expert_rows[e];
        first_win[p] = nw;
        num_win[p] = c > 0 ? (c + win_cap - 1) / win_cap : 0;
        for (int w = 0; w < num_win[p]; ++w) {
            windows[(size_t)nw * 3 + 0] = e;
            windows[(size_t)nw * 3 + 1] = row_base[e] + w * win_cap;
            windows[(size_t)nw * 3 + 2] = std::min(win_cap, c - w * win_cap);
            ++nw;
        }
    }
    int n = 0;
    for (int kind = 0; kind < 2; ++kind) {
        const int nt = kind == 0 ? nt1 : nt2;
        for (int p = 0; p < EPR; ++p)
            for (int t = 0; t < nt; ++t)
                for (int w = 0; w < num_win[p]; ++w) {
                    const int wid = first_win[p] + w;
                    tasks[(size_t)n * 4 + 0] = kind;
                    tasks[(size_t)n * 4 + 1] = wid;
                    tasks[(size_t)n * 4 + 2] = t;
                    tasks[(size_t)n * 4 + 3] = windows[(size_t)wid * 3 + 2];
                    ++n;
                }
        if (kind == 0) *n_l1 = n;
    }
    *n_windows = nw;
    return n;
}

// Cross-rank window LPT of src/group_sched.cuh:164-205 with run-time EPR and
// group size (the reference fixes kEPR=8, kGroupRanks=4).  cg[ge] = rows of
// group expert ge = member*EPR + le; cost = ceil(rows/16) (:34-41); windows are
// visited by descending cost, then (ge, w) ascending; the least-loaded member
// takes the window, a tie going to the owner first, then the lowest member.
ORC_API int orc_gs_schedule_member(const int* cg, int EPR, int group_ranks,
                                   int win_cap, int member, int* out_ge,
                                   int* out_w, int cap) {
    std::vector<long long> load(group_ranks, 0);
    const int GE = EPR * group_ranks;
    const int maxcost = (win_cap + 15) / 16;
    int nout = 0;
    for (int cost = maxcost; cost >= 1; --cost)
        for (int ge = 0; ge < GE; ++ge) {
            const int c = cg[ge];
            const int nw = c > 0 ? (c + win_cap - 1) / win_cap : 0;
            for (int w = 0; w < nw; ++w) {
                int rows = std::max(0, std::min(win_cap, c - w * win_cap));
                if ((rows + 15) / 16 != cost) continue;
                const int owner = ge / EPR;
                long long minl = load[0];
                for (int m = 1; m < group_ranks; ++m) minl = std::min(minl, load[m]);
                int chosen = owner;
                if (load[owner] != minl) {
                    chosen = 0;
                    for (int m = 0; m < group_ranks; ++m)
                        if (load[m] == minl) { chosen = m; break; }
                }
                load[chosen] += cost;
                if (chosen == member) {
                    if (nout < cap) { out_ge[nout] = ge; out_w[nout] = w; }
                    ++nout;
                }
            }
        }
    return nout;
}

// The same schedule with the spreading limited to hot experts (not in the reference; what the
// CUDA path runs by default): an expert with fewer than hot_windows windows stays with its
// owner, its cost counted into the owner's load before the first window is placed.
ORC_API int orc_gs_schedule_member_hot(const int* cg, int EPR, int group_ranks, int win_cap, int member,
                                       int hot_windows, int* out_ge, int* out_w, int cap) {
    std::vector<long long> load(group_ranks, 0);
    const int GE = EPR * group_ranks;
    const int maxcost = (win_cap + 15) / 16;
    auto n_windows = [&](int c) { return c > 0 ? (c + win_cap - 1) / win_cap : 0; };
    auto hot = [&](int c) { return hot_windows <= 0 || n_windows(c) >= hot_windows; };
    for (int ge = 0; ge < GE; ++ge)
        if (!hot(cg[ge]))
            for (int w = 0; w < n_windows(cg[ge]); ++w)
                load[ge / EPR] += (std::min(win_cap, cg[ge] - w * win_cap) + 15) / 16;
    int nout = 0;
    for (int cost = maxcost; cost >= 1; --cost)
        for (int ge = 0; ge < GE; ++ge) {
            const int c = cg[ge];
            for (int w = 0; w < n_windows(c); ++w) {
                const int rows = std::min(win_cap, c - w * win_cap);
                if ((rows + 15) / 16 != cost) continue;
                const int owner = ge / EPR;
                int chosen = owner;
                if (hot(c)) {
                    long long minl = load[0];
                    for (int m = 1; m < group_ranks; ++m) minl = std::min(minl, load[m]);
                    if (load[owner] != minl)
                        for (int m = 0; m < group_ranks; ++m)
                            if (load[m] == minl) { chosen = m; break; }
                    load[chosen] += cost;
                }
                if (chosen == member) {
                    if (nout < cap) { out_ge[nout] = ge; out_w[nout] = w; }
                    ++nout;
                }
            }
        }
    return nout;
}

// LPT over (expert, window, slice) tasks of src/balance_partition.cuh:62-115:
// cost = rows of the window, stable descending sort, each task to the member
// with the strictly smallest load (ties to the lowest member).  experts[] lists
// the group's global expert ids.  member_of[i] refers to the sorted order;
// sorted_tasks [n][3] = (e, w, slice).
ORC_API int orc_lpt_assign(const int* counts, const int* experts, int n_experts,
                           int win_cap, int nslice, int nmembers, int* sorted_tasks,
                           int* member_of, long long* load) {
    struct T { int e, w, s; long long cost; };
    std::vector<T> t;
    for (int i = 0; i < n_experts; ++i) {
        const int e = experts[i], c = counts[e];
        const int nw = c > 0 ? (c + win_cap - 1) / win_cap : 0;
        for (int w = 0; w < nw; ++w) {
            const int rows = std::max(0, std::min(win_cap, c - w * win_cap));
            for (int s = 0; s < nslice; ++s) t.push_back({e, w, s, rows});
        }
    }
    std::stable_sort(t.begin(), t.end(), [](const T& a, const T& b) { return a.cost > b.cost; });
    for (int m = 0; m < nmembers; ++m) load[m] = 0;
    for (size_t i = 0; i < t.size(); ++i) {
        int best = 0;
        for (int m = 1; m < nmembers; ++m)
            if (load[m] < load[best]) best = m;
        member_of[i] = best;
        load[best] += t[i].cost;
        sorted_tasks[i * 3 + 0] = t[i].e;
        sorted_tasks[i * 3 + 1] = t[i].w;
        sorted_tasks[i * 3 + 2] = t[i].s;
    }
    return (int)t.size();
}

// Window chooser of src/win_select.cuh:62-128 with the slice count, grid size
// and ring depth as arguments (reference: 4, 28, 8) and the reference's own
// calibration table (Q8 fixed point, :52-58).
static const int kWinCand[5] = {32, 48, 64, 96, 128};
static const long long kWinTq[5] = {10375, 8251, 8904, 10051, 9792};
static unsigned long long win_cost(const uint32_t* counts, int E, int win, int nslice, int grid) {
    unsigned long long W = 0;
    for (int e = 0; e < E; ++e) W += (counts[e] + (uint32_t)win - 1u) / (uint32_t)win;
    const unsigned long long waves = (W * (unsigned long long)nslice + grid - 1) / grid;
    long long tq = kWinTq[4];
    for (int i = 0; i < 5; ++i)
        if (kWinCand[i] == win) tq = kWinTq[i];
    return waves * (unsigned long long)tq;
}
ORC_API int orc_select_win(const uint32_t* counts, int E, int cap_hint, int win_min,
                           int nslice, int grid, int ring) {
    uint32_t mx = 0;
    unsigned long long total = 0;
    for (int e = 0; e < E; ++e) { mx = std::max(mx, counts[e]); total += counts[e]; }
    int floor_w = win_min, cap = cap_hint;
    const bool skewed = E > 0 && (unsigned long long)mx * E > 3ull * total;
    if (skewed) {
        const int need = (int)((mx + (unsigned)ring - 1) / (unsigned)ring);
        floor_w = std::max(floor_w, need);
        if (floor_w <= 96 && cap > 96) cap = 96;
    }
    int best = -1;
    unsigned long long bc = 0;
    for (int i = 0; i < 5; ++i) {
        const int w = kWinCand[i];
        if (w < floor_w || w > cap) continue;
        const unsigned long long c = win_cost(counts, E, w, nslice, grid);
        if (best < 0 || c < bc) { best = w; bc = c; }
    }
    return best < 0 ? cap : best;
}

// Test-data generator WPROBE_VAL (src/megakernel.h:46-47): byte at logical
// (row, k) of a weight tensor = (seed + 131*row + 7*k) & 0x3f.  Row-major output
// (the reference packs the same bytes in lane order, src/megakernel.cu:66-105).
ORC_API void orc_fill_weights(uint8_t* w, long long n_rows, int k_cols, uint32_t seed) {
    for (long long r = 0; r < n_rows; ++r)
        for (int k = 0; k < k_cols; ++k)
            w[(size_t)r * k_cols + k] = (uint8_t)((seed + (uint32_t)r * 131u + (uint32_t)k * 7u) & 0x3f);
}

// 4-bit weights (the reference's MX_FP4_W build).  A code is sign(1) exponent(2, bias 1)
// mantissa(1); the kernel multiplies with the E4M3 byte of the same value
// (fp4_code_to_fp8, src/common.cuh:116-126): exponent 0 -> 0 or 0.5, else
// 2^(e-1) * (1 + m/2), i.e. E4M3 exponent field e - 1 + 7 and mantissa m << 2.
ORC_API uint8_t orc_e2m1_to_e4m3(uint8_t c) {
    const uint8_t sign = (c & 8u) ? 0x80u : 0u;
    const unsigned e = (c >> 1) & 3u, m = c & 1u;
    const uint8_t mag = e == 0 ? (m ? 0x30u : 0x00u) : (uint8_t)(((e - 1u + 7u) << 3) | (m ? 4u : 0u));
    return (uint8_t)(sign | mag);
}
// Packed codes [n_rows][k_cols / 2] (element of even k in the low nibble) -> E4M3 bytes
// [n_rows][k_cols]: what the CPU reference reads through w_lane_get in that build
// (src/bench_check.cuh:405-421; row-major here instead of the MetaX lane order).
ORC_API void orc_expand_e2m1(const uint8_t* packed, long long n_rows, int k_cols, uint8_t* out) {
    for (long long r = 0; r < n_rows; ++r)
        for (int k = 0; k < k_cols; ++k) {
            const uint8_t b = packed[(size_t)r * (k_cols / 2) + k / 2];
            out[(size_t)r * k_cols + k] = orc_e2m1_to_e4m3((uint8_t)((b >> (4 * (k & 1))) & 0xfu));
        }
}
// Test-data generator WPROBE_FP4_CODE (src/common.cuh:127-131): code at logical (row, k) =
// ((seed + 131*row + 7*k) >> 1) & 0xf, packed two per byte.
ORC_API void orc_fill_weights_e2m1(uint8_t* w, long long n_rows, int k_cols, uint32_t seed) {
    for (long long r = 0; r < n_rows; ++r)
        for (int k = 0; k < k_cols; k += 2) {
            const uint32_t lo = ((seed + (uint32_t)r * 131u + (uint32_t)k * 7u) >> 1) & 0xfu;
            const uint32_t hi = ((seed + (uint32_t)r * 131u + (uint32_t)(k + 1) * 7u) >> 1) & 0xfu;
            w[(size_t)r * (k_cols / 2) + k / 2] = (uint8_t)(lo | (hi << 4));
        }
}

// ------------------------------------------------------------------ numerics --
template <class F>
static void parallel_rows(int rows, int threads, F fn) {  // test/check.cu:155-165
    threads = std::max(1, std::min(threads, rows));
    if (threads == 1) { for (int r = 0; r < rows; ++r) fn(r); return; }
    std::vector<std::thread> th;
    for (int t = 0; t < threads; ++t)
        th.emplace_back([=] { for (int r = t; r < rows; r += threads) fn(r); });
    for (auto& x : th) x.join();
}

// One dot product, FP32.  Unscaled: strictly sequential over K as the reference
// (src/bench_check.cuh:446-451).  Scaled: sequential inside each 128-wide K
// block, the block sum multiplied by (sa*sb) (both exact powers of two) and
// added to the running total.  The CUDA path applies the same scales inside the
// block-scaled tensor-core MMA, whose summation order inside a K block is not
// specified: the comparison tolerance of the parity tests covers the difference.
static inline float dot_fp8(const float* a, const uint8_t* a_sf, const uint8_t* w,
                            const uint8_t* w_sf, int K) {
    if (!a_sf && !w_sf) {
        float acc = 0.0f;
        for (int k = 0; k < K; ++k) acc += a[k] * g_e4m3[w[k]];
        return acc;
    }
    float acc = 0.0f;
    for (int kb = 0; kb < K / 128; ++kb) {
        float part = 0.0f;
        for (int k = kb * 128; k < kb * 128 + 128; ++k) part += a[k] * g_e4m3[w[k]];
        const float s = (a_sf ? orc_ue8m0_to_f32(a_sf[kb]) : 1.0f) *
                        (w_sf ? orc_ue8m0_to_f32(w_sf[kb]) : 1.0f);
        acc += part * s;
    }
    return acc;
}

// L1: h[r][c] = silu(gate)*up with gate = x . W1[c], up = x . W1[I + c]
// (src/bench_check.cuh:435-455; SiLU as g/(1+exp(-g)), :452 and
// src/compute.cuh:242-244).  x [rows][H] E4M3 bytes (+ optional [rows][H/128]
// scales); w1 [2I][H] bytes of ONE expert (+ optional [2I/128][H/128] scales).
ORC_API void orc_l1(const uint8_t* x, const uint8_t* x_sf, const uint8_t* w1,
                    const uint8_t* w1_sf, int rows, int H, int I, float* h_out,
                    int threads) {
    const int kb = H / 128;
    parallel_rows(rows, threads, [=](int r) {
        std::vector<float> xd(H);
        for (int k = 0; k < H; ++k) xd[k] = g_e4m3[x[(size_t)r * H + k]];
        const uint8_t* xs = x_sf ? x_sf + (size_t)r * kb : nullptr;
        for (int c = 0; c < I; ++c) {
            const float g = dot_fp8(xd.data(), xs, w1 + (size_t)c * H,
                                    w1_sf ? w1_sf + (size_t)(c / 128) * kb : nullptr, H);
            const float u = dot_fp8(xd.data(), xs, w1 + (size_t)(I + c) * H,
                                    w1_sf ? w1_sf + (size_t)((I + c) / 128) * kb : nullptr, H);
            h_out[(size_t)r * I + c] = (g / (1.0f + std::exp(-g))) * u;
        }
    });
}

// Re-quantisation of the L1 output.  Unscaled: saturating RNE cast of the raw
// value (ref_quantize_fp8, src/bench_check.cuh:502-505; torch test clamps to
// +-448 first, torch/tests/test_fp8_mega_moe.py:43).  Scaled: per-row 1x128
// UE8M0 as per_token_cast_to_fp8.
ORC_API void orc_requant(const float* h, int rows, int I, int scaled, uint8_t* q,
                         uint8_t* sf) {
    if (scaled) { orc_quant_rows_1x128(h, rows, I, q, sf); return; }
    for (long long i = 0; i < (long long)rows * I; ++i) q[i] = orc_e4m3_quantize(h[i]);
}

// L2: out[r][n] = a[r] . W2[n] in FP32 (src/bench_check.cuh:461-476).
ORC_API void orc_l2(const uint8_t* a, const uint8_t* a_sf, const uint8_t* w2,
                    const uint8_t* w2_sf, int rows, int I, int H, float* out,
                    int threads) {
    const int kb = I / 128;
    parallel_rows(rows, threads, [=](int r) {
        std::vector<float> ad(I);
        for (int k = 0; k < I; ++k) ad[k] = g_e4m3[a[(size_t)r * I + k]];
        const uint8_t* as = a_sf ? a_sf + (size_t)r * kb : nullptr;
        for (int n = 0; n < H; ++n)
            out[(size_t)r * H + n] =
                dot_fp8(ad.data(), as, w2 + (size_t)n * I,
                        w2_sf ? w2_sf + (size_t)(n / 128) * kb : nullptr, I);
    });
}

// REDUCE for one token (src/bench_check.cuh:484-499): k ascending, FP32,
// product then sum (two roundings), invalid expert ids skipped.
ORC_API void orc_reduce(const uint16_t* combine_rows, const int64_t* topk_idx,
                        const float* weights, int token, int topk, int E,
                        int combine_cap, int H, float* y) {
    for (int c = 0; c < H; ++c) y[c] = 0.0f;
    if (token < 0 || token >= combine_cap) return;
    for (int k = 0; k < topk; ++k) {
        const int64_t e = topk_idx[(size_t)token * topk + k];
        if (e < 0 || e >= (int64_t)E) continue;
        const float wv = weights[(size_t)token * topk + k];
        const uint16_t* row = combine_rows + ((size_t)k * combine_cap + token) * H;
        for (int c = 0; c < H; ++c) {
            const volatile float prod = orc_bf16_to_f32(row[c]) * wv;  // no FMA contraction
            y[c] += prod;
        }
    }
}

// Row-parallel wrapper used by tests and the CPU baseline: all tokens of a rank.
ORC_API void orc_reduce_all(const uint16_t* combine_rows, const int64_t* topk_idx,
                            const float* weights, int tokens, int topk, int E,
                            int combine_cap, int H, float* y, int threads) {
    parallel_rows(tokens, threads, [=](int t) {
        orc_reduce(combine_rows, topk_idx, weights, t, topk, E, combine_cap, H,
                   y + (size_t)t * H);
    });
}

ORC_API void orc_f32_to_bf16_n(const float* in, long long n, uint16_t* out) {
    for (long long i = 0; i < n; ++i) out[i] = orc_f32_to_bf16(in[i]);
}
ORC_API void orc_e4m3_decode_n(const uint8_t* in, long long n, float* out) {
    for (long long i = 0; i < n; ++i) out[i] = g_e4m3[in[i]];
}
ORC_API void orc_e4m3_quantize_n(const float* in, long long n, uint8_t* out) {
    for (long long i = 0; i < n; ++i) out[i] = orc_e4m3_quantize(in[i]);
}
