// ============================================================================
// ref_shim.cpp — C entry points over the REFERENCE's own host-side pure
// functions (TEST INFRASTRUCTURE, never shipped, never on the product path).
//
// oracle/Makefile compiles this file against the reference sources where they
// lie (-I <reference>/src); nothing of the reference is copied into this
// repository.  The two sections of src/bench_check.cuh that are declared
// self-contained there (route model :30-69, numeric reference :326-625) are
// extracted at build time into the git-ignored output folder because the top of
// that header includes the MetaX runtime.  The result, oracle/_ref/libmoe_ref.so,
// is used to pin oracle/moe_oracle.cpp and as the "reference" CPU baseline.
// ============================================================================
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"             // reference: scene constants, MT_WSTRIDE, kBTileBytes
#include "flags_defs.cuh"         // reference: kGroupRanks / kGE
#include "group_sched.cuh"        // reference: gs_schedule_member
#include "win_select.cuh"         // reference: select_win
#include "balance_partition.cuh"  // reference: lpt_assign
#include "bench_check_routes.inc"   // reference src/bench_check.cuh:30-69
#include "bench_check_numeric.inc"  // reference src/bench_check.cuh:326-625

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API int ref_const(int which) {
    switch (which) {
        case 0: return kEPR;
        case 1: return kTopk;
        case 2: return kHidden;
        case 3: return kIntermediate;
        case 4: return kGroupRanks;
        case 5: return kGE;
        case 6: return mxk::kWinGrid;
        case 7: return mxk::kWinNSlice;
        case 8: return mxk::kWinRing;
        case 9: return kMaxTPR;
    }
    return -1;
}

REF_API float ref_e4m3_decode(uint8_t b) { return fp8_e4m3_decode(b); }
REF_API uint8_t ref_e4m3_quantize(float v) { return fp8_e4m3_quantize(v); }
REF_API float ref_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
REF_API uint16_t ref_f32_to_bf16(float v) { return f32_to_bf16_rne(v); }

// Byte at logical (row, k) of one expert's lane-tiled weight block.
REF_API uint8_t ref_w_lane_get(const uint8_t* w_e, int row, int k, int k_cols) {
    return w_lane_get(w_e, row, k, k_cols);
}

// Pack a logical row-major [n_rows][k_cols] matrix into the reference's lane
// order by inverting its own accessor (so the packing is defined by the
// reference, not by this shim).
REF_API void ref_pack_lane(const uint8_t* logical, int n_rows, int k_cols, uint8_t* packed) {
    const int k_iters = k_cols / 32;
    for (int row = 0; row < n_rows; ++row)
        for (int k = 0; k < k_cols; ++k) {
            const size_t tile = ((size_t)(row >> 5) * k_iters + (size_t)(k >> 5)) * kBTileBytes;
            const int lane = (row & 15) + (((k & 31) >> 3) << 4);
            const int sub = (row >> 4) & 1;
            packed[tile + (size_t)lane * 16 + (size_t)sub * 8 + (size_t)(k & 7)] =
                logical[(size_t)row * k_cols + k];
        }
}

template <class F>
static void par_rows(int rows, int threads, F fn) {
    threads = std::max(1, std::min(threads, rows));
    std::vector<std::thread> th;
    for (int t = 0; t < threads; ++t)
        th.emplace_back([=] { for (int r = t; r < rows; r += threads) fn(r); });
    for (auto& x : th) x.join();
}

// ref_l1 / ref_l2 / ref_reduce driven row-parallel the way test/check.cu:155-165 does.
REF_API void ref_l1_rows(const uint8_t* x, const uint8_t* w1_lane, int expert, int count,
                         float* ffn_expect, int threads) {
    par_rows(count, threads, [=](int r) {
        ref_l1(x + (size_t)r * kHidden, w1_lane, expert, 1, kHidden, kIntermediate,
               ffn_expect + (size_t)r * kIntermediate);
    });
}
REF_API void ref_l2_rows(const uint8_t* ffn, const uint8_t* w2_lane, int expert, int count,
                         float* out_expect, int threads) {
    par_rows(count, threads, [=](int r) {
        ref_l2(ffn + (size_t)r * kIntermediate, w2_lane, expert, 1, kIntermediate, kHidden,
               out_expect + (size_t)r * kHidden);
    });
}
REF_API void ref_reduce_tokens(const uint8_t* combine_rows, const int64_t* topk_idx,
                               const float* weights, int tokens, int E, int combine_cap,
                               float* y, int threads) {
    par_rows(tokens, threads, [=](int t) {
        ref_reduce(combine_rows, topk_idx, weights, t, kTopk, E, combine_cap, kHidden,
                   y + (size_t)t * kHidden);
    });
}
REF_API void ref_quantize(const float* expect, long long n, uint8_t* out) {
    ref_quantize_fp8(expect, n, out);
}

REF_API void ref_make_routes(int pattern, int rank, int R, int tokens, int salt, int64_t* out) {
    const auto v = make_routes((RoutePattern)pattern, rank, R, tokens, salt);
    std::memcpy(out, v.data(), v.size() * sizeof(int64_t));
}

REF_API int ref_gs_schedule_member(const int* cg, int win_cap, int member, int* out_ge,
                                   int* out_w, int cap) {
    return mxk::gs_schedule_member(cg, win_cap, member, out_ge, out_w, cap);
}
REF_API int ref_select_win(const uint32_t* counts, int E, int cap_hint, int win_min) {
    return mxk::select_win(counts, E, cap_hint, win_min);
}
// enumerate_group_tasks + lpt_assign for one group; sorted_tasks [n][3].
REF_API int ref_lpt_assign(const int* counts, int win_cap, int nslice, int group, int nmembers,
                           int* sorted_tasks, int* member_of, long long* load) {
    std::vector<mxk::BpTask> t(mxk::kBpExpertsPerGroup * 64 * std::max(1, nslice));
    int nt = 0;
    mxk::enumerate_group_tasks(counts, win_cap, nslice, group, t.data(), &nt);
    mxk::lpt_assign(t.data(), nt, nmembers, member_of, load);
    for (int i = 0; i < nt; ++i) {
        sorted_tasks[i * 3 + 0] = t[i].e;
        sorted_tasks[i * 3 + 1] = t[i].w;
        sorted_tasks[i * 3 + 2] = t[i].slice;
    }
    return nt;
}
