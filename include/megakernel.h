// ============================================================================
// megakernel.h — C++ host interface of the FP8xFP8 MoE layer, drop-in for the
// reference's src/megakernel.h (namespace fp8mega): same struct, same field
// names, same free functions, forwarding to the C ABI of mxk_b200.h.
//
//   #include "megakernel.h"          // link libmxk_b200.so
//   fp8mega::MegaLaunchArgs a{};     // fill as before (+ the new trailing fields)
//   fp8mega::launch_full(a, stream); // route/setup/dispatch/GEMM + reduce
//
// Differences a caller sees:
//   * mcStream_t is cudaStream_t;
//   * rwk / unk are opaque blocks whose sizes and table offsets come from
//     mxk_compute_layout() (the reference exposes fixed-size structs
//     rwk_data / unk_data, src/flags_defs.cuh:171-222);
//   * geometry (experts_per_rank, topk, hidden, intermediate, max_tokens) and
//     the UE8M0 scale planes are new trailing fields; left at zero / null they
//     select the reference's frozen scene (EPR=8, topk=8, H=6144, I=2048) and
//     its scale-free arithmetic;
//   * w1 / w2 are plain row-major E4M3 ([EPR][2I][H] gate rows then up rows,
//     [EPR][H][I]), not MetaX lane-tiled bytes;
//   * the launchers still return void like the reference's; a failed launch is
//     reported through fp8mega::last_status() / mxk_last_error().
// ============================================================================
#pragma once

#include <cstdint>

#include <cuda_runtime.h>

#include "mxk_b200.h"

struct rwk_data;  // opaque: layout given by MxkLayout
struct unk_data;

// Test-weight value function shared by host reference and device generator
// (reference: src/megakernel.h:46-47).
#define WPROBE_VAL(seed, row, k) ((uint8_t)(((seed) + (row) * 131 + (k) * 7) & 0x3f))

namespace fp8mega {

using mcStream_t = cudaStream_t;

// Field order and names of the reference's MegaLaunchArgs (src/megakernel.h:54-114),
// followed by the additions.
struct MegaLaunchArgs {
    int R = 0, rank = 0;
    int tokens = 0;
    int slot_capacity = 0;
    int win_cap = 0;
    int grid = 0, threads = 0;
    int64_t smem = 0;
    rwk_data* rwk = nullptr;
    unk_data* unk = nullptr;
    unk_data* const* unk_peers = nullptr;
    const uint8_t* self = nullptr;
    uint8_t* const* peer_bases = nullptr;
    const int64_t* topk_idx = nullptr;
    const uint8_t* w1 = nullptr;
    const uint8_t* w2 = nullptr;
    int group_weights_ready = 0;
    int64_t topk_idx_off = 0;
    int64_t x_off = 0, weights_off = 0;
    int in_bf16 = 0;
    int skip_combine = 0;
    float* y = nullptr;
    int max_spins = 0;
    int skip_prologue = 0;
    // ---- additions (zero / null == reference behaviour) ----
    int experts_per_rank = 0, topk = 0, hidden = 0, intermediate = 0, max_tokens = 0;
    int64_t x_sf_off = 0;
    const uint8_t* w1_sf = nullptr;
    const uint8_t* w2_sf = nullptr;
    uint16_t* y_bf16 = nullptr;
    int cta_pair = 0;   // 0 = choose by load, 1 = single CTAs, 2 = CTA pairs (256-row windows)
    int dispatch_mode = 0;   // prologue protocol, the same on every rank: 0 = by geometry, 1 = pull, 2 = push
    // cross-rank helper scheduling (reference: MX_GROUP_SCHED with rwk->ld.w1g / w2g): group size, skew
    // threshold (0 = the reference's 2, negative = always) and the group-replicated weights
    int group_ranks = 0, group_skew_num = 0;
    const uint8_t* w1_group = nullptr;
    const uint8_t* w2_group = nullptr;
    const uint8_t* w1_sf_group = nullptr;
    const uint8_t* w2_sf_group = nullptr;
    // 4-bit weights (reference: the MX_FP4_W build, src/common.cuh:99-134): MXK_WEIGHTS_E2M1 = every weight
    // tensor holds e2m1 codes, two per byte, row-major [experts][rows][k / 2]
    int weight_format = 0;
    // helper groups: experts with fewer windows than this stay with their owners (0 = 3, negative = the reference's
    // schedule, every window may move)
    int group_hot_windows = 0;
};

inline int& last_status() {
    static thread_local int s = 0;
    return s;
}

inline MxkLaunchArgs to_c(const MegaLaunchArgs& a) {
    MxkLaunchArgs c{};
    c.R = a.R; c.rank = a.rank; c.tokens = a.tokens; c.slot_capacity = a.slot_capacity; c.win_cap = a.win_cap;
    c.grid = a.grid; c.threads = a.threads; c.smem = a.smem;
    c.rwk = a.rwk; c.unk = a.unk;
    c.unk_peers = reinterpret_cast<void* const*>(a.unk_peers);
    c.self = a.self; c.peer_bases = a.peer_bases; c.topk_idx = a.topk_idx;
    c.w1 = a.w1; c.w2 = a.w2; c.group_weights_ready = a.group_weights_ready;
    c.topk_idx_off = a.topk_idx_off; c.x_off = a.x_off; c.weights_off = a.weights_off;
    c.in_bf16 = a.in_bf16; c.skip_combine = a.skip_combine; c.y = a.y;
    c.max_spins = a.max_spins; c.skip_prologue = a.skip_prologue;
    c.experts_per_rank = a.experts_per_rank; c.topk = a.topk; c.hidden = a.hidden;
    c.intermediate = a.intermediate; c.max_tokens = a.max_tokens;
    c.x_sf_off = a.x_sf_off; c.w1_sf = a.w1_sf; c.w2_sf = a.w2_sf; c.y_bf16 = a.y_bf16; c.cta_pair = a.cta_pair; c.dispatch_mode = a.dispatch_mode;
    c.group_ranks = a.group_ranks; c.group_skew_num = a.group_skew_num;
    c.w1_group = a.w1_group; c.w2_group = a.w2_group; c.w1_sf_group = a.w1_sf_group; c.w2_sf_group = a.w2_sf_group;
    c.weight_format = a.weight_format; c.group_hot_windows = a.group_hot_windows;
    return c;
}

// Prologue only (reference: launch_prelude, src/megakernel.cu:203-220).
inline void launch_prelude(const MegaLaunchArgs& a, mcStream_t stream) {
    const MxkLaunchArgs c = to_c(a);
    last_status() = mxk_launch_prelude(&c, stream);
}
// Everything up to the combine push, no reduce (reference: launch_compute, :222-242).
inline void launch_compute(const MegaLaunchArgs& a, mcStream_t stream) {
    const MxkLaunchArgs c = to_c(a);
    last_status() = mxk_launch_compute(&c, stream);
}
// Reduce only (reference: launch_reduce, :244-250).
inline void launch_reduce(const MegaLaunchArgs& a, mcStream_t stream) {
    const MxkLaunchArgs c = to_c(a);
    last_status() = mxk_launch_reduce(&c, stream);
}
// Whole layer on one stream (reference: launch_full, :252-259).
inline void launch_full(const MegaLaunchArgs& a, mcStream_t stream) {
    const MxkLaunchArgs c = to_c(a);
    last_status() = mxk_launch_full(&c, stream);
}
// Empty kernel, the graph-chain floor (reference: launch_empty, :261-264).
inline void launch_empty(int grid, int threads, int64_t smem, mcStream_t stream) {
    last_status() = mxk_launch_empty(grid, threads, smem, stream);
}
// Device-side deterministic weights (reference: fill_weights_lane, :66-105; row-major here).
inline void fill_weights_lane(uint8_t* w, int n_rows, int k_cols, uint32_t seed, mcStream_t stream) {
    last_status() = mxk_fill_weights(w, n_rows, k_cols, seed, stream);
}
// The same for 4-bit weights: packed e2m1 codes WPROBE_FP4_CODE (reference: src/common.cuh:127-131), row-major.
inline void fill_weights_e2m1(uint8_t* w, int n_rows, int k_cols, uint32_t seed, mcStream_t stream) {
    last_status() = mxk_fill_weights_e2m1(w, n_rows, k_cols, seed, stream);
}
// Registers / local / shared memory of the kernels (reference: dump_kernel_resources, :270-282).
inline void dump_kernel_resources() { last_status() = mxk_dump_kernel_resources(); }

}  // namespace fp8mega
