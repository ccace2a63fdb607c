// A C++ caller of include/megakernel.h, the way the reference's harness calls its own
// src/megakernel.h (test/check.cu:171-172,204-205,555-556; test/mybench.cu:222-237): it fills
// fp8mega::MegaLaunchArgs field by field and calls launch_prelude / launch_compute /
// launch_reduce / launch_full.  Built by tests/test_cpp_consumer.py into a small shared
// library; the test hands it device pointers through `ConsumerArgs` and compares the result
// with the oracle.  The static_asserts tie the C++ struct to its C twin field by field, so a
// field added to one and forgotten in the other (or in to_c()) fails at compile time.
#include <cstddef>
#include <cstdint>
#include <type_traits>

#include "megakernel.h"

using fp8mega::MegaLaunchArgs;

#define SAME_FIELD(f)                                                                        \
    static_assert(offsetof(MegaLaunchArgs, f) == offsetof(MxkLaunchArgs, f) &&               \
                      sizeof(MegaLaunchArgs::f) == sizeof(MxkLaunchArgs::f),                 \
                  "MegaLaunchArgs::" #f " and MxkLaunchArgs::" #f " differ in place or size")
SAME_FIELD(R); SAME_FIELD(rank); SAME_FIELD(tokens); SAME_FIELD(slot_capacity); SAME_FIELD(win_cap);
SAME_FIELD(grid); SAME_FIELD(threads); SAME_FIELD(smem); SAME_FIELD(rwk); SAME_FIELD(unk);
SAME_FIELD(unk_peers); SAME_FIELD(self); SAME_FIELD(peer_bases); SAME_FIELD(topk_idx);
SAME_FIELD(w1); SAME_FIELD(w2); SAME_FIELD(group_weights_ready); SAME_FIELD(topk_idx_off);
SAME_FIELD(x_off); SAME_FIELD(weights_off); SAME_FIELD(in_bf16); SAME_FIELD(skip_combine);
SAME_FIELD(y); SAME_FIELD(max_spins); SAME_FIELD(skip_prologue); SAME_FIELD(experts_per_rank);
SAME_FIELD(topk); SAME_FIELD(hidden); SAME_FIELD(intermediate); SAME_FIELD(max_tokens);
SAME_FIELD(x_sf_off); SAME_FIELD(w1_sf); SAME_FIELD(w2_sf); SAME_FIELD(y_bf16); SAME_FIELD(cta_pair);
SAME_FIELD(dispatch_mode); SAME_FIELD(group_ranks); SAME_FIELD(group_skew_num); SAME_FIELD(w1_group);
SAME_FIELD(w2_group); SAME_FIELD(w1_sf_group); SAME_FIELD(w2_sf_group); SAME_FIELD(weight_format); SAME_FIELD(group_hot_windows);
static_assert(sizeof(MegaLaunchArgs) == sizeof(MxkLaunchArgs), "MegaLaunchArgs and MxkLaunchArgs differ in size");
static_assert(std::is_standard_layout<MegaLaunchArgs>::value, "MegaLaunchArgs must stay a plain struct");

extern "C" {

struct ConsumerArgs {
    int32_t tokens, experts, topk, hidden, intermediate, max_tokens;
    void* rwk;
    void* unk;
    void* unk_peers;
    void* sym;
    void* peer_bases;
    const uint8_t* w1;
    const uint8_t* w2;
    const uint8_t* w1_sf;
    const uint8_t* w2_sf;
    float* y;
    uint16_t* y_bf16;
    int64_t topk_idx_off, x_off, weights_off, x_sf_off;
    int32_t mode;   // 0 launch_full, 1 launch_compute + launch_reduce, 2 launch_prelude only, 3 launch_empty
};

static MegaLaunchArgs fill(const ConsumerArgs* c) {
    MegaLaunchArgs a{};
    a.R = 1; a.rank = 0; a.tokens = c->tokens; a.slot_capacity = 0; a.win_cap = 128;
    a.rwk = static_cast<rwk_data*>(c->rwk);
    a.unk = static_cast<unk_data*>(c->unk);
    a.unk_peers = static_cast<unk_data* const*>(c->unk_peers);
    a.self = static_cast<const uint8_t*>(c->sym);
    a.peer_bases = static_cast<uint8_t* const*>(c->peer_bases);
    a.w1 = c->w1; a.w2 = c->w2; a.w1_sf = c->w1_sf; a.w2_sf = c->w2_sf;
    a.topk_idx_off = c->topk_idx_off; a.x_off = c->x_off; a.weights_off = c->weights_off; a.x_sf_off = c->x_sf_off;
    a.experts_per_rank = c->experts; a.topk = c->topk; a.hidden = c->hidden; a.intermediate = c->intermediate;
    a.max_tokens = c->max_tokens;
    a.y = c->y; a.y_bf16 = c->y_bf16;
    return a;
}

// Returns fp8mega::last_status() of the last call made.
int consumer_run(const ConsumerArgs* c, void* stream) {
    const MegaLaunchArgs a = fill(c);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (c->mode) {
        case 0: fp8mega::launch_full(a, st); break;
        case 1:
            fp8mega::launch_compute(a, st);
            if (fp8mega::last_status()) break;
            fp8mega::launch_reduce(a, st);
            break;
        case 2: fp8mega::launch_prelude(a, st); break;
        case 3: fp8mega::launch_empty(4, 64, 0, st); break;
        default: return -100;
    }
    return fp8mega::last_status();
}

// No device needed: null buffers must come back as MXK_ERR_BAD_ARG through last_status().
int consumer_null_buffers(void) {
    MegaLaunchArgs a{};
    a.R = 1; a.tokens = 4; a.experts_per_rank = 8; a.topk = 2; a.hidden = 512; a.intermediate = 256; a.max_tokens = 32;
    fp8mega::launch_full(a, nullptr);
    return fp8mega::last_status();
}

uint8_t consumer_wprobe(uint32_t seed, uint32_t row, uint32_t k) { return WPROBE_VAL(seed, row, k); }

}  // extern "C"
