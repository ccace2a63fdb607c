/* ============================================================================
 * mxk_b200.h — C ABI of the B200 (sm_100a) FP8xFP8 MoE layer library.
 *
 * Plain pointers and sizes only; no C++ or torch types.  This is the boundary a
 * foreign-function binding (ctypes, cgo, JNI ...) attaches to.  The C++
 * namespace fp8mega in include/megakernel.h forwards to these entry points and
 * keeps the reference's host interface (reference: src/megakernel.h:54-137).
 *
 * All launch functions are asynchronous on the given CUDA stream, allocate
 * nothing, keep no per-call host state and are CUDA-graph capturable.  They
 * return 0 on success or a negative MXK_ERR_* / positive cudaError_t value;
 * mxk_last_error() gives a message for the calling thread's last failure.
 * Device-side protocol failures (a bounded wait that expired) never trap: they
 * set the status word read by mxk_read_status() (reference: lf->dbg[8] slots,
 * src/flags.cuh:197-360, src/prologue.cuh:348,474, src/combine.cuh:562).
 * ========================================================================== */
#ifndef MXK_B200_H_
#define MXK_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MXK_ERR_BAD_ARG (-1)      /* geometry / pointer / size rejected          */
#define MXK_ERR_NO_DRIVER (-2)    /* cuTensorMapEncodeTiled entry point missing  */
#define MXK_ERR_TENSOR_MAP (-3)   /* tensor-map encoding failed                  */
#define MXK_ERR_DEVICE (-4)       /* device is not sm_100                        */

/* Geometry of the expert-parallel world.  The reference freezes these at compile
 * time (src/common.cuh:18-24: EPR=8, topk=8, H=6144, I=2048); here they are
 * run-time values.  hidden % 256 == 0, intermediate % 128 == 0. */
typedef struct MxkGeom {
    int32_t R;                /* ranks (GPUs) in the EP world                    */
    int32_t rank;             /* this rank                                       */
    int32_t experts_per_rank; /* local experts; global expert e lives on e / EPR */
    int32_t topk;
    int32_t hidden;           /* H                                               */
    int32_t intermediate;     /* I                                               */
    int32_t max_tokens;       /* token rows per rank the buffers are sized for   */
    int32_t slot_capacity;    /* accepted pairs per (source rank, expert);
                                 0 means max_tokens (src/prologue.cuh:171-174)  */
} MxkGeom;

/* Byte offsets of every table inside the three caller-allocated blocks.
 *   sym : inputs of this rank, peers READ it   (reference ProdLayout x_off /
 *         topk_idx_off / topk_weights_off, src/host_layout.cuh:79-82)
 *   unk : workspace peers WRITE into            (reference unk_data,
 *         src/flags_defs.cuh:121-222)
 *   rwk : private workspace                     (reference rwk_data, :61-175)
 * All three must be zero-filled once before the first launch. */
typedef struct MxkLayout {
    /* sym */
    int64_t sym_bytes;
    int64_t x_off;              /* uint8  [max_tokens][H]      E4M3 activations   */
    int64_t x_sf_off;           /* uint8  [max_tokens][H/128]  UE8M0 1x128 scales */
    int64_t topk_idx_off;       /* int64  [max_tokens][topk]                      */
    int64_t topk_weights_off;   /* float  [max_tokens][topk]                      */
    /* unk */
    int64_t unk_bytes;
    int64_t src_index_table_off;/* uint64 [2][EPR][R][slot_capacity]: low word = pair
                                   index token*topk+k, high word = launch epoch       */
    int64_t expert_recv_counts_off; /* uint64 [2][R][recv_stride]: low word = count
                                   (word EPR: checksum), high word = launch epoch     */
    int64_t combine_rows_off;   /* bf16   [topk][max_tokens][H]                   */
    int64_t combine_cnt_off;    /* uint32 [topk][max_tokens] arrivals per pair    */
    int32_t recv_stride;        /* words per expert_recv_counts row (>= EPR+1)    */
    /* rwk */
    int64_t rwk_bytes;
    int64_t flags_off;          /* MxkStatus-sized header, see mxk_read_status    */
    int64_t route_slot_counts_off; /* int32 [E]                                   */
    int64_t pair_state_off;     /* uint8  [max_tokens*topk] 1 = pair accepted     */
    int64_t prefix_tbl_off;     /* int32  [EPR][R+1]                              */
    int64_t expert_row_base_off;/* int32  [EPR+1] first pool row of each expert   */
    int64_t windows_off;        /* int32  [max_windows][4] expert,row0,rows,-     */
    int64_t tasks_off;          /* int32  [max_tasks][4]   kind,window,ntile,rows */
    int64_t l1_done_off;        /* uint32 [2][max_windows] (copy = launch parity)  */
    int64_t row_meta_off;       /* int32  [pool_rows][4] src,token,k,weight bits  */
    int64_t pool_off;           /* uint8  [pool_rows+128][H]   dispatched rows    */
    int64_t pool_sf_off;        /* uint8  [pool_rows][sf_stride_h]                */
    int64_t ffn_off;            /* uint8  [pool_rows+128][I]   L1 output          */
    int64_t ffn_sf_off;         /* uint8  [pool_rows][sf_stride_i]                */
    int64_t pool_rows;          /* = R * max_tokens * topk                        */
    int32_t sf_stride_h;        /* bytes per pool_sf row (H/128 rounded to 16)    */
    int32_t sf_stride_i;        /* bytes per ffn_sf row  (I/128 rounded to 16)    */
    int32_t max_windows;
    int32_t max_tasks;
    int64_t pool_ready_off;     /* uint32 [2][max_windows] rows of a window dispatched
                                   (copy = launch parity, like l1_done)                */
    int64_t expert_first_win_off; /* int32 [EPR] first window id of each expert      */
    /* push-mode prologue (small batches): every rank stores its tokens' routing, top-k
     * weights, scales and E4M3 rows into the owner ranks' staging area as epoch-tagged
     * 64-bit words {payload u32, epoch u32}; 0 bytes when the geometry is not eligible */
    int64_t xin_off;            /* unk: uint64 [2][R][xin_src_words]                  */
    int64_t xin_src_words;      /* words per (parity, source rank): 16 header words
                                   (word 0 = token count) + max_tokens * xin_row_words */
    int32_t xin_row_words;      /* per token: topk ids, topk weights, ceil(H/512) scale
                                   words (padded to even), H/4 row words              */
    int32_t push_eligible;      /* 1: this geometry may run the push-mode prologue    */
    int64_t route_scratch_off;  /* rwk: int32 [route_scratch_ctas][E] pairs per (CTA slice, expert),
                                   scratch of the one-pass route build for large batches */
    int32_t route_scratch_ctas;
    int32_t push_auto;          /* 1: dispatch_mode 0 runs the push-mode prologue here: eligible and
                                   max_tokens * topk <= 2048 per rank (1024 in a world of
                                   several ranks, where the doubled bytes cross NVLink).  A pushed row travels as
                                   tagged words (twice its bytes) once per routed pair and is copied
                                   again into the pool; beyond that size the pull protocol's three
                                   round trips cost less than the extra bytes                      */
} MxkLayout;

/* One launch.  Field names follow fp8mega::MegaLaunchArgs (reference
 * src/megakernel.h:54-114); the fields after max_spins/skip_prologue are new:
 * geometry and the UE8M0 scale planes (all-null planes == the reference's
 * scale-free mode). */
#define MXK_WEIGHTS_E4M3 0
#define MXK_WEIGHTS_E2M1 1

typedef struct MxkLaunchArgs {
    int32_t R, rank;
    int32_t tokens;            /* valid tokens of this rank in this launch        */
    int32_t slot_capacity;
    int32_t win_cap;           /* rows per window (M tile), 8..128; 0 => 128      */
    int32_t grid, threads;     /* grid: CTAs of the GEMM kernel, 0 => SM count;
                                  threads is accepted and ignored                 */
    int64_t smem;              /* accepted and ignored                            */
    void* rwk;
    void* unk;
    void* const* unk_peers;    /* DEVICE array [R] of every rank's unk base       */
    const uint8_t* self;       /* this rank's sym base                            */
    uint8_t* const* peer_bases;/* DEVICE array [R] of every rank's sym base       */
    const int64_t* topk_idx;   /* optional; NULL => self + topk_idx_off           */
    const uint8_t* w1;         /* [EPR][2I][H] E4M3 row-major, gate rows then up  */
    const uint8_t* w2;         /* [EPR][H][I]  E4M3 row-major                     */
    int32_t group_weights_ready; /* != 0: w1_group / w2_group below hold the helper group's weights */
    int64_t topk_idx_off, x_off, weights_off;
    int32_t in_bf16;           /* must be 0                                       */
    int32_t skip_combine;      /* >0: L2 results are not pushed (diagnostic)      */
    float* y;                  /* optional FP32 [tokens][H]                       */
    int32_t max_spins;         /* bound of every device wait, in units of 250 ns;
                                  0 => 2 s                                        */
    int32_t skip_prologue;     /* must be 0                                       */
    /* ---- additions ---- */
    int32_t experts_per_rank, topk, hidden, intermediate, max_tokens;
    int64_t x_sf_off;          /* valid when w1_sf != NULL                        */
    const uint8_t* w1_sf;      /* [EPR][2I/128][H/128] UE8M0 or NULL              */
    const uint8_t* w2_sf;      /* [EPR][H/128][I/128]  UE8M0 or NULL              */
    uint16_t* y_bf16;          /* optional bf16 [tokens][H]                       */
    int32_t cta_pair;          /* GEMM tiling: 1 = one CTA per 128-row window, 2 = clusters
                                  of two CTAs per 256-row window (2-CTA MMA; needs
                                  win_cap 128 and an even grid), 0 = choose by load:
                                  pairs when tokens*topk/experts_per_rank >= 256  */
    int32_t dispatch_mode;     /* prologue protocol, THE SAME ON EVERY RANK of a launch:
                                  1 = pull (route scatter, count barrier, owner ranks pull
                                  rows; reference r19_pull_flags), 2 = push (source ranks
                                  store ids + rows into the owners' staging area, every CTA
                                  derives the tables itself; needs layout.push_eligible),
                                  0 = push for small batches (layout.push_auto, or any eligible
                                  geometry when helper groups are on), else pull          */
    /* ---- cross-rank helper scheduling for skewed routing (reference: MX_GROUP_SCHED,
     * src/compute.cuh:700-835; group-replicated weights rwk->ld.w1g / w2g,
     * src/flags_defs.cuh:160-169, gated by group_weights_ready above) ----
     * Ranks form interleaved helper groups of group_ranks (group = rank % (R / group_ranks),
     * member = rank / (R / group_ranks)); every member holds the weights of ALL the group's
     * experts in the order ge = member * experts_per_rank + local expert.  When a launch finds
     * its group's load skewed, the (expert, window) units of the group are spread over the
     * members by the deterministic LPT of mxk_gs_schedule_member and a member computes windows
     * of other members' experts from its replica, pushing the results to the source ranks as
     * usual.  Needs group_weights_ready != 0, the push-mode prologue, R % group_ranks == 0 and
     * the inputs in their regular regions of sym; the same on every rank. */
    int32_t group_ranks;       /* 0 / 1 = no helper groups                                  */
    int32_t group_skew_num;    /* skew test max * n > num * sum: 0 = the reference's 2,
                                  negative = helpers on in every launch                     */
    const uint8_t* w1_group;   /* [group_ranks * EPR][2I][H]                                */
    const uint8_t* w2_group;   /* [group_ranks * EPR][H][I]                                 */
    const uint8_t* w1_sf_group;/* [group_ranks * EPR][2I/128][H/128] or NULL                */
    const uint8_t* w2_sf_group;/* [group_ranks * EPR][H/128][I/128]  or NULL                */
    /* ---- 4-bit weights (reference: the MX_FP4_W build, src/common.cuh:99-134) ----
     * MXK_WEIGHTS_E2M1: every weight tensor above (w1, w2 and the group replicas) holds e2m1
     * codes, two per byte, row-major [experts][rows][k / 2] with the element of even k in the
     * low nibble; a code stands for the E4M3 value of mxk_e2m1_to_e4m3 (0, 0.5, 1, 1.5, 2, 3,
     * 4, 6 and their negatives) and the 128x128 scale planes apply as for 8-bit weights.  The
     * layer reads half the weight bytes from HBM; its results are those of the 8-bit layer on
     * the expanded weights.  The tensors must be 32-byte aligned. */
    int32_t weight_format;     /* MXK_WEIGHTS_E4M3 (0) or MXK_WEIGHTS_E2M1 (1)              */
    int32_t group_hot_windows; /* helper groups spread the windows of experts with at least this many
                                  windows and leave the others with their owners (see
                                  mxk_gs_schedule_member_hot): 0 = 3, negative = every window may
                                  move (the reference's schedule); the same on every rank   */
} MxkLaunchArgs;

/* Host-readable copy of the device status header. */
typedef struct MxkStatus {
    int64_t launches;      /* completed prologues (reference current_time)       */
    int32_t status;        /* 0 = ok, else the first MXK_DEV_* code raised       */
    int32_t n_tasks, n_l1_tasks, n_windows, total_rows;
    int32_t helper_on;     /* 1: the last launch ran this rank's member list of the helper group
                              (n_windows / total_rows then count the windows and rows it computed) */
    int32_t dbg[8];        /* expiry counters, slot meaning as the reference:
                              0 barrier, 2 route, 3 task queue, 4 L1->L2 gate /
                              reduce wait, 5 pipeline barrier, 6 TMEM barrier    */
    uint64_t ticks[16];    /* SM cycles of the last layer summed over the GEMM CTAs
                              (reference: pre_ticks readers, torch/csrc/flags_bridge.cu:44-51):
                              0 TMA producer blocked on a free stage, 1 on the L1->L2 gate,
                              2 MMA issuer blocked on operand tiles, 3 on the accumulator
                              drain, 4 on scale tiles, 5 epilogue blocked on accumulators,
                              6 CTA lifetime, 7 producer blocked on the task ring,
                              8 epilogue busy; 9..13 phase ends in ns since CTA start
                              (route, set-up, dispatch, GEMM, reduce); 15 epilogue
                              draining accumulators (part of 8)                       */
    uint64_t trace[64];    /* MXK_TICKS=1: globaltimer stamps (ns) of the last layer, CTA 0
                              in [0,32) and the last CTA in [32,64): 0 kernel entry, 1 barriers /
                              tensor memory ready, 2 route or push issued, 3 route phase left,
                              4 barrier seen (all sources arrived), 5 tables built, 6 set-up
                              left, 7 dispatch left, 8 first task's gate passed, 9 first
                              operand tile requested, 10 first tile landed, 11 GEMM phase left,
                              12 reduce left                                               */
} MxkStatus;

#define MXK_DEV_TIMEOUT_BARRIER 1
#define MXK_DEV_TIMEOUT_GATE 2
#define MXK_DEV_TIMEOUT_PIPE 3
#define MXK_DEV_TIMEOUT_REDUCE 4
#define MXK_DEV_BAD_TABLE 5

const char* mxk_last_error(void);
int mxk_version(void);

/* Layout of sym / unk / rwk for a geometry (reference: compute_layout,
 * src/host_layout.cuh:63-113; sizeof(rwk_data)/sizeof(unk_data) exported as
 * mxk_rwk_bytes / mxk_unk_bytes, torch/csrc/flags_bridge.cu:12-53). */
int mxk_compute_layout(const MxkGeom* g, MxkLayout* out);
int64_t mxk_sym_bytes(const MxkGeom* g);
int64_t mxk_rwk_bytes(const MxkGeom* g);
int64_t mxk_unk_bytes(const MxkGeom* g);

/* Launchers (reference: fp8mega::launch_prelude / launch_compute / launch_reduce /
 * launch_full / launch_empty, src/megakernel.cu:203-268).
 *   prelude : route build + count publish + cross-rank barrier + task set-up
 *   compute : prelude + dispatch pull + L1 + L2 + combine push
 *   reduce  : top-k weighted sum of the rows pushed to this rank
 *   full    : compute + reduce */
int mxk_launch_prelude(const MxkLaunchArgs* a, void* stream);
int mxk_launch_compute(const MxkLaunchArgs* a, void* stream);
int mxk_launch_reduce(const MxkLaunchArgs* a, void* stream);
int mxk_launch_full(const MxkLaunchArgs* a, void* stream);
int mxk_launch_empty(int grid, int threads, int64_t smem, void* stream);
/* Number of kernels one mxk_launch_full enqueues (one persistent kernel). */
int mxk_kernels_per_layer(void);

/* Phase-split launcher for diagnostics and single-GPU tests of a multi-rank world
 * (reference precedent: launch_l1 / launch_l2 under CM_L1L2_SPLIT,
 * src/megakernel.h:120-126).  Enqueues only the kernels selected by phase_mask, in
 * layer order.  Kernels of different ranks wait on each other (barrier, arrival
 * counts), so on ONE device the ranks' phases must be issued phase by phase:
 * ROUTE for every rank, then SETUP for every rank, and so on. */
#define MXK_PHASE_ROUTE 1
#define MXK_PHASE_SETUP 2
#define MXK_PHASE_DISPATCH 4
#define MXK_PHASE_GEMM 8
#define MXK_PHASE_REDUCE 16
int mxk_launch_phases(const MxkLaunchArgs* a, int phase_mask, void* stream);

/* Whole layer for callers that must not allocate device memory.  No counterpart in the
 * reference (its callers always allocate rwk / unk themselves).
 *
 * Some hosts cannot call cudaMalloc when a layer has to run: an inference server whose
 * memory pool already owns the whole GPU (a fresh cudaMalloc simply fails there), a
 * plugin loaded into somebody else's runtime that forbids allocation after start-up, or
 * code running where an allocation would synchronise the device at a bad moment.  For
 * them this entry point keeps the two workspace blocks (unk and rwk) and the two
 * one-entry pointer tables in a fixed array inside the library image instead of taking
 * them from the caller.  It calls no cudaMalloc / cudaFree and no allocating library
 * routine; every GPU that loads the library carries the array (mxk_static_scratch_bytes(),
 * 32 MiB) from load until exit.
 *
 * Arguments are those of mxk_launch_full for a single-rank world (R = 1, rank = 0): the
 * caller still passes its input block `self` (x, x_sf, topk_idx, topk_weights at the
 * usual offsets), the weights and y / y_bf16; the fields rwk, unk, unk_peers and
 * peer_bases are ignored.  A geometry whose workspace (256 + unk_bytes + rwk_bytes of
 * mxk_compute_layout) exceeds the array is rejected with MXK_ERR_BAD_ARG and a message
 * that states both sizes.
 *
 * The first call on a device asks the CUDA runtime for the array's device address
 * (once per device, with that device current); make that first call outside any stream
 * capture.  All calls share the one array and it keeps the previous call's contents.  Calls
 * with one geometry continue on it exactly like launches on a caller-owned workspace; the
 * launch counter (first word of rwk, at a fixed place whatever the geometry) keeps running
 * from call to call, because the prologue's words are tagged with it.  When a call's geometry
 * differs from the previous call's on that device, everything behind the counter is cleared on
 * the caller's stream first (cudaMemsetAsync allocates nothing), since the old tables lie at
 * other offsets.  Two calls that overlap on the GPU (different streams, or several threads)
 * would race on the array: issue them on one stream or serialise them yourself.  The status
 * of the last call is read with mxk_read_status_static(). */
int mxk_launch_full_static(const MxkLaunchArgs* a, void* stream);
int64_t mxk_static_scratch_bytes(void);

/* Deterministic test weights, byte (seed + 131*row + 7*k) & 0x3f at logical
 * (row, k), row-major (reference: fill_weights_lane writes the same values in
 * MetaX lane order, src/megakernel.cu:66-105, src/megakernel.h:46-47). */
int mxk_fill_weights(uint8_t* w, int64_t n_rows, int32_t k_cols, uint32_t seed, void* stream);

/* 4-bit test weights: e2m1 code ((seed + 131*row + 7*k) >> 1) & 0xf at logical (row, k)
 * (reference: WPROBE_FP4_CODE, src/common.cuh:127-131), packed two per byte (even k in the
 * low nibble), row-major [n_rows][k_cols / 2]; k_cols must be even. */
int mxk_fill_weights_e2m1(uint8_t* w, int64_t n_rows, int32_t k_cols, uint32_t seed, void* stream);

/* The E4M3 byte an e2m1 code (low 4 bits) stands for (reference: fp4_code_to_fp8,
 * src/common.cuh:116-126): magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6; bit 3 is the sign. */
uint8_t mxk_e2m1_to_e4m3(uint8_t code);

/* bf16 activations -> E4M3 rows + one UE8M0 scale per 128 columns (x_sf [tokens][hidden/128]),
 * the reference's activation quantiser per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=128)
 * (torch/mxmegakernel/utils/math.py:26-36).  x_sf == NULL: plain saturating RNE cast, the
 * reference kernel's own bf16 prefold for its scale-free arithmetic (src/prologue.cuh:105-122,
 * MegaLaunchArgs::in_bf16).  A host that holds bf16 activations calls this on the launch stream
 * with x_fp8 / x_sf pointing at this rank's x / x_sf regions of `sym`, then launches the layer:
 * peers still pull one byte per element.  The launch structure's in_bf16 stays rejected. */
int mxk_quantize_rows(const void* x_bf16, int32_t tokens, int32_t hidden, void* x_fp8, void* x_sf, void* stream);

/* Registers / shared memory of every kernel, printed to stdout (reference:
 * dump_kernel_resources, src/megakernel.cu:270-282). */
int mxk_dump_kernel_resources(void);

/* Synchronous read of the status header of an rwk block. */
int mxk_read_status(const void* rwk, MxkStatus* out);
/* The same for the workspace of mxk_launch_full_static on the current device. */
int mxk_read_status_static(MxkStatus* out);
/* Where MxkStatus.ticks sits inside rwk (byte offset) and how many 64-bit counters there are
 * (reference: mxk_rwk_ticks_off / mxk_ticks_count, torch/csrc/flags_bridge.cu:44-51). */
int64_t mxk_rwk_ticks_off(void);
int64_t mxk_ticks_count(void);
/* Wait-time accounting and phase stamps of the kernel (MxkStatus.ticks / trace) for the launches
 * that follow: 1 on, 0 off, -1 back to the MXK_TICKS environment variable.  Returns the setting
 * that was in force (reference: the -DR24_DIAG_PHASE build switch, src/flags_defs.cuh:93-109). */
int mxk_set_ticks(int on);

/* Window chooser kept for the callers that bind it (reference: mxk_select_win,
 * torch/csrc/flags_bridge.cu:31-38 -> src/win_select.cuh:95-128). */
int mxk_select_win(const uint32_t* counts, int E, int cap_hint, int win_min);

/* Skew-aware schedulers as pure functions (host entry points; the kernels call the same source).
 *   mxk_group_ranks         ranks per helper group of the reference's build (kGroupRanks,
 *                           torch/csrc/flags_bridge.cu:15)
 *   mxk_gs_schedule_member  the (group expert, window) units one member of a helper group computes:
 *                           deterministic LPT, cost = ceil(rows / 16), ties to the owner then the
 *                           lowest member (reference: gs_schedule_member, src/group_sched.cuh:164-205).
 *                           rows_of_ge [group_ranks * EPR], ge = member * EPR + local expert.
 *                           Returns the member's window count (at most cap entries are written).
 *   mxk_gs_schedule_member_hot  the same with the spreading limited to HOT experts, those with at least
 *                           hot_windows windows (not in the reference: a window computed away from its
 *                           expert's owner costs the helper a pass over the expert's weights, worth several
 *                           windows of arithmetic on a memory-bound layer).  Every other expert stays with its
 *                           owner; its cost is in the owner's load before the first hot window is placed.
 *                           hot_windows 0 = mxk_gs_schedule_member.  What the kernels run (group_hot_windows).
 *   mxk_gs_group_skewed     1 when max * n_experts > skew_num * sum (reference: MX_GS_SKEW_NUM = 2,
 *                           src/group_sched.cuh:26-28)
 *   mxk_lpt_assign          LPT over (expert, window, slice) tasks with cost = rows (reference:
 *                           enumerate_group_tasks / lpt_assign, src/balance_partition.cuh:62-115);
 *                           tasks [n][3] and member_of [n] in assignment order, load [n_members].
 *   mxk_gs_schedule_on_device  the member lists of a whole group computed by a kernel (host arrays
 *                           in and out, [group_ranks][cap]); host and device results must agree,
 *                           as in the reference's check (test/check.cu:287-315). */
int mxk_group_ranks(void);
int mxk_gs_schedule_member(const int32_t* rows_of_ge, int EPR, int group_ranks, int win_cap, int member,
                           int32_t* out_ge, int32_t* out_w, int cap);
int mxk_gs_schedule_member_hot(const int32_t* rows_of_ge, int EPR, int group_ranks, int win_cap, int member, int hot_windows,
                               int32_t* out_ge, int32_t* out_w, int cap);
int mxk_gs_group_skewed(const int32_t* rows_of_ge, int n_experts, int skew_num);
int mxk_lpt_assign(const int32_t* counts, const int32_t* experts, int n_experts, int win_cap, int n_slice, int n_members,
                   int32_t* tasks, int32_t* member_of, int64_t* load, int cap);
int mxk_gs_schedule_on_device(const int32_t* rows_of_ge, int EPR, int group_ranks, int win_cap, int hot_windows,
                              int32_t* out_ge, int32_t* out_w, int32_t* out_n, int cap);

/* Symmetric-memory helpers (reference SymmBuffer C++ side,
 * torch/csrc/apis/mega.hpp:86-195): device allocation that can be exported to
 * the other ranks' processes, and import of their handles. */
int mxk_symm_alloc(void** ptr, int64_t bytes);          /* cudaMalloc + zero fill */
int mxk_symm_free(void* ptr);
int mxk_ipc_export(void* ptr, uint8_t handle[64]);
int mxk_ipc_import(const uint8_t handle[64], void** ptr);
int mxk_ipc_close(void* ptr);

#ifdef __cplusplus
}
#endif
#endif /* MXK_B200_H_ */
