// ============================================================================
// mxk_sched.cuh — the skew-aware schedulers of the MoE layer as pure functions,
// compiled for the host and for the device from the same source (no state, no
// memory traffic beyond their arguments; the same inputs give the same outputs
// bit for bit on either side).
//
//   group maps          ranks are partitioned into helper groups; inside a group
//                       every member holds the weights of all the group's experts
//                       (reference: gs_nGroups ... gs_expert_of_ge,
//                        src/group_sched.cuh:61-80)
//   sched_group_skewed  the test that switches helper scheduling on for a launch
//                       (reference: MX_GS_SKEW_NUM, src/group_sched.cuh:26-28,
//                        src/compute.cuh:716-760)
//   sched_member_windows the (group expert, window) units one member computes:
//                       deterministic longest-processing-time assignment with
//                       cost = ceil(rows / 16) (reference: gs_schedule_member,
//                        src/group_sched.cuh:164-205); optionally only the windows
//                       of HOT experts move (see there)
//   sched_lpt_assign    LPT over (expert, window, slice) tasks with cost = rows
//                       (reference: enumerate_group_tasks / bp_sort_lpt /
//                        lpt_assign, src/balance_partition.cuh:62-115)
//
// The reference freezes EPR = 8 and 4 ranks per group; here both are arguments.
// On NVSwitch every pair of GPUs has the same bandwidth, so how ranks are put
// together does not matter for traffic, and the weight replication a group
// costs (group_ranks x EPR experts per member) is the same for any partition;
// the interleaved map of the reference is kept so that its recorded schedules
// stay valid test vectors.
// ============================================================================
#pragma once

#if defined(__CUDACC__)
#define MXK_HD __host__ __device__ __forceinline__
#else
#define MXK_HD inline
#endif

namespace mxk {

constexpr int kSchedMaxGroupRanks = 16;   // members of a helper group
constexpr int kSchedCostRows = 16;        // a window of r rows costs ceil(r / 16)

// ---- interleaved helper groups: group = rank % n_groups, member = rank / n_groups
MXK_HD int sched_n_groups(int R, int group_ranks) { return R / group_ranks; }
MXK_HD int sched_group_of_rank(int R, int group_ranks, int r) { return r % sched_n_groups(R, group_ranks); }
MXK_HD int sched_member_of_rank(int R, int group_ranks, int r) { return r / sched_n_groups(R, group_ranks); }
MXK_HD int sched_rank_of_member(int R, int group_ranks, int g, int m) { return g + m * sched_n_groups(R, group_ranks); }
// global expert e <-> index inside its group's replicated weight block, ge = member * EPR + local expert
MXK_HD int sched_ge_of_expert(int R, int group_ranks, int EPR, int e) {
    return sched_member_of_rank(R, group_ranks, e / EPR) * EPR + e % EPR;
}
MXK_HD int sched_expert_of_ge(int R, int group_ranks, int EPR, int g, int ge) {
    return sched_rank_of_member(R, group_ranks, g, ge / EPR) * EPR + ge % EPR;
}

MXK_HD int sched_window_count(int rows, int win_cap) { return rows > 0 ? (rows + win_cap - 1) / win_cap : 0; }
MXK_HD int sched_window_cost(int rows) { return (rows + kSchedCostRows - 1) / kSchedCostRows; }

// A group's load is skewed when its hottest expert holds more than skew_num / n_experts of the rows:
// max * n_experts > skew_num * sum (skew_num = 2 in the reference's build; 0 = always).
MXK_HD bool sched_group_skewed(const int* rows_of_ge, int n_experts, int skew_num) {
    long long mx = 0, sum = 0;
    for (int i = 0; i < n_experts; ++i) {
        const long long c = rows_of_ge[i] > 0 ? rows_of_ge[i] : 0;
        mx = c > mx ? c : mx;
        sum += c;
    }
    return mx * n_experts > (long long)skew_num * sum;
}

// Windows of the group's experts handed to `member`, in the order they are assigned.
//
// Every expert ge with c rows has floor(c / win_cap) full windows of cost C = ceil(win_cap / 16)
// and, when c % win_cap != 0, one tail window of cost ceil((c % win_cap) / 16).  Windows are
// visited by descending cost and, inside one cost, by ascending (ge, w); each goes to the member
// with the smallest accumulated cost, a tie going to the expert's owner (ge / EPR) first and to
// the lowest member otherwise.  Writes at most `cap` entries and returns how many `member` got.
//
// hot_windows > 0 (not in the reference): only experts with at least that many windows are spread.
// A window computed away from the expert's owner costs the helper a pass over the expert's weights,
// which on a memory-bound layer is worth several windows of arithmetic, so an expert with one or
// two windows is cheaper left where its weights are already streamed.  Every other expert stays with
// its owner: its cost is in the owner's load before the first hot window is placed, and its windows
// appear in the owner's list at their usual position.  0 = every window may move (the reference).
MXK_HD bool sched_expert_hot(int rows, int win_cap, int hot_windows) {
    return hot_windows <= 0 || sched_window_count(rows, win_cap) >= hot_windows;
}
MXK_HD int sched_member_windows(const int* rows_of_ge, int EPR, int group_ranks, int win_cap, int member,
                                int* out_ge, int* out_w, int cap, int hot_windows = 0) {
    long long load[kSchedMaxGroupRanks];
    for (int m = 0; m < group_ranks; ++m) load[m] = 0;
    const int n_experts = EPR * group_ranks;
    const int full_cost = sched_window_cost(win_cap);
    int n_out = 0;
    if (hot_windows > 0)
        for (int ge = 0; ge < n_experts; ++ge) {
            const int c = rows_of_ge[ge];
            if (c <= 0 || sched_expert_hot(c, win_cap, hot_windows)) continue;
            load[ge / EPR] += (long long)(c / win_cap) * full_cost + (c % win_cap ? sched_window_cost(c % win_cap) : 0);
        }
    for (int level = full_cost; level >= 1; --level) {
        for (int ge = 0; ge < n_experts; ++ge) {
            const int c = rows_of_ge[ge];
            if (c <= 0) continue;
            const int n_full = c / win_cap, tail = c % win_cap;
            // windows of this expert at this cost level: [w_lo, w_hi)
            int w_lo = 0, w_hi = 0;
            if (level == full_cost) w_hi = n_full;
            if (tail != 0 && sched_window_cost(tail) == level) {
                if (w_hi == 0) w_lo = n_full;
                w_hi = n_full + 1;
            }
            const int owner = ge / EPR;
            const bool hot = sched_expert_hot(c, win_cap, hot_windows);
            for (int w = w_lo; w < w_hi; ++w) {
                int best = owner;
                if (hot) {
                    best = 0;
                    for (int m = 1; m < group_ranks; ++m)
                        if (load[m] < load[best]) best = m;
                    if (load[owner] == load[best]) best = owner;
                    load[best] += level;
                }
                if (best == member) {
                    if (n_out < cap) { out_ge[n_out] = ge; out_w[n_out] = w; }
                    ++n_out;
                }
            }
        }
    }
    return n_out;
}

// Longest-processing-time assignment of (expert, window, slice) tasks to `n_members`.
// Tasks: for every listed expert e (counts[e] rows) its windows w, each cut in `n_slice`
// slices; cost = rows of the window.  Order: descending cost, equal costs in enumeration
// order (expert list order, w, slice).  Each task goes to the member with the strictly
// smallest load, so ties fall to the lowest member.  `tasks` [n][3] receives (e, w, slice)
// in assignment order, `member_of` [n] the member, `load` [n_members] the totals.
// Returns the number of tasks (at most `cap` are written).
MXK_HD int sched_lpt_assign(const int* counts, const int* experts, int n_experts, int win_cap, int n_slice,
                            int n_members, int* tasks, int* member_of, long long* load, int cap) {
    for (int m = 0; m < n_members; ++m) load[m] = 0;
    int n = 0;
    // costs are row counts in [1, win_cap]: walk them downwards instead of sorting
    for (int cost = win_cap; cost >= 1; --cost) {
        for (int i = 0; i < n_experts; ++i) {
            const int e = experts[i], c = counts[e];
            if (c <= 0) continue;
            const int n_full = c / win_cap, tail = c % win_cap;
            int w_lo = 0, w_hi = 0;
            if (cost == win_cap) w_hi = n_full;
            if (tail == cost) {     // tail < win_cap, so it never meets the full windows' level
                w_lo = n_full;
                w_hi = n_full + 1;
            }
            for (int w = w_lo; w < w_hi; ++w)
                for (int s = 0; s < n_slice; ++s) {
                    int best = 0;
                    for (int m = 1; m < n_members; ++m)
                        if (load[m] < load[best]) best = m;
                    load[best] += cost;
                    if (n < cap) {
                        tasks[3 * n] = e; tasks[3 * n + 1] = w; tasks[3 * n + 2] = s;
                        member_of[n] = best;
                    }
                    ++n;
                }
        }
    }
    return n;
}

}  // namespace mxk
