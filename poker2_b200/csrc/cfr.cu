// Fused subgame CFR: one persistent kernel solves a whole batch of independent subgames.
//
// A thread block owns one subgame at a time and runs ALL of its iterations before it
// takes the next one from a queue, so the subgame's state (cumulative regrets, weight
// sums, average policy: [node][combo] fp32 rows, vector accesses) and the block's work
// rows stay hot in L2.  A thread owns VPT consecutive hand columns of every row.  What
// one iteration does (upstream: p2/search/cfr_evaluator.py:1331-1381) is reorganised into
// two sweeps over the internal nodes of the public tree:
//
//   top-down   regret matching of the children (:1168-1185), average-policy mix and
//              renormalisation (:1195-1258), reach of both players (:332-361) and the
//              normalisation sums of the children's beliefs (:254-273);
//   bottom-up  beliefs of the node (:363-380), opponent-conditioned child policy
//              (:1076-1093), leaf values (fold constants, showdown :484-601), value backup
//              (:1095-1115), then instantaneous regrets (:1117-1165) and the discounted
//              update of the NEXT iteration (:1346-1368) while the child values are still
//              in registers.
//
// Pass -1 evaluates the uniform start policy (:830-886, :1511-1513); the pass after the
// last iteration evaluates the average policy (`update_average_values_final`, :1276-1292).
//
// Numerics.  fp32 state arithmetic follows the upstream operation order exactly (the
// library is built with -fmad=false).  The belief normalisation sum reproduces the
// association order of the CPU row reduction upstream runs through.  Quantities upstream
// accumulates in fp64 and rounds to fp32 (unblocked mass, showdown prefix sums) are
// accumulated in fp64 here too, in a different order, which changes the rounded fp32
// result only when the fp64 value lies within ~1e-16 of a rounding boundary.
#include <atomic>
#include <mutex>

#include "cfr.cuh"
#include "cfr_dev.cuh"
#include "exactdiv.cuh"
#include "showdown.cuh"

namespace p2b {

namespace {

// This file is compiled twice: as it is, for trees of up to kIterMaxChildren actions per node (the kernel every
// shipped configuration runs), and from cfr_wide.cu with P2B_CFR_WIDE defined, which yields only the kernel
// for up to kCfrMaxChildren actions and its launcher.  Node bodies are unrolled per child count, so the two
// widest counts cost most of the compile time and stack frame; they stay out of the common kernel.
#ifdef P2B_CFR_WIDE
constexpr bool kWide = true;
#else
constexpr bool kWide = false;
#endif
constexpr int kMaxC = kWide ? kCfrMaxChildren : kIterMaxChildren;
constexpr int kBankRows = kMaxC;  // child rows staged per node in the top-down sweep
constexpr int kStageRows = 2 + 2 * kBankRows;  // top-down: two banks of child rows; bottom-up: 2 belief rows,
                                               // one marginal row and one leaf-belief row per child
constexpr int kCsRows = 2 + kBankRows;       // rows whose per-card sums are needed at one node

// ---- shared memory carve-up (bytes) ----
constexpr int kOffTab = 0;
constexpr int kOffNodes = kOffTab + kTabBytes;
constexpr int kOffXs = kOffNodes + kCfrMaxNodes * (int)sizeof(NodeRec);
constexpr int kOffPref = kOffXs + kStageRows * P2B_HPAD * 4;
constexpr int kOffPc = kOffPref + 2 * P2B_HPAD * 4;
constexpr int kOffCs = kOffPc + 2 * 52 * 52 * 4;
constexpr int kOffWarpTot = kOffCs + kCsRows * 52 * 8;
constexpr int kOffS = kOffWarpTot + 32 * 8;
constexpr int kOffSig = kOffS + kCsRows * 8;
constexpr int kOffSigB = kOffSig + kCfrMaxNodes * 2 * 4;  // the same sums for the beliefs under the average policy
constexpr int kOffMisc = kOffSigB + kCfrMaxNodes * 2 * 4;
constexpr int kOffIlist = kOffMisc + 64;  // node index of every internal node, in node order
constexpr int kCfrSmem = kOffIlist + ((kCfrMaxNodes * 2 + 15) / 16) * 16;
static_assert(kOffXs % 16 == 0 && kOffCs % 8 == 0 && kOffMisc % 16 == 0 && kOffSig % 8 == 0, "alignment");

enum PassMode { kPassInit = 0, kPassIter = 1, kPassFinal = 2 };

struct Block {
    // shared memory views
    unsigned char* tab;
    NodeRec* nodes;
    float* xs;     // [kStageRows][HPAD] staging rows
    float* pref;   // [2][HPAD] strength-order prefix sums
    float* pc;     // [2][52*52] per-card prefix sums
    double* cs;    // [2][52] per-card sums
    double* warp_tot;
    double* S;
    float* sig;    // [nodes][2] normalisation sums of the node beliefs of the current pass
    float* sigb;   // [nodes][2] the same for the beliefs under the average policy (iteration passes with cfr_avg)
    int* misc;
    uint16_t* ilist;  // [n_internal] node index of the ii-th internal node
    float* fsum;
    // current subgame
    SubgameRec sg;
    float* scr;
    __device__ __forceinline__ float* reach(int ii, int pl) const { return scr + (long long)(ii * 6 + pl) * P2B_HPAD; }
    __device__ __forceinline__ float* rbar(int ii, int pl) const { return scr + (long long)(ii * 6 + 2 + pl) * P2B_HPAD; }
    __device__ __forceinline__ float* val(int ii, int pl) const { return scr + (long long)(ii * 6 + 4 + pl) * P2B_HPAD; }
    // Reach under the NEW average policy of the pass (cfr_avg only).  Shares the value rows: the top-down
    // sweep writes it, the bottom-up visit of the node reads it before it stores the node's values there.
    __device__ __forceinline__ float* rnew(int ii, int pl) const { return val(ii, pl); }
    __device__ __forceinline__ float* row1(float* base, int node) const {
        return base + (long long)(sg.node_begin + node) * P2B_HPAD;
    }
    __device__ __forceinline__ float* row2(float* base, int node, int pl) const {
        return base + ((long long)(sg.node_begin + node) * 2 + pl) * P2B_HPAD;
    }
    __device__ __forceinline__ float* stage_row(int r) const { return xs + r * P2B_HPAD; }
    int sample_pass;  // pass whose policy is the sampling policy of the current subgame (-2: none)
    int leaf0;  // first model-leaf slot of the current subgame
    __device__ __forceinline__ long long leaf_row(int leaf_rank, int pl) const {
        return ((long long)(leaf0 + leaf_rank) * 2 + pl) * P2B_HPAD;
    }
};

// Policy of the K (== k) children of one node: uniform (start pass), the stored average policy
// (final pass) or regret matching on the cumulative regrets, which are returned in Rc.
template <int VPT, int K>
__device__ __forceinline__ void children_policy(int mode, const CfrParams& p, const Block& B, int fc, int k, int tid,
                                                FV<VPT> (&P)[K], FV<VPT> (&Rc)[K]) {
    constexpr float invk = 1.0f / (float)K;  // K == k; folded at compile time, correctly rounded
    if (mode == kPassInit) {
#pragma unroll
        for (int c = 0; c < K; ++c) {
            if (p.start_policy) P[c] = ldv<VPT>(B.row1(const_cast<float*>(p.start_policy), fc + c), tid);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                if (!p.start_policy) P[c].v[i] = invk;
                Rc[c].v[i] = 0.0f;
            }
        }
        return;
    }
    if (mode == kPassFinal) {
#pragma unroll
        for (int c = 0; c < K; ++c)
            P[c] = ldv<VPT>(B.row1(p.policy_avg, fc + c), tid);
        return;
    }
    FV<VPT> sum;
#pragma unroll
    for (int i = 0; i < VPT; ++i) sum.v[i] = 0.0f;
    // all loads first: the rows are independent, so their latencies overlap
#pragma unroll
    for (int c = 0; c < K; ++c)
        Rc[c] = ldv<VPT>(B.row1(p.regrets, fc + c), tid);
#pragma unroll
    for (int c = 0; c < K; ++c)
        {
#pragma unroll
            for (int i = 0; i < VPT; ++i) sum.v[i] = __fadd_rn(sum.v[i], fmaxf(Rc[c].v[i], 0.0f));
        }
    Divisor ds[VPT];  // the siblings share the divisor
#pragma unroll
    for (int i = 0; i < VPT; ++i) ds[i] = make_divisor(fmaxf(sum.v[i], 1e-8f));
    bool bad = false;
#pragma unroll
    for (int c = 0; c < K; ++c)
        {
#pragma unroll
            for (int i = 0; i < VPT; ++i) P[c].v[i] = div_fast<true>(fmaxf(Rc[c].v[i], 0.0f), ds[i], bad);
        }
    if (__builtin_expect(bad, 0)) {
#pragma unroll
        for (int c = 0; c < K; ++c)
            {
#pragma unroll
                for (int i = 0; i < VPT; ++i) P[c].v[i] = __fdiv_rn(fmaxf(Rc[c].v[i], 0.0f), ds[i].y);
            }
    }
#pragma unroll
    for (int c = 0; c < K; ++c)
        {
#pragma unroll
            for (int i = 0; i < VPT; ++i) P[c].v[i] = sum.v[i] > 1e-8f ? P[c].v[i] : invk;
        }
}

// x / sum, or the uniform distribution over the allowed hands when the row is
// (numerically) empty (cfr_evaluator.py:263-273).
template <int VPT>
__device__ __forceinline__ void apply_norm(const Block& B, const HandInfo<VPT>& hi, FV<VPT>& x, float sum) {
    const Divisor d = make_divisor(sum);
    bool bad = false;
    FV<VPT> q;
#pragma unroll
    for (int i = 0; i < VPT; ++i) q.v[i] = div_fast<true>(x.v[i], d, bad);
    if (__builtin_expect(bad, 0)) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) q.v[i] = __fdiv_rn(x.v[i], sum);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) x.v[i] = sum > 1e-5f ? q.v[i] : (hi.allowed[i] ? B.sg.allowed_prob : 0.0f);
}

// Normalises the two rows x[0], x[1] (one per player) over hands.  Uses staging rows 0 and
// 1, which must be free on entry and are free again on return; leaves the two sums in
// B.fsum.
template <int VPT>
__device__ __forceinline__ void normalize2(Block& B, const HandInfo<VPT>& hi, FV<VPT> (&x)[2]) {
    const int tid = threadIdx.x;
    stv<VPT>(B.stage_row(0), tid, x[0]);
    stv<VPT>(B.stage_row(1), tid, x[1]);
    __syncthreads();
    const int warp = tid >> 5;
    if (warp < 2) {
        const float sum = row_sum_reference_order(B.stage_row(warp));
        if ((tid & 31) == 0) B.fsum[warp] = sum;
    }
    __syncthreads();
    apply_norm<VPT>(B, hi, x[0], B.fsum[0]);
    apply_norm<VPT>(B, hi, x[1], B.fsum[1]);
}

// One block-wide round of the cross-hand work of a node.  For each of the `n_cs` staged rows
// cs_row0 .. cs_row0+n_cs-1: per-card sums (cs[i][52]) and total (S[i]).  For each of the
// `n_pc` rows listed in pc_rows: strength-order prefix sums (pref slot i) and per-card
// prefix sums (pc slot i) for the showdown formula.
//
// The work is cut into warp-sized units that the warps of the block take from a shared
// counter, largest first, so that all warps finish together whatever the mix:
//   * quarter scans: a warp produces the strength-order prefix of 352 consecutive sorted
//     positions; its starting offset is the sum of the earlier quarters, which it adds up
//     itself (no dependency on another warp);
//   * row totals: a warp adds up one row;
//   * list rounds: 32 threads = 8 groups of four threads, a group takes one (row, card) list
//     of 51 hands (13 entries per thread).
// Every unit's arithmetic is fixed, so the results do not depend on which warp ran it.
// The staged rows must be visible (barrier) before the call; it ends with a barrier.
constexpr int kScanQuarter = 352;  // 32 lanes x 11 sorted positions

__device__ __forceinline__ void node_tables(Block& B, int cs_row0, int n_cs, const int (&pc_rows)[2], int n_pc) {
    const BoardTabView tv = view_tables(B.tab);
    const int tid = threadIdx.x, lane = tid & 31;
    const int quads_cs = n_cs * 208, quads = quads_cs + n_pc * 208;
    const uint16_t* __restrict__ cardlist = tv.cardlist;
    const uint16_t* __restrict__ sorted = tv.sorted;
    const int n_scan = 4 * n_pc, n_units = n_scan + n_cs + (quads + 31) / 32;
    int* queue = B.misc + 2;
    while (true) {
        int unit = 0;
        if (lane == 0) unit = atomicAdd(queue, 1);
        unit = __shfl_sync(0xffffffffu, unit, 0);
        if (unit >= n_units) break;
        if (unit < n_scan) {
            // quarter scan; the last quarters (most preceding positions to add up) go first
            const int slot = unit % n_pc, qi = 3 - unit / n_pc;
            const float* __restrict__ x = B.stage_row(pc_rows[slot]);
            float* __restrict__ pref = B.pref + slot * P2B_HPAD;
            double before = 0.0;
            for (int r = 0; r < qi; ++r) {
                const int k0 = r * kScanQuarter + 11 * lane;  // all inside the row: r < 3
                float v[11];
#pragma unroll
                for (int i = 0; i < 11; ++i) v[i] = x[sorted[k0 + i]];
                double a0 = 0.0, a1 = 0.0;
#pragma unroll
                for (int i = 0; i < 11; ++i) {
                    if (i & 1) a1 += (double)v[i];
                    else a0 += (double)v[i];
                }
                before += a0 + a1;
            }
            before = warp_sum(before);
            const int k0 = qi * kScanQuarter + 11 * lane;
            float v[11];
#pragma unroll
            for (int i = 0; i < 11; ++i) v[i] = (k0 + i < P2B_NUM_HANDS) ? x[sorted[k0 + i]] : 0.0f;
            double local = 0.0;
#pragma unroll
            for (int i = 0; i < 11; ++i) local += (double)v[i];
            double incl = local;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const double up = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += up;
            }
            double run = before + (incl - local);
            if (qi == 0 && lane == 0) pref[0] = 0.0f;
#pragma unroll
            for (int i = 0; i < 11; ++i) {
                run += (double)v[i];
                if (k0 + i < P2B_NUM_HANDS) pref[k0 + i + 1] = (float)run;
            }
        } else if (unit < n_scan + n_cs) {
            // total mass of a row, on several independent accumulators (the 18 padding entries
            // of a staged row are zero, so all 1344 are added)
            const int wt = unit - n_scan;
            const float* __restrict__ x = B.stage_row(cs_row0 + wt);
            double acc[6] = {0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
#pragma unroll
            for (int b = 0; b < 7; ++b) {
                float v[6];
#pragma unroll
                for (int i = 0; i < 6; ++i) v[i] = x[lane + 32 * (6 * b + i)];
#pragma unroll
                for (int i = 0; i < 6; ++i) acc[i] += (double)v[i];
            }
            const double tot = warp_sum(((acc[0] + acc[1]) + (acc[2] + acc[3])) + (acc[4] + acc[5]));
            if (lane == 0) B.S[wt] = tot;
        } else {
            // list round: thread t of the round works on quarter q of list (row, card)
            const int t_raw = (unit - n_scan - n_cs) * 32 + lane;
            const bool valid = t_raw < quads;
            const int t = valid ? t_raw : quads - 1;  // idle threads of the last round redo the last task, unstored
            const bool is_cs = t < quads_cs;
            const int u = is_cs ? t : t - quads_cs;
            const int slot = u / 208, rem = u % 208, c = rem >> 2, q = rem & 3;
            const float* __restrict__ x = B.stage_row(is_cs ? cs_row0 + slot : pc_rows[slot > 1 ? 1 : slot]);
            // The (up to) 13 values of this quarter list, loaded before any arithmetic so that the
            // shared-memory latencies overlap.  Entry e = q + 4i (sums: interleaved) or 13q + i
            // (prefixes: contiguous); in both cases only i = 12 can fall outside the 51 entries,
            // and it does exactly when q = 3.
            float v[13];
            if (is_cs) {
                // e-th hand holding card c, in hand order: (e, c) for e < c, then (c, e + 1); its index
                // is computed, not looked up: the round is bound by shared-memory traffic
                const int row_part = combo_row_offset(c) - c;
#pragma unroll
                for (int i = 0; i < 13; ++i) {
                    const int e = q + 4 * i;
                    const int idx = e < c ? ((e * (103 - e)) >> 1) + (c - e - 1) : row_part + e;
                    v[i] = (i < 12 || q < 3) ? x[idx] : 0.0f;
                }
            } else {
                const uint16_t* __restrict__ idx_base = cardlist + 13 * q * 52 + c;
#pragma unroll
                for (int i = 0; i < 12; ++i) v[i] = x[idx_base[i * 52]];
                v[12] = q < 3 ? x[idx_base[12 * 52]] : 0.0f;
            }
            double t_even = 0.0, t_odd = 0.0;
#pragma unroll
            for (int i = 0; i < 13; ++i) {
                if (i & 1) t_odd += (double)v[i];
                else t_even += (double)v[i];
            }
            const double tot = t_even + t_odd;
            const int g = lane & ~3;
            const double t0 = __shfl_sync(0xffffffffu, tot, g), t1 = __shfl_sync(0xffffffffu, tot, g + 1);
            const double t2 = __shfl_sync(0xffffffffu, tot, g + 2), t3 = __shfl_sync(0xffffffffu, tot, g + 3);
            if (valid) {
                if (is_cs) {
                    if (q == 0) B.cs[slot * 52 + c] = ((t0 + t1) + t2) + t3;
                } else {
                    double acc = q == 0 ? 0.0 : (q == 1 ? t0 : (q == 2 ? t0 + t1 : (t0 + t1) + t2));
                    float* __restrict__ row = B.pc + slot * 52 * 52 + c * 52;
                    if (q == 0) row[0] = 0.0f;
                    float* __restrict__ out = row + 13 * q + 1;
#pragma unroll
                    for (int i = 0; i < 12; ++i) {
                        acc += (double)v[i];
                        out[i] = (float)acc;
                    }
                    if (q < 3) out[12] = (float)(acc + (double)v[12]);
                }
            }
        }
    }
    __syncthreads();
    if (tid == 0) *queue = 0;  // for the next round; the barrier that precedes it publishes the reset
}

// Showdown EV (before the pot scaling) of the hero's hands against the range x.
template <int VPT>
__device__ __forceinline__ void showdown_ev(const Block& B, const HandInfo<VPT>& hi, int tid, const float* __restrict__ x,
                                            const float* __restrict__ pref, const float* __restrict__ pc,
                                            FV<VPT>& ev) {
    const BoardTabView tv = view_tables(B.tab);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        float e = 0.0f;
        if (hi.valid[i]) {
            const int h = VPT * tid + i;
            e = showdown_hand_ev(tv.rec[h], hi.c1[i], hi.c2[i], x[h], hi.allowed[i], pref, pc);
        }
        ev.v[i] = e;
    }
}

// Runs body(ChildCount<k>) for the run-time child count k (uniform over the
// block): each instantiation is unrolled for exactly k children, so no instruction is spent
// on absent child slots.
template <int N>
struct ChildCount {
    static constexpr int value = N;
};
template <typename Body>
__device__ __forceinline__ void dispatch_children(int k, Body&& body) {
    switch (k) {
        case 1: body(ChildCount<1>{}); break;
        case 2: body(ChildCount<2>{}); break;
        case 3: body(ChildCount<3>{}); break;
        case 4: body(ChildCount<4>{}); break;
        case 5: body(ChildCount<5>{}); break;
        default:
            if constexpr (kMaxC > 6) {
                if (k == 6) body(ChildCount<6>{});
                else if (k == 7) body(ChildCount<7>{});
                else body(ChildCount<kMaxC>{});
            } else {
                body(ChildCount<kMaxC>{});
            }
            break;
    }
}

// sum over hands of x*y in the reference row-reduction order; stage rows 0/1 must be free.
template <int VPT>
__device__ __forceinline__ void dot2_reference_order(Block& B, const FV<VPT>& x0, const FV<VPT>& x1, float (&out)[2]) {
    const int tid = threadIdx.x;
    __syncthreads();
    stv<VPT>(B.stage_row(0), tid, x0);
    stv<VPT>(B.stage_row(1), tid, x1);
    __syncthreads();
    const int warp = tid >> 5;
    if (warp < 2) {
        const float sum = row_sum_reference_order(B.stage_row(warp));
        if ((tid & 31) == 0) B.fsum[warp] = sum;
    }
    __syncthreads();
    out[0] = B.fsum[0];
    out[1] = B.fsum[1];
}

// Zero-sum shift of the value outputs of one node (cfr_evaluator.py:957-980): the mean over the two
// players of sum_h values * beliefs, the sums in the reference row-reduction order.  Block-wide
// (barriers inside); stage rows 0/1 must be free.
template <int VPT>
__device__ __forceinline__ float zero_sum_shift(Block& B, const FV<VPT>& v0, const FV<VPT>& b0, const FV<VPT>& v1,
                                                const FV<VPT>& b1) {
    FV<VPT> x0, x1;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        x0.v[i] = __fmul_rn(v0.v[i], b0.v[i]);
        x1.v[i] = __fmul_rn(v1.v[i], b1.v[i]);
    }
    float sums[2];
    dot2_reference_order<VPT>(B, x0, x1, sums);
    return __fmul_rn(__fadd_rn(sums[0], sums[1]), 0.5f);
}

// ---- top-down sweep of one pass -------------------------------------------------------
template <int VPT, int MAXC, int FIXED_MODE, bool PLAIN>
__device__ __forceinline__ void sweep_down(int mode_rt, int pass, const CfrParams& p_in, Block& B, const HandInfo<VPT>& hi,
                                           const FV<VPT> (&prior)[2], int tid) {
    // PLAIN: a solve without model leaves, sampling outputs or a kept current policy; their code
    // is compiled out of this variant
    CfrParams p = p_in;
    if (PLAIN) {
        p.leaf_beliefs = nullptr;
        p.leaf_values = nullptr;
        p.policy_sample = nullptr;
        p.beliefs_last = nullptr;
        p.policy = nullptr;
        p.start_policy = nullptr;
        p.cfr_avg = 0;
        p.iter_values = 0;
    }
    // FIXED_MODE >= 0: compiled for that kind of pass alone (the iteration passes of a plain solve:
    // the start- and final-pass code stays out of the hot loop); otherwise the kind is a run-time value
    const int mode = FIXED_MODE >= 0 ? FIXED_MODE : mode_rt;
    const bool mix = (mode == kPassIter) && (p.scalars[pass].do_mix & 1) != 0;
    // cfr_avg (cfr_evaluator.py:1029, :1133): the bottom-up sweep of an iteration pass takes leaf values and
    // regret weights at the beliefs under the average policy this sweep has just updated
    const bool avgb = (mode == kPassIter) && p.cfr_avg != 0;
    // the reach and the normalisation sums under the updated average policy are also needed when the node
    // values of every iteration are kept (their zero-sum shift uses the average beliefs, :1260-1274)
    const bool avgd = (mode == kPassIter) && (p.cfr_avg != 0 || p.iter_values != 0);
    FV<VPT> mask;
#pragma unroll
    for (int i = 0; i < VPT; ++i) mask.v[i] = hi.allowed[i] ? 1.0f : 0.0f;
    int parity = 0;
    for (int ii = 0; ii < B.sg.n_internal; ++ii) {
        const int j = B.ilist[ii];
        const NodeRec nd = B.nodes[j];
        const int a = nd.to_act, k = nd.n_children, fc = nd.first_child;
        auto node_body = [&](auto kc) {
        constexpr int K = decltype(kc)::value;
        FV<VPT> ra = mask, rna = mask, rba = mask, rbna = mask;
        if (j != 0) {
            ra = ldv<VPT>(B.reach(ii, a), tid);
            rna = ldv<VPT>(B.reach(ii, 1 - a), tid);
            if (mix) {
                rba = ldv<VPT>(B.rbar(ii, a), tid);
                rbna = ldv<VPT>(B.rbar(ii, 1 - a), tid);
            }
        }
        if (mode != kPassInit) {
            // the next internal node's state rows are streamed from HBM: start them now
            if (ii + 1 < B.sg.n_internal) {
                const NodeRec nn = B.nodes[B.ilist[ii + 1]];
                prefetch_rows<VPT>(B.row1(mode == kPassFinal ? p.policy_avg : p.regrets, nn.first_child), nn.n_children, tid);
                if (mix) prefetch_rows<VPT>(B.row1(p.policy_avg, nn.first_child), nn.n_children, tid);
            }
        }
        FV<VPT> P[K], Rc[K], Pbs[K];
        if (mix) {
#pragma unroll
            for (int c = 0; c < K; ++c)
                Pbs[c] = ldv<VPT>(B.row1(p.policy_avg, fc + c), tid);
        }
        children_policy<VPT, K>(mode, p, B, fc, k, tid, P, Rc);

        if (mode == kPassInit) {
            // Start beliefs.  Upstream pushes beliefs down one level at a time and re-normalises
            // EVERY row after each level (cfr_evaluator.py:855-875), so a node at level L is
            // normalised init_depth-L+1 times and its children derive from its once-normalised
            // row.  During this pass the work rows hold: reach = once-normalised beliefs,
            // rbar = final start beliefs.
            FV<VPT> b1a, b1o;  // once-normalised beliefs of the acting / the other player
            if (j == 0) {
                b1a = pick<VPT>(prior, a);
                b1o = pick<VPT>(prior, 1 - a);
            } else {
                b1a = ldv<VPT>(B.reach(ii, a), tid);
                b1o = ldv<VPT>(B.reach(ii, 1 - a), tid);
            }
#pragma unroll
            for (int c = 0; c < K; ++c) {
                const NodeRec ch = B.nodes[fc + c];
                stv<VPT>(B.row1(p.policy_avg, fc + c), tid, P[c]);
                if (ch.kind != kInternal && !(ch.kind == kModelLeaf && p.leaf_beliefs)) continue;
                FV<VPT> x[2];
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const float xa = __fmul_rn(b1a.v[i], P[c].v[i]);
                    x[0].v[i] = a == 0 ? xa : b1o.v[i];
                    x[1].v[i] = a == 0 ? b1o.v[i] : xa;
                }
                if (ch.kind == kModelLeaf) {  // a leaf row is normalised once per level from its own down
                    for (int rep = ch.depth; rep <= p.init_depth; ++rep) normalize2<VPT>(B, hi, x);
                    stv<VPT>(p.leaf_beliefs + B.leaf_row(ch.internal_idx, 0), tid, x[0]);
                    stv<VPT>(p.leaf_beliefs + B.leaf_row(ch.internal_idx, 1), tid, x[1]);
                    continue;
                }
                normalize2<VPT>(B, hi, x);
                stv<VPT>(B.reach(ch.internal_idx, 0), tid, x[0]);
                stv<VPT>(B.reach(ch.internal_idx, 1), tid, x[1]);
                for (int rep = ch.depth; rep < p.init_depth; ++rep) normalize2<VPT>(B, hi, x);
                stv<VPT>(B.rbar(ch.internal_idx, 0), tid, x[0]);
                stv<VPT>(B.rbar(ch.internal_idx, 1), tid, x[1]);
            }
            return;
        }

        if (mode == kPassIter) {
            // average policy of the children
            FV<VPT> Pn[K];
            if (mix) {
                const IterScalars sc = p.scalars[pass];
                // weights of the old average and of the new policy: reach-weighted, or the plain
                // iteration weights where the hand has (numerically) no reach (:1231-1239)
                FV<VPT> ro, rn, sum;
                Divisor dmix[VPT];
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    ro.v[i] = __fmul_rn(rba.v[i], sc.mix_old);
                    rn.v[i] = __fmul_rn(ra.v[i], sc.mix_new);
                    const float den = __fadd_rn(ro.v[i], rn.v[i]);
                    const bool weighted = den > 1e-5f;
                    ro.v[i] = weighted ? ro.v[i] : sc.mix_old;
                    rn.v[i] = weighted ? rn.v[i] : sc.mix_new;
                    dmix[i] = make_divisor(weighted ? den : sc.mix_total);
                    sum.v[i] = 0.0f;
                }
#pragma unroll
                for (int c = 0; c < K; ++c)
                    {
                        const FV<VPT> Pb = Pbs[c];
                        const NodeRec ch = B.nodes[fc + c];
                        if (ch.kind == kInternal) {  // average reach under the OLD average policy
                            FV<VPT> t;
#pragma unroll
                            for (int i = 0; i < VPT; ++i) t.v[i] = __fmul_rn(rba.v[i], Pb.v[i]);
                            stv<VPT>(B.rbar(ch.internal_idx, a), tid, t);
                            stv<VPT>(B.rbar(ch.internal_idx, 1 - a), tid, rbna);
                        }
                        bool bad = false;
                        FV<VPT> num;
#pragma unroll
                        for (int i = 0; i < VPT; ++i) {
                            num.v[i] = __fadd_rn(__fmul_rn(ro.v[i], Pb.v[i]), __fmul_rn(rn.v[i], P[c].v[i]));
                            Pn[c].v[i] = div_fast<true>(num.v[i], dmix[i], bad);
                        }
                        if (__builtin_expect(bad, 0)) {
#pragma unroll
                            for (int i = 0; i < VPT; ++i) Pn[c].v[i] = __fdiv_rn(num.v[i], dmix[i].y);
                        }
#pragma unroll
                        for (int i = 0; i < VPT; ++i) sum.v[i] = __fadd_rn(sum.v[i], Pn[c].v[i]);
                    }
                Divisor dsum[VPT];
#pragma unroll
                for (int i = 0; i < VPT; ++i) dsum[i] = make_divisor(sum.v[i]);
                {
                    bool bad = false;
                    FV<VPT> Q[K];
#pragma unroll
                    for (int c = 0; c < K; ++c)
                        {
#pragma unroll
                            for (int i = 0; i < VPT; ++i) Q[c].v[i] = div_fast<true>(Pn[c].v[i], dsum[i], bad);
                        }
                    if (__builtin_expect(bad, 0)) {
#pragma unroll
                        for (int c = 0; c < K; ++c)
                            {
#pragma unroll
                                for (int i = 0; i < VPT; ++i) Q[c].v[i] = __fdiv_rn(Pn[c].v[i], sum.v[i]);
                            }
                    }
#pragma unroll
                    for (int c = 0; c < K; ++c)
                        {
#pragma unroll
                            for (int i = 0; i < VPT; ++i)
                                if (sum.v[i] > 1e-5f) Pn[c].v[i] = Q[c].v[i];
                            stv<VPT>(B.row1(p.policy_avg, fc + c), tid, Pn[c]);
                        }
                }
            } else {
#pragma unroll
                for (int c = 0; c < K; ++c)
                    stv<VPT>(B.row1(p.policy_avg, fc + c), tid, P[c]);
            }
            if (p.policy && pass == p.iterations - 1) {
#pragma unroll
                for (int c = 0; c < K; ++c)
                    stv<VPT>(B.row1(p.policy, fc + c), tid, P[c]);
            }
            if (p.policy_sample && pass == B.sample_pass) {
#pragma unroll
                for (int c = 0; c < K; ++c)
                    stv<VPT>(B.row1(p.policy_sample, fc + c), tid, P[c]);
            }
        }
        // reach of the children under the policy of this pass, and the rows whose sums
        // normalise the children's beliefs (only the acting player's row is new: the other
        // player's row, hence its sum, is the parent's)
        const int bank = parity * kBankRows;
        parity ^= 1;
        const FV<VPT> prior_a = pick<VPT>(prior, a);
#pragma unroll
        for (int c = 0; c < K; ++c)
            {
                const NodeRec ch = B.nodes[fc + c];
                if (ch.kind == kFoldLeaf || (ch.kind == kModelLeaf && !p.leaf_beliefs)) continue;
                FV<VPT> t, u;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    t.v[i] = __fmul_rn(ra.v[i], P[c].v[i]);
                    u.v[i] = __fmul_rn(prior_a.v[i], t.v[i]);
                }
                stv<VPT>(B.stage_row(bank + c), tid, u);
                if (ch.kind == kModelLeaf && !avgb) {
                    // unnormalised rows now; normalised in place at the end of the sweep, when
                    // the sums are known
                    const FV<VPT> prior_o = pick<VPT>(prior, 1 - a);
                    FV<VPT> w;
#pragma unroll
                    for (int i = 0; i < VPT; ++i) w.v[i] = __fmul_rn(prior_o.v[i], rna.v[i]);
                    stv<VPT>(p.leaf_beliefs + B.leaf_row(ch.internal_idx, a), tid, u);
                    stv<VPT>(p.leaf_beliefs + B.leaf_row(ch.internal_idx, 1 - a), tid, w);
                }
                if (ch.kind == kInternal) {
                    stv<VPT>(B.reach(ch.internal_idx, a), tid, t);
                    stv<VPT>(B.reach(ch.internal_idx, 1 - a), tid, rna);
                }
            }
        __syncthreads();
        const int warp = tid >> 5;
        if (warp < k) {
            const NodeRec ch = B.nodes[fc + warp];
            if (ch.kind == kInternal || ch.kind == kShowdownLeaf || (ch.kind == kModelLeaf && p.leaf_beliefs)) {
                const float sum = row_sum_reference_order(B.stage_row(bank + warp));
                if ((tid & 31) == 0) {
                    B.sig[(fc + warp) * 2 + a] = sum;
                    B.sig[(fc + warp) * 2 + 1 - a] = B.sig[j * 2 + 1 - a];
                }
            }
        }
        if (avgd) {
            // the same once more under the average policy as updated above (its rows were just stored by
            // this thread): reach, the rows whose sums normalise the children's average beliefs
            FV<VPT> rwa = mask, rwna = mask;
            if (j != 0) {
                rwa = ldv<VPT>(B.rnew(ii, a), tid);
                rwna = ldv<VPT>(B.rnew(ii, 1 - a), tid);
            }
            __syncthreads();  // the warps are done adding up the bank
#pragma unroll
            for (int c = 0; c < K; ++c) {
                const NodeRec ch = B.nodes[fc + c];
                if (ch.kind == kFoldLeaf || (ch.kind == kModelLeaf && !p.leaf_beliefs)) continue;
                const FV<VPT> Pa = ldv<VPT>(B.row1(p.policy_avg, fc + c), tid);
                FV<VPT> t, u;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    t.v[i] = __fmul_rn(rwa.v[i], Pa.v[i]);
                    u.v[i] = __fmul_rn(prior_a.v[i], t.v[i]);
                }
                stv<VPT>(B.stage_row(bank + c), tid, u);
                if (ch.kind == kModelLeaf && avgb) {  // the caller's model sees the average beliefs
                    const FV<VPT> prior_o = pick<VPT>(prior, 1 - a);
                    FV<VPT> w;
#pragma unroll
                    for (int i = 0; i < VPT; ++i) w.v[i] = __fmul_rn(prior_o.v[i], rwna.v[i]);
                    stv<VPT>(p.leaf_beliefs + B.leaf_row(ch.internal_idx, a), tid, u);
                    stv<VPT>(p.leaf_beliefs + B.leaf_row(ch.internal_idx, 1 - a), tid, w);
                }
                if (ch.kind == kInternal) {
                    stv<VPT>(B.rnew(ch.internal_idx, a), tid, t);
                    stv<VPT>(B.rnew(ch.internal_idx, 1 - a), tid, rwna);
                }
            }
            __syncthreads();
            if (warp < k) {
                const NodeRec ch = B.nodes[fc + warp];
                if (ch.kind == kInternal || ch.kind == kShowdownLeaf || (ch.kind == kModelLeaf && p.leaf_beliefs)) {
                    const float sum = row_sum_reference_order(B.stage_row(bank + warp));
                    if ((tid & 31) == 0) {
                        B.sigb[(fc + warp) * 2 + a] = sum;
                        B.sigb[(fc + warp) * 2 + 1 - a] = B.sigb[j * 2 + 1 - a];
                    }
                }
            }
        }
        };
        dispatch_children(k, node_body);
    }
    __syncthreads();
    if (p.leaf_beliefs && mode != kPassInit) {
        // beliefs at the model leaves: divide the rows written above by their sums
        for (int j = 1; j < B.sg.n_nodes; ++j) {
            const NodeRec nd = B.nodes[j];
            if (nd.kind != kModelLeaf) continue;
#pragma unroll
            for (int pl = 0; pl < 2; ++pl) {
                float* row = p.leaf_beliefs + B.leaf_row(nd.internal_idx, pl);
                FV<VPT> x = ldv<VPT>(row, tid);
                apply_norm<VPT>(B, hi, x, (avgb ? B.sigb : B.sig)[j * 2 + pl]);
                stv<VPT>(row, tid, x);
            }
        }
    }
}

// ---- bottom-up sweep of one pass ------------------------------------------------------
// Suffix _a: the player acting at the node, _o: the other player.  Per node: stage every
// row that needs cross-hand work, one block-wide round of that work (node_tables), then
// the per-hand arithmetic with no further barrier.  Staging rows: 0 = beliefs of the
// acting player, 1 = of the other player, 2+c = marginal policy of child c, 8+c = beliefs
// of the acting player at showdown child c.
template <int VPT, int MAXC, int FIXED_MODE, bool PLAIN>
__device__ __forceinline__ void sweep_up(int mode_rt, int pass, const CfrParams& p_in, Block& B, const HandInfo<VPT>& hi,
                                         const FV<VPT> (&prior)[2], const FV<VPT> (&root_b)[2], int s, int tid) {
    // PLAIN: a solve without model leaves, sampling outputs or a kept current policy; their code
    // is compiled out of this variant
    CfrParams p = p_in;
    if (PLAIN) {
        p.leaf_beliefs = nullptr;
        p.leaf_values = nullptr;
        p.policy_sample = nullptr;
        p.beliefs_last = nullptr;
        p.policy = nullptr;
        p.start_policy = nullptr;
        p.cfr_avg = 0;
        p.iter_values = 0;
    }
    const int mode = FIXED_MODE >= 0 ? FIXED_MODE : mode_rt;
    const bool update = (mode != kPassFinal) && (pass + 1 < p.iterations);
    const bool avgb = (mode == kPassIter) && p.cfr_avg != 0;  // see sweep_down
    const bool avgd = (mode == kPassIter) && (p.cfr_avg != 0 || p.iter_values != 0);
    const bool keep_values = (mode == kPassFinal || p.iter_values != 0) && p.values_avg != nullptr;
    const bool keep_avg_beliefs = mode == kPassIter && p.iter_values != 0 && p.beliefs_avg != nullptr;
    constexpr int kRowM = 2, kRowLeaf = 2 + kBankRows;
    FV<VPT> mask;
#pragma unroll
    for (int i = 0; i < VPT; ++i) mask.v[i] = hi.allowed[i] ? 1.0f : 0.0f;
    for (int ii = B.sg.n_internal - 1; ii >= 0; --ii) {
        const int j = B.ilist[ii];
        const NodeRec nd = B.nodes[j];
        const int a = nd.to_act, o = 1 - a, k = nd.n_children, fc = nd.first_child;
        auto node_body = [&](auto kc) {
        constexpr int K = decltype(kc)::value;
        const FV<VPT> prior_a = pick<VPT>(prior, a), prior_o = pick<VPT>(prior, o);
        // r: reach of both players (start pass: once-normalised start beliefs, see sweep_down)
        FV<VPT> r_a, r_o, b_a, b_o;
        if (j == 0) {
            r_a = mode == kPassInit ? prior_a : mask;
            r_o = mode == kPassInit ? prior_o : mask;
            b_a = pick<VPT>(root_b, a);
            b_o = pick<VPT>(root_b, o);
        } else {
            r_a = ldv<VPT>(B.reach(ii, a), tid);
            r_o = ldv<VPT>(B.reach(ii, o), tid);
            if (mode == kPassInit) {
                b_a = ldv<VPT>(B.rbar(ii, a), tid);
                b_o = ldv<VPT>(B.rbar(ii, o), tid);
            } else {
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    b_a.v[i] = __fmul_rn(prior_a.v[i], r_a.v[i]);
                    b_o.v[i] = __fmul_rn(prior_o.v[i], r_o.v[i]);
                }
                apply_norm<VPT>(B, hi, b_a, B.sig[j * 2 + a]);
                apply_norm<VPT>(B, hi, b_o, B.sig[j * 2 + o]);
            }
        }
        // x_o: the other player's beliefs that weight the regrets and meet the acting player's hands at a
        // showdown; rw_a: the acting player's reach the showdown leaves' beliefs derive from.  With cfr_avg
        // both are taken under the average policy (at the root the two kinds of beliefs are the same row).
        FV<VPT> x_o = b_o, rw_a = r_a;
        FV<VPT> bbar_o = b_o, rbar_a = mask;  // average beliefs of the other player, average reach of the acting one
        if (avgd && j != 0) {
            rbar_a = ldv<VPT>(B.rnew(ii, a), tid);
            const FV<VPT> rw_o = ldv<VPT>(B.rnew(ii, o), tid);
#pragma unroll
            for (int i = 0; i < VPT; ++i) bbar_o.v[i] = __fmul_rn(prior_o.v[i], rw_o.v[i]);
            apply_norm<VPT>(B, hi, bbar_o, B.sigb[j * 2 + o]);
        }
        if (avgb) {
            rw_a = rbar_a;
            x_o = bbar_o;
        }
        if (keep_avg_beliefs) {
            // beliefs under the average policy at this node and at the leaves below it that the caller's
            // model values (terminal nodes are exempt from the zero-sum shift that reads them)
            FV<VPT> bbar_a = b_a;
            if (j != 0) {
#pragma unroll
                for (int i = 0; i < VPT; ++i) bbar_a.v[i] = __fmul_rn(prior_a.v[i], rbar_a.v[i]);
                apply_norm<VPT>(B, hi, bbar_a, B.sigb[j * 2 + a]);
            }
            stv<VPT>(B.row2(p.beliefs_avg, j, a), tid, bbar_a);
            stv<VPT>(B.row2(p.beliefs_avg, j, o), tid, bbar_o);
            for (int c = 0; c < k; ++c) {
                if (B.nodes[fc + c].kind != kModelLeaf) continue;
                const FV<VPT> Pa = ldv<VPT>(B.row1(p.policy_avg, fc + c), tid);
                FV<VPT> bl;
#pragma unroll
                for (int i = 0; i < VPT; ++i) bl.v[i] = __fmul_rn(prior_a.v[i], __fmul_rn(rbar_a.v[i], Pa.v[i]));
                apply_norm<VPT>(B, hi, bl, B.sigb[(fc + c) * 2 + a]);
                stv<VPT>(B.row2(p.beliefs_avg, fc + c, a), tid, bl);
                stv<VPT>(B.row2(p.beliefs_avg, fc + c, o), tid, bbar_o);
            }
        }
        {
            if (ii > 0) {
                const NodeRec nn = B.nodes[B.ilist[ii - 1]];
                prefetch_rows<VPT>(B.row1(mode == kPassFinal ? p.policy_avg : p.regrets, nn.first_child), nn.n_children, tid);
                if (update && p.weight_sums) prefetch_rows<VPT>(B.row1(p.weight_sums, nn.first_child), nn.n_children, tid);
            }
        }
        FV<VPT> P[K], Rc[K], Va[K], acc_a, acc_o;
        children_policy<VPT, K>(mode, p, B, fc, k, tid, P, Rc);

        // ---- stage ----
        int first_sd = -1;
#pragma unroll
        for (int c = 0; c < K; ++c) {
            const NodeRec ch = B.nodes[fc + c];
            if (ch.kind != kShowdownLeaf) continue;
            if (first_sd < 0) first_sd = c;
            FV<VPT> bca;  // beliefs of the acting player at the leaf
            if (mode == kPassInit) {
                FV<VPT> x[2];
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const float xa = __fmul_rn(r_a.v[i], P[c].v[i]);
                    x[0].v[i] = a == 0 ? xa : r_o.v[i];
                    x[1].v[i] = a == 0 ? r_o.v[i] : xa;
                }
                for (int rep = ch.depth; rep <= p.init_depth; ++rep) normalize2<VPT>(B, hi, x);
                bca = pick<VPT>(x, a);
            } else if (avgb) {
                const FV<VPT> Pa = ldv<VPT>(B.row1(p.policy_avg, fc + c), tid);
#pragma unroll
                for (int i = 0; i < VPT; ++i) bca.v[i] = __fmul_rn(prior_a.v[i], __fmul_rn(rw_a.v[i], Pa.v[i]));
                apply_norm<VPT>(B, hi, bca, B.sigb[(fc + c) * 2 + a]);
            } else {
#pragma unroll
                for (int i = 0; i < VPT; ++i) bca.v[i] = __fmul_rn(prior_a.v[i], __fmul_rn(r_a.v[i], P[c].v[i]));
                apply_norm<VPT>(B, hi, bca, B.sig[(fc + c) * 2 + a]);
            }
            stv<VPT>(B.stage_row(kRowLeaf + c), tid, bca);
            if (mode == kPassFinal && p.beliefs_avg) {
                stv<VPT>(B.row2(p.beliefs_avg, fc + c, a), tid, bca);
                stv<VPT>(B.row2(p.beliefs_avg, fc + c, o), tid, b_o);
            }
        }
        stv<VPT>(B.stage_row(0), tid, b_a);
        stv<VPT>(B.stage_row(1), tid, x_o);
#pragma unroll
        for (int c = 0; c < K; ++c)
            {
                FV<VPT> m;
#pragma unroll
                for (int i = 0; i < VPT; ++i) m.v[i] = __fmul_rn(b_a.v[i], P[c].v[i]);
                stv<VPT>(B.stage_row(kRowM + c), tid, m);
            }
        if (mode == kPassFinal && p.beliefs_avg) {
            stv<VPT>(B.row2(p.beliefs_avg, j, a), tid, b_a);
            stv<VPT>(B.row2(p.beliefs_avg, j, o), tid, b_o);
        }
        if (p.beliefs_last && mode == kPassIter && pass == p.iterations - 1) {
            stv<VPT>(B.row2(p.beliefs_last, j, a), tid, b_a);
            stv<VPT>(B.row2(p.beliefs_last, j, o), tid, b_o);
        }
        __syncthreads();

        // ---- cross-hand work: per-card sums of every row, showdown tables of the other
        // player's beliefs (they serve the acting player at every showdown child) and of the
        // first showdown child ----
        {
            int pc_rows[2] = {1, first_sd >= 0 ? kRowLeaf + first_sd : 1};
            node_tables(B, 0, 2 + k, pc_rows, first_sd >= 0 ? 2 : 0);
        }
        // ---- per-hand arithmetic ----
        FV<VPT> wgt, denm, eva;
        Divisor ddenm[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            wgt.v[i] = unblocked(B.cs + 52, B.S[1], hi.c1[i], hi.c2[i], x_o.v[i]);
            denm.v[i] = unblocked(B.cs, B.S[0], hi.c1[i], hi.c2[i], b_a.v[i]);
            ddenm[i] = make_divisor(denm.v[i]);
            eva.v[i] = 0.0f;
            acc_a.v[i] = acc_o.v[i] = 0.0f;
        }
        if (first_sd >= 0) showdown_ev<VPT>(B, hi, tid, B.stage_row(1), B.pref, B.pc, eva);
        // Further showdown children (rare: none in a river tree): one more round each builds the
        // child's tables in slot 0 (the acting player's EV, the only user of slot 0, is already in
        // registers) and the opponent's EV replaces the child's staged beliefs, of which a thread
        // reads its own two entries only.  Kept out of the unrolled loop below: one copy of the
        // round's code per node body instead of one per child.
        if (first_sd >= 0) {
#pragma unroll 1
            for (int c = first_sd + 1; c < k; ++c) {
                if (B.nodes[fc + c].kind != kShowdownLeaf) continue;
                __syncthreads();
                int pc_rows[2] = {kRowLeaf + c, kRowLeaf + c};
                node_tables(B, 0, 0, pc_rows, 1);
                FV<VPT> evo;
                showdown_ev<VPT>(B, hi, tid, B.stage_row(kRowLeaf + c), B.pref, B.pc, evo);
                stv<VPT>(B.stage_row(kRowLeaf + c), tid, evo);
            }
        }

#pragma unroll
        for (int c = 0; c < K; ++c) {
            const NodeRec ch = B.nodes[fc + c];
            // policy of this child as seen by each opponent hand (cfr_evaluator.py:1083-1093)
            FV<VPT> pio, blk;
            {
                bool bad = false;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const float m = __fmul_rn(b_a.v[i], P[c].v[i]);
                    blk.v[i] = unblocked(B.cs + (kRowM + c) * 52, B.S[kRowM + c], hi.c1[i], hi.c2[i], m);
                    pio.v[i] = div_fast<true>(blk.v[i], ddenm[i], bad);
                }
                if (__builtin_expect(bad, 0)) {
#pragma unroll
                    for (int i = 0; i < VPT; ++i) pio.v[i] = __fdiv_rn(blk.v[i], denm.v[i]);
                }
#pragma unroll
                for (int i = 0; i < VPT; ++i) pio.v[i] = denm.v[i] > 1e-5f ? pio.v[i] : 0.0f;
            }
            FV<VPT> V_a, V_o;
            if (ch.kind == kFoldLeaf) {
                const float va = a == 0 ? ch.v0 : -ch.v0;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    V_a.v[i] = va;
                    V_o.v[i] = -va;
                }
            } else if (ch.kind == kInternal) {
                V_a = ldv<VPT>(B.val(ch.internal_idx, a), tid);
                V_o = ldv<VPT>(B.val(ch.internal_idx, o), tid);
            } else if (ch.kind == kShowdownLeaf) {
                FV<VPT> evo;
                if (c == first_sd) {
                    showdown_ev<VPT>(B, hi, tid, B.stage_row(kRowLeaf + c), B.pref + P2B_HPAD, B.pc + 52 * 52, evo);
                } else {
                    evo = ldv<VPT>(B.stage_row(kRowLeaf + c), tid);  // computed above
                }
                const float pot_a = a == 0 ? ch.v0 : ch.v1, pot_o = a == 0 ? ch.v1 : ch.v0;
                const Divisor dscale = make_divisor(B.sg.scale);
                bool bad = false;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    V_a.v[i] = div_fast(__fmul_rn(eva.v[i], pot_a), dscale, bad);
                    V_o.v[i] = div_fast(__fmul_rn(evo.v[i], pot_o), dscale, bad);
                }
                if (__builtin_expect(bad, 0)) {
#pragma unroll
                    for (int i = 0; i < VPT; ++i) {
                        V_a.v[i] = __fdiv_rn(__fmul_rn(eva.v[i], pot_a), B.sg.scale);
                        V_o.v[i] = __fdiv_rn(__fmul_rn(evo.v[i], pot_o), B.sg.scale);
                    }
                }
            } else if (p.leaf_values) {  // valued by the caller's model between the sweeps
                V_a = ldv<VPT>(p.leaf_values + B.leaf_row(ch.internal_idx, a), tid);
                V_o = ldv<VPT>(p.leaf_values + B.leaf_row(ch.internal_idx, o), tid);
            } else {
#pragma unroll
                for (int i = 0; i < VPT; ++i) V_a.v[i] = V_o.v[i] = 0.0f;
            }
            if (keep_values && ch.kind != kInternal) {
                FV<VPT> out_a = V_a, out_o = V_o;
                if (mode == kPassFinal && p.enforce_zero_sum && ch.kind == kModelLeaf && p.leaf_beliefs) {
                    // a leaf that is not terminal is shifted like an inner node, by its own beliefs
                    const FV<VPT> la = ldv<VPT>(p.leaf_beliefs + B.leaf_row(ch.internal_idx, a), tid);
                    const FV<VPT> lo = ldv<VPT>(p.leaf_beliefs + B.leaf_row(ch.internal_idx, o), tid);
                    const float shift = zero_sum_shift<VPT>(B, V_a, la, V_o, lo);
#pragma unroll
                    for (int i = 0; i < VPT; ++i) {
                        out_a.v[i] = __fsub_rn(V_a.v[i], shift);
                        out_o.v[i] = __fsub_rn(V_o.v[i], shift);
                    }
                }
                stv<VPT>(B.row2(p.values_avg, fc + c, a), tid, out_a);
                stv<VPT>(B.row2(p.values_avg, fc + c, o), tid, out_o);
            }
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                acc_a.v[i] = __fadd_rn(acc_a.v[i], __fmul_rn(V_a.v[i], P[c].v[i]));
                acc_o.v[i] = __fadd_rn(acc_o.v[i], __fmul_rn(V_o.v[i], pio.v[i]));
            }
            Va[c] = V_a;
        }
        if (j != 0) {
            stv<VPT>(B.val(ii, a), tid, acc_a);
            stv<VPT>(B.val(ii, o), tid, acc_o);
        }
        if (mode != kPassFinal && keep_values) {  // the values of this iteration, as they are
            stv<VPT>(B.row2(p.values_avg, j, a), tid, acc_a);
            stv<VPT>(B.row2(p.values_avg, j, o), tid, acc_o);
        }
        if (mode == kPassFinal) {
            // the outputs may be shifted to zero sum; the work rows the parent backs up from are not
            FV<VPT> out_a = acc_a, out_o = acc_o;
            if (p.enforce_zero_sum && (p.values_avg || j == 0)) {
                const float shift = zero_sum_shift<VPT>(B, acc_a, b_a, acc_o, b_o);
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    out_a.v[i] = __fsub_rn(acc_a.v[i], shift);
                    out_o.v[i] = __fsub_rn(acc_o.v[i], shift);
                }
            }
            if (p.values_avg) {
                stv<VPT>(B.row2(p.values_avg, j, a), tid, out_a);
                stv<VPT>(B.row2(p.values_avg, j, o), tid, out_o);
            }
            if (j == 0) {
                stv<VPT>(p.root_values + ((long long)s * 2 + a) * P2B_HPAD, tid, out_a);
                stv<VPT>(p.root_values + ((long long)s * 2 + o) * P2B_HPAD, tid, out_o);
            }
        }
        if (update) {
            // instantaneous regrets of this pass folded into the discounted update of the next
            const IterScalars sc = p.scalars[pass + 1];
            const Divisor d_pos = make_divisor(sc.den_pos), d_neg = make_divisor(sc.den_neg);
            // linear CFR: at that iteration the actions of one player get no regret (:1348-1349)
            const bool no_regret = ((sc.do_mix >> 1) & 3) == a + 1;
            FV<VPT> ws[K];
#pragma unroll
            for (int c = 0; c < K; ++c) {
#pragma unroll
                for (int i = 0; i < VPT; ++i) ws[c].v[i] = 0.0f;
                if (p.weight_sums && mode != kPassInit) ws[c] = ldv<VPT>(B.row1(p.weight_sums, fc + c), tid);
            }
#pragma unroll
            for (int c = 0; c < K; ++c)
                {
                    FV<VPT> w = ws[c], rn, wn, rq, wq;
                    Divisor d[VPT];
                    bool bad = false;
#pragma unroll
                    for (int i = 0; i < VPT; ++i) {
                        const bool pos = Rc[c].v[i] > 0.0f;
                        const float num = pos ? sc.num_pos : sc.num_neg;
                        d[i].y = pos ? d_pos.y : d_neg.y;
                        d[i].r = pos ? d_pos.r : d_neg.r;
                        d[i].ok = d_pos.ok && d_neg.ok;
                        rn.v[i] = __fmul_rn(Rc[c].v[i], num);
                        wn.v[i] = __fmul_rn(w.v[i], num);
                        rq.v[i] = div_fast(rn.v[i], d[i], bad);
                        wq.v[i] = div_fast<true>(wn.v[i], d[i], bad);
                    }
                    if (__builtin_expect(bad, 0)) {
#pragma unroll
                        for (int i = 0; i < VPT; ++i) {
                            rq.v[i] = __fdiv_rn(rn.v[i], d[i].y);
                            wq.v[i] = __fdiv_rn(wn.v[i], d[i].y);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < VPT; ++i) {
                        const float reg = no_regret ? 0.0f : __fmul_rn(wgt.v[i], __fsub_rn(Va[c].v[i], acc_a.v[i]));
                        float rr = __fadd_rn(rq.v[i], reg);
                        if (p.cfr_plus) rr = fmaxf(rr, 0.0f);
                        Rc[c].v[i] = rr;
                        w.v[i] = __fadd_rn(wq.v[i], 1.0f);
                    }
                    stv<VPT>(B.row1(p.regrets, fc + c), tid, Rc[c]);
                    if (p.weight_sums) stv<VPT>(B.row1(p.weight_sums, fc + c), tid, w);
                }
        }
        };
        dispatch_children(k, node_body);
    }
}

// ---- best-response sweeps (local exploitability of the average policy) -------------------
// Upstream: `_compute_exploitability` / `_best_response_values`
// (p2/search/cfr_evaluator.py:603-764).  Runs after the final pass, whose reach rows and
// normalisation sums are still in place.  Leaf values are the final-pass values clamped to
// [-1,1] (:730), read back from p.values_avg.  deviator < 0: plain expectation under the
// average policy (`base_values`, :732-735); deviator = d: player d plays a best response.
// Returns the root values of both players in root_v (index = player).
//
// warm = true: the best-response pass of a warm start of type `model_br` (:927-955), run after the start
// pass.  Beliefs are the start beliefs (kept in the rbar rows by that pass), the policy is the start policy
// (stored as the average policy), leaf values are the start pass's own (values_avg, not clamped), and at
// every node where the deviator acts the regrets of its children are SET to
// unblocked(other player's beliefs) x (best-response value of the child - the node's value under the
// start policy) -- `compute_instantaneous_regrets(values_br, latest_values)`; the caller scales them.
template <int VPT, int MAXC>
__device__ __forceinline__ void sweep_br(int deviator, const CfrParams& p, Block& B, const HandInfo<VPT>& hi,
                                         const FV<VPT> (&prior)[2], const FV<VPT> (&root_b)[2], int tid,
                                         FV<VPT> (&root_v)[2], bool warm = false) {
    constexpr int kRowM = 2;
    FV<VPT> mask;
#pragma unroll
    for (int i = 0; i < VPT; ++i) mask.v[i] = hi.allowed[i] ? 1.0f : 0.0f;
    for (int j = B.sg.n_nodes - 1; j >= 0; --j) {
        const NodeRec nd = B.nodes[j];
        if (nd.kind != kInternal) continue;
        const int a = nd.to_act, o = 1 - a, k = nd.n_children, fc = nd.first_child, ii = nd.internal_idx;
        auto node_body = [&](auto kc) {
        constexpr int K = decltype(kc)::value;
        const bool deviates = deviator == a;
        FV<VPT> b_a;  // beliefs of the acting player under the average policy
        FV<VPT> b_o;  // warm start only: the other player's
        if (j == 0) {
            b_a = pick<VPT>(root_b, a);
            b_o = pick<VPT>(root_b, o);
        } else if (warm) {
            b_a = ldv<VPT>(B.rbar(ii, a), tid);
            b_o = ldv<VPT>(B.rbar(ii, o), tid);
        } else {
            const FV<VPT> prior_a = pick<VPT>(prior, a);
            const FV<VPT> r_a = ldv<VPT>(B.reach(ii, a), tid);
#pragma unroll
            for (int i = 0; i < VPT; ++i) b_a.v[i] = __fmul_rn(prior_a.v[i], r_a.v[i]);
            apply_norm<VPT>(B, hi, b_a, B.sig[j * 2 + a]);
        }
        // child values of both players (leaves: clamped final values; internal: this sweep)
        FV<VPT> Va[K], Vo[K], P[K];
#pragma unroll
        for (int c = 0; c < K; ++c) {
            const NodeRec ch = B.nodes[fc + c];
            if (ch.kind == kInternal) {
                Va[c] = ldv<VPT>(B.val(ch.internal_idx, a), tid);
                Vo[c] = ldv<VPT>(B.val(ch.internal_idx, o), tid);
            } else {
                Va[c] = ldv<VPT>(B.row2(p.values_avg, fc + c, a), tid);
                Vo[c] = ldv<VPT>(B.row2(p.values_avg, fc + c, o), tid);
                if (!warm) {
#pragma unroll
                    for (int i = 0; i < VPT; ++i) {
                        Va[c].v[i] = fminf(fmaxf(Va[c].v[i], -1.0f), 1.0f);
                        Vo[c].v[i] = fminf(fmaxf(Vo[c].v[i], -1.0f), 1.0f);
                    }
                }
            }
            P[c] = ldv<VPT>(B.row1(p.policy_avg, fc + c), tid);
        }
        // best action of the deviating player per hand: first maximum (argmax, :653-660)
        FV<VPT> best_v;
        int best_c[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            best_v.v[i] = Va[0].v[i];
            best_c[i] = 0;
        }
#pragma unroll
        for (int c = 1; c < K; ++c)
            {
#pragma unroll
                for (int i = 0; i < VPT; ++i)
                    if (Va[c].v[i] > best_v.v[i]) {
                        best_v.v[i] = Va[c].v[i];
                        best_c[i] = c;
                    }
            }
        // rows whose unblocked mass is needed: the acting player's beliefs (matchup mass) and,
        // per child, either the belief mass that picks it (deviator) or belief x policy
        stv<VPT>(B.stage_row(0), tid, b_a);
        stv<VPT>(B.stage_row(1), tid, warm ? b_o : b_a);
#pragma unroll
        for (int c = 0; c < K; ++c)
            {
                FV<VPT> m;
#pragma unroll
                for (int i = 0; i < VPT; ++i)
                    m.v[i] = deviates ? (best_c[i] == c ? b_a.v[i] : 0.0f) : __fmul_rn(P[c].v[i], b_a.v[i]);
                stv<VPT>(B.stage_row(kRowM + c), tid, m);
            }
        __syncthreads();
        {
            int pc_rows[2] = {0, 0};
            node_tables(B, 0, 2 + k, pc_rows, 0);
        }
        FV<VPT> acc_a, acc_o;
#pragma unroll
        for (int i = 0; i < VPT; ++i) acc_a.v[i] = acc_o.v[i] = 0.0f;
#pragma unroll
        for (int c = 0; c < K; ++c)
            {
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const float m = deviates ? (best_c[i] == c ? b_a.v[i] : 0.0f) : __fmul_rn(P[c].v[i], b_a.v[i]);
                    const float blk = unblocked(B.cs + (kRowM + c) * 52, B.S[kRowM + c], hi.c1[i], hi.c2[i], m);
                    const float den = unblocked(B.cs, B.S[0], hi.c1[i], hi.c2[i], b_a.v[i]);
                    const float w = den > 1e-5f ? __fdiv_rn(blk, den) : 0.0f;
                    acc_o.v[i] = __fadd_rn(acc_o.v[i], __fmul_rn(w, Vo[c].v[i]));
                    acc_a.v[i] = __fadd_rn(acc_a.v[i], __fmul_rn(Va[c].v[i], P[c].v[i]));
                }
            }
        if (warm && deviates) {
            const FV<VPT> ev_a = ldv<VPT>(B.row2(p.values_avg, j, a), tid);  // value of the node under the start policy
#pragma unroll
            for (int c = 0; c < K; ++c) {
                FV<VPT> r;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    const float wgt = unblocked(B.cs + 52, B.S[1], hi.c1[i], hi.c2[i], b_o.v[i]);
                    r.v[i] = __fmul_rn(wgt, __fsub_rn(Va[c].v[i], ev_a.v[i]));
                }
                stv<VPT>(B.row1(p.regrets, fc + c), tid, r);
            }
        }
        if (deviates) acc_a = best_v;
        if (j != 0) {
            stv<VPT>(B.val(ii, a), tid, acc_a);
            stv<VPT>(B.val(ii, o), tid, acc_o);
        } else {
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                root_v[0].v[i] = a == 0 ? acc_a.v[i] : acc_o.v[i];
                root_v[1].v[i] = a == 0 ? acc_o.v[i] : acc_a.v[i];
            }
        }
        };
        dispatch_children(k, node_body);
    }
}

template <int VPT, int MAXC>
__global__ void __launch_bounds__(CfrThreads<VPT>::value, 1) cfr_solve_kernel(const CfrParams p) {
    constexpr int NT = CfrThreads<VPT>::value;
    extern __shared__ __align__(16) unsigned char smem[];
    Block B;
    B.tab = smem + kOffTab;
    B.nodes = reinterpret_cast<NodeRec*>(smem + kOffNodes);
    B.xs = reinterpret_cast<float*>(smem + kOffXs);
    B.pref = reinterpret_cast<float*>(smem + kOffPref);
    B.pc = reinterpret_cast<float*>(smem + kOffPc);
    B.cs = reinterpret_cast<double*>(smem + kOffCs);
    B.warp_tot = reinterpret_cast<double*>(smem + kOffWarpTot);
    B.S = reinterpret_cast<double*>(smem + kOffS);
    B.sig = reinterpret_cast<float*>(smem + kOffSig);
    B.sigb = reinterpret_cast<float*>(smem + kOffSigB);
    B.misc = reinterpret_cast<int*>(smem + kOffMisc);
    B.ilist = reinterpret_cast<uint16_t*>(smem + kOffIlist);
    B.fsum = reinterpret_cast<float*>(smem + kOffMisc + 16);
    if (threadIdx.x == 0) B.misc[2] = 0;  // unit counter of node_tables
    const int tid = threadIdx.x;

    HandInfo<VPT> hi;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int h = VPT * tid + i;
        hi.valid[i] = h < P2B_NUM_HANDS;
        const int hc = h < P2B_NUM_HANDS ? h : P2B_NUM_HANDS - 1;
        hi.c1[i] = p.combos->c1[hc];
        hi.c2[i] = p.combos->c2[hc];
    }

    while (true) {
        __syncthreads();
        if (tid == 0) B.misc[0] = atomicAdd(p.work_counter, 1);
        __syncthreads();
        if (B.misc[0] >= p.num_subgames) break;
        const int s = p.queue_order ? p.queue_order[B.misc[0]] : B.misc[0];
        B.sg = p.subgames[s];
        if (p.large_only && B.sg.n_nodes <= kIterMaxNodes) continue;  // the lean iteration kernel has solved these passes
        // work rows: one set per block, or one per subgame when state is carried between launches
        B.scr = p.scratch + (long long)((p.stepped && !p.scratch_per_block) ? s : (int)blockIdx.x) * p.scratch_stride;
        B.leaf0 = p.leaf_begin ? p.leaf_begin[s] : 0;
        B.sample_pass = p.sample_pass ? p.sample_pass[s] : -2;
        {
            for (int i = tid; i < B.sg.n_nodes; i += NT) B.nodes[i] = load_node(p.nodes + B.sg.node_begin + i);
            if (B.sg.table_index >= 0) {
                const uint4* t = reinterpret_cast<const uint4*>(p.tables + (long long)B.sg.table_index * kTabBytes);
                for (int i = tid; i < kTabBytes / 16; i += NT) reinterpret_cast<uint4*>(B.tab)[i] = t[i];
            }
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i)
            hi.allowed[i] = hi.valid[i] && (((B.sg.board_mask >> hi.c1[i]) | (B.sg.board_mask >> hi.c2[i])) & 1ull) == 0;
        // prior = root beliefs the node beliefs of a pass are derived from; root_b = the
        // root's own row, renormalised once per pass like every other row upstream.
        FV<VPT> prior[2], root_b[2];
        const int pass_first = p.stepped ? p.pass_begin : -1, pass_last = p.stepped ? p.pass_end : p.iterations;
        // phases 16: the bottom-up sweep of pass_begin and the top-down sweep of pass_begin + 1 in one visit
        const bool joint = p.stepped && p.phases == 16;
        const bool run_down = !p.stepped || (p.phases & 1) || joint, run_up = !p.stepped || (p.phases & 2) || joint;
        const bool resume = p.stepped && !(pass_first < 0 && run_down && !joint);  // continue from carried state
        if (resume) {
            const float* cr = p.carry_roots + (long long)s * 4 * P2B_HPAD;
            prior[0] = ldv<VPT>(cr, tid);
            prior[1] = ldv<VPT>(cr + P2B_HPAD, tid);
            root_b[0] = ldv<VPT>(cr + 2 * P2B_HPAD, tid);
            root_b[1] = ldv<VPT>(cr + 3 * P2B_HPAD, tid);
            for (int i = tid; i < 2 * B.sg.n_nodes; i += NT) B.sig[i] = p.carry_sums[(long long)B.sg.node_begin * 2 + i];
            if (p.cfr_avg || p.iter_values)  // the sums under the average policy follow the [rows][2] block of the current ones
                for (int i = tid; i < 2 * B.sg.n_nodes; i += NT)
                    B.sigb[i] = p.carry_sums[(p.rows + B.sg.node_begin) * 2 + i];
        } else {
            root_b[0] = ldv<VPT>(p.root_beliefs + ((long long)s * 2 + 0) * P2B_HPAD, tid);
            root_b[1] = ldv<VPT>(p.root_beliefs + ((long long)s * 2 + 1) * P2B_HPAD, tid);
        }
        __syncthreads();
        for (int i = tid; i < B.sg.n_nodes; i += NT) {
            const NodeRec nd = B.nodes[i];
            if (nd.kind == kInternal && nd.internal_idx < B.sg.n_internal) B.ilist[nd.internal_idx] = (uint16_t)i;
        }
        __syncthreads();

        // a one-launch solve without optional outputs takes the leanest copy of the sweeps
        const bool plain = !p.stepped && !p.leaf_beliefs && !p.leaf_values && !p.policy_sample && !p.beliefs_last &&
                           !p.policy && !p.start_policy && !p.cfr_avg && !p.linear;
        for (int pass = pass_first; pass <= pass_last; ++pass) {
            const int mode = pass < 0 ? kPassInit : (pass == p.iterations ? kPassFinal : kPassIter);
            const bool down_now = run_down && !(joint && pass == pass_first);
            const bool up_now = run_up && !(joint && pass == pass_last);
            if (!down_now) {
                // the top-down sweep of this pass ran in an earlier launch
            } else if (mode == kPassInit) {
                // prior = the given ranges restricted to the allowed hands; the root's own row is
                // normalised once per tree level during the start pass (see sweep_down)
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    prior[0].v[i] = hi.allowed[i] ? root_b[0].v[i] : 0.0f;
                    prior[1].v[i] = hi.allowed[i] ? root_b[1].v[i] : 0.0f;
                }
                root_b[0] = prior[0];
                root_b[1] = prior[1];
                const int reps = p.init_depth > 1 ? p.init_depth : 1;
                for (int rep = 0; rep < reps; ++rep) normalize2<VPT>(B, hi, root_b);
            } else if (mode == kPassIter) {
                prior[0] = root_b[0];
                prior[1] = root_b[1];
                normalize2<VPT>(B, hi, root_b);
                // a child's row of the player who did not act is the root's row; so is its sum
                if (tid < 2) B.sig[tid] = B.sigb[tid] = B.fsum[tid];
            }
            bool done_plain = false;
            if constexpr (!kWide) {
                if (mode == kPassIter && plain) {
                    sweep_down<VPT, MAXC, kPassIter, true>(mode, pass, p, B, hi, prior, tid);
                    sweep_up<VPT, MAXC, kPassIter, true>(mode, pass, p, B, hi, prior, root_b, s, tid);
                    done_plain = true;
                }
            }
            if (!done_plain) {  // start and final passes; every pass of a stepped solve or one with optional outputs
                if (down_now) sweep_down<VPT, MAXC, -1, false>(mode, pass, p, B, hi, prior, tid);
                if (up_now) sweep_up<VPT, MAXC, -1, false>(mode, pass, p, B, hi, prior, root_b, s, tid);
            }
        }
        if (p.stepped) {
            __syncthreads();
            float* cr = p.carry_roots + (long long)s * 4 * P2B_HPAD;
            stv<VPT>(cr, tid, prior[0]);
            stv<VPT>(cr + P2B_HPAD, tid, prior[1]);
            stv<VPT>(cr + 2 * P2B_HPAD, tid, root_b[0]);
            stv<VPT>(cr + 3 * P2B_HPAD, tid, root_b[1]);
            for (int i = tid; i < 2 * B.sg.n_nodes; i += NT) p.carry_sums[(long long)B.sg.node_begin * 2 + i] = B.sig[i];
            if (p.cfr_avg || p.iter_values)
                for (int i = tid; i < 2 * B.sg.n_nodes; i += NT)
                    p.carry_sums[(p.rows + B.sg.node_begin) * 2 + i] = B.sigb[i];
        }
        if (p.stepped && (p.phases & 8) && p.values_avg) {
            // best-response pass of a `model_br` warm start: one sweep per deviating player
            FV<VPT> unused[2];
            for (int d = 0; d < 2; ++d) {
                __syncthreads();
                sweep_br<VPT, MAXC>(d, p, B, hi, prior, root_b, tid, unused, true);
            }
        }
        if (p.exploitability && p.values_avg && !joint && (run_up || (p.stepped && (p.phases & 4))) &&
            pass_last == p.iterations) {
            // local exploitability of the average policy (cfr_evaluator.py:718-764)
            __syncthreads();
            FV<VPT> base[2], br[2];
            float total = 0.0f;
            for (int d = -1; d < 2; ++d) {
                __syncthreads();
                sweep_br<VPT, MAXC>(d, p, B, hi, prior, root_b, tid, br);
                if (d < 0) {
                    base[0] = br[0];
                    base[1] = br[1];
                    continue;
                }
                const FV<VPT> rb = pick<VPT>(root_b, d), bv = pick<VPT>(br, d), sv = pick<VPT>(base, d);
                FV<VPT> gain, val;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    gain.v[i] = __fmul_rn(__fsub_rn(bv.v[i], sv.v[i]), rb.v[i]);
                    val.v[i] = __fmul_rn(bv.v[i], rb.v[i]);
                }
                float sums[2];
                dot2_reference_order<VPT>(B, gain, val, sums);
                total = d == 0 ? sums[0] : __fadd_rn(total, sums[0]);
                if (tid == 0 && p.br_values) p.br_values[(long long)s * 2 + d] = sums[1];
            }
            if (tid == 0) p.exploitability[s] = total;
        }
    }
}

#ifndef P2B_CFR_WIDE
// Checks every subgame's records against the solver kernels' limits before they run: a
// malformed tree would make them index shared memory or the work rows out of range.  One block
// per subgame, one thread per node.  On a violation the status word (work_counter[1]) receives
// 1 + the subgame index and the subgame queue (work_counter[0]) is set past its end, so that the
// solver kernel launched next on the stream finds no work at all.
__global__ void __launch_bounds__(kCfrMaxNodes) cfr_validate_kernel(const CfrParams p) {
    const int s = blockIdx.x, i = threadIdx.x;
    const SubgameRec sg = p.subgames[s];
    int bad = sg.n_nodes < 1 || sg.n_nodes > kCfrMaxNodes || sg.n_internal > p.max_internal || sg.node_begin < 0 ||
              (p.rows > 0 && (long long)sg.node_begin + sg.n_nodes > p.rows) ||
              (p.queue_order && (unsigned)p.queue_order[s] >= (unsigned)p.num_subgames);
    if (!bad && i < sg.n_nodes) {
        const NodeRecPacked raw = p.nodes[sg.node_begin + i];
        const NodeRec nd = unpack_node(raw);
        if (raw.kind_act & 0x7c) bad = 1;  // bits that carry nothing must be zero
        if (nd.kind > kModelLeaf || (nd.kind == kShowdownLeaf && (sg.table_index < 0 || p.tables == nullptr))) bad = 1;
        if (i == 0 && nd.kind != kInternal) bad = 1;
        if (nd.kind == kInternal &&
            (nd.n_children < 1 || nd.n_children > kCfrMaxChildren || nd.first_child <= i ||
             nd.first_child + nd.n_children > sg.n_nodes || nd.internal_idx >= p.max_internal || nd.to_act > 1))
            bad = 1;
        // a leaf valued by the caller's model must own a slot of the leaf arrays
        if (nd.kind == kModelLeaf && p.leaf_begin && (p.leaf_beliefs || p.leaf_values) &&
            (p.leaf_begin[s] < 0 || p.leaf_begin[s] + (int)nd.internal_idx >= p.leaf_slots))
            bad = 1;
    }
    // internal_idx must be the rank among the subgame's internal nodes (the solver walks them
    // through a list indexed by it) and n_internal their number
    __shared__ uint8_t s_internal[kCfrMaxNodes];
    const bool in_tree = !bad && i < sg.n_nodes;
    s_internal[i] = in_tree && (p.nodes[sg.node_begin + i].kind_act & 3) == kInternal;
    __syncthreads();
    if (in_tree) {
        int before = 0;
        for (int j = 0; j < i; ++j) before += s_internal[j];
        if (s_internal[i] && before != p.nodes[sg.node_begin + i].internal_idx) bad = 1;
        if (i == sg.n_nodes - 1 && before + s_internal[i] != sg.n_internal) bad = 1;
    }
    if (__syncthreads_or(bad) && i == 0) {
        atomicMax(p.work_counter + 1, s + 1);
        atomicMax(p.work_counter, p.num_subgames);
    }
}

// Warm start of type `model` (p2/search/cfr_evaluator.py:913-926), applied between the start
// pass and the first iteration pass of a stepped solve.  After the start pass a regret row
// holds the instantaneous regrets of the start policy.  Per non-root row: weight = `weight` x
// mean over the 1326 hands of max(regret, 0) (the sum in the reference row-reduction order),
// then regrets = start policy x weight and weight sums = weight.  One block per row.
__global__ void __launch_bounds__(256) cfr_warm_seed_kernel(const NodeRecPacked* __restrict__ nodes, long long rows,
                                                            const float* __restrict__ start_policy, float weight,
                                                            float* __restrict__ regrets, float* __restrict__ weight_sums) {
    __shared__ __align__(16) float pos[P2B_HPAD];
    __shared__ float s_sum;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        if (nodes[row].depth == 0) continue;  // roots are reached by no action (uniform per block)
        float* r = regrets + row * P2B_HPAD;
        for (int h = threadIdx.x; h < P2B_HPAD; h += blockDim.x) pos[h] = h < P2B_NUM_HANDS ? fmaxf(r[h], 0.0f) : 0.0f;
        __syncthreads();
        if (threadIdx.x < 32) {
            const float sum = row_sum_reference_order(pos);
            if (threadIdx.x == 0) s_sum = sum;
        }
        __syncthreads();
        const float w = __fmul_rn(weight, __fdiv_rn(s_sum, (float)P2B_NUM_HANDS));
        const float* sp = start_policy + row * P2B_HPAD;
        for (int h = threadIdx.x; h < P2B_HPAD; h += blockDim.x) {
            r[h] = __fmul_rn(sp[h], w);
            if (weight_sums) weight_sums[row * P2B_HPAD + h] = w;
        }
        __syncthreads();
    }
}

#endif  // !P2B_CFR_WIDE

template <int VPT, int MAXC>
int launch_kernel(const CfrParams& p, int num_blocks, cudaStream_t stream) {
    int rc = check_cuda(cudaFuncSetAttribute(cfr_solve_kernel<VPT, MAXC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kCfrSmem),
                        "cfr_solve_kernel shared-memory attribute");
    if (rc) return rc;
    cfr_solve_kernel<VPT, MAXC><<<num_blocks, CfrThreads<VPT>::value, kCfrSmem, stream>>>(p);
    return check_cuda(cudaGetLastError(), "cfr_solve_kernel");
}

}  // namespace

#ifdef P2B_CFR_WIDE
// the launcher of the kernel for up to kCfrMaxChildren actions per node (the record check runs before it)
int launch_cfr_wide(const CfrParams& p, int num_blocks, cudaStream_t stream) {
    return launch_kernel<2, kMaxC>(p, num_blocks, stream);
}

}  // namespace p2b
#else

int launch_cfr_wide(const CfrParams& p, int num_blocks, cudaStream_t stream);  // cfr_wide.cu

int sm_count();

int cfr_default_blocks() { return sm_count(); }

static int dispatch_cfr(const CfrParams& p, int num_blocks, int max_children, cudaStream_t stream) {
    if (max_children > kCfrMaxChildren)
        return set_error(P2B_ERR_ARG, "at most %d actions per node are supported, got %d", kCfrMaxChildren, max_children);
    // every launch is checked, also the later steps of a stepped solve: the launcher has cleared the
    // status word and the queue, and the kernel must not walk records the check refuses
    cfr_validate_kernel<<<p.num_subgames, kCfrMaxNodes, 0, stream>>>(p);
    const int rc = check_cuda(cudaGetLastError(), "cfr_validate_kernel");
    if (rc) return rc;
    // one kernel serves every child count up to its width: node bodies are specialised per count inside it
    if (max_children <= kMaxC) return launch_kernel<2, kMaxC>(p, num_blocks, stream);
    return launch_cfr_wide(p, num_blocks, stream);
}

int launch_cfr_warm_seed(const NodeRecPacked* nodes, long long rows, const float* start_policy, float weight, float* regrets,
                         float* weight_sums, cudaStream_t stream) {
    if (rows <= 0) return P2B_OK;
    long long grid = rows < (long long)sm_count() * 8 ? rows : (long long)sm_count() * 8;
    cfr_warm_seed_kernel<<<(unsigned)grid, 256, 0, stream>>>(nodes, rows, start_policy, weight, regrets, weight_sums);
    return check_cuda(cudaGetLastError(), "cfr_warm_seed_kernel");
}

// ---- optional timing of the iteration kernel of a split solve (for benchmarks) ----------------
namespace {
struct IterTiming {
    bool enabled = false;
    bool recorded = false;
    cudaEvent_t start = nullptr, stop = nullptr;
};
IterTiming g_iter_timing[64];
IterTiming* iter_timing_of_current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return &g_iter_timing[dev];
}
}  // namespace

// Which kernel runs the iteration passes of a plain one-call solve.  0 (default): the lean kernel, unless the
// batch is so small that the general kernel is quicker -- at most one subgame per SM (a lone 448-thread block
// leaves an SM idler than the general kernel's 672 threads: 22.3 against 30.2 ms for 148 subgames x 64
// iterations), or fewer than eight per SM when some subgame may exceed the lean kernel's node limit (the lean
// launch and the launch for the large subgames would then both run half empty, one after the other: 36 against
// 64 ms for 192 ragged subgames of up to 237 nodes x 24 iterations).  1: the lean kernel whenever it applies.
static std::atomic<int> g_path_policy{0};

int cfr_path_policy(int policy) {
    const int before = g_path_policy.load();
    if (policy >= 0) g_path_policy.store(policy != 0);
    return before;
}

int cfr_iteration_timing(int enable) {
    IterTiming* t = iter_timing_of_current_device();
    if (!t) return set_error(P2B_ERR_STATE, "no current device");
    if (enable && !t->start) {
        int rc = check_cuda(cudaEventCreate(&t->start), "cudaEventCreate");
        if (rc) return rc;
        rc = check_cuda(cudaEventCreate(&t->stop), "cudaEventCreate");
        if (rc) return rc;
    }
    t->enabled = enable != 0;
    t->recorded = false;
    return P2B_OK;
}

int cfr_iteration_ms(float* ms) {
    IterTiming* t = iter_timing_of_current_device();
    if (!t || !t->recorded) return set_error(P2B_ERR_STATE, "no timed iteration kernel has run on this device");
    int rc = check_cuda(cudaEventSynchronize(t->stop), "cudaEventSynchronize");
    if (rc) return rc;
    return check_cuda(cudaEventElapsedTime(ms, t->start, t->stop), "cudaEventElapsedTime");
}

static int clear_counters(int32_t* work_counter, cudaStream_t stream) {
    // [0] subgame queue, [1] status, [2], [3] spare
    return check_cuda(cudaMemsetAsync(work_counter, 0, 4 * sizeof(int32_t), stream), "cudaMemsetAsync(work counter)");
}

long long cfr_solve_scratch_floats(int max_internal, int max_children, int num_blocks, int num_subgames, long long rows) {
    long long per_block = cfr_scratch_floats(max_internal);
    const long long iter_block = cfr_iter_scratch_floats(max_internal, max_children);
    if (iter_block > per_block) per_block = iter_block;
    const long long carry_sums = rows * 4;  // current-policy sums and, for cfr_avg, average-policy sums
    return per_block * num_blocks + (long long)num_subgames * 4 * P2B_HPAD + carry_sums;
}

int launch_cfr_solve(const CfrParams& params, int num_blocks, int max_children, cudaStream_t stream, bool fast_scratch) {
    if (params.num_subgames == 0) return P2B_OK;
    if (params.iterations < 1) return set_error(P2B_ERR_ARG, "at least one iteration is required");
    int rc = ensure_tables();
    if (rc) return rc;
    CfrParams p = params;
    p.combos = device_combo_table();
    // leaves all terminal, uniform start policy, all passes in this call: the iteration kernel applies
    if (p.warm_weight > 0.0f && (!p.start_policy || !p.rows))
        return set_error(P2B_ERR_ARG, "a warm start needs a start policy and the row count of the state arrays");
    // leaves all terminal, all passes in this call: the iteration kernel applies (a start policy only concerns
    // the start pass, a warm start of type `model` is a kernel of its own between that pass and the iterations)
    const bool plain = !p.stepped && !p.leaf_beliefs && !p.leaf_values && !p.cfr_avg && !p.linear;
    long long per_block = cfr_scratch_floats(p.max_internal);
    const long long iter_block = cfr_iter_scratch_floats(p.max_internal, max_children);
    if (iter_block > per_block) per_block = iter_block;
    const bool maybe_large = (long long)p.max_internal * max_children + 1 > kIterMaxNodes;
    const bool few = g_path_policy.load() == 0 &&
                     (p.num_subgames <= sm_count() || (maybe_large && p.num_subgames < 8 * sm_count()));
    if (!(plain && fast_scratch && max_children <= kIterMaxChildren && !few)) {
        if (p.warm_weight > 0.0f) {
            // the general kernel in two launches around the seeding: start pass, then every other pass
            if (p.stepped) return set_error(P2B_ERR_ARG, "a stepped solve seeds its warm start itself");
            if (!fast_scratch)
                return set_error(P2B_ERR_ARG, "a warm start needs the scratch area of p2b_cfr_solve_scratch_floats "
                                              "(hand-over rows between the launches)");
            CfrParams q = p;
            q.scratch_stride = per_block;
            q.carry_roots = p.scratch + per_block * num_blocks;
            q.carry_sums = q.carry_roots + (long long)p.num_subgames * 4 * P2B_HPAD;
            q.stepped = 1;
            q.scratch_per_block = 1;
            q.phases = 3;
            for (int part = 0; part < 2; ++part) {
                q.pass_begin = part == 0 ? -1 : 0;
                q.pass_end = part == 0 ? -1 : p.iterations;
                rc = clear_counters(q.work_counter, stream);
                if (rc) return rc;
                rc = dispatch_cfr(q, num_blocks, max_children, stream);
                if (rc) return rc;
                if (part == 0) {
                    rc = launch_cfr_warm_seed(p.nodes, p.rows, p.start_policy, p.warm_weight, p.regrets, p.weight_sums, stream);
                    if (rc) return rc;
                }
            }
            return P2B_OK;
        }
        rc = clear_counters(p.work_counter, stream);
        if (rc) return rc;
        return dispatch_cfr(p, num_blocks, max_children, stream);
    }
    // A plain solve runs as: start pass (cfr_solve_kernel), iteration passes (cfr_iter_kernel), final
    // pass with the best responses (cfr_solve_kernel).  Root rows and their sums travel between the
    // launches in the tail of the scratch area; work rows do not, so each launch keeps one set per block.
    p.scratch_stride = per_block;
    p.carry_roots = p.scratch + per_block * num_blocks;
    p.carry_sums = p.carry_roots + (long long)p.num_subgames * 4 * P2B_HPAD;
    p.stepped = 1;
    p.scratch_per_block = 1;
    p.phases = 3;
    for (int part = 0; part < 3; ++part) {
        CfrParams q = p;
        q.pass_begin = part == 0 ? -1 : (part == 1 ? 0 : p.iterations);
        q.pass_end = part == 0 ? -1 : (part == 1 ? p.iterations - 1 : p.iterations);
        rc = clear_counters(q.work_counter, stream);
        if (rc) return rc;
        if (part == 1) {
            cfr_validate_kernel<<<q.num_subgames, kCfrMaxNodes, 0, stream>>>(q);
            rc = check_cuda(cudaGetLastError(), "cfr_validate_kernel");
            if (rc) return rc;
            IterTiming* timing = iter_timing_of_current_device();
            const bool timed = timing && timing->enabled;
            if (timed) cudaEventRecord(timing->start, stream);
            rc = launch_cfr_iter(q, num_blocks, stream);
            if (timed) {
                cudaEventRecord(timing->stop, stream);
                timing->recorded = true;
            }
            // Subgames with more nodes than the iteration kernel holds in shared memory were skipped by it:
            // the general kernel runs their iteration passes.  The batch can only contain such a subgame
            // if the bound below exceeds the limit.
            if (!rc && maybe_large) {
                rc = clear_counters(q.work_counter, stream);
                if (rc) return rc;
                q.large_only = 1;
                rc = dispatch_cfr(q, num_blocks, max_children, stream);
            }
        } else {
            rc = dispatch_cfr(q, num_blocks, max_children, stream);
        }
        if (rc) return rc;
        if (part == 0 && p.warm_weight > 0.0f) {
            rc = launch_cfr_warm_seed(p.nodes, p.rows, p.start_policy, p.warm_weight, p.regrets, p.weight_sums, stream);
            if (rc) return rc;
        }
    }
    return P2B_OK;
}

// ---- variant that allocates nothing --------------------------------------------------
// Work rows, the subgame queue counter and the combo table live in file-scope device
// arrays, so every GPU that loads this library holds them (about 32 MiB) until the process
// exits.  In host code these names are only stand-ins: the device addresses are obtained
// once per device with cudaGetSymbolAddress and handed to the kernel.
constexpr long long kStaticScratchFloats = 8ll << 20;  // 32 MiB of work rows
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
static __device__ __align__(256) int32_t g_static_counter[64];
static __device__ __align__(256) ComboTable g_static_combos;

namespace {
struct StaticPointers {
    float* scratch = nullptr;
    int32_t* counter = nullptr;
    ComboTable* combos = nullptr;
    bool ready = false;
};
constexpr int kStaticMaxDevices = 64;
StaticPointers g_static[kStaticMaxDevices];
}  // namespace

long long cfr_static_scratch_floats() { return kStaticScratchFloats; }

// First call on a device: resolves the three symbols and uploads the combo table with a
// synchronous copy.  Later calls only enqueue a 16-byte memset, the record check and the kernel.
int launch_cfr_solve_static(const CfrParams& params, int max_children, cudaStream_t stream) {
    if (params.num_subgames == 0) return P2B_OK;
    if (params.iterations < 1) return set_error(P2B_ERR_ARG, "at least one iteration is required");
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (dev < 0 || dev >= kStaticMaxDevices) return set_error(P2B_ERR_STATE, "device ordinal %d out of range", dev);
    StaticPointers& sp = g_static[dev];
    static std::mutex setup_lock;  // first calls on a device may come from several host threads
    std::lock_guard<std::mutex> hold(setup_lock);
    if (!sp.ready) {
        rc = check_cuda(cudaGetSymbolAddress((void**)&sp.scratch, g_static_scratch), "cudaGetSymbolAddress(scratch)");
        if (rc) return rc;
        rc = check_cuda(cudaGetSymbolAddress((void**)&sp.counter, g_static_counter), "cudaGetSymbolAddress(counter)");
        if (rc) return rc;
        rc = check_cuda(cudaGetSymbolAddress((void**)&sp.combos, g_static_combos), "cudaGetSymbolAddress(combos)");
        if (rc) return rc;
        ComboTable host;
        int h = 0;
        for (int a = 0; a < P2B_NUM_CARDS; ++a)
            for (int b = a + 1; b < P2B_NUM_CARDS; ++b, ++h) {
                host.c1[h] = (uint8_t)a;
                host.c2[h] = (uint8_t)b;
            }
        rc = check_cuda(cudaMemcpy(sp.combos, &host, sizeof(ComboTable), cudaMemcpyHostToDevice),
                        "cudaMemcpy(static combo table)");
        if (rc) return rc;
        sp.ready = true;
    }
    const long long per_block = cfr_scratch_floats(params.max_internal);
    if (per_block > kStaticScratchFloats)
        return set_error(P2B_ERR_ARG,
                         "a subgame with %d internal nodes needs %lld floats of work rows per block; the built-in "
                         "work area holds %lld floats (use p2b_cfr_solve with caller-provided scratch instead)",
                         params.max_internal, per_block, kStaticScratchFloats);
    long long blocks = kStaticScratchFloats / per_block;
    if (blocks > sm_count()) blocks = sm_count();
    if (blocks > params.num_subgames) blocks = params.num_subgames;
    CfrParams p = params;
    p.combos = sp.combos;
    p.scratch = sp.scratch;
    p.scratch_stride = per_block;
    p.work_counter = sp.counter;
    // the queue counter must start at zero; the work rows need no clearing (every row is
    // written before it is read within a solve)
    rc = check_cuda(cudaMemsetAsync(sp.counter, 0, 4 * sizeof(int32_t), stream), "cudaMemsetAsync(static counter)");
    if (rc) return rc;
    return dispatch_cfr(p, (int)blocks, max_children, stream);
}

// Status word of the last allocation-free solve on the current device (0, or 1 + the index of a
// subgame whose records the check refused, in which case nothing was solved).  Waits for `stream`.
int cfr_static_status(int32_t* host_status, cudaStream_t stream) {
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (dev < 0 || dev >= kStaticMaxDevices || !g_static[dev].ready)
        return set_error(P2B_ERR_STATE, "no allocation-free solve has run on device %d yet", dev);
    rc = check_cuda(cudaMemcpyAsync(host_status, g_static[dev].counter + 1, sizeof(int32_t), cudaMemcpyDeviceToHost, stream),
                    "cudaMemcpyAsync(static status)");
    if (rc) return rc;
    return check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize(static status)");
}

}  // namespace p2b
#endif  // P2B_CFR_WIDE
