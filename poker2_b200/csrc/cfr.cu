// Fused subgame CFR: one persistent kernel solves a whole batch of independent subgames.
//
// A thread block owns one subgame at a time and runs ALL of its iterations before it
// takes the next one from a queue, so the subgame's state (cumulative regrets, weight
// sums, average policy: [node][combo] fp32 rows, 128-bit accesses) and the block's work
// rows stay hot in L2.  A thread owns four consecutive hand columns of every row.  What
// one iteration does (upstream: p2/search/cfr_evaluator.py:1331-1381) is reorganised into
// two sweeps over the internal nodes of the public tree:
//
//   top-down   regret matching of the children (:1168-1185), average-policy mix and
//              renormalisation (:1195-1258), reach of both players (:332-361);
//   bottom-up  beliefs of the node (:363-380, :254-273), opponent-conditioned child
//              policy (:1076-1093), leaf values (fold constants, showdown :484-601), value
//              backup (:1095-1115), then instantaneous regrets (:1117-1165) and the
//              discounted update of the NEXT iteration (:1346-1368) while the child values
//              are still in registers.
//
// Pass -1 evaluates the uniform start policy (:830-886, :1511-1513); the pass after the
// last iteration evaluates the average policy (`update_average_values_final`, :1276-1292).
// Arithmetic on fp32 state follows the upstream operation order (the library is built
// with -fmad=false); sums over hands are accumulated in fp64.
#include "cfr.cuh"
#include "showdown.cuh"

namespace p2b {

namespace {

constexpr int NT = kCfrThreads;
constexpr int NW = NT / 32;        // 11 warps
constexpr int kActive = P2B_HPAD / 4;  // 332 threads hold hands
constexpr int kNatEntries = 52 * 51;

// ---- shared memory carve-up (bytes) ----
constexpr int kOffTab = 0;
constexpr int kOffNodes = kOffTab + kTabBytes;
constexpr int kOffXs = kOffNodes + kCfrMaxNodes * 16;
constexpr int kOffPref = kOffXs + 2 * P2B_HPAD * 4;
constexpr int kOffPc = kOffPref + 2 * P2B_HPAD * 4;
constexpr int kOffCs = kOffPc + 2 * 52 * 52 * 4;
constexpr int kOffRed = kOffCs + 2 * 52 * 8;
constexpr int kOffWarpTot = kOffRed + 2 * NW * 2 * 8;
constexpr int kOffS = kOffWarpTot + 16 * 8;
constexpr int kOffNat = kOffS + 4 * 8;
constexpr int kOffMisc = kOffNat + ((kNatEntries * 2 + 15) / 16) * 16;
constexpr int kCfrSmem = kOffMisc + 64;
static_assert(kOffXs % 16 == 0 && kOffCs % 8 == 0 && kOffNat % 16 == 0, "alignment");

struct F4 {
    float v[4];
};

__device__ __forceinline__ F4 ld4(const float* row, int tid) {
    F4 r;
    if (tid < kActive) {
        const float4 t = *reinterpret_cast<const float4*>(row + 4 * tid);
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else {
        r.v[0] = r.v[1] = r.v[2] = r.v[3] = 0.0f;
    }
    return r;
}
__device__ __forceinline__ void st4(float* row, int tid, const F4& r) {
    if (tid < kActive) *reinterpret_cast<float4*>(row + 4 * tid) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// Sums two per-thread values over the block.  `red` holds two alternating buffers so that
// one barrier per call is enough.
__device__ __forceinline__ void block_sum2(double a, double b, double* red, int& phase, double& sa, double& sb) {
    a = warp_sum(a);
    b = warp_sum(b);
    double* buf = red + phase * (NW * 2);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        buf[warp * 2] = a;
        buf[warp * 2 + 1] = b;
    }
    __syncthreads();
    sa = 0.0;
    sb = 0.0;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
        sa += buf[w * 2];
        sb += buf[w * 2 + 1];
    }
    phase ^= 1;
}

// Per-card sums of `nrows` (1 or 2) ranges staged in xs[row][HPAD]: cs[row][c] = mass of the
// hands holding card c, S[row] = total mass.  Four threads share one card.  Ends with a
// barrier; the caller must have made xs visible with a barrier before the call.
__device__ __forceinline__ void block_cardsums(const float* xs, int nrows, const uint16_t* nat, double* cs, double* S) {
    const int tid = threadIdx.x;
    const int ntasks = nrows * 208;
    for (int base = 0; base < ntasks; base += NT) {
        const int task = base + tid;
        const bool valid = task < ntasks;
        const int row = task / 208, rem = task % 208, c = rem >> 2, q = rem & 3;
        double s = 0.0;
        if (valid) {
            const float* x = xs + row * P2B_HPAD;
            const uint16_t* list = nat + c * 51;
            for (int i = q; i < 51; i += 4) s += (double)x[list[i]];
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if (valid && q == 0) cs[row * 52 + c] = s;
    }
    __syncthreads();
    const int lane = tid & 31, warp = tid >> 5;
    if (warp < nrows) {
        double v = cs[warp * 52 + lane] + (lane + 32 < 52 ? cs[warp * 52 + lane + 32] : 0.0);
        v = warp_sum(v);
        if (lane == 0) S[warp] = 0.5 * v;  // every hand was counted under both of its cards
    }
    __syncthreads();
}

// Mass of the hands that share no card with (c1,c2): total - card sums + own mass,
// evaluated in fp64, rounded to fp32 and clamped at zero (p2/env/card_utils.py:196-222).
__device__ __forceinline__ float unblocked(const double* cs, double S, int c1, int c2, float x) {
    const double m = S - cs[c1] - cs[c2] + (double)x;
    return fmaxf((float)m, 0.0f);
}

struct HandInfo {
    int c1[4], c2[4];
    bool valid[4];    // a real combo (not row padding)
    bool allowed[4];  // and not blocked by the board of the current subgame
};

enum PassMode { kPassInit = 0, kPassIter = 1, kPassFinal = 2 };

struct Block {
    // shared memory views
    unsigned char* tab;
    NodeRec* nodes;
    float* xs;
    float* pref;
    float* pc;
    double* cs;
    double* red;
    double* warp_tot;
    double* S;
    uint16_t* nat;
    int* misc;
    float* fsum;
    int red_phase;
    // current subgame
    SubgameRec sg;
    float* scr;
    __device__ __forceinline__ float* reach(int ii, int pl) const { return scr + (long long)(ii * 6 + pl) * P2B_HPAD; }
    __device__ __forceinline__ float* rbar(int ii, int pl) const { return scr + (long long)(ii * 6 + 2 + pl) * P2B_HPAD; }
    __device__ __forceinline__ float* val(int ii, int pl) const { return scr + (long long)(ii * 6 + 4 + pl) * P2B_HPAD; }
    __device__ __forceinline__ float* row1(float* base, int node) const {
        return base + (long long)(sg.node_begin + node) * P2B_HPAD;
    }
    __device__ __forceinline__ float* row2(float* base, int node, int pl) const {
        return base + ((long long)(sg.node_begin + node) * 2 + pl) * P2B_HPAD;
    }
};

// Policy of the k children of one node: uniform (start pass), the stored average policy
// (final pass) or regret matching on the cumulative regrets, which are returned in Rc.
template <int MAXC>
__device__ __forceinline__ void children_policy(int mode, const CfrParams& p, const Block& B, int fc, int k, int tid,
                                                F4 (&P)[MAXC], F4 (&Rc)[MAXC]) {
    const float invk = __fdiv_rn(1.0f, (float)k);
    if (mode == kPassInit) {
#pragma unroll
        for (int c = 0; c < MAXC; ++c)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                P[c].v[i] = invk;
                Rc[c].v[i] = 0.0f;
            }
        return;
    }
    if (mode == kPassFinal) {
#pragma unroll
        for (int c = 0; c < MAXC; ++c)
            if (c < k) P[c] = ld4(B.row1(p.policy_avg, fc + c), tid);
        return;
    }
    F4 sum;
#pragma unroll
    for (int i = 0; i < 4; ++i) sum.v[i] = 0.0f;
#pragma unroll
    for (int c = 0; c < MAXC; ++c)
        if (c < k) {
            Rc[c] = ld4(B.row1(p.regrets, fc + c), tid);
#pragma unroll
            for (int i = 0; i < 4; ++i) sum.v[i] = __fadd_rn(sum.v[i], fmaxf(Rc[c].v[i], 0.0f));
        }
#pragma unroll
    for (int c = 0; c < MAXC; ++c)
        if (c < k) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                P[c].v[i] = sum.v[i] > 1e-8f ? __fdiv_rn(fmaxf(Rc[c].v[i], 0.0f), fmaxf(sum.v[i], 1e-8f)) : invk;
        }
}

__device__ __forceinline__ void stage(float* dst, int tid, const F4& v) {
    if (tid < kActive) *reinterpret_cast<float4*>(dst + 4 * tid) = make_float4(v.v[0], v.v[1], v.v[2], v.v[3]);
}

// fp32 sum of x[0..1325] in exactly the association order of the vectorised CPU row
// reduction the upstream normalisation runs through (`target.sum(dim=-1)`,
// cfr_evaluator.py:263): 8-wide vectors x 4 interleaved accumulators = 32 chains, each
// cascaded in blocks of 16, then the 165th vector, the four accumulators, the 6 scalar
// tail elements and finally the 8 vector lanes, all sequentially.  One warp computes it;
// every lane returns the sum.
__device__ __forceinline__ float row_sum_reference_order(const float* __restrict__ x) {
    const int lane = threadIdx.x & 31;
    float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) s1 = __fadd_rn(s1, x[32 * i + lane]);
#pragma unroll
    for (int i = 16; i < 32; ++i) s2 = __fadd_rn(s2, x[32 * i + lane]);
#pragma unroll
    for (int i = 32; i < 41; ++i) s3 = __fadd_rn(s3, x[32 * i + lane]);
    float c = __fadd_rn(s3, __fadd_rn(s1, s2));
    if (lane < 8) c = __fadd_rn(c, x[1312 + lane]);
    const float c1 = __shfl_down_sync(0xffffffffu, c, 8);
    const float c2 = __shfl_down_sync(0xffffffffu, c, 16);
    const float c3 = __shfl_down_sync(0xffffffffu, c, 24);
    const float pv = __fadd_rn(__fadd_rn(__fadd_rn(c, c1), c2), c3);  // meaningful on lanes 0..7
    float fa = 0.0f;
#pragma unroll
    for (int t = 1320; t < P2B_NUM_HANDS; ++t) fa = __fadd_rn(fa, x[t]);
#pragma unroll
    for (int v = 0; v < 8; ++v) fa = __fadd_rn(fa, __shfl_sync(0xffffffffu, pv, v));
    return fa;
}

// Normalises the two rows x[0], x[1] (one per player) over hands; a row whose sum is not
// above 1e-5 becomes uniform over the allowed hands (cfr_evaluator.py:254-273).  B.xs must
// be free on entry and is free again on return.
__device__ __forceinline__ void normalize2(Block& B, const HandInfo& hi, F4 (&x)[2]) {
    const int tid = threadIdx.x;
    stage(B.xs, tid, x[0]);
    stage(B.xs + P2B_HPAD, tid, x[1]);
    __syncthreads();
    const int warp = tid >> 5;
    if (warp < 2) {
        const float sum = row_sum_reference_order(B.xs + warp * P2B_HPAD);
        if ((tid & 31) == 0) B.fsum[warp] = sum;
    }
    __syncthreads();
    const float f[2] = {B.fsum[0], B.fsum[1]};
#pragma unroll
    for (int pl = 0; pl < 2; ++pl)
#pragma unroll
        for (int i = 0; i < 4; ++i)
            x[pl].v[i] = f[pl] > 1e-5f ? __fdiv_rn(x[pl].v[i], f[pl]) : (hi.allowed[i] ? B.sg.allowed_prob : 0.0f);
}

// beliefs of a node in an iteration: prior * reach, normalised (cfr_evaluator.py:363-380).
__device__ __forceinline__ void node_beliefs(Block& B, const HandInfo& hi, const F4 (&prior)[2], const F4 (&r)[2],
                                             F4 (&b)[2]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        b[0].v[i] = __fmul_rn(prior[0].v[i], r[0].v[i]);
        b[1].v[i] = __fmul_rn(prior[1].v[i], r[1].v[i]);
    }
    normalize2(B, hi, b);
}

// Showdown values of both players at a leaf whose beliefs are staged in B.xs[0..1].
__device__ __forceinline__ void leaf_showdown(Block& B, const HandInfo& hi, const NodeRec& leaf, int tid, F4 (&V)[2]) {
    const BoardTabView tv = view_tables(B.tab);
    if (tid < 2 * 52) {
        const int pl = tid / 52, c = tid % 52;
        const float* xp = B.xs + pl * P2B_HPAD;
        float* pcr = B.pc + pl * 52 * 52 + c * 52;
        double acc = 0.0;
        pcr[0] = 0.0f;
#pragma unroll 3
        for (int k = 0; k < 51; ++k) {
            acc += (double)xp[tv.cardlist[k * 52 + c]];
            pcr[k + 1] = (float)acc;
        }
    }
    for (int pl = 0; pl < 2; ++pl) {
        const float* xp = B.xs + pl * P2B_HPAD;
        block_prefix_f64([&](int k) { return xp[tv.sorted[k]]; }, P2B_NUM_HANDS, B.pref + pl * P2B_HPAD, B.warp_tot);
    }
    const float pot[2] = {leaf.v0, leaf.v1};
#pragma unroll
    for (int hero = 0; hero < 2; ++hero) {
        const int opp = 1 - hero;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float ev = 0.0f;
            if (hi.valid[i]) {
                const int h = 4 * tid + i;
                ev = showdown_hand_ev(tv.rec[h], hi.c1[i], hi.c2[i], B.xs[opp * P2B_HPAD + h], hi.allowed[i],
                                      B.pref + opp * P2B_HPAD, B.pc + opp * 52 * 52);
            }
            V[hero].v[i] = __fdiv_rn(__fmul_rn(ev, pot[hero]), B.sg.scale);
        }
    }
    __syncthreads();  // xs / pref / pc are free again
}

// ---- top-down sweep of one pass -------------------------------------------------------
template <int MAXC>
__device__ __forceinline__ void sweep_down(int mode, int pass, const CfrParams& p, Block& B, const HandInfo& hi,
                                           const F4 (&prior)[2], int tid) {
    const bool mix = (mode == kPassIter) && p.scalars[pass].do_mix != 0;
    F4 mask;
#pragma unroll
    for (int i = 0; i < 4; ++i) mask.v[i] = hi.allowed[i] ? 1.0f : 0.0f;
    for (int j = 0; j < B.sg.n_nodes; ++j) {
        const NodeRec nd = B.nodes[j];
        if (nd.kind != kInternal) continue;
        const int a = nd.to_act, k = nd.n_children, fc = nd.first_child, ii = nd.internal_idx;
        F4 ra = mask, rna = mask, rba = mask, rbna = mask;
        if (j != 0) {
            ra = ld4(B.reach(ii, a), tid);
            rna = ld4(B.reach(ii, 1 - a), tid);
            if (mix) {
                rba = ld4(B.rbar(ii, a), tid);
                rbna = ld4(B.rbar(ii, 1 - a), tid);
            }
        }
        F4 P[MAXC], Rc[MAXC];
        children_policy<MAXC>(mode, p, B, fc, k, tid, P, Rc);

        if (mode == kPassInit) {
            // Start beliefs.  Upstream pushes beliefs down one level at a time and re-normalises
            // EVERY row after each level (cfr_evaluator.py:855-875), so a node at level L is
            // normalised init_depth-L+1 times and its children derive from its once-normalised
            // row.  During this pass the work rows hold: reach = once-normalised beliefs,
            // rbar = final start beliefs.
            F4 b1[2];
            if (j == 0) {
                b1[0] = prior[0];
                b1[1] = prior[1];
            } else {
                b1[0] = ld4(B.reach(ii, 0), tid);
                b1[1] = ld4(B.reach(ii, 1), tid);
            }
#pragma unroll
            for (int c = 0; c < MAXC; ++c) {
                if (c >= k) continue;
                const NodeRec ch = B.nodes[fc + c];
                st4(B.row1(p.policy_avg, fc + c), tid, P[c]);
                if (ch.kind != kInternal) continue;
                F4 x[2];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    x[a].v[i] = __fmul_rn(b1[a].v[i], P[c].v[i]);
                    x[1 - a].v[i] = b1[1 - a].v[i];
                }
                normalize2(B, hi, x);
                st4(B.reach(ch.internal_idx, 0), tid, x[0]);
                st4(B.reach(ch.internal_idx, 1), tid, x[1]);
                for (int rep = ch.depth; rep < p.init_depth; ++rep) normalize2(B, hi, x);
                st4(B.rbar(ch.internal_idx, 0), tid, x[0]);
                st4(B.rbar(ch.internal_idx, 1), tid, x[1]);
            }
            continue;
        }

        if (mode != kPassFinal) {
            // average policy of the children
            F4 Pn[MAXC];
            if (mix) {
                const IterScalars sc = p.scalars[pass];
                F4 ro, rn, sum;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    ro.v[i] = __fmul_rn(rba.v[i], sc.mix_old);
                    rn.v[i] = __fmul_rn(ra.v[i], sc.mix_new);
                    sum.v[i] = 0.0f;
                }
#pragma unroll
                for (int c = 0; c < MAXC; ++c)
                    if (c < k) {
                        const F4 Pb = ld4(B.row1(p.policy_avg, fc + c), tid);
                        const NodeRec ch = B.nodes[fc + c];
                        if (ch.kind == kInternal) {  // average reach under the OLD average policy
                            F4 t;
#pragma unroll
                            for (int i = 0; i < 4; ++i) t.v[i] = __fmul_rn(rba.v[i], Pb.v[i]);
                            st4(B.rbar(ch.internal_idx, a), tid, t);
                            st4(B.rbar(ch.internal_idx, 1 - a), tid, rbna);
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float num = __fadd_rn(__fmul_rn(ro.v[i], Pb.v[i]), __fmul_rn(rn.v[i], P[c].v[i]));
                            const float den = __fadd_rn(ro.v[i], rn.v[i]);
                            const float plain = __fdiv_rn(
                                __fadd_rn(__fmul_rn(sc.mix_old, Pb.v[i]), __fmul_rn(sc.mix_new, P[c].v[i])), sc.mix_total);
                            Pn[c].v[i] = den > 1e-5f ? __fdiv_rn(num, den) : plain;
                            sum.v[i] = __fadd_rn(sum.v[i], Pn[c].v[i]);
                        }
                    }
#pragma unroll
                for (int c = 0; c < MAXC; ++c)
                    if (c < k) {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (sum.v[i] > 1e-5f) Pn[c].v[i] = __fdiv_rn(Pn[c].v[i], sum.v[i]);
                        st4(B.row1(p.policy_avg, fc + c), tid, Pn[c]);
                    }
            } else {
#pragma unroll
                for (int c = 0; c < MAXC; ++c)
                    if (c < k) st4(B.row1(p.policy_avg, fc + c), tid, P[c]);
            }
            if (p.policy && pass == p.iterations - 1) {
#pragma unroll
                for (int c = 0; c < MAXC; ++c)
                    if (c < k) st4(B.row1(p.policy, fc + c), tid, P[c]);
            }
        }
        // reach of the internal children under the policy of this pass
#pragma unroll
        for (int c = 0; c < MAXC; ++c)
            if (c < k) {
                const NodeRec ch = B.nodes[fc + c];
                if (ch.kind == kInternal) {
                    F4 t;
#pragma unroll
                    for (int i = 0; i < 4; ++i) t.v[i] = __fmul_rn(ra.v[i], P[c].v[i]);
                    st4(B.reach(ch.internal_idx, a), tid, t);
                    st4(B.reach(ch.internal_idx, 1 - a), tid, rna);
                }
            }
    }
}

// ---- bottom-up sweep of one pass ------------------------------------------------------
template <int MAXC>
__device__ __forceinline__ void sweep_up(int mode, int pass, const CfrParams& p, Block& B, const HandInfo& hi,
                                         const F4 (&prior)[2], const F4 (&root_b)[2], int s, int tid) {
    const bool update = (mode != kPassFinal) && (pass + 1 < p.iterations);
    F4 mask;
#pragma unroll
    for (int i = 0; i < 4; ++i) mask.v[i] = hi.allowed[i] ? 1.0f : 0.0f;
    for (int j = B.sg.n_nodes - 1; j >= 0; --j) {
        const NodeRec nd = B.nodes[j];
        if (nd.kind != kInternal) continue;
        const int a = nd.to_act, k = nd.n_children, fc = nd.first_child, ii = nd.internal_idx;
        // r: reach of both players (start pass: once-normalised start beliefs, see sweep_down)
        F4 r[2], b[2];
        if (j == 0) {
            r[0] = mode == kPassInit ? prior[0] : mask;
            r[1] = mode == kPassInit ? prior[1] : mask;
            b[0] = root_b[0];
            b[1] = root_b[1];
        } else {
            r[0] = ld4(B.reach(ii, 0), tid);
            r[1] = ld4(B.reach(ii, 1), tid);
            if (mode == kPassInit) {
                b[0] = ld4(B.rbar(ii, 0), tid);
                b[1] = ld4(B.rbar(ii, 1), tid);
            } else {
                node_beliefs(B, hi, prior, r, b);
            }
        }
        stage(B.xs, tid, b[0]);
        stage(B.xs + P2B_HPAD, tid, b[1]);
        __syncthreads();
        block_cardsums(B.xs, 2, B.nat, B.cs, B.S);
        F4 wgt, denm;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            wgt.v[i] = unblocked(B.cs + (1 - a) * 52, B.S[1 - a], hi.c1[i], hi.c2[i], b[1 - a].v[i]);
            denm.v[i] = unblocked(B.cs + a * 52, B.S[a], hi.c1[i], hi.c2[i], b[a].v[i]);
        }
        if (mode == kPassFinal && p.beliefs_avg) {
            st4(B.row2(p.beliefs_avg, j, 0), tid, b[0]);
            st4(B.row2(p.beliefs_avg, j, 1), tid, b[1]);
        }
        F4 P[MAXC], Rc[MAXC], Va[MAXC], acc[2];
        children_policy<MAXC>(mode, p, B, fc, k, tid, P, Rc);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[0].v[i] = acc[1].v[i] = 0.0f;

#pragma unroll
        for (int c = 0; c < MAXC; ++c) {
            if (c >= k) continue;  // uniform across the block
            const NodeRec ch = B.nodes[fc + c];
            // policy of this child as seen by each opponent hand (cfr_evaluator.py:1083-1093)
            F4 m, pio;
#pragma unroll
            for (int i = 0; i < 4; ++i) m.v[i] = __fmul_rn(b[a].v[i], P[c].v[i]);
            stage(B.xs, tid, m);
            __syncthreads();
            block_cardsums(B.xs, 1, B.nat, B.cs, B.S);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float blk = unblocked(B.cs, B.S[0], hi.c1[i], hi.c2[i], m.v[i]);
                pio.v[i] = denm.v[i] > 1e-5f ? __fdiv_rn(blk, denm.v[i]) : 0.0f;
            }
            F4 V[2];
            if (ch.kind == kFoldLeaf) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    V[0].v[i] = ch.v0;
                    V[1].v[i] = -ch.v0;
                }
            } else if (ch.kind == kInternal) {
                V[0] = ld4(B.val(ch.internal_idx, 0), tid);
                V[1] = ld4(B.val(ch.internal_idx, 1), tid);
            } else if (ch.kind == kShowdownLeaf) {
                F4 rc[2], bc[2];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    rc[a].v[i] = __fmul_rn(r[a].v[i], P[c].v[i]);
                    rc[1 - a].v[i] = r[1 - a].v[i];
                }
                if (mode == kPassInit) {
                    bc[0] = rc[0];
                    bc[1] = rc[1];
                    for (int rep = ch.depth; rep <= p.init_depth; ++rep) normalize2(B, hi, bc);
                } else {
                    node_beliefs(B, hi, prior, rc, bc);
                }
                stage(B.xs, tid, bc[0]);
                stage(B.xs + P2B_HPAD, tid, bc[1]);
                __syncthreads();
                leaf_showdown(B, hi, ch, tid, V);
                if (mode == kPassFinal && p.beliefs_avg) {
                    st4(B.row2(p.beliefs_avg, fc + c, 0), tid, bc[0]);
                    st4(B.row2(p.beliefs_avg, fc + c, 1), tid, bc[1]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) V[0].v[i] = V[1].v[i] = 0.0f;
            }
            if (mode == kPassFinal && p.values_avg && ch.kind != kInternal) {
                st4(B.row2(p.values_avg, fc + c, 0), tid, V[0]);
                st4(B.row2(p.values_avg, fc + c, 1), tid, V[1]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[a].v[i] = __fadd_rn(acc[a].v[i], __fmul_rn(V[a].v[i], P[c].v[i]));
                acc[1 - a].v[i] = __fadd_rn(acc[1 - a].v[i], __fmul_rn(V[1 - a].v[i], pio.v[i]));
            }
            Va[c] = V[a];
        }
        if (j != 0) {
            st4(B.val(ii, 0), tid, acc[0]);
            st4(B.val(ii, 1), tid, acc[1]);
        }
        if (mode == kPassFinal) {
            if (p.values_avg) {
                st4(B.row2(p.values_avg, j, 0), tid, acc[0]);
                st4(B.row2(p.values_avg, j, 1), tid, acc[1]);
            }
            if (j == 0) {
                st4(p.root_values + ((long long)s * 2 + 0) * P2B_HPAD, tid, acc[0]);
                st4(p.root_values + ((long long)s * 2 + 1) * P2B_HPAD, tid, acc[1]);
            }
        }
        if (update) {
            // instantaneous regrets of this pass folded into the discounted update of the next
            const IterScalars sc = p.scalars[pass + 1];
#pragma unroll
            for (int c = 0; c < MAXC; ++c)
                if (c < k) {
                    F4 w;
                    if (p.weight_sums) {
                        if (mode == kPassInit) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) w.v[i] = 0.0f;
                        } else {
                            w = ld4(B.row1(p.weight_sums, fc + c), tid);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float reg = __fmul_rn(wgt.v[i], __fsub_rn(Va[c].v[i], acc[a].v[i]));
                        const bool pos = Rc[c].v[i] > 0.0f;
                        const float num = pos ? sc.num_pos : sc.num_neg, den = pos ? sc.den_pos : sc.den_neg;
                        float rr = __fdiv_rn(__fmul_rn(Rc[c].v[i], num), den);
                        rr = __fadd_rn(rr, reg);
                        if (p.cfr_plus) rr = fmaxf(rr, 0.0f);
                        Rc[c].v[i] = rr;
                        if (p.weight_sums) w.v[i] = __fadd_rn(__fdiv_rn(__fmul_rn(w.v[i], num), den), 1.0f);
                    }
                    st4(B.row1(p.regrets, fc + c), tid, Rc[c]);
                    if (p.weight_sums) st4(B.row1(p.weight_sums, fc + c), tid, w);
                }
        }
    }
}

template <int MAXC>
__global__ void __launch_bounds__(NT, 1) cfr_solve_kernel(const CfrParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    Block B;
    B.tab = smem + kOffTab;
    B.nodes = reinterpret_cast<NodeRec*>(smem + kOffNodes);
    B.xs = reinterpret_cast<float*>(smem + kOffXs);
    B.pref = reinterpret_cast<float*>(smem + kOffPref);
    B.pc = reinterpret_cast<float*>(smem + kOffPc);
    B.cs = reinterpret_cast<double*>(smem + kOffCs);
    B.red = reinterpret_cast<double*>(smem + kOffRed);
    B.warp_tot = reinterpret_cast<double*>(smem + kOffWarpTot);
    B.S = reinterpret_cast<double*>(smem + kOffS);
    B.nat = reinterpret_cast<uint16_t*>(smem + kOffNat);
    B.misc = reinterpret_cast<int*>(smem + kOffMisc);
    B.fsum = reinterpret_cast<float*>(smem + kOffMisc + 16);
    B.red_phase = 0;
    B.scr = p.scratch + (long long)blockIdx.x * p.scratch_stride;
    const int tid = threadIdx.x;

    // hands holding each card, in combo order (used by the per-card sums)
    for (int idx = tid; idx < kNatEntries; idx += NT) {
        const int c = idx / 51, i = idx % 51, d = i < c ? i : i + 1;
        B.nat[idx] = (uint16_t)(c < d ? combo_index(c, d) : combo_index(d, c));
    }
    HandInfo hi;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int h = 4 * tid + i;
        hi.valid[i] = tid < kActive && h < P2B_NUM_HANDS;
        const int hc = h < P2B_NUM_HANDS ? h : P2B_NUM_HANDS - 1;
        hi.c1[i] = p.combos->c1[hc];
        hi.c2[i] = p.combos->c2[hc];
    }

    while (true) {
        __syncthreads();
        if (tid == 0) B.misc[0] = atomicAdd(p.work_counter, 1);
        __syncthreads();
        const int s = B.misc[0];
        if (s >= p.num_subgames) break;
        B.sg = p.subgames[s];
        {
            const uint4* src = reinterpret_cast<const uint4*>(p.nodes + B.sg.node_begin);
            for (int i = tid; i < B.sg.n_nodes; i += NT) reinterpret_cast<uint4*>(B.nodes)[i] = src[i];
            if (B.sg.table_index >= 0) {
                const uint4* t = reinterpret_cast<const uint4*>(p.tables + (long long)B.sg.table_index * kTabBytes);
                for (int i = tid; i < kTabBytes / 16; i += NT) reinterpret_cast<uint4*>(B.tab)[i] = t[i];
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
            hi.allowed[i] = hi.valid[i] && (((B.sg.board_mask >> hi.c1[i]) | (B.sg.board_mask >> hi.c2[i])) & 1ull) == 0;
        // prior = root beliefs the node beliefs of a pass are derived from; root_b = the
        // root's own row, renormalised once per pass like every other row upstream.
        F4 prior[2], root_b[2];
        root_b[0] = ld4(p.root_beliefs + ((long long)s * 2 + 0) * P2B_HPAD, tid);
        root_b[1] = ld4(p.root_beliefs + ((long long)s * 2 + 1) * P2B_HPAD, tid);
        __syncthreads();

        for (int pass = -1; pass <= p.iterations; ++pass) {
            const int mode = pass < 0 ? kPassInit : (pass == p.iterations ? kPassFinal : kPassIter);
            if (mode == kPassInit) {
                // prior = the given ranges restricted to the allowed hands; the root's own row is
                // normalised once per tree level during the start pass (see sweep_down)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    prior[0].v[i] = hi.allowed[i] ? root_b[0].v[i] : 0.0f;
                    prior[1].v[i] = hi.allowed[i] ? root_b[1].v[i] : 0.0f;
                }
                root_b[0] = prior[0];
                root_b[1] = prior[1];
                const int reps = p.init_depth > 1 ? p.init_depth : 1;
                for (int rep = 0; rep < reps; ++rep) normalize2(B, hi, root_b);
            } else if (mode == kPassIter) {
                prior[0] = root_b[0];
                prior[1] = root_b[1];
                normalize2(B, hi, root_b);
            }
            sweep_down<MAXC>(mode, pass, p, B, hi, prior, tid);
            sweep_up<MAXC>(mode, pass, p, B, hi, prior, root_b, s, tid);
        }
    }
}

}  // namespace

int sm_count();

int cfr_default_blocks() { return sm_count(); }

int launch_cfr_solve(const CfrParams& params, int num_blocks, int max_children, cudaStream_t stream) {
    if (params.num_subgames == 0) return P2B_OK;
    int rc = ensure_tables();
    if (rc) return rc;
    CfrParams p = params;
    p.combos = device_combo_table();
    rc = check_cuda(cudaMemsetAsync(p.work_counter, 0, sizeof(int32_t), stream), "cudaMemsetAsync(work counter)");
    if (rc) return rc;
    if (max_children <= 5) {
        rc = check_cuda(cudaFuncSetAttribute(cfr_solve_kernel<5>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCfrSmem),
                        "cfr_solve_kernel smem attribute");
        if (rc) return rc;
        cfr_solve_kernel<5><<<num_blocks, NT, kCfrSmem, stream>>>(p);
    } else if (max_children <= kCfrMaxChildren) {
        rc = check_cuda(cudaFuncSetAttribute(cfr_solve_kernel<kCfrMaxChildren>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, kCfrSmem),
                        "cfr_solve_kernel smem attribute");
        if (rc) return rc;
        cfr_solve_kernel<kCfrMaxChildren><<<num_blocks, NT, kCfrSmem, stream>>>(p);
    } else {
        return set_error(P2B_ERR_ARG, "at most %d actions per node are supported, got %d", kCfrMaxChildren, max_children);
    }
    return check_cuda(cudaGetLastError(), "cfr_solve_kernel");
}

}  // namespace p2b
