// Iteration passes of a subgame solve whose leaves are all terminal (no model leaves, no start policy): the lean
// copy of the two sweeps of cfr.cu, used for the passes 0..iterations-1 between the start pass
// and the final pass, which stay in cfr_solve_kernel.  Same arithmetic, bit for bit; what
// differs is how the work is laid out on the SM:
//
//   * One regret matching per iteration instead of two: the bottom-up sweep, which has just
//     updated the regrets of a node's children (p2/search/cfr_evaluator.py:1346-1368), turns
//     them into the next policy (:1168-1185) while they are in registers and keeps it in the
//     block's work rows; both sweeps of the next pass read that row.  The regrets are read
//     and written once per iteration.
//   * The child loops are rolled (one copy of the code for every child count) with the next
//     child's rows loaded while the current one is worked on, so the instruction footprint of
//     a pass is a few KB instead of one unrolled body per child count.
//   * The cross-hand work of a node (per-card sums, strength-order and per-card prefix sums)
//     runs one node ahead of the per-hand arithmetic, on the same warps: a warp takes its
//     share of the next node's units, then does its hands of the current node.  Staged rows and
//     tables are double buffered, and there is one block-wide barrier per node.
//   * A player's reach changes only where that player acts, so a node stores one reach row
//     (the player who acted at its parent); the other player's row is found at an ancestor.
//   * The range check of the short division sequence is two integer min/max per quotient,
//     evaluated once per group of quotients.
#include "cfr.cuh"
#include "cfr_dev.cuh"
#include "exactdiv.cuh"
#include "showdown.cuh"

// Hands per thread and blocks per SM of the iteration kernel: 3 x 448 threads x 2 blocks (28 warps
// per SM, two subgames interleaving on one SM, single-buffered tables) or 2 x 672 threads x 1 block
// (21 warps, double-buffered tables with the cross-hand units one node ahead).
#ifndef P2B_ITER_VPT
#define P2B_ITER_VPT 3
#endif
#ifndef P2B_ITER_CTAS
#define P2B_ITER_CTAS 2
#endif

namespace p2b {

namespace {

constexpr int kVpt = P2B_ITER_VPT;    // hands per thread
constexpr int kCtas = P2B_ITER_CTAS;  // blocks per SM
static_assert((kVpt == 2 && kCtas == 1) || (kVpt == 3 && kCtas == 2) || (kVpt == 4 && kCtas == 2), "supported configurations");
constexpr int kHT = P2B_HPAD / kVpt;          // threads that own hands
constexpr int kNT = (kHT + 31) / 32 * 32;     // threads per block: whole warps; the extra ones repeat the last hand thread's
                                              // per-hand work (same loads, same values stored) and share the cross-hand units
constexpr bool kDouble = kCtas == 1;  // staged rows and tables double buffered, units one node ahead
constexpr int kSets = kDouble ? 2 : 1;
constexpr int kK = kIterMaxChildren;
constexpr int kSetRows = 2 + kK + 1;  // beliefs of the acting / the other player, one row per child, one leaf row
constexpr int kRowM = 2;
constexpr int kRowLeaf = 2 + kK;
constexpr int kCsRows = 2 + kK;  // rows of a node whose per-card sums are needed

// ---- one set of cross-hand tables (bytes) ----
constexpr int kTsCs = 0;                                // double [kCsRows][52] per-card sums
constexpr int kTsS = kTsCs + kCsRows * 52 * 8;          // double [kCsRows] row totals
constexpr int kTsPref = kTsS + kCsRows * 8;             // float [2][HPAD] strength-order prefix sums
constexpr int kTsPc = kTsPref + 2 * P2B_HPAD * 4;       // float [2][52*52] per-card prefix sums
constexpr int kTsTot = kTsPc + 2 * 52 * 52 * 4;         // float [2][64] whole mass per card (consecutive cards, consecutive banks)
constexpr int kTsBytes = kTsTot + 2 * 64 * 4;

// ---- shared memory carve-up (bytes) ----
constexpr int kOffTab = 0;
constexpr int kOffNodes = kOffTab + kTabBytes;
constexpr int kOffStage = kOffNodes + kIterMaxNodes * (int)sizeof(NodeRec);  // float [kSets][kSetRows][HPAD]
constexpr int kOffTs = kOffStage + kSets * kSetRows * P2B_HPAD * 4;    // kSets table sets, right behind the rows
constexpr int kOffSig = kOffTs + kSets * kTsBytes;                     // float [nodes][2]
constexpr int kOffRsrc = kOffSig + kIterMaxNodes * 2 * 4;              // uint8 [nodes][2]
constexpr int kOffIlist = kOffRsrc + kIterMaxNodes * 2;                // uint8 [internal nodes]
constexpr int kOffSdc = kOffIlist + kIterMaxNodes;                     // uint8 [internal nodes]
constexpr int kOffMisc = kOffSdc + kIterMaxNodes;
constexpr int kOffCsIdx = kOffMisc + 64;                               // uint16 [52][52] hand index of the e-th hand holding a card
constexpr int kIterSmem = kOffCsIdx + 52 * 52 * 2;
static_assert(kOffStage % 16 == 0 && kOffTs % 16 == 0 && kTsBytes % 16 == 0 && kOffSig % 16 == 0 && kOffMisc % 16 == 0,
              "alignment");
static_assert(kIterSmem + 1024 <= 227 * 1024 / kCtas, "the blocks' shared memory must fit one SM");
// The top-down sweep uses the staging rows and the (then idle) table area behind them as kSets banks
// of child rows plus one stash row per child; with two table sets the rest of the table area
// receives the asynchronous copies of the children's policy rows.
constexpr int kDownRows = (kSets + 1) * kK;
static_assert(kDownRows * P2B_HPAD * 4 <= kOffSig - kOffStage, "top-down rows must fit the staging and table areas");
constexpr bool kDownAsync = kDouble && kVpt == 2;
static_assert(!kDownAsync || (kDownRows + 2 * kK) * P2B_HPAD * 4 <= kOffSig - kOffStage, "landing rows must fit");

constexpr uint8_t kNoRow = 0xFF;

// Hands of a thread: two consecutive ones (64-bit accesses), or three a third of a row apart
// (32-bit accesses, consecutive threads on consecutive hands).
template <int VPT>
__device__ __forceinline__ int hand_of(int tid, int i) {
    return VPT == 2 ? 2 * tid + i : tid + i * (P2B_HPAD / VPT);
}
template <int VPT>
__device__ __forceinline__ FV<VPT> ldh(const float* row, int tid) {
    if constexpr (VPT == 2) {
        return ldv<2>(row, tid);
    } else {
        FV<VPT> r;
#pragma unroll
        for (int i = 0; i < VPT; ++i) r.v[i] = row[tid + i * (P2B_HPAD / VPT)];
        return r;
    }
}
template <int VPT>
__device__ __forceinline__ void sth(float* row, int tid, const FV<VPT>& r) {
    if constexpr (VPT == 2) {
        stv<2>(row, tid, r);
    } else {
#pragma unroll
        for (int i = 0; i < VPT; ++i) row[tid + i * (P2B_HPAD / VPT)] = r.v[i];
    }
}
// State rows (regrets, weight sums, average policy) are read once and written once per pass and not touched again
// before the next pass, by which time the other blocks have pushed far more than the L2 holds through it; the
// streaming forms mark their lines as the first to evict, in favour of the block's work rows (bit 0: loads,
// bit 1: stores).  Measured on 1184 subgames x 64 iterations: stores 0.5 % faster, loads no effect.
#ifndef P2B_ITER_STREAM
#define P2B_ITER_STREAM 2
#endif
template <int VPT>
__device__ __forceinline__ FV<VPT> ldh_state(const float* row, int tid) {
    if constexpr ((P2B_ITER_STREAM & 1) != 0 && VPT != 2) {
        FV<VPT> r;
#pragma unroll
        for (int i = 0; i < VPT; ++i) r.v[i] = __ldcs(row + tid + i * (P2B_HPAD / VPT));
        return r;
    } else {
        return ldh<VPT>(row, tid);
    }
}
template <int VPT>
__device__ __forceinline__ void sth_state(float* row, int tid, const FV<VPT>& r) {
    if constexpr ((P2B_ITER_STREAM & 2) != 0 && VPT != 2) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) __stcs(row + tid + i * (P2B_HPAD / VPT), r.v[i]);
    } else {
        sth<VPT>(row, tid, r);
    }
}
// Pulls n consecutive rows into L2: a row is 42 lines of 128 bytes, thread t takes line t of each.
__device__ __forceinline__ void prefetch_lines(const float* row, int n, int tid) {
    if (tid < P2B_HPAD / 32) {
        const float* mine = row + 32 * tid;
#pragma unroll
        for (int c = 0; c < kK; ++c)
            if (c < n) asm volatile("prefetch.global.L2 [%0];" ::"l"(mine + c * P2B_HPAD));
    }
}

// Asynchronous copy of this thread's slice of a global row into its slice of a shared row.  The
// issuing thread sees the data after async_wait(); no other thread reads these slices.
template <int VPT>
__device__ __forceinline__ void async_row(float* smem_row, const float* global_row, int tid) {
    if constexpr (VPT == 2) {
        const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_row + VPT * tid);
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(global_row + VPT * tid) : "memory");
    } else {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int h = tid + i * (P2B_HPAD / VPT);
            const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_row + h);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(global_row + h) : "memory");
        }
    }
}
__device__ __forceinline__ void async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void async_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

struct IterBlock {
    unsigned char* tab;
    NodeRec* nodes;
    float* stage;
    unsigned char* ts;
    float* sig;
    uint8_t* rsrc;   // [node][player] internal index of the node whose reach row holds this player's reach (kNoRow: the mask)
    uint8_t* ilist;  // [ii] node index of the ii-th internal node
    uint8_t* sdc;    // [ii] child slot of the showdown leaf below the ii-th internal node (kNoRow: none)
    const uint16_t* csidx;  // [card][e] index of the e-th hand holding the card, hands in their natural order
    int* misc;       // [0] subgame taken from the queue, [2],[3] unit counters of the two table sets, [6] of an extra round
                     // ([4],[5] hold fsum)
    float* fsum;
    SubgameRec sg;
    float* scr;
    int max_internal;
    int sample_pass;  // pass whose policy is the sampling policy of the current subgame (-2: none)
    // work rows of the block: per internal node one reach row, one average-reach row and the values of
    // both players; then one current-policy row per node
    __device__ __forceinline__ float* row_reach(int x) const { return scr + (long long)(x * 4) * P2B_HPAD; }
    __device__ __forceinline__ float* row_rbar(int x) const { return scr + (long long)(x * 4 + 1) * P2B_HPAD; }
    __device__ __forceinline__ float* row_val(int x, int pl) const { return scr + (long long)(x * 4 + 2 + pl) * P2B_HPAD; }
    __device__ __forceinline__ float* row_pcur(int node) const {
        return scr + (long long)(max_internal * 4 + node) * P2B_HPAD;
    }
    __device__ __forceinline__ float* state_row(float* base, int node) const {
        return base + (long long)(sg.node_begin + node) * P2B_HPAD;
    }
    __device__ __forceinline__ float* set_row(int set, int r) const { return stage + (set * kSetRows + r) * P2B_HPAD; }
    // top-down sweep: kSets banks of child rows (rows whose sums normalise the children's beliefs), a stash
    // row per child and, with asynchronous copies, landing rows for the current policy and the average
    // policy of the children of one node
    __device__ __forceinline__ float* bank_row(int parity, int c) const { return stage + (parity * kK + c) * P2B_HPAD; }
    __device__ __forceinline__ float* stash_row(int c) const { return stage + (kSets * kK + c) * P2B_HPAD; }
    __device__ __forceinline__ float* land_row(int which, int c) const {
        return stage + (kDownRows + which * kK + c) * P2B_HPAD;
    }
};

// x / sum, or the uniform distribution over the allowed hands when the row is (numerically)
// empty (cfr_evaluator.py:263-273)
template <int VPT>
__device__ __forceinline__ void norm_row(float allowed_prob, const HandInfo<VPT>& hi, FV<VPT>& x, float sum) {
    const Divisor d = make_divisor(sum);
    DivGuard g = guard_begin(d.ok);
    FV<VPT> q;
#pragma unroll
    for (int i = 0; i < VPT; ++i) q.v[i] = div_g<true>(x.v[i], d.y, d.r, g);
    if (__builtin_expect(guard_bad(g), 0)) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) q.v[i] = __fdiv_rn(x.v[i], sum);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) x.v[i] = sum > 1e-5f ? q.v[i] : (hi.allowed[i] ? allowed_prob : 0.0f);
}

// Normalises the rows x[0], x[1] over hands through rows 0 and 1 of staging set 0; leaves the sums in B.fsum.
template <int VPT>
__device__ __forceinline__ void normalize_pair(IterBlock& B, const HandInfo<VPT>& hi, FV<VPT> (&x)[2], int tid) {
    sth<VPT>(B.set_row(0, 0), tid, x[0]);
    sth<VPT>(B.set_row(0, 1), tid, x[1]);
    __syncthreads();
    const int warp = tid >> 5;
    if (warp < 2) {
        const float sum = row_sum_reference_order(B.set_row(0, warp));
        if ((tid & 31) == 0) B.fsum[warp] = sum;
    }
    __syncthreads();
    norm_row<VPT>(B.sg.allowed_prob, hi, x[0], B.fsum[0]);
    norm_row<VPT>(B.sg.allowed_prob, hi, x[1], B.fsum[1]);
}

// Regret matching of the children of one node from the stored regrets into the current-policy rows
// (used once per subgame, before the first pass; later the bottom-up sweep keeps the rows current).
template <int VPT>
__device__ __forceinline__ void policy_from_regrets(const CfrParams& p, IterBlock& B, int j, int tid) {
    const NodeRec nd = B.nodes[j];
    const int k = nd.n_children, fc = nd.first_child;
    const float invk = __fdiv_rn(1.0f, (float)k);
    FV<VPT> sum;
#pragma unroll
    for (int i = 0; i < VPT; ++i) sum.v[i] = 0.0f;
#pragma unroll 1
    for (int c = 0; c < k; ++c) {
        FV<VPT> R = ldh<VPT>(B.state_row(p.regrets, fc + c), tid);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            R.v[i] = fmaxf(R.v[i], 0.0f);
            sum.v[i] = __fadd_rn(sum.v[i], R.v[i]);
        }
        sth<VPT>(B.stash_row(c), tid, R);
    }
    Divisor ds[VPT];
    bool dok = true;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        ds[i] = make_divisor(fmaxf(sum.v[i], 1e-8f));
        dok = dok && ds[i].ok;
    }
#pragma unroll 1
    for (int c = 0; c < k; ++c) {
        const FV<VPT> pos = ldh<VPT>(B.stash_row(c), tid);
        DivGuard g = guard_begin(dok);
        FV<VPT> P;
#pragma unroll
        for (int i = 0; i < VPT; ++i) P.v[i] = div_g<true>(pos.v[i], ds[i].y, ds[i].r, g);
        if (__builtin_expect(guard_bad(g), 0)) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) P.v[i] = __fdiv_rn(pos.v[i], ds[i].y);
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i) P.v[i] = sum.v[i] > 1e-8f ? P.v[i] : invk;
        sth<VPT>(B.row_pcur(fc + c), tid, P);
    }
}

// ---- top-down sweep of one iteration pass ------------------------------------------------
// Average-policy mix and renormalisation (cfr_evaluator.py:1195-1258), reach of both players
// (:332-361) and the normalisation sums of the children's beliefs (:254-273).
template <int VPT>
__device__ __forceinline__ void iter_down(int pass, const CfrParams& p, IterBlock& B, const HandInfo<VPT>& hi,
                                          const float* __restrict__ cr, int tid) {
    const IterScalars sc = p.scalars[pass];
    const bool mix = sc.do_mix != 0;
    const bool keep_policy = p.policy != nullptr && pass == p.iterations - 1;
    const bool keep_sample = p.policy_sample != nullptr && pass == B.sample_pass;
    FV<VPT> mask;
#pragma unroll
    for (int i = 0; i < VPT; ++i) mask.v[i] = hi.allowed[i] ? 1.0f : 0.0f;
    int parity = 0;
    const int n_internal = B.sg.n_internal;
    // the children's policy rows (and average-policy rows) land in shared memory one node ahead
    auto fetch_children = [&](int ii) {
        const NodeRec nn = B.nodes[B.ilist[ii]];
        for (int c = 0; c < nn.n_children; ++c) {
            async_row<VPT>(B.land_row(0, c), B.row_pcur(nn.first_child + c), tid);
            if (mix) async_row<VPT>(B.land_row(1, c), B.state_row(p.policy_avg, nn.first_child + c), tid);
        }
        async_commit();
    };
    if (kDownAsync) fetch_children(0);
#pragma unroll 1
    for (int ii = 0; ii < n_internal; ++ii) {
        const int j = B.ilist[ii];
        const NodeRec nd = B.nodes[j];
        const int a = nd.to_act, k = nd.n_children, fc = nd.first_child;
        if (mix && ii + 2 < n_internal) {  // average-policy rows are streamed from HBM: pull them into L2 two nodes ahead
            const NodeRec nn = B.nodes[B.ilist[ii + 2]];
            prefetch_lines(B.state_row(p.policy_avg, nn.first_child), nn.n_children, tid);
        }
        FV<VPT> ra = mask, rba = mask;
        const int sa = B.rsrc[j * 2 + a];
        if (sa != kNoRow) {
            ra = ldh<VPT>(B.row_reach(sa), tid);
            if (mix) rba = ldh<VPT>(B.row_rbar(sa), tid);
        }
        const FV<VPT> prior_a = ldh<VPT>(cr + a * P2B_HPAD, tid);
        // weights of the old average and of the new policy: reach-weighted, or the plain iteration
        // weights where the hand has (numerically) no reach (:1231-1239)
        FV<VPT> ro, rn, psum;
        Divisor dmix[VPT];
        bool dmix_ok = true;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            ro.v[i] = __fmul_rn(rba.v[i], sc.mix_old);
            rn.v[i] = __fmul_rn(ra.v[i], sc.mix_new);
            const float den = __fadd_rn(ro.v[i], rn.v[i]);
            const bool weighted = den > 1e-5f;
            ro.v[i] = weighted ? ro.v[i] : sc.mix_old;
            rn.v[i] = weighted ? rn.v[i] : sc.mix_new;
            dmix[i] = make_divisor(weighted ? den : sc.mix_total);
            dmix_ok = dmix_ok && dmix[i].ok;
            psum.v[i] = 0.0f;
        }
        const int bank = parity;
        if (kDouble) parity ^= 1;
        if (kDownAsync) async_wait();
        // with one bank, the warps that add up the previous node's rows must be done with them
        if (!kDouble && ii > 0) __syncthreads();
        FV<VPT> Pn, Pbn;
        if (!kDownAsync) {
            Pn = ldh<VPT>(B.row_pcur(fc), tid);
            if (mix) Pbn = ldh_state<VPT>(B.state_row(p.policy_avg, fc), tid);
        }
#pragma unroll 1
        for (int c = 0; c < k; ++c) {
            FV<VPT> P, Pb;
            if (kDownAsync) {
                P = ldh<VPT>(B.land_row(0, c), tid);
                if (mix) Pb = ldh<VPT>(B.land_row(1, c), tid);
            } else {
                P = Pn;
                Pb = Pbn;
                if (c + 1 < k) {
                    Pn = ldh<VPT>(B.row_pcur(fc + c + 1), tid);
                    if (mix) Pbn = ldh_state<VPT>(B.state_row(p.policy_avg, fc + c + 1), tid);
                }
            }
            const NodeRec ch = B.nodes[fc + c];
            // optional outputs: the current policy of the last iteration and of the subgame's sampling pass
            if (keep_policy) sth<VPT>(B.state_row(p.policy, fc + c), tid, P);
            if (keep_sample) sth<VPT>(B.state_row(p.policy_sample, fc + c), tid, P);
            FV<VPT> t;
#pragma unroll
            for (int i = 0; i < VPT; ++i) t.v[i] = __fmul_rn(ra.v[i], P.v[i]);
            if (ch.kind == kInternal) {
                sth<VPT>(B.row_reach(ch.internal_idx), tid, t);
                if (mix) {  // average reach under the OLD average policy
                    FV<VPT> tb;
#pragma unroll
                    for (int i = 0; i < VPT; ++i) tb.v[i] = __fmul_rn(rba.v[i], Pb.v[i]);
                    sth<VPT>(B.row_rbar(ch.internal_idx), tid, tb);
                }
            }
            if (ch.kind == kInternal || ch.kind == kShowdownLeaf) {
                FV<VPT> u;
#pragma unroll
                for (int i = 0; i < VPT; ++i) u.v[i] = __fmul_rn(prior_a.v[i], t.v[i]);
                sth<VPT>(B.bank_row(bank, c), tid, u);
            }
            if (mix) {
                DivGuard g = guard_begin(dmix_ok);
                FV<VPT> num, q;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    num.v[i] = __fadd_rn(__fmul_rn(ro.v[i], Pb.v[i]), __fmul_rn(rn.v[i], P.v[i]));
                    q.v[i] = div_g<true>(num.v[i], dmix[i].y, dmix[i].r, g);
                }
                if (__builtin_expect(guard_bad(g), 0)) {
#pragma unroll
                    for (int i = 0; i < VPT; ++i) q.v[i] = __fdiv_rn(num.v[i], dmix[i].y);
                }
#pragma unroll
                for (int i = 0; i < VPT; ++i) psum.v[i] = __fadd_rn(psum.v[i], q.v[i]);
                sth<VPT>(B.stash_row(c), tid, q);
            } else {
                sth_state<VPT>(B.state_row(p.policy_avg, fc + c), tid, P);
            }
        }
        if (kDownAsync && ii + 1 < n_internal) fetch_children(ii + 1);  // the landing rows are free again
        if (mix) {  // renormalise over the siblings (:1241-1258)
            Divisor dsum[VPT];
            bool dsum_ok = true;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                dsum[i] = make_divisor(psum.v[i]);
                dsum_ok = dsum_ok && dsum[i].ok;
            }
#pragma unroll 1
            for (int c = 0; c < k; ++c) {
                FV<VPT> q = ldh<VPT>(B.stash_row(c), tid), r;
                DivGuard g = guard_begin(dsum_ok);
#pragma unroll
                for (int i = 0; i < VPT; ++i) r.v[i] = div_g<true>(q.v[i], dsum[i].y, dsum[i].r, g);
                if (__builtin_expect(guard_bad(g), 0)) {
#pragma unroll
                    for (int i = 0; i < VPT; ++i) r.v[i] = __fdiv_rn(q.v[i], psum.v[i]);
                }
#pragma unroll
                for (int i = 0; i < VPT; ++i)
                    if (psum.v[i] > 1e-5f) q.v[i] = r.v[i];
                sth_state<VPT>(B.state_row(p.policy_avg, fc + c), tid, q);
            }
        }
        __syncthreads();
        // only the acting player's row is new: the other player's row, hence its sum, is the parent's
        const int warp = tid >> 5;
        if (warp < k) {
            const NodeRec ch = B.nodes[fc + warp];
            if (ch.kind == kInternal || ch.kind == kShowdownLeaf) {
                const float sum = row_sum_reference_order(B.bank_row(bank, warp));
                if ((tid & 31) == 0) {
                    B.sig[(fc + warp) * 2 + a] = sum;
                    B.sig[(fc + warp) * 2 + 1 - a] = B.sig[j * 2 + 1 - a];
                }
            }
        }
    }
}

// ---- cross-hand units of one node ----------------------------------------------------------
// Per-card sums and totals of the rows 0..n_cs-1 of a staging set and, when the node has a
// showdown child, strength-order and per-card prefix sums of row 1 (the other player's beliefs,
// slot 0) and of the leaf row (slot 1).  The warps take warp-sized units from a shared counter,
// largest first; every unit's arithmetic is fixed, so results do not depend on which warp ran it.
constexpr int kScanQuarter = 352;  // 32 lanes x 11 sorted positions

__device__ __forceinline__ void table_units(const IterBlock& B, const float* __restrict__ rows, unsigned char* ts,
                                            int n_cs, bool leaf, int* queue) {
    const BoardTabView tv = view_tables(B.tab);
    const int lane = threadIdx.x & 31;
    const int n_pc = leaf ? 2 : 0;
    const int quads_cs = n_cs * 208, quads = quads_cs + n_pc * 208;
    const uint16_t* __restrict__ cardlist = tv.cardlist;
    const uint16_t* __restrict__ sorted = tv.sorted;
    const int n_scan = 4 * n_pc, n_units = n_scan + n_cs + (quads + 31) / 32;
    double* __restrict__ cs_out = reinterpret_cast<double*>(ts + kTsCs);
    double* __restrict__ S_out = reinterpret_cast<double*>(ts + kTsS);
    float* __restrict__ pref_out = reinterpret_cast<float*>(ts + kTsPref);
    float* __restrict__ pc_out = reinterpret_cast<float*>(ts + kTsPc);
    float* __restrict__ tot_out = reinterpret_cast<float*>(ts + kTsTot);
    while (true) {
        int unit = 0;
        if (lane == 0) unit = atomicAdd(queue, 1);
        unit = __shfl_sync(0xffffffffu, unit, 0);
        if (unit >= n_units) break;
        if (unit < n_scan) {
            // quarter scan; the last quarters (most preceding positions to add up) go first
            const int slot = unit & 1, qi = 3 - (unit >> 1);
            const float* __restrict__ x = rows + (slot ? kRowLeaf : 1) * P2B_HPAD;
            float* __restrict__ pref = pref_out + slot * P2B_HPAD;
            double before = 0.0;
            for (int r = 0; r < qi; ++r) {
                const int k0 = r * kScanQuarter + 11 * lane;
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
            // total mass of a row (the 18 padding entries of a staged row are zero)
            const int wt = unit - n_scan;
            const float* __restrict__ x = rows + wt * P2B_HPAD;
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
            if (lane == 0) S_out[wt] = tot;
        } else {
            // list round: thread t of the round works on quarter q of list (row, card)
            const int t_raw = (unit - n_scan - n_cs) * 32 + lane;
            const bool valid = t_raw < quads;
            const int t = valid ? t_raw : quads - 1;  // idle threads of the last round redo the last task, unstored
            const bool is_cs = t < quads_cs;
            const int u = is_cs ? t : t - quads_cs;
            const int slot = u / 208, rem = u % 208, c = rem >> 2, q = rem & 3;
            const float* __restrict__ x = rows + (is_cs ? slot : (slot ? kRowLeaf : 1)) * P2B_HPAD;
            float v[13];
            if (is_cs) {
                // e-th hand holding card c, in hand order ((e, c) for e < c, then (c, e + 1)): its index comes from
                // a table of the block; computing it costs more issue slots than the load costs shared-memory cycles
                const uint16_t* __restrict__ ib = B.csidx + c * 52 + q;
#pragma unroll
                for (int i = 0; i < 12; ++i) v[i] = x[ib[4 * i]];
                v[12] = q < 3 ? x[ib[48]] : 0.0f;
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
                    if (q == 0) cs_out[slot * 52 + c] = ((t0 + t1) + t2) + t3;
                } else {
                    double acc = q == 0 ? 0.0 : (q == 1 ? t0 : (q == 2 ? t0 + t1 : (t0 + t1) + t2));
                    float* __restrict__ row = pc_out + slot * 52 * 52 + c * 52;
                    if (q == 0) row[0] = 0.0f;
                    float* __restrict__ out = row + 13 * q + 1;
#pragma unroll
                    for (int i = 0; i < 12; ++i) {
                        acc += (double)v[i];
                        out[i] = (float)acc;
                    }
                    if (q < 3) out[12] = (float)(acc + (double)v[12]);
                    else tot_out[slot * 64 + c] = (float)acc;  // == row[51]
                }
            }
        }
    }
}

// ---- bottom-up sweep, first half of a node: beliefs, staged rows ---------------------------
// Beliefs of the node (cfr_evaluator.py:363-380), marginal policy rows b_a * P[c] whose
// unblocked mass conditions the child policy on the other player's hand (:1076-1093), and the
// acting player's beliefs at the showdown child.
template <int VPT>
__device__ __forceinline__ void iter_up_stage(int pass, const CfrParams& p, IterBlock& B, const HandInfo<VPT>& hi,
                                              const float* __restrict__ cr, int ii, int set, int tid) {
    const int j = B.ilist[ii];
    const NodeRec nd = B.nodes[j];
    const int a = nd.to_act, o = 1 - a, k = nd.n_children, fc = nd.first_child;
    const FV<VPT> prior_a = ldh<VPT>(cr + a * P2B_HPAD, tid);
    FV<VPT> r_a, b_a, b_o;
#pragma unroll
    for (int i = 0; i < VPT; ++i) r_a.v[i] = hi.allowed[i] ? 1.0f : 0.0f;
    if (j == 0) {
        b_a = ldh<VPT>(cr + (2 + a) * P2B_HPAD, tid);
        b_o = ldh<VPT>(cr + (2 + o) * P2B_HPAD, tid);
    } else {
        const FV<VPT> prior_o = ldh<VPT>(cr + o * P2B_HPAD, tid);
        FV<VPT> r_o = r_a;
        const int sa = B.rsrc[j * 2 + a], so = B.rsrc[j * 2 + o];
        if (sa != kNoRow) r_a = ldh<VPT>(B.row_reach(sa), tid);
        if (so != kNoRow) r_o = ldh<VPT>(B.row_reach(so), tid);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            b_a.v[i] = __fmul_rn(prior_a.v[i], r_a.v[i]);
            b_o.v[i] = __fmul_rn(prior_o.v[i], r_o.v[i]);
        }
        norm_row<VPT>(B.sg.allowed_prob, hi, b_a, B.sig[j * 2 + a]);
        norm_row<VPT>(B.sg.allowed_prob, hi, b_o, B.sig[j * 2 + o]);
    }
    if (pass + 1 < p.iterations) {  // rows the second half of this node updates, streamed from HBM
        prefetch_lines(B.state_row(p.regrets, fc), k, tid);
        if (p.weight_sums) prefetch_lines(B.state_row(p.weight_sums, fc), k, tid);
    }
    sth<VPT>(B.set_row(set, 0), tid, b_a);
    sth<VPT>(B.set_row(set, 1), tid, b_o);
    if (p.beliefs_last && pass == p.iterations - 1) {  // optional output: what leaf sampling continues from
        sth<VPT>(p.beliefs_last + ((long long)(B.sg.node_begin + j) * 2 + a) * P2B_HPAD, tid, b_a);
        sth<VPT>(p.beliefs_last + ((long long)(B.sg.node_begin + j) * 2 + o) * P2B_HPAD, tid, b_o);
    }
    const int sd = B.sdc[ii];
#pragma unroll 1
    for (int c = 0; c < k; ++c) {
        const FV<VPT> Pc = ldh<VPT>(B.row_pcur(fc + c), tid);
        FV<VPT> m;
#pragma unroll
        for (int i = 0; i < VPT; ++i) m.v[i] = __fmul_rn(b_a.v[i], Pc.v[i]);
        sth<VPT>(B.set_row(set, kRowM + c), tid, m);
        if (c == sd) {
            FV<VPT> bca;
#pragma unroll
            for (int i = 0; i < VPT; ++i) bca.v[i] = __fmul_rn(prior_a.v[i], __fmul_rn(r_a.v[i], Pc.v[i]));
            norm_row<VPT>(B.sg.allowed_prob, hi, bca, B.sig[(fc + c) * 2 + a]);
            sth<VPT>(B.set_row(set, kRowLeaf), tid, bca);
        }
    }
}

// Showdown EV (before the pot scaling) of this thread's hands against the staged range x.
template <int VPT>
__device__ __forceinline__ void showdown_ev(const IterBlock& B, const HandInfo<VPT>& hi, int tid,
                                            const float* __restrict__ x, const float* __restrict__ pref,
                                            const float* __restrict__ pc, const float* __restrict__ tot, FV<VPT>& ev) {
    const BoardTabView tv = view_tables(B.tab);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        float e = 0.0f;
        if (hi.valid[i]) {
            const int h = hand_of<VPT>(tid, i);
            e = showdown_hand_ev(tv.rec[h], hi.c1[i], hi.c2[i], x[h], hi.allowed[i], pref, pc, tot[hi.c1[i]], tot[hi.c2[i]]);
        }
        ev.v[i] = e;
    }
}

// ---- bottom-up sweep, second half of a node: per-hand arithmetic ---------------------------
// Opponent-conditioned child policy (cfr_evaluator.py:1083-1093), leaf values (fold constants,
// showdown :484-601), value backup (:1095-1115), instantaneous regrets (:1117-1165) folded into the
// discounted update of the next iteration (:1346-1368), and regret matching of the updated
// regrets (:1168-1185) into the current-policy rows of the next pass.
template <int VPT>
__device__ __forceinline__ void iter_up_hands(int pass, const CfrParams& p, IterBlock& B, const HandInfo<VPT>& hi,
                                              const float* __restrict__ cr, int ii, int set, int tid) {
    const int j = B.ilist[ii];
    const NodeRec nd = B.nodes[j];
    const int a = nd.to_act, o = 1 - a, k = nd.n_children, fc = nd.first_child;
    const unsigned char* ts = B.ts + set * kTsBytes;
    const double* __restrict__ cs = reinterpret_cast<const double*>(ts + kTsCs);
    const double* __restrict__ St = reinterpret_cast<const double*>(ts + kTsS);
    const float* __restrict__ pref = reinterpret_cast<const float*>(ts + kTsPref);
    const float* __restrict__ pc = reinterpret_cast<const float*>(ts + kTsPc);
    const float* __restrict__ tot = reinterpret_cast<const float*>(ts + kTsTot);
    const FV<VPT> b_a = ldh<VPT>(B.set_row(set, 0), tid), b_o = ldh<VPT>(B.set_row(set, 1), tid);
    FV<VPT> wgt, denm, acc_a, acc_o;
    Divisor ddenm[VPT];
    bool ddenm_ok = true;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        wgt.v[i] = unblocked(cs + 52, St[1], hi.c1[i], hi.c2[i], b_o.v[i]);
        denm.v[i] = unblocked(cs, St[0], hi.c1[i], hi.c2[i], b_a.v[i]);
        ddenm[i] = make_divisor(denm.v[i]);
        ddenm_ok = ddenm_ok && ddenm[i].ok;
        acc_a.v[i] = acc_o.v[i] = 0.0f;
    }
    sth<VPT>(B.set_row(set, 0), tid, wgt);  // needed again for the regrets; the beliefs row is spent
    const int sd = B.sdc[ii];
    // ---- policy of every child as seen by each hand of the other player; replaces the marginal rows ----
#pragma unroll 1
    for (int c = 0; c < k; ++c) {
        const FV<VPT> m = ldh<VPT>(B.set_row(set, kRowM + c), tid);
        FV<VPT> pio, blk;
        DivGuard g = guard_begin(ddenm_ok);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            blk.v[i] = unblocked(cs + (kRowM + c) * 52, St[kRowM + c], hi.c1[i], hi.c2[i], m.v[i]);
            pio.v[i] = div_g<true>(blk.v[i], ddenm[i].y, ddenm[i].r, g);
        }
        if (__builtin_expect(guard_bad(g), 0)) {
#pragma unroll
            for (int i = 0; i < VPT; ++i) pio.v[i] = __fdiv_rn(blk.v[i], denm.v[i]);
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i) pio.v[i] = denm.v[i] > 1e-5f ? pio.v[i] : 0.0f;
        sth<VPT>(B.set_row(set, kRowM + c), tid, pio);
    }
    // ---- children: values and backup ----
    {
#pragma unroll 1
        for (int c = 0; c < k; ++c) {
            const NodeRec ch = B.nodes[fc + c];
            const FV<VPT> P = ldh<VPT>(B.row_pcur(fc + c), tid);
            FV<VPT> V_a, V_o;
            if (ch.kind == kInternal) {
                V_a = ldh<VPT>(B.row_val(ch.internal_idx, a), tid);
                V_o = ldh<VPT>(B.row_val(ch.internal_idx, o), tid);
            }
            const FV<VPT> pio = ldh<VPT>(B.set_row(set, kRowM + c), tid);  // computed by the loop above
            if (ch.kind == kFoldLeaf) {
                const float va = a == 0 ? ch.v0 : -ch.v0;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    V_a.v[i] = va;
                    V_o.v[i] = -va;
                }
            } else if (ch.kind == kShowdownLeaf) {
                // the acting player's hands against the other player's beliefs, and the reverse at the leaf
                FV<VPT> eva, evo;
                showdown_ev<VPT>(B, hi, tid, B.set_row(set, 1), pref, pc, tot, eva);
                if (c == sd) showdown_ev<VPT>(B, hi, tid, B.set_row(set, kRowLeaf), pref + P2B_HPAD, pc + 52 * 52, tot + 64, evo);
                if (c != sd) {
                    // A further showdown child (a call and an all-in of the same size; rare): its tables
                    // are built here, in one more block-wide round, in place of the first one's.
                    const FV<VPT> prior_a = ldh<VPT>(cr + a * P2B_HPAD, tid);
                    FV<VPT> bca;
#pragma unroll
                    for (int i = 0; i < VPT; ++i) bca.v[i] = hi.allowed[i] ? 1.0f : 0.0f;
                    const int sa = B.rsrc[j * 2 + a];
                    if (j != 0 && sa != kNoRow) bca = ldh<VPT>(B.row_reach(sa), tid);
#pragma unroll
                    for (int i = 0; i < VPT; ++i) bca.v[i] = __fmul_rn(prior_a.v[i], __fmul_rn(bca.v[i], P.v[i]));
                    norm_row<VPT>(B.sg.allowed_prob, hi, bca, B.sig[(fc + c) * 2 + a]);
                    __syncthreads();  // every thread is done with the leaf tables of the first showdown child
                    sth<VPT>(B.set_row(set, kRowLeaf), tid, bca);
                    if (tid == 0) B.misc[6] = 0;
                    __syncthreads();
                    table_units(B, B.set_row(set, 0), B.ts + set * kTsBytes, 0, true, B.misc + 6);
                    __syncthreads();
                    showdown_ev<VPT>(B, hi, tid, B.set_row(set, kRowLeaf), pref + P2B_HPAD, pc + 52 * 52, tot + 64, evo);
                }
                const float pot_a = a == 0 ? ch.v0 : ch.v1, pot_o = a == 0 ? ch.v1 : ch.v0;
                const Divisor dscale = make_divisor(B.sg.scale);
                DivGuard g = guard_begin(dscale.ok);
                FV<VPT> na, no;
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    na.v[i] = __fmul_rn(eva.v[i], pot_a);
                    no.v[i] = __fmul_rn(evo.v[i], pot_o);
                    V_a.v[i] = div_g<false>(na.v[i], dscale.y, dscale.r, g);
                    V_o.v[i] = div_g<false>(no.v[i], dscale.y, dscale.r, g);
                }
                if (__builtin_expect(guard_bad(g), 0)) {
#pragma unroll
                    for (int i = 0; i < VPT; ++i) {
                        V_a.v[i] = __fdiv_rn(na.v[i], B.sg.scale);
                        V_o.v[i] = __fdiv_rn(no.v[i], B.sg.scale);
                    }
                }
            } else if (ch.kind != kInternal) {  // a leaf no model values in a plain solve
#pragma unroll
                for (int i = 0; i < VPT; ++i) V_a.v[i] = V_o.v[i] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                acc_a.v[i] = __fadd_rn(acc_a.v[i], __fmul_rn(V_a.v[i], P.v[i]));
                acc_o.v[i] = __fadd_rn(acc_o.v[i], __fmul_rn(V_o.v[i], pio.v[i]));
            }
            sth<VPT>(B.set_row(set, kRowM + c), tid, V_a);  // kept for the regrets below; the row's pio is spent
        }
    }
    if (j != 0) {
        sth<VPT>(B.row_val(ii, a), tid, acc_a);
        sth<VPT>(B.row_val(ii, o), tid, acc_o);
    }
    if (pass + 1 >= p.iterations) return;  // the last iteration leaves the regrets as they are
    // ---- regrets of this pass folded into the discounted update of the next, then its policy ----
    const IterScalars sc = p.scalars[pass + 1];
    const Divisor d_pos = make_divisor(sc.den_pos), d_neg = make_divisor(sc.den_neg);
    const bool d_ok = d_pos.ok && d_neg.ok;
    const bool tracked = p.weight_sums != nullptr;
    wgt = ldh<VPT>(B.set_row(set, 0), tid);
    FV<VPT> psum;
#pragma unroll
    for (int i = 0; i < VPT; ++i) psum.v[i] = 0.0f;
    {
#pragma unroll 1
        for (int c = 0; c < k; ++c) {
            FV<VPT> R = ldh_state<VPT>(B.state_row(p.regrets, fc + c), tid), W;
            if (tracked) W = ldh_state<VPT>(B.state_row(p.weight_sums, fc + c), tid);
            const FV<VPT> Va = ldh<VPT>(B.set_row(set, kRowM + c), tid);
            FV<VPT> rn, wn, rq, wq, dy;
            DivGuard g = guard_begin(d_ok);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const bool pos = R.v[i] > 0.0f;
                const float num = pos ? sc.num_pos : sc.num_neg;
                const float dr = pos ? d_pos.r : d_neg.r;
                dy.v[i] = pos ? d_pos.y : d_neg.y;
                rn.v[i] = __fmul_rn(R.v[i], num);
                rq.v[i] = div_g<false>(rn.v[i], dy.v[i], dr, g);
                if (tracked) {
                    wn.v[i] = __fmul_rn(W.v[i], num);
                    wq.v[i] = div_g<true>(wn.v[i], dy.v[i], dr, g);
                }
            }
            if (__builtin_expect(guard_bad(g), 0)) {
#pragma unroll
                for (int i = 0; i < VPT; ++i) {
                    rq.v[i] = __fdiv_rn(rn.v[i], dy.v[i]);
                    if (tracked) wq.v[i] = __fdiv_rn(wn.v[i], dy.v[i]);
                }
            }
            FV<VPT> posn;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const float reg = __fmul_rn(wgt.v[i], __fsub_rn(Va.v[i], acc_a.v[i]));
                float rr = __fadd_rn(rq.v[i], reg);
                if (p.cfr_plus) rr = fmaxf(rr, 0.0f);
                R.v[i] = rr;
                if (tracked) W.v[i] = __fadd_rn(wq.v[i], 1.0f);
                posn.v[i] = fmaxf(rr, 0.0f);
                psum.v[i] = __fadd_rn(psum.v[i], posn.v[i]);
            }
            sth_state<VPT>(B.state_row(p.regrets, fc + c), tid, R);
            if (tracked) sth_state<VPT>(B.state_row(p.weight_sums, fc + c), tid, W);
            sth<VPT>(B.set_row(set, kRowM + c), tid, posn);
        }
    }
    {
        const float invk = __fdiv_rn(1.0f, (float)k);
        Divisor ds[VPT];
        bool ds_ok = true;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            ds[i] = make_divisor(fmaxf(psum.v[i], 1e-8f));
            ds_ok = ds_ok && ds[i].ok;
        }
#pragma unroll 1
        for (int c = 0; c < k; ++c) {
            const FV<VPT> posn = ldh<VPT>(B.set_row(set, kRowM + c), tid);
            DivGuard g = guard_begin(ds_ok);
            FV<VPT> P;
#pragma unroll
            for (int i = 0; i < VPT; ++i) P.v[i] = div_g<true>(posn.v[i], ds[i].y, ds[i].r, g);
            if (__builtin_expect(guard_bad(g), 0)) {
#pragma unroll
                for (int i = 0; i < VPT; ++i) P.v[i] = __fdiv_rn(posn.v[i], ds[i].y);
            }
#pragma unroll
            for (int i = 0; i < VPT; ++i) P.v[i] = psum.v[i] > 1e-8f ? P.v[i] : invk;
            sth<VPT>(B.row_pcur(fc + c), tid, P);
        }
    }
}

template <int VPT>
__global__ void __launch_bounds__(kNT, kCtas) cfr_iter_kernel(const CfrParams p) {
    constexpr int NT = kNT;
    extern __shared__ __align__(16) unsigned char smem[];
    IterBlock B;
    B.tab = smem + kOffTab;
    B.nodes = reinterpret_cast<NodeRec*>(smem + kOffNodes);
    B.stage = reinterpret_cast<float*>(smem + kOffStage);
    B.ts = smem + kOffTs;
    B.sig = reinterpret_cast<float*>(smem + kOffSig);
    B.rsrc = smem + kOffRsrc;
    B.ilist = smem + kOffIlist;
    B.sdc = smem + kOffSdc;
    B.misc = reinterpret_cast<int*>(smem + kOffMisc);
    {
        uint16_t* t = reinterpret_cast<uint16_t*>(smem + kOffCsIdx);
        for (int i = threadIdx.x; i < 52 * 52; i += kNT) {
            const int c = i / 52, e = i % 52;
            const int ee = e < 51 ? e : 50;
            t[i] = (uint16_t)(ee < c ? ((ee * (103 - ee)) >> 1) + (c - ee - 1) : combo_row_offset(c) - c + ee);
        }
        B.csidx = t;
    }
    B.fsum = reinterpret_cast<float*>(smem + kOffMisc + 16);
    B.max_internal = p.max_internal;
    B.scr = p.scratch + (long long)(blockIdx.x / kCtas) * p.scratch_stride +
            (long long)(blockIdx.x % kCtas) * (p.scratch_stride / kCtas);
    const int rtid = threadIdx.x;                        // this thread
    const int tid = rtid < kHT ? rtid : kHT - 1;         // the hand thread whose per-hand work it does

    HandInfo<VPT> hi;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int h = hand_of<VPT>(tid, i);
        hi.valid[i] = h < P2B_NUM_HANDS;
        const int hc = h < P2B_NUM_HANDS ? h : P2B_NUM_HANDS - 1;
        hi.c1[i] = p.combos->c1[hc];
        hi.c2[i] = p.combos->c2[hc];
    }

    while (true) {
        __syncthreads();
        if (rtid == 0) B.misc[0] = atomicAdd(p.work_counter, 1);
        __syncthreads();
        if (B.misc[0] >= p.num_subgames) break;
        const int s = p.queue_order ? p.queue_order[B.misc[0]] : B.misc[0];
        B.sg = p.subgames[s];
        if (B.sg.n_nodes > kIterMaxNodes) continue;  // too large for this kernel's tables: the general kernel runs its passes
        B.sample_pass = p.sample_pass ? p.sample_pass[s] : -2;
        {
            for (int i = rtid; i < B.sg.n_nodes; i += NT) B.nodes[i] = load_node(p.nodes + B.sg.node_begin + i);
            if (B.sg.table_index >= 0) {
                const uint4* t = reinterpret_cast<const uint4*>(p.tables + (long long)B.sg.table_index * kTabBytes);
                for (int i = rtid; i < kTabBytes / 16; i += NT) reinterpret_cast<uint4*>(B.tab)[i] = t[i];
            }
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i)
            hi.allowed[i] = hi.valid[i] && (((B.sg.board_mask >> hi.c1[i]) | (B.sg.board_mask >> hi.c2[i])) & 1ull) == 0;
        // The root rows stay in the hand-over area of the subgame: rows 0, 1 = the root beliefs the node
        // beliefs of a pass derive from, rows 2, 3 = the root's own rows (renormalised once per pass, like
        // every other row upstream), as the start pass left them.
        float* cr = p.carry_roots + (long long)s * 4 * P2B_HPAD;
        __syncthreads();
        // per node: list of the internal nodes, where each player's reach is stored, the showdown child
        for (int i = rtid; i < B.sg.n_nodes; i += NT) {
            const NodeRec nd = B.nodes[i];
            if (nd.kind != kInternal) continue;
            B.ilist[nd.internal_idx] = (uint8_t)i;
            uint8_t sdc = kNoRow;
            for (int c = nd.n_children - 1; c >= 0; --c)
                if (B.nodes[nd.first_child + c].kind == kShowdownLeaf) sdc = (uint8_t)c;
            B.sdc[nd.internal_idx] = sdc;
            for (int pl = 0; pl < 2; ++pl) {
                uint8_t src = kNoRow;
                int x = i;
                while (x != 0) {
                    const int par = B.nodes[x].parent;
                    if (B.nodes[par].to_act == pl) {
                        src = B.nodes[x].internal_idx;
                        break;
                    }
                    x = par;
                }
                B.rsrc[i * 2 + pl] = src;
            }
        }
        __syncthreads();
        const int n_internal = B.sg.n_internal;
        // current policy of the first pass: regret matching on the regrets the start pass left
        for (int ii = 0; ii < n_internal; ++ii) policy_from_regrets<VPT>(p, B, B.ilist[ii], tid);

        for (int pass = 0; pass < p.iterations; ++pass) {
            {
                FV<VPT> root_b[2];
                root_b[0] = ldh<VPT>(cr + 2 * P2B_HPAD, tid);
                root_b[1] = ldh<VPT>(cr + 3 * P2B_HPAD, tid);
                sth<VPT>(cr, tid, root_b[0]);
                sth<VPT>(cr + P2B_HPAD, tid, root_b[1]);
                normalize_pair<VPT>(B, hi, root_b, tid);
                sth<VPT>(cr + 2 * P2B_HPAD, tid, root_b[0]);
                sth<VPT>(cr + 3 * P2B_HPAD, tid, root_b[1]);
            }
            // a child's row of the player who did not act is the root's row; so is its sum
            if (tid < 2) B.sig[tid] = B.fsum[tid];
            __syncthreads();
            iter_down<VPT>(pass, p, B, hi, cr, tid);
            if (tid == 0) B.misc[2] = B.misc[3] = 0;
            __syncthreads();
            if (kDouble) {
                // bottom-up: the cross-hand units of a node run while the hands of the node above it
                // (in sweep order: the one before) are worked on
                int set = 0;
                iter_up_stage<VPT>(pass, p, B, hi, cr, n_internal - 1, set, tid);
                __syncthreads();
                {
                    const NodeRec nd = B.nodes[B.ilist[n_internal - 1]];
                    table_units(B, B.set_row(set, 0), B.ts + set * kTsBytes, 2 + nd.n_children,
                                B.sdc[n_internal - 1] != kNoRow, B.misc + 2 + set);
                }
                for (int ii = n_internal - 1; ii >= 0; --ii) {
                    if (ii > 0) {
                        iter_up_stage<VPT>(pass, p, B, hi, cr, ii - 1, set ^ 1, tid);
                        if (tid == 0) B.misc[2 + (set ^ 1)] = 0;
                    }
                    __syncthreads();  // staged rows of node ii-1 and the tables of node ii are complete
                    if (ii > 0) {
                        const NodeRec nd = B.nodes[B.ilist[ii - 1]];
                        table_units(B, B.set_row(set ^ 1, 0), B.ts + (set ^ 1) * kTsBytes, 2 + nd.n_children,
                                    B.sdc[ii - 1] != kNoRow, B.misc + 2 + (set ^ 1));
                    }
                    iter_up_hands<VPT>(pass, p, B, hi, cr, ii, set, tid);
                    set ^= 1;
                }
            } else {
                // bottom-up with one set of rows and tables: stage, units, hands, two barriers per node;
                // the other block of the SM fills the gaps
                for (int ii = n_internal - 1; ii >= 0; --ii) {
                    iter_up_stage<VPT>(pass, p, B, hi, cr, ii, 0, tid);
                    if (tid == 0) B.misc[2] = 0;
                    __syncthreads();  // rows staged; every thread is done with the tables of the node before
                    const NodeRec nd = B.nodes[B.ilist[ii]];
                    table_units(B, B.set_row(0, 0), B.ts, 2 + nd.n_children, B.sdc[ii] != kNoRow, B.misc + 2);
                    __syncthreads();
                    iter_up_hands<VPT>(pass, p, B, hi, cr, ii, 0, tid);
                }
            }
            __syncthreads();
        }
        // the root rows are in place for the final pass; hand over their sums
        if (tid < 2) p.carry_sums[(long long)B.sg.node_begin * 2 + tid] = B.sig[tid];
    }
}

}  // namespace

// floats of work rows the blocks of the iteration kernel on one SM need
long long cfr_iter_scratch_floats(int max_internal, int max_children) {
    long long nodes = (long long)max_internal * max_children + 1;
    if (nodes > kIterMaxNodes) nodes = kIterMaxNodes;
    return kCtas * ((long long)max_internal * 4 + nodes) * P2B_HPAD;
}

int launch_cfr_iter(const CfrParams& p, int num_blocks, cudaStream_t stream) {
    int rc = check_cuda(cudaFuncSetAttribute(cfr_iter_kernel<kVpt>, cudaFuncAttributeMaxDynamicSharedMemorySize, kIterSmem),
                        "cfr_iter_kernel shared-memory attribute");
    if (rc) return rc;
    cfr_iter_kernel<kVpt><<<num_blocks * kCtas, kNT, kIterSmem, stream>>>(p);
    return check_cuda(cudaGetLastError(), "cfr_iter_kernel");
}

}  // namespace p2b
