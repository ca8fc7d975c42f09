// Blocker-aware river showdown: per-board strength tables and the per-range evaluation.
//
// What is computed (p2/search/cfr_evaluator.py:406-601): for a hero hand h=(c1,c2) against
// an opponent range x over the 1326 combos, with hands sorted by strength and tie groups
// [L,R) in sorted positions,
//   win  = P[L] - PC[c1][<L] - PC[c2][<L]
//   tie  = (P[R]-P[L]) - (PC[c1][<R]-PC[c1][<L]) - (PC[c2][<R]-PC[c2][<L]) + x[h]
//   den  = max(1 - PC[c1][all] - PC[c2][all] + x[h], 1e-8)
//   EV   = win/den - (1 - win/den - tie/den),   0 for hands that use a board card
// where P is the prefix sum of x in strength order and PC[c] the prefix sum restricted to
// hands holding card c.  The upstream code materialises PC as an [1327,52] table per
// node; here each card keeps its own list of 51 hands in strength order, and a hand
// stores how many entries of its two lists lie before L and before R, so PC is a
// 52x52 table in shared memory.  Prefix sums are accumulated in fp64 and rounded to
// fp32 per element, which is what the upstream CPU cumsum does; the remaining
// arithmetic is fp32 in the upstream operation order.
#pragma once

#include "common.cuh"
#include "exactdiv.cuh"
#include "rank7.cuh"

namespace p2b {

// ---- per-board table blob (global memory and shared memory use the same layout) ----
struct HandRec {          // 8 bytes per hand, natural combo order
    uint16_t lpos, rpos;  // tie group [lpos, rpos) in sorted positions
    uint8_t nb0, ne0;     // entries of card c1's list before lpos / before rpos
    uint8_t nb1, ne1;     // same for card c2
};
constexpr int kTabHeaderBytes = 16;                 // uint64 board-card mask + padding
constexpr int kTabRecBytes = P2B_NUM_HANDS * 8;     // 10608
constexpr int kTabSortedPad = 1328;                 // entries reserved for the strength order (1326 used)
constexpr int kTabSortedBytes = kTabSortedPad * 2;  // 2656
constexpr int kTabCardListBytes = 5312;             // uint16 [51][52] = 5304 used
constexpr int kTabBytes = kTabHeaderBytes + kTabRecBytes + kTabSortedBytes + kTabCardListBytes;  // 18592
static_assert(kTabBytes % 16 == 0, "table blob must be a whole number of 16-byte vectors");
static_assert(kTabBytes == 18592, "the table size is part of the C ABI (P2B_TABLE_BYTES)");

struct BoardTabView {
    const unsigned long long* board_mask;
    const HandRec* rec;
    const uint16_t* sorted;     // [1326] combo at sorted position k
    const uint16_t* cardlist;   // [51][52]: t-th weakest hand holding card c at [t*52+c]
};
__host__ __device__ __forceinline__ BoardTabView view_tables(const unsigned char* blob) {
    BoardTabView v;
    v.board_mask = reinterpret_cast<const unsigned long long*>(blob);
    v.rec = reinterpret_cast<const HandRec*>(blob + kTabHeaderBytes);
    v.sorted = reinterpret_cast<const uint16_t*>(blob + kTabHeaderBytes + kTabRecBytes);
    v.cardlist = reinterpret_cast<const uint16_t*>(blob + kTabHeaderBytes + kTabRecBytes + kTabSortedBytes);
    return v;
}

// One hero hand of the showdown formula.  P: [1327] prefix in strength order; PC: [52][52]
// per-card prefix (PC[c*52+t] = mass of the t weakest hands holding c); x: opponent range;
// tot1, tot2: the whole mass of the hands holding c1 / c2 (PC[c*52+51], which a caller may keep in a
// table of its own).
__device__ __forceinline__ float showdown_hand_ev(const HandRec r, int c1, int c2, float xh, bool allowed,
                                                  const float* __restrict__ P, const float* __restrict__ PC, float tot1,
                                                  float tot2) {
    const float PL = P[r.lpos], PR = P[r.rpos];
    const float* pc1 = PC + c1 * 52;
    const float* pc2 = PC + c2 * 52;
    const float a0 = pc1[r.nb0], a1 = pc1[r.ne0], b0 = pc2[r.nb1], b1 = pc2[r.ne1];
    const float win = __fsub_rn(__fsub_rn(PL, a0), b0);
    const float seg = __fsub_rn(PR, PL);
    const float tie = __fadd_rn(__fsub_rn(__fsub_rn(seg, __fsub_rn(a1, a0)), __fsub_rn(b1, b0)), xh);
    float den = __fadd_rn(__fsub_rn(__fsub_rn(1.0f, tot1), tot2), xh);
    den = fmaxf(den, 1e-8f);
    const Divisor d = make_divisor(den);
    bool bad = false;
    float wp = div_fast(win, d, bad), tp = div_fast(tie, d, bad);
    if (__builtin_expect(bad, 0)) {
        wp = __fdiv_rn(win, den);
        tp = __fdiv_rn(tie, den);
    }
    const float lp = __fsub_rn(__fsub_rn(1.0f, wp), tp);
    const float ev = __fsub_rn(wp, lp);
    return (allowed && den > 1e-8f) ? ev : 0.0f;
}
__device__ __forceinline__ float showdown_hand_ev(const HandRec r, int c1, int c2, float xh, bool allowed,
                                                  const float* __restrict__ P, const float* __restrict__ PC) {
    return showdown_hand_ev(r, c1, c2, xh, allowed, P, PC, PC[c1 * 52 + 51], PC[c2 * 52 + 51]);
}

}  // namespace p2b
