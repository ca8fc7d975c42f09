// 7-card hand scoring on suit bit masks (device functions shared by the rank, board-setup
// and compare kernels).
//
// Output convention (bit-exact with the upstream evaluator, p2/env/rules.py:136-299 and
// p2/env/rules_triton.py:415-581): six 4-bit fields [type,k1..k5] packed as
// type<<20 | k1<<16 | k2<<12 | k3<<8 | k4<<4 | k5, where
//   * kickers are the ranks ordered by (count desc, rank desc);
//   * the straight field is the LOWEST complete 5-window (window 0 = wheel A2345,
//     window w>=1 covers ranks w-1..w+3);
//   * the straight-flush field is the HIGHEST complete window inside one suit;
//   * the flush fields are the five highest ranks of the first suit holding >= 5 cards.
#pragma once

#include <stdint.h>

namespace p2b {

struct RankClasses {
    uint32_t quads, trips, pairs, singles;  // 13-bit rank masks by multiplicity
};

// Multiplicity classes when every card is distinct: the count of a rank is the number of
// suit masks that hold it (bit-sliced 4-input adder).
__device__ __forceinline__ RankClasses classes_from_suits(uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3) {
    const uint32_t x = m0 ^ m1, y = m2 ^ m3, a = m0 & m1, b = m2 & m3;
    const uint32_t b0 = x ^ y;
    const uint32_t b1 = a ^ b ^ (x & y);
    RankClasses rc;
    rc.quads = a & b;
    rc.trips = b1 & b0;
    rc.pairs = b1 & ~b0;
    rc.singles = b0 & ~b1;
    return rc;
}

// Multiplicity classes when card ids may repeat: every occurrence counts, saturating at
// four (p2/env/rules_triton.py:431-446).
struct RankChain {
    uint32_t seen = 0, p2 = 0, p3 = 0, p4 = 0;
    __device__ __forceinline__ void add(uint32_t bit) {
        p4 |= p3 & bit;
        p3 |= p2 & bit;
        p2 |= seen & bit;
        seen |= bit;
    }
    __device__ __forceinline__ RankClasses classes() const {
        RankClasses rc;
        rc.quads = p4;
        rc.trips = p3 & ~p4;
        rc.pairs = p2 & ~p3;
        rc.singles = seen & ~p2;
        return rc;
    }
};

// Bit w of the result is set iff the 5-window w is complete in the 13-bit rank mask.
__device__ __forceinline__ uint32_t straight_windows(uint32_t ranks) {
    const uint32_t ext = (ranks << 1) | ((ranks >> 12) & 1u);  // bit 0 = ace below the deuce
    return ext & (ext >> 1) & (ext >> 2) & (ext >> 3) & (ext >> 4);
}

// The part of the score that depends on the ranks alone: the multiplicity category with its kickers
// and the straight.  `seen` is the union of the ranks.
__device__ __forceinline__ int32_t score_rank_part(const RankClasses& rc, uint32_t seen) {
    // ---- rank-multiplicity categories: pop ranks by (count desc, rank desc) ----
    uint64_t w = ((uint64_t)((rc.quads << 13) | rc.trips) << 26) | (uint64_t)((rc.pairs << 13) | rc.singles);
    uint32_t zeros = ~seen & 0x1fffu;
    uint32_t k[5], v[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 5; ++i) {
        if (w != 0) {
            const int pos = 63 - __clzll((long long)w);
            w ^= 1ull << pos;
            const int cls = (pos * 20) >> 8;  // pos / 13 for pos < 52
            k[i] = pos - 13 * cls;
            if (i < 2) v[i] = cls + 1;
        } else {  // fewer distinct ranks than fields: continue with absent ranks
            const int pos = 31 - __clz((int)zeros);
            zeros ^= 1u << pos;
            k[i] = pos;
        }
    }
    int type, nf;
    if (v[0] >= 4) { type = 8; nf = 2; }
    else if (v[0] >= 3 && v[1] >= 2) { type = 7; nf = 2; }
    else if (v[0] >= 3) { type = 4; nf = 3; }
    else if (v[0] >= 2 && v[1] >= 2) { type = 3; nf = 3; }
    else if (v[0] >= 2) { type = 2; nf = 4; }
    else { type = 1; nf = 5; }
    const uint32_t kick = (k[0] << 16) | (k[1] << 12) | (k[2] << 8) | (k[3] << 4) | k[4];
    const uint32_t keep = (0xFFFFFu << (4 * (5 - nf))) & 0xFFFFFu;
    int32_t best = (int32_t)(((uint32_t)type << 20) | (kick & keep));

    // ---- straight (lowest window) ----
    const uint32_t sw = straight_windows(seen);
    if (sw) best = max(best, (int32_t)((5u << 20) | ((uint32_t)(__ffs((int)sw) - 1) << 16)));
    return best;
}

__device__ __forceinline__ int32_t score_from_masks(uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3,
                                                    const RankClasses& rc) {
    int32_t best = score_rank_part(rc, m0 | m1 | m2 | m3);

    // ---- flush / straight flush ----
    const int c0 = __popc(m0), c1 = __popc(m1), c2 = __popc(m2), c3 = __popc(m3);
    if (max(max(c0, c1), max(c2, c3)) >= 5) {
        uint32_t fm = c0 >= 5 ? m0 : (c1 >= 5 ? m1 : (c2 >= 5 ? m2 : m3));
        uint32_t f = 0;
#pragma unroll
        for (int i = 0; i < 5; ++i) {
            const int pos = 31 - __clz((int)fm);
            fm ^= 1u << pos;
            f = (f << 4) | (uint32_t)pos;
        }
        best = max(best, (int32_t)((6u << 20) | f));
        const uint32_t sf = (c0 >= 5 ? straight_windows(m0) : 0u) | (c1 >= 5 ? straight_windows(m1) : 0u) |
                            (c2 >= 5 ? straight_windows(m2) : 0u) | (c3 >= 5 ? straight_windows(m3) : 0u);
        if (sf) best = max(best, (int32_t)((9u << 20) | ((uint32_t)(31 - __clz((int)sf)) << 16)));
    }
    return best;
}

// ---- table walk for hands of distinct cards --------------------------------------------
// One 32-bit entry per 13-bit rank mask:
//   bits 19:0   the (up to) five highest ranks of the mask as 4-bit fields, highest first,
//               left-aligned, zero-filled;
//   bits 27:24  1 + the LOWEST complete straight window of the mask (0 = no straight);
//   bits 31:28  1 + the HIGHEST complete straight window.
// With the four multiplicity masks of a hand, the kicker fields (ranks by count desc, rank
// desc) are the concatenation of the entries of quads, trips, pairs and singles, each
// shifted right by four bits per rank already placed; the hand type and the number of
// fields it keeps follow from the three counts (quads, trips, pairs) through a 24-entry
// table.  Straight and flush candidates come from the entries of the rank union and of the
// flush suit.
constexpr int kRankLutEntries = 8192;
constexpr int kTypeLutEntries = 24;
struct RankLut {
    uint32_t mask_entry[kRankLutEntries];
    uint32_t type_entry[kTypeLutEntries];  // index quads*12 + trips*4 + pairs: type << 24 | kept-field mask
    uint32_t pad[8];
};

inline uint32_t rank_lut_mask_entry(uint32_t mask) {  // host side, plain loops
    uint32_t fields = 0;
    int placed = 0;
    for (int r = 12; r >= 0 && placed < 5; --r)
        if (mask & (1u << r)) {
            fields |= (uint32_t)r << (16 - 4 * placed);
            ++placed;
        }
    const uint32_t ext = (mask << 1) | ((mask >> 12) & 1u);
    int lowest = -1, highest = -1;
    for (int w = 0; w <= 9; ++w)
        if (((ext >> w) & 0x1fu) == 0x1fu) {
            if (lowest < 0) lowest = w;
            highest = w;
        }
    return fields | ((uint32_t)(lowest + 1) << 24) | ((uint32_t)(highest + 1) << 28);
}

inline uint32_t rank_lut_type_entry(int quads, int trips, int pairs) {
    int type, nf;
    if (quads) { type = 8; nf = 2; }
    else if (trips && (trips >= 2 || pairs)) { type = 7; nf = 2; }
    else if (trips) { type = 4; nf = 3; }
    else if (pairs >= 2) { type = 3; nf = 3; }
    else if (pairs) { type = 2; nf = 4; }
    else { type = 1; nf = 5; }
    const uint32_t keep = (0xFFFFFu << (4 * (5 - nf))) & 0xFFFFFu;
    return ((uint32_t)type << 24) | keep;
}

// Score of a hand of DISTINCT cards given as four suit masks; T / TT are the two tables
// (shared or global memory).  Bit-identical to score_from_masks for such hands.
__device__ __forceinline__ int32_t score_distinct_lut(uint32_t m0, uint32_t m1, uint32_t m2, uint32_t m3,
                                                      const uint32_t* __restrict__ T, const uint32_t* __restrict__ TT) {
    const RankClasses rc = classes_from_suits(m0, m1, m2, m3);
    const uint32_t seen = m0 | m1 | m2 | m3;
    const uint32_t eq = T[rc.quads] & 0xFFFFFu, et = T[rc.trips] & 0xFFFFFu, ep = T[rc.pairs] & 0xFFFFFu;
    const uint32_t es = T[rc.singles] & 0xFFFFFu, en = T[seen];
    const int nq = __popc(rc.quads), nt = __popc(rc.trips), np = __popc(rc.pairs);
    const uint32_t kick = eq | (et >> (4 * nq)) | (ep >> (4 * (nq + nt))) | (es >> (4 * (nq + nt + np)));
    const uint32_t tt = TT[nq * 12 + nt * 4 + np];
    int32_t best = (int32_t)(((tt >> 24) << 20) | (kick & tt & 0xFFFFFu));
    const uint32_t sw = (en >> 24) & 15u;
    if (sw) best = max(best, (int32_t)((5u << 20) | ((sw - 1u) << 16)));
    const int c0 = __popc(m0), c1 = __popc(m1), c2 = __popc(m2), c3 = __popc(m3);
    if (max(max(c0, c1), max(c2, c3)) >= 5) {
        const uint32_t fm = c0 >= 5 ? m0 : (c1 >= 5 ? m1 : (c2 >= 5 ? m2 : m3));
        const uint32_t ef = T[fm];
        best = max(best, (int32_t)((6u << 20) | (ef & 0xFFFFFu)));
        const uint32_t sf = ef >> 28;
        if (sf) best = max(best, (int32_t)((9u << 20) | ((sf - 1u) << 16)));
    }
    return best;
}

// Position of card id c (0..51) in a 64-bit word made of four 16-bit suit lanes.
__device__ __forceinline__ int card_bit(int c) {
    const int s = (c * 79) >> 10;  // c / 13 for 0 <= c < 52
    return c + 3 * s;              // 16*s + (c - 13*s)
}

// Scores n (<= 7) card ids; repeated ids follow the "ids" convention described above.
template <int N>
__device__ __forceinline__ int32_t score_cards(const int (&cards)[N]) {
    uint64_t suits = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) suits |= 1ull << card_bit(cards[i]);
    const uint32_t lo = (uint32_t)suits, hi = (uint32_t)(suits >> 32);
    const uint32_t m0 = lo & 0x1fffu, m1 = (lo >> 16) & 0x1fffu, m2 = hi & 0x1fffu, m3 = (hi >> 16) & 0x1fffu;
    RankClasses rc;
    if (__popcll(suits) == N) {
        rc = classes_from_suits(m0, m1, m2, m3);
    } else {
        RankChain ch;
#pragma unroll
        for (int i = 0; i < N; ++i) ch.add(1u << (card_bit(cards[i]) & 15));
        rc = ch.classes();
    }
    return score_from_masks(m0, m1, m2, m3, rc);
}

}  // namespace p2b
