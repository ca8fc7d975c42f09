/*
 * CPU oracle for the 7-card hand ranker.  TEST INFRASTRUCTURE ONLY: nothing in the
 * product path links or calls this file; it exists to check the CUDA kernels and to
 * serve as the timed CPU baseline.
 *
 * It restates, step by step and without bit tricks, what the upstream evaluator
 * computes (p2/env/rules.py:136-299 `create_comparison_vector`, packed as in
 * rules.py:108-112 / rules_triton.py:158-174):
 *
 *   fields = [type, k1..k5], packed = type<<20 | k1<<16 | k2<<12 | k3<<8 | k4<<4 | k5
 *   type: 9 straight flush, 8 quads, 7 full house, 6 flush, 5 straight, 4 trips,
 *         3 two pair, 2 pair, 1 high card                       (rules.py:17-28)
 *   kickers come from the top-5 ranks ordered by (count desc, rank desc), ranks with
 *   count 0 included                                             (rules.py:157-162)
 *   straight field  = LOWEST complete 5-window (window 0 = wheel) (rules.py:241-254)
 *   straight flush  = HIGHEST complete 5-window in one suit      (rules.py:164-186)
 *   flush           = top-5 ranks of the first suit holding >=5   (rules.py:213-237)
 *
 * Two counting conventions exist upstream for inputs that repeat a card id:
 *   mode 0 ("planes"): cards are OR-ed into 4x13 one-hot planes first, so a repeated
 *          id counts once (rules.py:87-102, used by `rank_hands`);
 *   mode 1 ("ids"):    rank multiplicity counts every occurrence, saturating at 4,
 *          while suit masks are still OR-ed (rules_triton.py:415-446).
 * For 7 distinct cards both modes give the same value.
 */
#include <stdint.h>
#include <stddef.h>

static int32_t pack6(const int f[6]) {
    return (int32_t)((f[0] << 20) | (f[1] << 16) | (f[2] << 12) | (f[3] << 8) | (f[4] << 4) | f[5]);
}

int32_t p2o_rank_cards(const int16_t *cards, int ncards, int mode) {
    int plane[4][13] = {{0}};
    int mult[13] = {0};
    for (int i = 0; i < ncards; ++i) {
        int c = cards[i];
        int s = c / 13, r = c % 13;
        plane[s][r] = 1;
        if (mult[r] < 4) mult[r]++;
    }
    int count[13];
    for (int r = 0; r < 13; ++r) {
        if (mode == 0) count[r] = plane[0][r] + plane[1][r] + plane[2][r] + plane[3][r];
        else count[r] = mult[r];
    }
    /* top-5 of key = count<<8 | rank, descending (rules.py:158-162) */
    int idx[5], val[5], used[13] = {0};
    for (int k = 0; k < 5; ++k) {
        int best = -1, bestkey = -1;
        for (int r = 0; r < 13; ++r) {
            if (used[r]) continue;
            int key = (count[r] << 8) | r;
            if (key > bestkey) { bestkey = key; best = r; }
        }
        used[best] = 1;
        idx[k] = best;
        val[k] = count[best];
    }
    int table[10][6] = {{0}};
    /* straight flush: windows over [A,2,3,...,A] per suit, keep the highest */
    int has_sf = 0, sf_last = 0;
    for (int w = 0; w < 10; ++w) {
        for (int s = 0; s < 4; ++s) {
            int n = 0;
            for (int j = 0; j < 5; ++j) {
                int e = w + j;               /* index in the 14-long extended row */
                int r = (e == 0) ? 12 : e - 1;
                n += plane[s][r];
            }
            if (n == 5) { has_sf = 1; sf_last = w; }
        }
    }
    if (has_sf) { table[9][0] = 9; table[9][1] = sf_last; }
    if (val[0] >= 4) { table[8][0] = 8; table[8][1] = idx[0]; table[8][2] = idx[1]; }
    if (val[0] >= 3 && val[1] >= 2) { table[7][0] = 7; table[7][1] = idx[0]; table[7][2] = idx[1]; }
    /* flush: first suit with the maximum count, if that count >= 5 */
    int suit_sum[4], fs = 0;
    for (int s = 0; s < 4; ++s) {
        suit_sum[s] = 0;
        for (int r = 0; r < 13; ++r) suit_sum[s] += plane[s][r];
    }
    for (int s = 1; s < 4; ++s) if (suit_sum[s] > suit_sum[fs]) fs = s;
    if (suit_sum[fs] >= 5) {
        table[6][0] = 6;
        int k = 1;
        for (int r = 12; r >= 0 && k <= 5; --r) if (plane[fs][r]) table[6][k++] = r;
    }
    /* straight: lowest complete window on rank presence */
    for (int w = 0; w < 10; ++w) {
        int n = 0;
        for (int j = 0; j < 5; ++j) {
            int e = w + j;
            int r = (e == 0) ? 12 : e - 1;
            n += (plane[0][r] | plane[1][r] | plane[2][r] | plane[3][r]);
        }
        if (n == 5) { table[5][0] = 5; table[5][1] = w; break; }
    }
    if (val[0] >= 3) { table[4][0] = 4; table[4][1] = idx[0]; table[4][2] = idx[1]; table[4][3] = idx[2]; }
    if (val[0] >= 2 && val[1] >= 2) { table[3][0] = 3; table[3][1] = idx[0]; table[3][2] = idx[1]; table[3][3] = idx[2]; }
    if (val[0] >= 2) { table[2][0] = 2; for (int k = 0; k < 4; ++k) table[2][1 + k] = idx[k]; }
    table[1][0] = 1;
    for (int k = 0; k < 5; ++k) table[1][1 + k] = idx[k];
    for (int t = 9; t >= 1; --t) if (table[t][0]) return pack6(table[t]);
    return 0;
}

/* hands: [n,7] int16, out: [n] int32 */
void p2o_rank7_batch(const int16_t *hands, int64_t n, int mode, int32_t *out) {
    for (int64_t i = 0; i < n; ++i) out[i] = p2o_rank_cards(hands + 7 * i, 7, mode);
}

/* boards: [m,5] int16 -> scores [m,1326] in the lexicographic (c1<c2) combo order
 * (p2/env/card_utils.py:58-68); combos that overlap the board are still scored. */
void p2o_rank_boards(const int16_t *boards, int64_t m, int mode, int32_t *out) {
    for (int64_t b = 0; b < m; ++b) {
        int h = 0;
        for (int c1 = 0; c1 < 52; ++c1) {
            for (int c2 = c1 + 1; c2 < 52; ++c2, ++h) {
                int16_t cards[7];
                cards[0] = (int16_t)c1;
                cards[1] = (int16_t)c2;
                for (int j = 0; j < 5; ++j) cards[2 + j] = boards[5 * b + j];
                out[b * 1326 + h] = p2o_rank_cards(cards, 7, mode);
            }
        }
    }
}

/* two hands per row: cards [n,2,7] -> {1,-1,0} (rules.py:390-409) */
void p2o_compare7_batch(const int16_t *cards, int64_t n, int mode, int32_t *out) {
    for (int64_t i = 0; i < n; ++i) {
        int32_t a = p2o_rank_cards(cards + 14 * i, 7, mode);
        int32_t b = p2o_rank_cards(cards + 14 * i + 7, 7, mode);
        out[i] = (a > b) - (a < b);
    }
}

/* planes: [n,4,13] bytes, non-zero = card present -> packed score of the card SET
 * (any number of cards; rules.py:136-299 works on such planes directly). */
void p2o_rank_planes(const int8_t *planes, int64_t n, int32_t *out) {
    for (int64_t i = 0; i < n; ++i) {
        int16_t cards[52];
        int k = 0;
        for (int c = 0; c < 52; ++c) if (planes[i * 52 + c]) cards[k++] = (int16_t)c;
        out[i] = p2o_rank_cards(cards, k, 0);
    }
}
