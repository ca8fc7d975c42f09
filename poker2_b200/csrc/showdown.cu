// Board set-up (rank all 1326 combos, stable sort, tie groups, per-card lists) and the
// stand-alone showdown evaluation kernel.
#include "common.cuh"
#include "showdown.cuh"

namespace p2b {

constexpr int kSetupThreads = 1024;
constexpr int kSortN = 2048;

// One block per board.  boards: [m,5] int16.  Any of tabs / scores / order may be null.
//   tabs   : [m, kTabBytes] table blobs used by the showdown evaluation
//   scores : [m,1326] int32 packed strength of every combo (combos that overlap the board
//            are scored with repeated card ids, as p2/env/rules_triton.py:139-146 does)
//   order  : [m,1326] int64 stable ascending argsort of scores
__global__ void __launch_bounds__(kSetupThreads) board_setup_kernel(const int16_t* __restrict__ boards, int64_t m,
                                                                    const ComboTable* __restrict__ combos,
                                                                    unsigned char* __restrict__ tabs,
                                                                    int32_t* __restrict__ scores,
                                                                    long long* __restrict__ order) {
    __shared__ unsigned long long keys[kSortN];
    __shared__ uint16_t pos[P2B_NUM_HANDS];   // sorted position of combo h
    __shared__ uint16_t lgrp[kSortN];         // tie-group start per sorted position
    __shared__ uint16_t rgrp[kSortN];         // tie-group end (exclusive) per sorted position
    __shared__ uint16_t tmp16[kSortN];
    __shared__ int bcard[5];
    const int tid = threadIdx.x;
    const int64_t b = blockIdx.x;
    if (tid < 5) bcard[tid] = boards[b * 5 + tid];
    __syncthreads();

    // 1. strength of every combo
    for (int h = tid; h < kSortN; h += kSetupThreads) {
        if (h < P2B_NUM_HANDS) {
            int c[7] = {combos->c1[h], combos->c2[h], bcard[0], bcard[1], bcard[2], bcard[3], bcard[4]};
            const int32_t s = score_cards<7>(c);
            if (scores) scores[b * P2B_NUM_HANDS + h] = s;
            keys[h] = ((unsigned long long)(uint32_t)s << 11) | (unsigned long long)h;
        } else {
            keys[h] = ~0ull;
        }
    }
    __syncthreads();

    // 2. bitonic sort, ascending; the combo index in the low bits makes it stable
    for (int k = 2; k <= kSortN; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            const int i = ((tid & ~(j - 1)) << 1) | (tid & (j - 1));  // lower index of the pair
            const int p = i | j;
            const unsigned long long a = keys[i], c = keys[p];
            const bool up = (i & k) == 0;
            if ((a > c) == up) {
                keys[i] = c;
                keys[p] = a;
            }
            __syncthreads();
        }
    }

    // 3. positions and tie groups
    for (int k = tid; k < kSortN; k += kSetupThreads) {
        if (k < P2B_NUM_HANDS) {
            const int h = (int)(keys[k] & 2047ull);
            pos[h] = (uint16_t)k;
            if (order) order[b * P2B_NUM_HANDS + k] = h;
            const bool start = (k == 0) || ((keys[k] >> 11) != (keys[k - 1] >> 11));
            const bool last = (k == P2B_NUM_HANDS - 1) || ((keys[k] >> 11) != (keys[k + 1] >> 11));
            lgrp[k] = start ? (uint16_t)k : 0;            // max-scan from the left
            rgrp[k] = last ? (uint16_t)(k + 1) : 0xFFFF;  // min-scan from the right
        } else {
            lgrp[k] = 0;
            rgrp[k] = 0xFFFF;
        }
    }
    __syncthreads();
    for (int d = 1; d < kSortN; d <<= 1) {
        for (int k = tid; k < kSortN; k += kSetupThreads) tmp16[k] = (k >= d) ? max(lgrp[k], lgrp[k - d]) : lgrp[k];
        __syncthreads();
        for (int k = tid; k < kSortN; k += kSetupThreads) lgrp[k] = tmp16[k];
        __syncthreads();
        for (int k = tid; k < kSortN; k += kSetupThreads) tmp16[k] = (k + d < kSortN) ? min(rgrp[k], rgrp[k + d]) : rgrp[k];
        __syncthreads();
        for (int k = tid; k < kSortN; k += kSetupThreads) rgrp[k] = tmp16[k];
        __syncthreads();
    }
    if (!tabs) return;

    unsigned char* blob = tabs + b * (int64_t)kTabBytes;
    HandRec* rec = reinterpret_cast<HandRec*>(blob + kTabHeaderBytes);
    uint16_t* sorted = reinterpret_cast<uint16_t*>(blob + kTabHeaderBytes + kTabRecBytes);
    uint16_t* cardlist = reinterpret_cast<uint16_t*>(blob + kTabHeaderBytes + kTabRecBytes + kTabSortedBytes);
    if (tid == 0) {
        unsigned long long mask = 0;
        for (int i = 0; i < 5; ++i) mask |= 1ull << bcard[i];
        reinterpret_cast<unsigned long long*>(blob)[0] = mask;
        reinterpret_cast<unsigned long long*>(blob)[1] = 0ull;
    }
    for (int k = tid; k < kTabSortedPad; k += kSetupThreads) sorted[k] = k < P2B_NUM_HANDS ? (uint16_t)(keys[k] & 2047ull) : 0;

    // 4. per-card lists in strength order, 5. per-hand counts before L and before R.
    // Task (c, i): the i-th other card d of card c names the hand g = {c,d}.
    for (int task = tid; task < P2B_NUM_CARDS * 51; task += kSetupThreads) {
        const int c = task / 51, i = task % 51;
        const int d = i < c ? i : i + 1;
        const int g = c < d ? combo_index(c, d) : combo_index(d, c);
        const int pg = pos[g];
        const int L = lgrp[pg], R = rgrp[pg];
        int before = 0, nb = 0, ne = 0;
        for (int j = 0; j < 51; ++j) {
            const int e = j < c ? j : j + 1;
            const int q = pos[c < e ? combo_index(c, e) : combo_index(e, c)];
            before += q < pg;
            nb += q < L;
            ne += q < R;
        }
        cardlist[before * 52 + c] = (uint16_t)g;
        HandRec* r = rec + g;
        if (c < d) {  // c is the hand's lower card
            r->lpos = (uint16_t)L;
            r->rpos = (uint16_t)R;
            r->nb0 = (uint8_t)nb;
            r->ne0 = (uint8_t)ne;
        } else {
            r->nb1 = (uint8_t)nb;
            r->ne1 = (uint8_t)ne;
        }
    }
    if (tid < (kTabCardListBytes - 51 * 52 * 2) / 2) cardlist[51 * 52 + tid] = 0;
}

constexpr int kEvalThreads = 384;
constexpr int kEvalSmem = kTabBytes + 2 * P2B_HPAD * 4 /*x*/ + 2 * P2B_HPAD * 4 /*P*/ + 2 * 52 * 52 * 4 /*PC*/ + 32 * 8;

// One block per showdown row.  beliefs: [rows,2,1326] fp32 (row stride given in floats so
// that padded layouts work); values: same shape.  tab_of_row: which table blob a row uses
// (null = row index).  potential: [rows,2] int64 chips won by each player at showdown,
// scale: [rows] fp32; value = EV * potential / scale (cfr_evaluator.py:597-601).
__global__ void __launch_bounds__(kEvalThreads) showdown_eval_kernel(
    const unsigned char* __restrict__ tabs, const int32_t* __restrict__ tab_of_row, const ComboTable* __restrict__ combos,
    const float* __restrict__ beliefs, int64_t belief_row_stride, const long long* __restrict__ potential,
    const float* __restrict__ scale, float* __restrict__ values, int64_t value_row_stride, int64_t rows) {
    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* tab_s = smem;
    float* x = reinterpret_cast<float*>(smem + kTabBytes);  // [2][HPAD]: x[p] = range of player p
    float* P = x + 2 * P2B_HPAD;                            // [2][HPAD]: prefix of the range of player p
    float* PC = P + 2 * P2B_HPAD;                           // [2][52*52]
    double* warp_tot = reinterpret_cast<double*>(PC + 2 * 52 * 52);
    const int tid = threadIdx.x;

    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const int64_t t = tab_of_row ? tab_of_row[row] : row;
        const uint4* src = reinterpret_cast<const uint4*>(tabs + t * (int64_t)kTabBytes);
        for (int i = tid; i < kTabBytes / 16; i += kEvalThreads) reinterpret_cast<uint4*>(tab_s)[i] = src[i];
        const float* brow = beliefs + row * belief_row_stride;
        for (int i = tid; i < 2 * P2B_NUM_HANDS; i += kEvalThreads) {
            const int p = i >= P2B_NUM_HANDS;
            x[p * P2B_HPAD + (i - p * P2B_NUM_HANDS)] = __ldcs(brow + i);
        }
        __syncthreads();
        const BoardTabView tv = view_tables(tab_s);

        // per-card prefix sums: thread (p,c) walks card c's list in strength order
        if (tid < 2 * 52) {
            const int p = tid / 52, c = tid % 52;
            const float* xp = x + p * P2B_HPAD;
            float* pc = PC + p * 52 * 52 + c * 52;
            double acc = 0.0;
            pc[0] = 0.0f;
#pragma unroll 3
            for (int k = 0; k < 51; ++k) {
                acc += (double)xp[tv.cardlist[k * 52 + c]];
                pc[k + 1] = (float)acc;
            }
        }
        // strength-order prefix sums of both ranges
        for (int p = 0; p < 2; ++p) {
            const float* xp = x + p * P2B_HPAD;
            block_prefix_f64([&](int k) { return xp[tv.sorted[k]]; }, P2B_NUM_HANDS, P + p * P2B_HPAD, warp_tot);
        }
        const unsigned long long bmask = *tv.board_mask;
        float* vrow = values + row * value_row_stride;
        for (int i = tid; i < 2 * P2B_NUM_HANDS; i += kEvalThreads) {
            const int hero = i >= P2B_NUM_HANDS, h = i - hero * P2B_NUM_HANDS, opp = 1 - hero;
            const int c1 = combos->c1[h], c2 = combos->c2[h];
            const bool allowed = (((bmask >> c1) | (bmask >> c2)) & 1ull) == 0;
            const float ev = showdown_hand_ev(tv.rec[h], c1, c2, x[opp * P2B_HPAD + h], allowed, P + opp * P2B_HPAD,
                                              PC + opp * 52 * 52);
            const float pot = (float)potential[row * 2 + hero];
            __stcs(vrow + i, __fdiv_rn(__fmul_rn(ev, pot), scale[row]));
        }
        __syncthreads();
    }
}

int sm_count();

int launch_board_setup(const int16_t* boards, int64_t m, unsigned char* tabs, int32_t* scores, long long* order,
                       cudaStream_t stream) {
    if (m == 0) return P2B_OK;
    int rc = ensure_tables();
    if (rc) return rc;
    board_setup_kernel<<<(unsigned)m, kSetupThreads, 0, stream>>>(boards, m, device_combo_table(), tabs, scores, order);
    return check_cuda(cudaGetLastError(), "board_setup_kernel");
}

int launch_showdown_eval(const unsigned char* tabs, const int32_t* tab_of_row, const float* beliefs,
                         int64_t belief_row_stride, const long long* potential, const float* scale, float* values,
                         int64_t value_row_stride, int64_t rows, cudaStream_t stream) {
    if (rows == 0) return P2B_OK;
    int rc = ensure_tables();
    if (rc) return rc;
    rc = check_cuda(cudaFuncSetAttribute(showdown_eval_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kEvalSmem),
                    "showdown_eval_kernel smem attribute");
    if (rc) return rc;
    int64_t grid = rows;
    const int64_t cap = (int64_t)sm_count() * 3;
    if (grid > cap) grid = cap;
    showdown_eval_kernel<<<(unsigned)grid, kEvalThreads, kEvalSmem, stream>>>(
        tabs, tab_of_row, device_combo_table(), beliefs, belief_row_stride, potential, scale, values, value_row_stride,
        rows);
    return check_cuda(cudaGetLastError(), "showdown_eval_kernel");
}

}  // namespace p2b
