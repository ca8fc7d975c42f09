// Board set-up (rank all 1326 combos, stable sort, tie groups, per-card lists) and the
// stand-alone showdown evaluation kernel.
#include "common.cuh"
#include "showdown.cuh"

namespace p2b {

// ---------------------------------------------------------------------------------------
// Board set-up.  One block per board, 352 threads, four keys per thread.
//   1. strength of every combo (board cards + two hole cards; combos that overlap the board
//      are scored with repeated card ids, as p2/env/rules_triton.py:139-146 does).  On a fixed
//      board the rank part of the score (multiplicity category, kickers, straight) depends on
//      the two hole RANKS only: it is computed once per rank pair (169 threads) and looked up
//      per combo; only the board's suit with three or more cards, if any, can make a flush,
//      which costs a combo one table entry of the suit's rank mask;
//   2. stable LSD radix sort of the 24-bit strengths, four passes of six bits.  A warp ranks
//      32 consecutive keys with a match instruction; counts per (digit, chunk of 32) are
//      bytes, scanned in digit-major order to give every key its destination;
//   3. tie groups [L,R) from the sorted strengths (one block-wide max scan);
//   4. per card, a bit mask over the sorted positions of the hands that hold it, and the
//      running bit counts per 32-position word;
//   5. per hand: its index in the strength-ordered list of each of its two cards, and how
//      many entries of those lists lie before L and before R -- each a count of mask bits
//      below a position.
// The table blob is assembled in shared memory and written out with 16-byte stores.
// ---------------------------------------------------------------------------------------
constexpr int kSetupThreads = 352;
constexpr int kSetupWarps = kSetupThreads / 32;         // 11
constexpr int kSortChunks = 44;                         // chunks of 32 keys
constexpr int kSortN = kSortChunks * 32;                // 1408 >= 1326
constexpr int kSortRounds = kSortChunks / kSetupWarps;  // 4 chunks per warp
constexpr int kDigitBits = 6, kDigits = 1 << kDigitBits, kSortPasses = 4;
static_assert(kSortChunks % 4 == 0, "count bytes are scanned four at a time");
static_assert(kSortChunks == kSortRounds * kSetupWarps, "every warp sorts the same number of chunks");
constexpr int kSortCntWords = kDigits * kSortChunks / 4;  // 704 words of four byte counters
constexpr int kMaskWords = 42;                            // 32-position words of a card's mask (1326 positions, and 1326 itself)
constexpr int kMaskStride = 43;                           // odd: the cards of one word fall into distinct banks
static_assert(kMaskWords * 32 > P2B_NUM_HANDS && kMaskStride >= kMaskWords, "a mask covers positions 0..1326");

// shared-memory carve-up (bytes)
constexpr int kSuKey = 0;                                // uint32 [2][kSortN]
constexpr int kSuVal = kSuKey + 2 * kSortN * 4;          // uint16 [2][kSortN]
constexpr int kSuCnt = kSuVal + 2 * kSortN * 2;          // uint32: sort counters [kSortCntWords], then card masks [52][kMaskStride]
constexpr int kSuCntWords = 52 * kMaskStride;            // 2236 >= kSortCntWords
constexpr int kSuOff = kSuCnt + kSuCntWords * 4;         // rank-pair scores int32 [169], then sort offsets uint16 [64*44],
constexpr int kSuOffBytes = kDigits * kSortChunks * 2;   // then mask bit counts uint16 [52][kMaskStride]
static_assert(kSuOffBytes >= 52 * kMaskStride * 2 && kSuOffBytes >= 169 * 4 && kSuCntWords >= kSortCntWords, "shared areas");
constexpr int kSuLg = kSuOff + kSuOffBytes;              // uint16 [kSortN]   tie-group start per sorted position
constexpr int kSuRt = kSuLg + kSortN * 2;                // uint16 [kSortN]   tie-group end, indexed by group start
constexpr int kSuBlob = (kSuRt + kSortN * 2 + 15) / 16 * 16;  // the table blob
constexpr int kSuWarp = kSuBlob + kTabBytes;             // uint32 [16] warp totals of the block scan
constexpr int kSetupSmem = kSuWarp + 64;
static_assert(kSuCnt % 4 == 0 && kSuOff % 4 == 0 && kSuBlob % 16 == 0 && kSuWarp % 4 == 0, "alignment");

// Exclusive prefix over `words*4` byte counters (in memory order) -> uint16 offsets.  Every
// thread takes `words_per_thread` consecutive words.  Ends with a barrier.
template <int WPT>
__device__ __forceinline__ void scan_byte_counts(const uint32_t* __restrict__ cnt, int words, uint16_t* __restrict__ off,
                                                 uint32_t* warp_tot) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t w[WPT];
    uint32_t local = 0;
#pragma unroll
    for (int i = 0; i < WPT; ++i) {
        const int idx = tid * WPT + i;
        w[i] = idx < words ? cnt[idx] : 0u;
        local += (w[i] & 0xffu) + ((w[i] >> 8) & 0xffu) + ((w[i] >> 16) & 0xffu) + (w[i] >> 24);
    }
    uint32_t incl = local;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    uint32_t base = incl - local;
    for (int k = 0; k < warp; ++k) base += warp_tot[k];
#pragma unroll
    for (int i = 0; i < WPT; ++i) {
        const int idx = tid * WPT + i;
        if (idx < words) {
            uint32_t run = base;
            ushort4 o;
            o.x = (uint16_t)run; run += w[i] & 0xffu;
            o.y = (uint16_t)run; run += (w[i] >> 8) & 0xffu;
            o.z = (uint16_t)run; run += (w[i] >> 16) & 0xffu;
            o.w = (uint16_t)run; run += w[i] >> 24;
            *reinterpret_cast<ushort4*>(off + 4 * idx) = o;
            base = run;
        }
    }
    __syncthreads();
}

// boards: [m,5] int16.  Any of tabs / scores / order may be null.
//   tabs   : [m, kTabBytes] table blobs used by the showdown evaluation
//   scores : [m,1326] int32 packed strength of every combo
//   order  : [m,1326] int64 stable ascending argsort of scores
__global__ void __launch_bounds__(kSetupThreads, 3) board_setup_kernel(const int16_t* __restrict__ boards, int64_t m,
                                                                       const ComboTable* __restrict__ combos,
                                                                       const RankLut* __restrict__ lut,
                                                                       unsigned char* __restrict__ tabs,
                                                                       int32_t* __restrict__ scores,
                                                                       long long* __restrict__ order) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint32_t* key = reinterpret_cast<uint32_t*>(smem + kSuKey);
    uint16_t* val = reinterpret_cast<uint16_t*>(smem + kSuVal);
    uint32_t* cnt = reinterpret_cast<uint32_t*>(smem + kSuCnt);
    unsigned char* cnt8 = smem + kSuCnt;
    uint32_t* cmask = reinterpret_cast<uint32_t*>(smem + kSuCnt);   // [52][kMaskStride], after the sort
    uint16_t* off = reinterpret_cast<uint16_t*>(smem + kSuOff);
    int32_t* pair_score = reinterpret_cast<int32_t*>(smem + kSuOff);  // [13][13], before the sort
    uint16_t* cpre = reinterpret_cast<uint16_t*>(smem + kSuOff);      // [52][kMaskStride], after the sort
    uint16_t* lg = reinterpret_cast<uint16_t*>(smem + kSuLg);
    uint16_t* rt = reinterpret_cast<uint16_t*>(smem + kSuRt);
    unsigned char* blob = smem + kSuBlob;
    uint32_t* warp_tot = reinterpret_cast<uint32_t*>(smem + kSuWarp);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t lt_mask = (1u << lane) - 1u;
    const int64_t b = blockIdx.x;

    // ---- 1. strengths ----
    int bc[5];
#pragma unroll
    for (int i = 0; i < 5; ++i) bc[i] = boards[b * 5 + i];
    uint64_t bsuits = 0;
    RankChain bchain;
#pragma unroll
    for (int i = 0; i < 5; ++i) {
        const int bit = card_bit(bc[i]);
        bsuits |= 1ull << bit;
        bchain.add(1u << (bit & 15));
    }
    if (tid < 169) {  // rank part per pair of hole ranks (every occurrence of a rank counts, repeated card ids included)
        const int r1 = tid / 13, r2 = tid - 13 * r1;
        RankChain ch = bchain;
        ch.add(1u << r1);
        ch.add(1u << r2);
        pair_score[tid] = score_rank_part(ch.classes(), ch.seen);
    }
    // the one suit of the board that can make a flush (three or more cards), if any
    int fsuit = -1;
    uint32_t fboard = 0;
#pragma unroll
    for (int su = 0; su < 4; ++su) {
        const uint32_t ms = (uint32_t)(bsuits >> (16 * su)) & 0x1fffu;
        if (__popc(ms) >= 3) {
            fsuit = su;
            fboard = ms;
        }
    }
    for (int i = tid; i < kSortCntWords; i += kSetupThreads) cnt[i] = 0u;
    __syncthreads();
    for (int h = tid; h < kSortN; h += kSetupThreads) {
        uint32_t k = 0xffffffffu;
        if (h < P2B_NUM_HANDS) {
            const int b1 = card_bit(combos->c1[h]), b2 = card_bit(combos->c2[h]);
            int32_t s = pair_score[(b1 & 15) * 13 + (b2 & 15)];
            if (fsuit >= 0) {
                const uint32_t fm = fboard | ((b1 >> 4) == fsuit ? 1u << (b1 & 15) : 0u) |
                                    ((b2 >> 4) == fsuit ? 1u << (b2 & 15) : 0u);
                if (__popc(fm) >= 5) {  // flush: the five highest ranks of the suit; straight flush: its highest window
                    const uint32_t ef = lut->mask_entry[fm];
                    s = max(s, (int32_t)((6u << 20) | (ef & 0xFFFFFu)));
                    const uint32_t sf = ef >> 28;
                    if (sf) s = max(s, (int32_t)((9u << 20) | ((sf - 1u) << 16)));
                }
            }
            if (scores) scores[b * P2B_NUM_HANDS + h] = s;
            k = (uint32_t)s;
        }
        key[h] = k;
        val[h] = (uint16_t)h;
    }
    __syncthreads();

    // ---- 2. stable radix sort; buffers alternate, the result ends in buffer 0 ----
#pragma unroll 1
    for (int pass = 0; pass < kSortPasses; ++pass) {
        const uint32_t* ksrc = key + (pass & 1) * kSortN;
        const uint16_t* vsrc = val + (pass & 1) * kSortN;
        uint32_t* kdst = key + ((pass & 1) ^ 1) * kSortN;
        uint16_t* vdst = val + ((pass & 1) ^ 1) * kSortN;
        const int shift = kDigitBits * pass;
        uint32_t kk[kSortRounds];
        uint16_t vv[kSortRounds];
        int slot[kSortRounds], rnk[kSortRounds];
#pragma unroll
        for (int i = 0; i < kSortRounds; ++i) {
            const int chunk = warp + kSetupWarps * i, p = 32 * chunk + lane;
            kk[i] = ksrc[p];
            vv[i] = vsrc[p];
            const int d = (int)((kk[i] >> shift) & (kDigits - 1));
            const uint32_t peers = __match_any_sync(0xffffffffu, d);
            rnk[i] = __popc(peers & lt_mask);
            slot[i] = d * kSortChunks + chunk;
            if (rnk[i] == 0) cnt8[slot[i]] = (unsigned char)__popc(peers);
        }
        __syncthreads();
        scan_byte_counts<2>(cnt, kSortCntWords, off, warp_tot);
#pragma unroll
        for (int i = 0; i < kSortRounds; ++i) {
            const int dest = off[slot[i]] + rnk[i];
            kdst[dest] = kk[i];
            vdst[dest] = vv[i];
        }
        // the counters of the next pass, or (after the last one) the card masks that take their place
        for (int i = tid; i < (pass + 1 < kSortPasses ? kSortCntWords : kSuCntWords); i += kSetupThreads) cnt[i] = 0u;
        __syncthreads();
    }

    // ---- 3. tie groups: lg[k] = first position of the run of equal strengths holding k ----
    {
        const int k0 = 4 * tid;
        uint32_t kprev = k0 > 0 ? key[k0 - 1] : ~key[0];
        int run[4];
        int best = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t kc = key[k0 + i];
            if (kc != kprev) best = k0 + i;
            run[i] = best;
            kprev = kc;
        }
        int incl = best;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl = max(incl, up);
        }
        if (lane == 31) warp_tot[warp] = (uint32_t)incl;
        __syncthreads();
        int base = __shfl_up_sync(0xffffffffu, incl, 1);
        if (lane == 0) base = 0;
        for (int w = 0; w < warp; ++w) base = max(base, (int)warp_tot[w]);
#pragma unroll
        for (int i = 0; i < 4; ++i) lg[k0 + i] = (uint16_t)max(run[i], base);
        __syncthreads();
        // the end of a group is the start of the next one; position 1326 (first pad) closes the last
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + i;
            if (k > 0 && k <= P2B_NUM_HANDS && lg[k] == k) rt[lg[k - 1]] = (uint16_t)k;
        }
    }

    // ---- 4. per card: which sorted positions hold a hand with that card ----
    BoardTabView tv = view_tables(blob);
    uint16_t* sorted_s = const_cast<uint16_t*>(tv.sorted);
    uint16_t* cardlist_s = const_cast<uint16_t*>(tv.cardlist);
    HandRec* rec_s = const_cast<HandRec*>(tv.rec);
    int hh[kSortRounds], c1s[kSortRounds], c2s[kSortRounds];
#pragma unroll
    for (int i = 0; i < kSortRounds; ++i) {
        const int k = tid + kSetupThreads * i;
        hh[i] = k < P2B_NUM_HANDS ? val[k] : 0;
        c1s[i] = combos->c1[hh[i]];
        c2s[i] = combos->c2[hh[i]];
        if (k < P2B_NUM_HANDS) {
            atomicOr(cmask + c1s[i] * kMaskStride + (k >> 5), 1u << (k & 31));
            atomicOr(cmask + c2s[i] * kMaskStride + (k >> 5), 1u << (k & 31));
        }
    }
    if (tid < (kTabCardListBytes - 51 * 52 * 2) / 2) cardlist_s[51 * 52 + tid] = 0;
    for (int k = tid; k < kTabSortedPad; k += kSetupThreads) {
        const uint16_t h = k < P2B_NUM_HANDS ? val[k] : (uint16_t)0;
        sorted_s[k] = h;
        if (order && k < P2B_NUM_HANDS) order[b * P2B_NUM_HANDS + k] = h;
    }
    if (tid == 0) {
        unsigned long long mask = 0;
        for (int i = 0; i < 5; ++i) mask |= 1ull << bc[i];
        reinterpret_cast<unsigned long long*>(blob)[0] = mask;
        reinterpret_cast<unsigned long long*>(blob)[1] = 0ull;
    }
    __syncthreads();
    // bits of a card's mask before each of its words: a warp per card, a lane per word (and word + 32)
    for (int card = warp; card < 52; card += kSetupWarps) {
        const uint32_t* mrow = cmask + card * kMaskStride;
        const int v0 = __popc(mrow[lane]), v1 = lane + 32 < kMaskWords ? __popc(mrow[lane + 32]) : 0;
        int i0 = v0, i1 = v1;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u0 = __shfl_up_sync(0xffffffffu, i0, d), u1 = __shfl_up_sync(0xffffffffu, i1, d);
            if (lane >= d) {
                i0 += u0;
                i1 += u1;
            }
        }
        const int first32 = __shfl_sync(0xffffffffu, i0, 31);
        cpre[card * kMaskStride + lane] = (uint16_t)(i0 - v0);
        if (lane + 32 < kMaskWords) cpre[card * kMaskStride + lane + 32] = (uint16_t)(first32 + i1 - v1);
    }
    __syncthreads();

    // ---- 5. per hand: place it in its two cards' lists; list entries before its tie group and before the group's end ----
    auto below = [&](int card, int pos) {  // entries of the card's list at sorted positions < pos (pos <= 1326)
        const int w = pos >> 5;
        return (int)cpre[card * kMaskStride + w] + __popc(cmask[card * kMaskStride + w] & ((1u << (pos & 31)) - 1u));
    };
#pragma unroll
    for (int i = 0; i < kSortRounds; ++i) {
        const int k = tid + kSetupThreads * i;
        if (k >= P2B_NUM_HANDS) continue;
        const int h = hh[i], c1 = c1s[i], c2 = c2s[i];
        const int L = lg[k], R = rt[L];
        cardlist_s[below(c1, k) * 52 + c1] = (uint16_t)h;
        cardlist_s[below(c2, k) * 52 + c2] = (uint16_t)h;
        HandRec r;
        r.lpos = (uint16_t)L;
        r.rpos = (uint16_t)R;
        r.nb0 = (uint8_t)below(c1, L);
        r.ne0 = (uint8_t)below(c1, R);
        r.nb1 = (uint8_t)below(c2, L);
        r.ne1 = (uint8_t)below(c2, R);
        rec_s[h] = r;
    }
    __syncthreads();
    if (tabs) {
        uint4* dst = reinterpret_cast<uint4*>(tabs + b * (int64_t)kTabBytes);
        const uint4* src = reinterpret_cast<const uint4*>(blob);
        for (int i = tid; i < kTabBytes / 16; i += kSetupThreads) dst[i] = src[i];
    }
}

// ---------------------------------------------------------------------------------------
// Stand-alone showdown evaluation.  One block (448 threads) per showdown row at a time.
// beliefs: [rows,2,1326] fp32 (row stride given in floats so that padded layouts work);
// values: same shape.  tab_of_row: which table blob a row uses (null = row index).
// potential: [rows,2] int64 chips won by each player at showdown, scale: [rows] fp32;
// value = EV * potential / scale (cfr_evaluator.py:597-601).
//
// Per row: (A) the 2 x 52 per-card prefix lists, four threads per list, and the totals of
// the four quarters of both strength-order scans; (B) the eight quarter scans, one warp
// each; (C) the per-hand formula.  All sums are fp64, rounded to fp32 per element.
// ---------------------------------------------------------------------------------------
constexpr int kEvalThreads = 448;
constexpr int kEvalWarps = kEvalThreads / 32;
constexpr int kQuarter = 352;  // sorted positions per quarter scan: 32 lanes x 11
constexpr int kEvX = kTabBytes;                         // float [2*1326 (+pad)]
constexpr int kEvStage = kTabBytes + 2 * P2B_HPAD * 4;  // one staging buffer: table blob + both ranges
constexpr int kEvP = 2 * kEvStage;                      // float [2][HPAD]   (two staging buffers come first)
constexpr int kEvPC = kEvP + 2 * P2B_HPAD * 4;          // float [2][52*52]
constexpr int kEvQ = kEvPC + 2 * 52 * 52 * 4;           // double [8]
constexpr int kEvCombo = kEvQ + 64;                     // uint8 [2][1326 (+pad)]
constexpr int kEvTot = kEvCombo + 2 * 1328;             // float [2][64] mass of all hands holding a card
constexpr int kEvalSmem = kEvTot + 2 * 64 * 4;
static_assert(kEvQ % 8 == 0, "alignment");

__global__ void __launch_bounds__(kEvalThreads, 2) showdown_eval_kernel(
    const unsigned char* __restrict__ tabs, const int32_t* __restrict__ tab_of_row, const ComboTable* __restrict__ combos,
    const float* __restrict__ beliefs, int64_t belief_row_stride, const long long* __restrict__ potential,
    const float* __restrict__ scale, float* __restrict__ values, int64_t value_row_stride, int64_t rows) {
    extern __shared__ __align__(16) unsigned char smem[];
    float* P = reinterpret_cast<float*>(smem + kEvP);   // P[p*HPAD + k] = prefix of player p's range, strength order
    float* PC = reinterpret_cast<float*>(smem + kEvPC);
    double* qtot = reinterpret_cast<double*>(smem + kEvQ);
    uint8_t* c1s = smem + kEvCombo;
    uint8_t* c2s = c1s + 1328;
    float* PCT = reinterpret_cast<float*>(smem + kEvTot);  // consecutive cards in consecutive banks
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int h = tid; h < P2B_NUM_HANDS; h += kEvalThreads) {
        c1s[h] = combos->c1[h];
        c2s[h] = combos->c2[h];
    }
    const bool vec_in = ((reinterpret_cast<uintptr_t>(beliefs) | (uintptr_t)(belief_row_stride * 4)) & 15) == 0;

    // The table blob and the two ranges of a row are copied into one of two staging buffers
    // asynchronously, one row ahead of the row being evaluated.
    auto stage_row = [&](int64_t row, int buf) {
        if (row < rows) {
            unsigned char* dst = smem + buf * kEvStage;
            const int64_t t = tab_of_row ? tab_of_row[row] : row;
            const unsigned char* src = tabs + t * (int64_t)kTabBytes;
            for (int i = tid; i < kTabBytes / 16; i += kEvalThreads) {
                const unsigned d = (unsigned)__cvta_generic_to_shared(dst + 16 * i);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + 16 * i) : "memory");
            }
            const float* brow = beliefs + row * belief_row_stride;
            float* xd = reinterpret_cast<float*>(dst + kEvX);
            if (vec_in) {
                for (int i = tid; i < 2 * P2B_NUM_HANDS / 4; i += kEvalThreads) {
                    const unsigned d = (unsigned)__cvta_generic_to_shared(xd + 4 * i);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(brow + 4 * i) : "memory");
                }
            } else {
                for (int i = tid; i < 2 * P2B_NUM_HANDS; i += kEvalThreads) {
                    const unsigned d = (unsigned)__cvta_generic_to_shared(xd + i);
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(brow + i) : "memory");
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int buf = 0;
    stage_row(blockIdx.x, 0);
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, buf ^= 1) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // every thread's share of this row has landed; the other buffer is free
        stage_row(row + gridDim.x, buf ^ 1);
        unsigned char* tab_s = smem + buf * kEvStage;
        float* x = reinterpret_cast<float*>(tab_s + kEvX);  // x[p*1326 + h] = range of player p
        const BoardTabView tv = view_tables(tab_s);

        // ---- A. per-card prefix lists (threads 0..415: player, card, quarter of the list) ----
        {
            const bool valid = tid < 2 * 52 * 4;
            const int p = tid / 208, rem = tid % 208, c = rem >> 2, q = rem & 3;
            const float* xp = x + (valid ? p : 0) * P2B_NUM_HANDS;
            float v[13];
#pragma unroll
            for (int i = 0; i < 13; ++i) {
                const int e = 13 * q + i;
                v[i] = (valid && e < 51) ? xp[tv.cardlist[e * 52 + c]] : 0.0f;
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
            const double t2 = __shfl_sync(0xffffffffu, tot, g + 2);
            if (valid) {
                double acc = q == 0 ? 0.0 : (q == 1 ? t0 : (q == 2 ? t0 + t1 : (t0 + t1) + t2));
                float* out = PC + p * 52 * 52 + c * 52;
                if (q == 0) out[0] = 0.0f;
#pragma unroll
                for (int i = 0; i < 13; ++i)
                    if (13 * q + i < 51) {
                        acc += (double)v[i];
                        out[13 * q + i + 1] = (float)acc;
                    }
                if (q == 3) PCT[p * 64 + c] = (float)acc;  // == out[51]
            }
        }
        // quarter totals of the strength-order scans: task = player*4 + quarter, last warps first
        for (int wt = kEvalWarps - 1 - warp; wt < 8; wt += kEvalWarps) {
            const int p = wt >> 2, k0 = (wt & 3) * kQuarter + 11 * lane;
            const float* xp = x + p * P2B_NUM_HANDS;
            float v[11];
#pragma unroll
            for (int i = 0; i < 11; ++i) v[i] = (k0 + i < P2B_NUM_HANDS) ? xp[tv.sorted[k0 + i]] : 0.0f;
            double a = 0.0;
#pragma unroll
            for (int i = 0; i < 11; ++i) a += (double)v[i];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) a += __shfl_xor_sync(0xffffffffu, a, d);
            if (lane == 0) qtot[wt] = a;
        }
        __syncthreads();

        // ---- B. the eight quarter scans ----
        for (int wt = warp; wt < 8; wt += kEvalWarps) {
            const int p = wt >> 2, qi = wt & 3, k0 = qi * kQuarter + 11 * lane;
            const float* xp = x + p * P2B_NUM_HANDS;
            float* pref = P + p * P2B_HPAD;
            double start = 0.0;
            for (int r = 0; r < qi; ++r) start += qtot[p * 4 + r];
            float v[11];
#pragma unroll
            for (int i = 0; i < 11; ++i) v[i] = (k0 + i < P2B_NUM_HANDS) ? xp[tv.sorted[k0 + i]] : 0.0f;
            double local = 0.0;
#pragma unroll
            for (int i = 0; i < 11; ++i) local += (double)v[i];
            double incl = local;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const double up = __shfl_up_sync(0xffffffffu, incl, d);
                if (lane >= d) incl += up;
            }
            double run = start + (incl - local);
            if (wt == p * 4 && lane == 0) pref[0] = 0.0f;
#pragma unroll
            for (int i = 0; i < 11; ++i) {
                run += (double)v[i];
                if (k0 + i < P2B_NUM_HANDS) pref[k0 + i + 1] = (float)run;
            }
        }
        __syncthreads();

        // ---- C. per-hand formula ----
        const unsigned long long bmask = *tv.board_mask;
        float* vrow = values + row * value_row_stride;
        const float pot0 = (float)potential[row * 2], pot1 = (float)potential[row * 2 + 1];
        const Divisor dscale = make_divisor(scale[row]);
        // a thread takes a hand for both players: cards, board check and the hand's record are shared
        for (int h = tid; h < P2B_NUM_HANDS; h += kEvalThreads) {
            const int c1 = c1s[h], c2 = c2s[h];
            const bool allowed = (((bmask >> c1) | (bmask >> c2)) & 1ull) == 0;
            const HandRec r = tv.rec[h];
            const float ev0 = showdown_hand_ev(r, c1, c2, x[P2B_NUM_HANDS + h], allowed, P + P2B_HPAD, PC + 52 * 52,
                                               PCT[64 + c1], PCT[64 + c2]);
            const float ev1 = showdown_hand_ev(r, c1, c2, x[h], allowed, P, PC, PCT[c1], PCT[c2]);
            __stcs(vrow + h, div_exact(__fmul_rn(ev0, pot0), dscale));
            __stcs(vrow + P2B_NUM_HANDS + h, div_exact(__fmul_rn(ev1, pot1), dscale));
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

int sm_count();

int launch_board_setup(const int16_t* boards, int64_t m, unsigned char* tabs, int32_t* scores, long long* order,
                       cudaStream_t stream) {
    if (m == 0) return P2B_OK;
    int rc = ensure_tables();
    if (rc) return rc;
    rc = check_cuda(cudaFuncSetAttribute(board_setup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSetupSmem),
                    "board_setup_kernel smem attribute");
    if (rc) return rc;
    board_setup_kernel<<<(unsigned)m, kSetupThreads, kSetupSmem, stream>>>(boards, m, device_combo_table(),
                                                                         device_rank_lut(), tabs, scores, order);
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
    const int64_t cap = (int64_t)sm_count() * 2;
    if (grid > cap) grid = cap;
    showdown_eval_kernel<<<(unsigned)grid, kEvalThreads, kEvalSmem, stream>>>(
        tabs, tab_of_row, device_combo_table(), beliefs, belief_row_stride, potential, scale, values, value_row_stride,
        rows);
    return check_cuda(cudaGetLastError(), "showdown_eval_kernel");
}

// ---- showdown EV straight from strength-sorted inputs ------------------------------------
// Counterpart of `showdown_ev_triton` (p2/search/fused_cfr_triton.py:2271-2320): per row the opponent
// range in strength order, the two hole cards of every sorted position and its tie group [L,R); out is
// the EV of every sorted position, before the caller permutes it back, masks the hands on the board and
// scales by the pot.  The upstream kernel scans all 1326 positions for each hero position; here the
// row gets one prefix over the positions and one prefix per card over that card's (at most 51)
// positions, found through a bit mask of the positions per card.  Prefixes are accumulated in fp64 and
// rounded to fp32 one by one and the formula runs in the operation order of `_showdown_value`
// (p2/search/cfr_evaluator.py:544-596), so a row equals that function's sorted-order EV.
constexpr int kEvsThreads = 384;
constexpr int kEvsWarps = kEvsThreads / 32;
constexpr int kEvsMaxHands = 1344;
constexpr int kEvsWords = kEvsMaxHands / 32;  // 42 mask words per card

__global__ void __launch_bounds__(kEvsThreads) showdown_ev_sorted_kernel(
    const float* __restrict__ b_sorted, const int32_t* __restrict__ c1_sorted, const int32_t* __restrict__ c2_sorted,
    const int32_t* __restrict__ l_idx, const int32_t* __restrict__ r_idx, int64_t rows, int hands, float eps,
    float* __restrict__ out) {
    __shared__ float s_b[kEvsMaxHands];
    __shared__ float s_P[kEvsMaxHands + 1];        // s_P[k] = rounded mass of the positions before k
    __shared__ float s_pc[52 * 52];                // first the card's values in list order, then their prefixes
    __shared__ uint32_t s_mask[52 * kEvsWords];    // bit k of card c: position k holds c
    __shared__ uint16_t s_pre[52 * (kEvsWords + 1)];  // set bits of card c in the words before w
    __shared__ uint8_t s_c1[kEvsMaxHands], s_c2[kEvsMaxHands];
    __shared__ double s_warp[kEvsWarps];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const int64_t base = row * hands;
        for (int k = tid; k < kEvsMaxHands; k += kEvsThreads) {
            const bool in = k < hands;
            const int a = in ? c1_sorted[base + k] : -1, c = in ? c2_sorted[base + k] : -1;
            s_b[k] = in ? b_sorted[base + k] : 0.0f;
            s_c1[k] = (unsigned)a < 52u ? (uint8_t)a : 255;
            s_c2[k] = ((unsigned)c < 52u && c != a) ? (uint8_t)c : 255;
        }
        for (int i = tid; i < 52 * kEvsWords; i += kEvsThreads) s_mask[i] = 0u;
        for (int i = tid; i < 52 * 52; i += kEvsThreads) s_pc[i] = 0.0f;
        __syncthreads();
        for (int k = tid; k < hands; k += kEvsThreads) {
            if (s_c1[k] != 255) atomicOr(&s_mask[s_c1[k] * kEvsWords + (k >> 5)], 1u << (k & 31));
            if (s_c2[k] != 255) atomicOr(&s_mask[s_c2[k] * kEvsWords + (k >> 5)], 1u << (k & 31));
        }
        __syncthreads();
        for (int c = warp; c < 52; c += kEvsWarps) {  // bit counts before every word
            const int n0 = __popc(s_mask[c * kEvsWords + lane]);
            const int n1 = lane + 32 < kEvsWords ? __popc(s_mask[c * kEvsWords + lane + 32]) : 0;
            int i0 = n0, i1 = n1;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int u0 = __shfl_up_sync(0xffffffffu, i0, d), u1 = __shfl_up_sync(0xffffffffu, i1, d);
                if (lane >= d) {
                    i0 += u0;
                    i1 += u1;
                }
            }
            const int first = __shfl_sync(0xffffffffu, i0, 31);
            s_pre[c * (kEvsWords + 1) + lane] = (uint16_t)(i0 - n0);
            if (lane + 32 <= kEvsWords) s_pre[c * (kEvsWords + 1) + lane + 32] = (uint16_t)(first + i1 - n1);
        }
        __syncthreads();
        for (int k = tid; k < hands; k += kEvsThreads) {  // the card lists: values in strength order
            const uint32_t below = (1u << (k & 31)) - 1u;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = j == 0 ? s_c1[k] : s_c2[k];
                if (c == 255) continue;
                const int t = s_pre[c * (kEvsWords + 1) + (k >> 5)] + __popc(s_mask[c * kEvsWords + (k >> 5)] & below);
                if (t < 52) s_pc[c * 52 + t] = s_b[k];
            }
        }
        __syncthreads();
        for (int c = warp; c < 52; c += kEvsWarps) {  // per card: mass of its t weakest hands, t = 0..51
            const double v0 = s_pc[c * 52 + lane], v1 = lane + 32 < 52 ? s_pc[c * 52 + lane + 32] : 0.0;
            double i0 = v0, i1 = v1;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const double u0 = __shfl_up_sync(0xffffffffu, i0, d), u1 = __shfl_up_sync(0xffffffffu, i1, d);
                if (lane >= d) {
                    i0 += u0;
                    i1 += u1;
                }
            }
            const double first = __shfl_sync(0xffffffffu, i0, 31);
            __syncwarp();
            s_pc[c * 52 + lane] = (float)(i0 - v0);
            if (lane + 32 < 52) s_pc[c * 52 + lane + 32] = (float)(first + (i1 - v1));
        }
        {  // prefix over all positions: four consecutive positions per thread
            double v[4], run = 0.0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int k = 4 * tid + i;
                v[i] = k < kEvsMaxHands ? (double)s_b[k] : 0.0;
                run += v[i];
            }
            double inc = run;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const double u = __shfl_up_sync(0xffffffffu, inc, d);
                if (lane >= d) inc += u;
            }
            if (lane == 31) s_warp[warp] = inc;
            __syncthreads();
            double before = inc - run;
            for (int w = 0; w < warp; ++w) before += s_warp[w];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int k = 4 * tid + i;
                if (k == 0) s_P[0] = 0.0f;
                before += v[i];
                if (k < kEvsMaxHands) s_P[k + 1] = (float)before;
            }
        }
        __syncthreads();
        for (int k = tid; k < hands; k += kEvsThreads) {
            int L = l_idx[base + k], R = r_idx[base + k];
            L = min(max(L, 0), hands);
            R = min(max(R, 0), hands);
            const float x = s_b[k];
            float at[2][3];  // per card: mass before L, before R, in all
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = j == 0 ? s_c1[k] : s_c2[k];
                at[j][0] = at[j][1] = at[j][2] = 0.0f;
                if (c == 255) continue;
                const uint32_t* m = s_mask + c * kEvsWords;
                const uint16_t* pre = s_pre + c * (kEvsWords + 1);
                const int tl = pre[L >> 5] + ((L >> 5) < kEvsWords ? __popc(m[L >> 5] & ((1u << (L & 31)) - 1u)) : 0);
                const int tr = pre[R >> 5] + ((R >> 5) < kEvsWords ? __popc(m[R >> 5] & ((1u << (R & 31)) - 1u)) : 0);
                at[j][0] = s_pc[c * 52 + min(tl, 51)];
                at[j][1] = s_pc[c * 52 + min(tr, 51)];
                at[j][2] = s_pc[c * 52 + 51];
            }
            const float PL = s_P[L], PR = s_P[R];
            const float win = __fsub_rn(__fsub_rn(PL, at[0][0]), at[1][0]);
            const float seg = __fsub_rn(PR, PL);
            const float tie = __fadd_rn(
                __fsub_rn(__fsub_rn(seg, __fsub_rn(at[0][1], at[0][0])), __fsub_rn(at[1][1], at[1][0])), x);
            const float den = __fadd_rn(__fsub_rn(__fsub_rn(1.0f, at[0][2]), at[1][2]), x);
            const float safe = fmaxf(den, eps);
            const float wp = __fdiv_rn(win, safe), tp = __fdiv_rn(tie, safe);
            const float lp = __fsub_rn(__fsub_rn(1.0f, wp), tp);
            out[base + k] = den > eps ? __fsub_rn(wp, lp) : 0.0f;
        }
        __syncthreads();
    }
}

int launch_showdown_ev_sorted(const float* b_sorted, const int32_t* c1_sorted, const int32_t* c2_sorted,
                              const int32_t* l_idx, const int32_t* r_idx, int64_t rows, int hands, float eps, float* out,
                              cudaStream_t stream) {
    if (rows == 0 || hands == 0) return P2B_OK;
    if (hands < 0 || hands > kEvsMaxHands) return set_error(P2B_ERR_ARG, "a row holds at most %d hands", kEvsMaxHands);
    int64_t grid = rows;
    const int64_t cap = (int64_t)sm_count() * 4;
    if (grid > cap) grid = cap;
    showdown_ev_sorted_kernel<<<(unsigned)grid, kEvsThreads, 0, stream>>>(b_sorted, c1_sorted, c2_sorted, l_idx, r_idx,
                                                                        rows, hands, eps, out);
    return check_cuda(cudaGetLastError(), "showdown_ev_sorted_kernel");
}

}  // namespace p2b
