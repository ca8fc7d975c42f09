// Chance-node helpers: belief expansion over the next public card and the ordered
// indexed add that averages the leaf-model values back per root
// (p2/search/chance_node_helper.py:359-479, `single_card_chance_values`).
#include "common.cuh"
#include "exactdiv.cuh"

#include <cuda_bf16.h>

namespace p2b {
namespace {

constexpr int kThreads = 256;

// One block per (root, next card) sample.  boards: [B, board_len] int64, -1 = empty slot.
// Sample s of root b is the s-th card (ascending id) not on b's board; sample rows are
// grouped by root in root order, which is the order upstream's nonzero() produces
// (:402-414).  Writes, per sample: the root index, the board with the new card in the first
// empty slot (:416-418), and both players' beliefs with every combo touching the extended
// board zeroed and the row renormalised; a row whose mass is <= 1e-12 becomes uniform over
// the allowed combos (:434-444).
__global__ void chance_expand_kernel(const float* __restrict__ pre_beliefs, const long long* __restrict__ boards,
                                     int board_len, const long long* __restrict__ sample_offsets, long long num_roots,
                                     const ComboTable* __restrict__ combos, float* __restrict__ post_beliefs,
                                     long long* __restrict__ root_lookup, long long* __restrict__ board_samples) {
    __shared__ double red[kThreads / 32];
    __shared__ int s_root;
    __shared__ int s_card;
    __shared__ unsigned long long s_mask;
    const long long total = sample_offsets[num_roots];
    for (long long smp = blockIdx.x; smp < total; smp += gridDim.x) {
        if (threadIdx.x == 0) {
            // root of this sample: last b with sample_offsets[b] <= smp
            long long lo = 0, hi = num_roots - 1;
            while (lo < hi) {
                const long long mid = (lo + hi + 1) >> 1;
                if (sample_offsets[mid] <= smp) lo = mid;
                else hi = mid - 1;
            }
            unsigned long long mask = 0;
            int ncards = 0;
            for (int j = 0; j < board_len; ++j) {
                const long long c = boards[lo * board_len + j];
                if (c >= 0) {
                    mask |= 1ull << c;
                    ++ncards;
                }
            }
            // the k-th free card, k = smp - offset
            int k = (int)(smp - sample_offsets[lo]), card = 0;
            for (;; ++card)
                if (!((mask >> card) & 1ull) && k-- == 0) break;
            s_root = (int)lo;
            s_card = card;
            s_mask = mask | (1ull << card);
            root_lookup[smp] = lo;
            for (int j = 0; j < board_len; ++j) {
                long long c = boards[lo * board_len + j];
                if (j == ncards) c = card;
                board_samples[smp * board_len + j] = c;
            }
        }
        __syncthreads();
        const unsigned long long mask = s_mask;
        const long long b = s_root;
        for (int p = 0; p < 2; ++p) {
            const float* src = pre_beliefs + (b * 2 + p) * P2B_NUM_HANDS;
            float* dst = post_beliefs + (smp * 2 + p) * P2B_NUM_HANDS;
            double s = 0.0;
            int n_allowed = 0;
            for (int h = threadIdx.x; h < P2B_NUM_HANDS; h += blockDim.x) {
                const bool ok = (((mask >> combos->c1[h]) | (mask >> combos->c2[h])) & 1ull) == 0;
                const float v = ok ? src[h] : 0.0f;
                dst[h] = v;
                s += (double)v;
                n_allowed += ok;
            }
            // block sums (mass and number of allowed combos)
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) {
                s += __shfl_xor_sync(0xffffffffu, s, d);
                n_allowed += __shfl_xor_sync(0xffffffffu, n_allowed, d);
            }
            __shared__ int cnt[kThreads / 32];
            __syncthreads();
            if ((threadIdx.x & 31) == 0) {
                red[threadIdx.x >> 5] = s;
                cnt[threadIdx.x >> 5] = n_allowed;
            }
            __syncthreads();
            double tot = 0.0;
            int nall = 0;
            for (int w = 0; w < kThreads / 32; ++w) {
                tot += red[w];
                nall += cnt[w];
            }
            const float sum = (float)tot;
            const float uni = __fdiv_rn(1.0f, fmaxf((float)nall, 1.0f));
            for (int h = threadIdx.x; h < P2B_NUM_HANDS; h += blockDim.x) {
                const bool ok = (((mask >> combos->c1[h]) | (mask >> combos->c2[h])) & 1ull) == 0;
                dst[h] = sum > 1e-12f ? __fdiv_rn(dst[h], fmaxf(sum, 1e-12f)) : (ok ? uni : 0.0f);
            }
        }
        __syncthreads();
    }
}

// out[index[i], :] += src[i, :] for i in ascending order; `index` must be sorted
// (non-decreasing), as the chance helper's root_lookup is.  Each output element is owned
// by one thread, so the additions happen in index order: deterministic, no atomics.  With
// `mean` the sum is divided by max(count, 1) (:468-477).
__global__ void indexed_add_rows_kernel(float* __restrict__ out, const long long* __restrict__ index,
                                        const float* __restrict__ src, long long num_src, long long num_out,
                                        long long width, int mean, int accumulate) {
    const long long n = num_out * width;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {
        const long long row = e / width, col = e % width;
        // first i with index[i] >= row
        long long lo = 0, hi = num_src;
        while (lo < hi) {
            const long long mid = (lo + hi) >> 1;
            if (index[mid] < row) lo = mid + 1;
            else hi = mid;
        }
        float acc = accumulate ? out[e] : 0.0f;
        long long i = lo;
        for (; i < num_src && index[i] == row; ++i) acc = __fadd_rn(acc, src[i * width + col]);
        if (mean) acc = __fdiv_rn(acc, fmaxf((float)(i - lo), 1.0f));
        out[e] = acc;
    }
}

// Fused form of the expansion for a bf16 value network: per (root, next card)
// sample writes the network's input row directly -- both players' re-blocked, re-normalised
// beliefs (the arithmetic of chance_expand_kernel, then rounded to bf16), the one-hot of the
// extended board, the root's three context scalars and zero padding up to `feature_stride`
// -- so that no fp32 copy of the expanded beliefs ever exists.  The two belief rows of a root
// are `player_stride` floats apart (1326 for packed rows, 1344 for the solver's padded rows).
constexpr int kHandsPerThread = (P2B_NUM_HANDS + kThreads - 1) / kThreads;  // 6

// A block takes up to kCardsPerBlock consecutive next cards of one root: the root's two belief rows are
// read once into registers, every card's block-wide sums (mass of the combos that stay allowed, their
// number) are gathered with one barrier pair for the whole group, then the rows are written.  The
// per-thread partial sums, the shuffle tree and the order over warps are those of chance_expand_kernel,
// so the normalised values are the same bits.
constexpr int kCardsPerBlock = 8;
constexpr int kCardGroups = (P2B_NUM_CARDS + kCardsPerBlock - 1) / kCardsPerBlock;  // groups per root (the last ones may be empty)

__global__ void __launch_bounds__(kThreads) chance_expand_features_kernel(
    const float* __restrict__ pre_beliefs, long long player_stride, const long long* __restrict__ boards, int board_len,
    const long long* __restrict__ sample_offsets, long long num_roots, const float* __restrict__ context,
    const ComboTable* __restrict__ combos, __nv_bfloat16* __restrict__ features, long long feature_stride,
    long long* __restrict__ root_lookup) {
    __shared__ double red[kCardsPerBlock][2][kThreads / 32];
    __shared__ int cnt[kCardsPerBlock][kThreads / 32];
    // the two cards of this thread's hands do not depend on the root
    int c1[kHandsPerThread], c2[kHandsPerThread];
#pragma unroll
    for (int i = 0; i < kHandsPerThread; ++i) {
        const int h = threadIdx.x + i * kThreads;
        c1[i] = h < P2B_NUM_HANDS ? combos->c1[h] : 0;
        c2[i] = h < P2B_NUM_HANDS ? combos->c2[h] : 0;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long long task = blockIdx.x; task < num_roots * kCardGroups; task += gridDim.x) {
        const long long b = task / kCardGroups;
        const int k0 = (int)(task - b * kCardGroups) * kCardsPerBlock;
        const long long first = sample_offsets[b];
        const int n_free = (int)(sample_offsets[b + 1] - first);
        if (k0 >= n_free) continue;  // uniform over the block
        const int n_here = min(kCardsPerBlock, n_free - k0);
        unsigned long long board_mask = 0;
        for (int j = 0; j < board_len; ++j) {
            const long long c = boards[b * board_len + j];
            if (c >= 0) board_mask |= 1ull << c;
        }
        // the k0-th free card, in ascending order; the following ones are the next set bits
        unsigned long long free_cards = ~board_mask & ((1ull << P2B_NUM_CARDS) - 1ull);
        for (int k = 0; k < k0; ++k) free_cards &= free_cards - 1ull;
        const float* src0 = pre_beliefs + (b * 2) * player_stride;
        const float* src1 = src0 + player_stride;
        float v0[kHandsPerThread], v1[kHandsPerThread];
#pragma unroll
        for (int i = 0; i < kHandsPerThread; ++i) {
            const int h = threadIdx.x + i * kThreads;
            const bool on = h < P2B_NUM_HANDS && (((board_mask >> c1[i]) | (board_mask >> c2[i])) & 1ull) == 0;
            v0[i] = on ? src0[h] : 0.0f;
            v1[i] = on ? src1[h] : 0.0f;
            if (!on) c1[i] |= 64;  // marks a hand that no card of this root allows
        }
        __syncthreads();  // the previous task's sums have been read
        {
            unsigned long long rest = free_cards;
            for (int k = 0; k < n_here; ++k) {
                const int card = __ffsll((long long)rest) - 1;
                rest &= rest - 1ull;
                double s0 = 0.0, s1 = 0.0;
                int n_allowed = 0;
#pragma unroll
                for (int i = 0; i < kHandsPerThread; ++i) {
                    const bool ok = c1[i] != card && c2[i] != card && c1[i] < 64;
                    s0 += (double)(ok ? v0[i] : 0.0f);
                    s1 += (double)(ok ? v1[i] : 0.0f);
                    n_allowed += ok;
                }
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) {
                    s0 += __shfl_xor_sync(0xffffffffu, s0, d);
                    s1 += __shfl_xor_sync(0xffffffffu, s1, d);
                    n_allowed += __shfl_xor_sync(0xffffffffu, n_allowed, d);
                }
                if (lane == 0) {
                    red[k][0][warp] = s0;
                    red[k][1][warp] = s1;
                    cnt[k][warp] = n_allowed;
                }
            }
        }
        __syncthreads();
        unsigned long long rest = free_cards;
        for (int k = 0; k < n_here; ++k) {
            const int card = __ffsll((long long)rest) - 1;
            rest &= rest - 1ull;
            const long long smp = first + k0 + k;
            if (threadIdx.x == 0 && root_lookup) root_lookup[smp] = b;
            __nv_bfloat16* row = features + smp * feature_stride;
            double tot0 = 0.0, tot1 = 0.0;
            int nall = 0;
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) {
                tot0 += red[k][0][w];
                tot1 += red[k][1][w];
                nall += cnt[k][w];
            }
            const float uni = __fdiv_rn(1.0f, fmaxf((float)nall, 1.0f));
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const float sum = (float)(p ? tot1 : tot0);
                const Divisor d = make_divisor(fmaxf(sum, 1e-12f));  // one divisor per row: exactly rounded quotients
#pragma unroll
                for (int i = 0; i < kHandsPerThread; ++i) {
                    const int h = threadIdx.x + i * kThreads;
                    if (h < P2B_NUM_HANDS) {
                        const bool ok = c1[i] != card && c2[i] != card && c1[i] < 64;
                        const float v = ok ? (p ? v1[i] : v0[i]) : 0.0f;
                        const float x = sum > 1e-12f ? div_exact(v, d) : (ok ? uni : 0.0f);
                        row[p * P2B_NUM_HANDS + h] = __float2bfloat16_rn(x);
                    }
                }
            }
            // board one-hot, context, padding
            const unsigned long long mask = board_mask | (1ull << card);
            for (long long j = 2 * P2B_NUM_HANDS + threadIdx.x; j < feature_stride; j += kThreads) {
                const int r = (int)(j - 2 * P2B_NUM_HANDS);
                float x = 0.0f;
                if (r < 52) x = ((mask >> r) & 1ull) ? 1.0f : 0.0f;
                else if (r < 55) x = context[b * 3 + (r - 52)];
                row[j] = __float2bfloat16_rn(x);
            }
        }
#pragma unroll
        for (int i = 0; i < kHandsPerThread; ++i) c1[i] &= 63;
    }
}

// out[r, p, h] = mean over the samples of root r (rows sample_offsets[r] .. sample_offsets[r+1])
// of src[sample, p*1326 + h], bf16 -> fp32, added in ascending sample order and divided by
// max(count, 1) (chance_node_helper.py:462-477).  Each output element is owned by one thread.
__global__ void indexed_mean_bf16_kernel(const __nv_bfloat16* __restrict__ src, long long src_stride,
                                         const long long* __restrict__ sample_offsets, long long num_roots,
                                         float* __restrict__ out, long long out_player_stride) {
    const long long n = num_roots * 2 * P2B_NUM_HANDS;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {
        const long long r = e / (2 * P2B_NUM_HANDS);
        const int c = (int)(e - r * 2 * P2B_NUM_HANDS), p = c >= P2B_NUM_HANDS, h = c - p * P2B_NUM_HANDS;
        const long long a = sample_offsets[r], b = sample_offsets[r + 1];
        float acc = 0.0f;
        for (long long i = a; i < b; ++i) acc = __fadd_rn(acc, __bfloat162float(src[i * src_stride + c]));
        out[(r * 2 + p) * out_player_stride + h] = __fdiv_rn(acc, fmaxf((float)(b - a), 1.0f));
    }
}

// Beliefs re-blocked and re-normalised on explicitly given boards (the flop chance node,
// chance_node_helper.py:262-284): sample s = root * num_boards + board.  Same arithmetic as
// chance_expand_kernel; every card of `boards[board]` that is >= 0 blocks.
__global__ void expand_on_boards_kernel(const float* __restrict__ pre_beliefs, long long player_stride,
                                        const long long* __restrict__ boards, int board_len, long long num_roots,
                                        long long num_boards, const ComboTable* __restrict__ combos,
                                        float* __restrict__ post_beliefs) {
    __shared__ double red[kThreads / 32];
    __shared__ int cnt[kThreads / 32];
    const long long total = num_roots * num_boards;
    for (long long smp = blockIdx.x; smp < total; smp += gridDim.x) {
        const long long b = smp / num_boards, f = smp - b * num_boards;
        unsigned long long mask = 0;
        for (int j = 0; j < board_len; ++j) {
            const long long c = boards[f * board_len + j];
            if (c >= 0) mask |= 1ull << c;
        }
        for (int p = 0; p < 2; ++p) {
            const float* src = pre_beliefs + (b * 2 + p) * player_stride;
            float* dst = post_beliefs + (smp * 2 + p) * P2B_NUM_HANDS;
            float v[kHandsPerThread];
            bool ok[kHandsPerThread];
            double s = 0.0;
            int n_allowed = 0;
#pragma unroll
            for (int i = 0; i < kHandsPerThread; ++i) {
                const int h = threadIdx.x + i * kThreads;
                ok[i] = false;
                v[i] = 0.0f;
                if (h < P2B_NUM_HANDS) {
                    ok[i] = (((mask >> combos->c1[h]) | (mask >> combos->c2[h])) & 1ull) == 0;
                    v[i] = ok[i] ? src[h] : 0.0f;
                    s += (double)v[i];
                    n_allowed += ok[i];
                }
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) {
                s += __shfl_xor_sync(0xffffffffu, s, d);
                n_allowed += __shfl_xor_sync(0xffffffffu, n_allowed, d);
            }
            __syncthreads();
            if ((threadIdx.x & 31) == 0) {
                red[threadIdx.x >> 5] = s;
                cnt[threadIdx.x >> 5] = n_allowed;
            }
            __syncthreads();
            double tot = 0.0;
            int nall = 0;
            for (int w = 0; w < kThreads / 32; ++w) {
                tot += red[w];
                nall += cnt[w];
            }
            const float sum = (float)tot;
            const float uni = __fdiv_rn(1.0f, fmaxf((float)nall, 1.0f));
#pragma unroll
            for (int i = 0; i < kHandsPerThread; ++i) {
                const int h = threadIdx.x + i * kThreads;
                if (h < P2B_NUM_HANDS)
                    dst[h] = sum > 1e-12f ? __fdiv_rn(v[i], fmaxf(sum, 1e-12f)) : (ok[i] ? uni : 0.0f);
            }
        }
        __syncthreads();
    }
}

// out[n, h] = (sum over p of values[n, perms[p, h]]) / num_perms, added in ascending p: the mean
// of a row over the hand-index permutations of a set of suit permutations
// (`_avg_over_perms`, chance_node_helper.py:17-27).  Rows are 1326 floats, packed.
__global__ void mean_over_hand_perms_kernel(const float* __restrict__ values, const int* __restrict__ perms,
                                            int num_perms, long long rows, float* __restrict__ out) {
    const long long n = rows * P2B_NUM_HANDS;
    for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n; e += (long long)gridDim.x * blockDim.x) {
        const long long r = e / P2B_NUM_HANDS;
        const int h = (int)(e - r * P2B_NUM_HANDS);
        const float* row = values + r * P2B_NUM_HANDS;
        float acc = 0.0f;
        for (int p = 0; p < num_perms; ++p) acc = __fadd_rn(acc, row[perms[p * P2B_NUM_HANDS + h]]);
        out[e] = __fdiv_rn(acc, (float)num_perms);
    }
}

}  // namespace

int sm_count();

}  // namespace p2b

using namespace p2b;

extern "C" {

int p2b_chance_expand(const float* pre_beliefs, const int64_t* boards, int32_t board_len, const int64_t* sample_offsets,
                      int64_t num_roots, int64_t num_samples, float* post_beliefs, int64_t* root_lookup,
                      int64_t* board_samples, void* stream) {
    if (num_roots <= 0 || num_samples <= 0) return P2B_OK;
    if (!pre_beliefs || !boards || !sample_offsets || !post_beliefs || !root_lookup || !board_samples)
        return set_error(P2B_ERR_ARG, "p2b_chance_expand: null pointer");
    int rc = ensure_tables();
    if (rc) return rc;
    long long grid = num_samples;
    if (grid > (long long)sm_count() * 16) grid = (long long)sm_count() * 16;
    chance_expand_kernel<<<(unsigned)grid, kThreads, 0, (cudaStream_t)stream>>>(
        pre_beliefs, (const long long*)boards, board_len, (const long long*)sample_offsets, num_roots,
        device_combo_table(), post_beliefs, (long long*)root_lookup, (long long*)board_samples);
    return check_cuda(cudaGetLastError(), "chance_expand_kernel");
}

int p2b_chance_expand_features(const float* pre_beliefs, int64_t player_stride, const int64_t* boards, int32_t board_len,
                               const int64_t* sample_offsets, int64_t num_roots, int64_t num_samples,
                               const float* context, void* features_bf16, int64_t feature_stride, int64_t* root_lookup,
                               void* stream) {
    if (num_roots <= 0 || num_samples <= 0) return P2B_OK;
    if (!pre_beliefs || !boards || !sample_offsets || !context || !features_bf16)
        return set_error(P2B_ERR_ARG, "p2b_chance_expand_features: null pointer");
    if (player_stride < P2B_NUM_HANDS || feature_stride < 2 * P2B_NUM_HANDS + 55)
        return set_error(P2B_ERR_ARG, "p2b_chance_expand_features: stride too small");
    int rc = ensure_tables();
    if (rc) return rc;
    long long grid = num_roots * kCardGroups;
    if (grid > (long long)sm_count() * 16) grid = (long long)sm_count() * 16;
    chance_expand_features_kernel<<<(unsigned)grid, kThreads, 0, (cudaStream_t)stream>>>(
        pre_beliefs, player_stride, (const long long*)boards, board_len, (const long long*)sample_offsets, num_roots,
        context, device_combo_table(), static_cast<__nv_bfloat16*>(features_bf16), feature_stride,
        (long long*)root_lookup);
    return check_cuda(cudaGetLastError(), "chance_expand_features_kernel");
}

int p2b_indexed_mean_bf16(const void* src_bf16, int64_t src_stride, const int64_t* sample_offsets, int64_t num_roots,
                          float* out, int64_t out_player_stride, void* stream) {
    if (num_roots <= 0) return P2B_OK;
    if (!src_bf16 || !sample_offsets || !out) return set_error(P2B_ERR_ARG, "p2b_indexed_mean_bf16: null pointer");
    if (src_stride < 2 * P2B_NUM_HANDS || out_player_stride < P2B_NUM_HANDS)
        return set_error(P2B_ERR_ARG, "p2b_indexed_mean_bf16: stride too small");
    long long blocks = (num_roots * 2 * P2B_NUM_HANDS + kThreads - 1) / kThreads;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
    indexed_mean_bf16_kernel<<<(unsigned)blocks, kThreads, 0, (cudaStream_t)stream>>>(
        static_cast<const __nv_bfloat16*>(src_bf16), src_stride, (const long long*)sample_offsets, num_roots, out,
        out_player_stride);
    return check_cuda(cudaGetLastError(), "indexed_mean_bf16_kernel");
}

int p2b_expand_on_boards(const float* pre_beliefs, int64_t player_stride, const int64_t* boards, int32_t board_len,
                         int64_t num_roots, int64_t num_boards, float* post_beliefs, void* stream) {
    if (num_roots <= 0 || num_boards <= 0) return P2B_OK;
    if (!pre_beliefs || !boards || !post_beliefs) return set_error(P2B_ERR_ARG, "p2b_expand_on_boards: null pointer");
    if (player_stride < P2B_NUM_HANDS) return set_error(P2B_ERR_ARG, "p2b_expand_on_boards: stride too small");
    int rc = ensure_tables();
    if (rc) return rc;
    long long grid = num_roots * num_boards;
    if (grid > (long long)sm_count() * 16) grid = (long long)sm_count() * 16;
    expand_on_boards_kernel<<<(unsigned)grid, kThreads, 0, (cudaStream_t)stream>>>(
        pre_beliefs, player_stride, (const long long*)boards, board_len, num_roots, num_boards, device_combo_table(),
        post_beliefs);
    return check_cuda(cudaGetLastError(), "expand_on_boards_kernel");
}

int p2b_mean_over_hand_perms(const float* values, const int32_t* perms, int32_t num_perms, int64_t rows, float* out,
                             void* stream) {
    if (rows <= 0) return P2B_OK;
    if (!values || !perms || !out || num_perms < 1)
        return set_error(P2B_ERR_ARG, "p2b_mean_over_hand_perms: null pointer or no permutation");
    long long blocks = (rows * P2B_NUM_HANDS + kThreads - 1) / kThreads;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
    mean_over_hand_perms_kernel<<<(unsigned)blocks, kThreads, 0, (cudaStream_t)stream>>>(values, perms, num_perms, rows, out);
    return check_cuda(cudaGetLastError(), "mean_over_hand_perms_kernel");
}

int p2b_indexed_add_rows(float* out, const int64_t* index, const float* src, int64_t num_src, int64_t num_out,
                         int64_t width, int mean, int accumulate, void* stream) {
    if (num_out <= 0 || width <= 0) return P2B_OK;
    if (!out || (num_src > 0 && (!index || !src))) return set_error(P2B_ERR_ARG, "p2b_indexed_add_rows: null pointer");
    long long blocks = (num_out * width + kThreads - 1) / kThreads;
    if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
    indexed_add_rows_kernel<<<(unsigned)blocks, kThreads, 0, (cudaStream_t)stream>>>(
        out, (const long long*)index, src, num_src, num_out, width, mean, accumulate);
    return check_cuda(cudaGetLastError(), "indexed_add_rows_kernel");
}

}  // extern "C"
