// Hand-ranking kernels: packed score of [N,7] card ids, pairwise comparison of card-id
// and one-hot-plane hands.  HBM-bound by design: 14 B in + 4 B out per hand; a thread owns
// four consecutive hands (56 B, seven 8-byte loads) and prefetches its next four while it
// scores the current ones.
#include "common.cuh"
#include "rank7.cuh"

namespace p2b {

constexpr int kRankThreads = 256;
constexpr int kHandsPerThread = 4;
constexpr int kTileHands = kRankThreads * kHandsPerThread;  // 1024 hands = 14336 B per tile

// cards: [n,7] int16; out: [n] int32.  VEC = base pointer is 8-byte aligned.
// A block keeps the 32 KB rank table, the type table and a card -> suit-lane-bit table in
// shared memory; a hand of distinct cards is scored by the table walk of rank7.cuh
// (score_distinct_lut), a hand with repeated ids by the general bit-mask scorer.
template <bool VEC>
__global__ void __launch_bounds__(kRankThreads) rank7_cards_kernel(const int16_t* __restrict__ cards,
                                                                   int32_t* __restrict__ out, int64_t n,
                                                                   const RankLut* __restrict__ lut) {
    __shared__ __align__(16) uint32_t T[kRankLutEntries];
    __shared__ uint32_t TT[32];
    {
        const uint4* src = reinterpret_cast<const uint4*>(lut->mask_entry);
        for (int i = threadIdx.x; i < kRankLutEntries / 4; i += kRankThreads) reinterpret_cast<uint4*>(T)[i] = __ldg(src + i);
        if (threadIdx.x < 32) TT[threadIdx.x] = threadIdx.x < kTypeLutEntries ? lut->type_entry[threadIdx.x] : 0u;
    }
    __syncthreads();
    // A thread takes four consecutive hands: 56 bytes = seven 8-byte words (VEC: 8-byte aligned),
    // read straight from global memory; the words of its next tile are fetched while the current
    // four hands are scored, so no barrier separates loading from scoring.
    const int64_t num_tiles = (n + kTileHands - 1) / kTileHands;
    auto load_words = [&](int64_t t, uint32_t (&w)[14]) {
        const int64_t h0 = t * kTileHands + kHandsPerThread * threadIdx.x;
        if (t < num_tiles && VEC && h0 + kHandsPerThread <= n) {
            const uint2* mine = reinterpret_cast<const uint2*>(cards + h0 * 7);
#pragma unroll
            for (int i = 0; i < 7; ++i) {
                const uint2 v = __ldcs(mine + i);
                w[2 * i] = v.x;
                w[2 * i + 1] = v.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 14; ++i) {
                const int64_t e = h0 * 7 + 2 * i;
                const uint32_t a0 = (t < num_tiles && e < n * 7) ? (uint16_t)cards[e] : 0u;
                const uint32_t a1 = (t < num_tiles && e + 1 < n * 7) ? (uint16_t)cards[e + 1] : 0u;
                w[i] = a0 | (a1 << 16);
            }
        }
    };
    uint32_t w[14], wn[14];
    load_words(blockIdx.x, w);
    for (int64_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        const int64_t hand0 = t * kTileHands;
        const int64_t remaining = n - hand0;
        const int hands = remaining < kTileHands ? (int)remaining : kTileHands;
        load_words(t + gridDim.x, wn);
        // card id -> bit position in the four 16-bit suit lanes (id + 3 * suit), for both 16-bit
        // halves of a word at once: (id * 79) >> 10 is id / 13 for ids below 52 and the product
        // of the low half cannot carry into the high half
        uint32_t bp[14];
#pragma unroll
        for (int k = 0; k < 14; ++k) bp[k] = w[k] + 3u * (((w[k] * 79u) >> 10) & 0x003F003Fu);
        int32_t score[kHandsPerThread];
#pragma unroll
        for (int j = 0; j < kHandsPerThread; ++j) {
            uint32_t lo = 0, hi = 0;
#pragma unroll
            for (int i = 0; i < 7; ++i) {
                const int e = 7 * j + i;  // 16-bit element of the thread's 28
                const uint32_t bit = (e & 1) ? (bp[e >> 1] >> 16) : (bp[e >> 1] & 0xffffu);
                uint32_t blo, bhi;  // 1 << bit as two words: shl.b32 gives 0 for shift counts above 31
                asm("shl.b32 %0, 1, %1;" : "=r"(blo) : "r"(bit));
                asm("shl.b32 %0, 1, %1;" : "=r"(bhi) : "r"(bit - 32u));
                lo |= blo;
                hi |= bhi;
            }
            if (__popc(lo) + __popc(hi) == 7) {
                score[j] = score_distinct_lut(lo & 0x1fffu, (lo >> 16) & 0x1fffu, hi & 0x1fffu, (hi >> 16) & 0x1fffu, T, TT);
            } else {  // repeated (or out-of-range) ids: the general scorer on the ids themselves
                int c[7];
#pragma unroll
                for (int i = 0; i < 7; ++i) {
                    const int e = 7 * j + i;
                    c[i] = (int)(int16_t)((e & 1) ? (w[e >> 1] >> 16) : (w[e >> 1] & 0xffffu));
                }
                score[j] = score_cards<7>(c);
            }
        }
        const int h0 = kHandsPerThread * threadIdx.x;
        if (h0 + kHandsPerThread <= hands && ((reinterpret_cast<uintptr_t>(out + hand0) & 15) == 0)) {
            __stcs(reinterpret_cast<int4*>(out + hand0 + h0), make_int4(score[0], score[1], score[2], score[3]));
        } else {
#pragma unroll
            for (int j = 0; j < kHandsPerThread; ++j)
                if (h0 + j < hands) out[hand0 + h0 + j] = score[j];
        }
#pragma unroll
        for (int i = 0; i < 14; ++i) w[i] = wn[i];
    }
}

// cards: [n,2,7] int16 -> {1,-1,0}
__global__ void __launch_bounds__(256) compare7_cards_kernel(const int16_t* __restrict__ cards,
                                                            int32_t* __restrict__ out, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int a[7], b[7];
#pragma unroll
        for (int k = 0; k < 7; ++k) {
            a[k] = cards[i * 14 + k];
            b[k] = cards[i * 14 + 7 + k];
        }
        const int32_t sa = score_cards<7>(a), sb = score_cards<7>(b);
        out[i] = (sa > sb) - (sa < sb);
    }
}

// planes: [n,2,4,13] bytes (non-zero = card present) -> {1,-1,0}.  A plane set is a set of
// cards, so a rank's count is the number of suits holding it (p2/env/rules.py:157).
__device__ __forceinline__ int32_t score_planes(const int8_t* __restrict__ p) {
    uint32_t m[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        uint32_t bits = 0;
#pragma unroll
        for (int r = 0; r < 13; ++r) bits |= (p[s * 13 + r] != 0 ? 1u : 0u) << r;
        m[s] = bits;
    }
    return score_from_masks(m[0], m[1], m[2], m[3], classes_from_suits(m[0], m[1], m[2], m[3]));
}

__global__ void __launch_bounds__(256) compare7_planes_kernel(const int8_t* __restrict__ planes,
                                                             int32_t* __restrict__ out, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int32_t sa = score_planes(planes + i * 104), sb = score_planes(planes + i * 104 + 52);
        out[i] = (sa > sb) - (sa < sb);
    }
}

static int grid_for(int64_t work_items, int per_block, int max_blocks) {
    int64_t g = (work_items + per_block - 1) / per_block;
    if (g < 1) g = 1;
    if (g > max_blocks) g = max_blocks;
    return (int)g;
}

int sm_count();

int launch_rank7_cards(const int16_t* cards, int64_t n, int32_t* out, cudaStream_t stream) {
    if (n == 0) return P2B_OK;
    int rc = ensure_tables();
    if (rc) return rc;
    const bool vec = (reinterpret_cast<uintptr_t>(cards) & 7) == 0;
    // one wave of resident blocks: the tile loop is strided by the grid, so a partial second wave
    // would leave most SMs idle at the end
    static int resident[2] = {0, 0};
    if (resident[vec] == 0) {
        int per_sm = 0;
        cudaError_t e = vec ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rank7_cards_kernel<true>, kRankThreads, 0)
                            : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rank7_cards_kernel<false>, kRankThreads, 0);
        if (e != cudaSuccess) return check_cuda(e, "rank7 occupancy query");
        resident[vec] = per_sm > 0 ? per_sm : 1;
    }
    const int grid = grid_for(n, kTileHands, sm_count() * resident[vec]);
    if (vec) rank7_cards_kernel<true><<<grid, kRankThreads, 0, stream>>>(cards, out, n, device_rank_lut());
    else rank7_cards_kernel<false><<<grid, kRankThreads, 0, stream>>>(cards, out, n, device_rank_lut());
    return check_cuda(cudaGetLastError(), "rank7_cards_kernel");
}

int launch_compare7_cards(const int16_t* cards, int64_t n, int32_t* out, cudaStream_t stream) {
    if (n == 0) return P2B_OK;
    compare7_cards_kernel<<<grid_for(n, 256, sm_count() * 8), 256, 0, stream>>>(cards, out, n);
    return check_cuda(cudaGetLastError(), "compare7_cards_kernel");
}

int launch_compare7_planes(const int8_t* planes, int64_t n, int32_t* out, cudaStream_t stream) {
    if (n == 0) return P2B_OK;
    compare7_planes_kernel<<<grid_for(n, 256, sm_count() * 8), 256, 0, stream>>>(planes, out, n);
    return check_cuda(cudaGetLastError(), "compare7_planes_kernel");
}

}  // namespace p2b
