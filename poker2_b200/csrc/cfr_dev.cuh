// Device helpers shared by the subgame-CFR kernels (cfr.cu, cfr_iter.cu): a thread's slice of a
// [node][combo] row, row prefetch, the fp64 unblocked-mass formula and the row sum in the
// association order of the CPU reduction the upstream normalisation runs through.
#pragma once

#include "cfr.cuh"

namespace p2b {
namespace {

// VPT consecutive hands of one row
template <int VPT>
struct FV {
    float v[VPT];
};

static_assert(P2B_HPAD == 1344, "rows are covered exactly by 672 x 2 or 336 x 4 hands");

template <int VPT>
__device__ __forceinline__ FV<VPT> ldv(const float* row, int tid) {
    FV<VPT> r;
    if (VPT == 4) {
        const float4 t = *reinterpret_cast<const float4*>(row + 4 * tid);
        r.v[0] = t.x; r.v[1] = t.y; r.v[VPT - 2] = t.z; r.v[VPT - 1] = t.w;
    } else {
        const float2 t = *reinterpret_cast<const float2*>(row + 2 * tid);
        r.v[0] = t.x; r.v[1] = t.y;
    }
    return r;
}
template <int VPT>
__device__ __forceinline__ void stv(float* row, int tid, const FV<VPT>& r) {
    if (VPT == 4) *reinterpret_cast<float4*>(row + 4 * tid) = make_float4(r.v[0], r.v[1], r.v[VPT - 2], r.v[VPT - 1]);
    else *reinterpret_cast<float2*>(row + 2 * tid) = make_float2(r.v[0], r.v[1]);
}

// Hint that this thread's slice of a row will be read soon: pulls the line into L2.
template <int VPT>
__device__ __forceinline__ void prefetch_row(const float* row, int tid) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(row + VPT * tid));
}
// The same for the n (<= kCfrMaxChildren) consecutive rows that start at `row` (the rows of the
// children of one node): one address computation, fixed offsets.
template <int VPT>
__device__ __forceinline__ void prefetch_rows(const float* row, int n, int tid) {
    const float* mine = row + VPT * tid;
#pragma unroll
    for (int c = 0; c < kCfrMaxChildren; ++c)
        if (c < n) asm volatile("prefetch.global.L2 [%0];" ::"l"(mine + c * P2B_HPAD));
}

// x[which] without indexing a register array by a run-time value
template <int VPT>
__device__ __forceinline__ FV<VPT> pick(const FV<VPT> (&x)[2], int which) {
    FV<VPT> r;
#pragma unroll
    for (int i = 0; i < VPT; ++i) r.v[i] = which ? x[1].v[i] : x[0].v[i];
    return r;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// Mass of the hands that share no card with (c1,c2): total - card sums + own mass,
// evaluated in fp64, rounded to fp32 and clamped at zero (p2/env/card_utils.py:196-222).
__device__ __forceinline__ float unblocked(const double* cs, double S, int c1, int c2, float x) {
    const double m = S - cs[c1] - cs[c2] + (double)x;
    return fmaxf((float)m, 0.0f);
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

template <int VPT>
struct HandInfo {
    int c1[VPT], c2[VPT];
    bool valid[VPT];    // a real combo (not row padding)
    bool allowed[VPT];  // and not blocked by the board of the current subgame
};

template <int VPT>
struct CfrThreads {
    static constexpr int value = P2B_HPAD / VPT;  // 672 threads for two hands per thread, 336 for four
};

}  // namespace
}  // namespace p2b
