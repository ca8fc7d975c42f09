// Device self-test of the shared-divisor division (exactdiv.cuh) against the compiler's
// correctly rounded division, on generated operand pairs.
#include "../../include/poker2_b200.h"

#include "common.cuh"
#include "exactdiv.cuh"

namespace p2b {
namespace {

__device__ __forceinline__ uint32_t scramble(uint64_t z) {  // splitmix64 finaliser, upper bits
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return (uint32_t)((z ^ (z >> 31)) >> 16);
}

// exponent field moved into [lo, lo+span)
__device__ __forceinline__ uint32_t confine(uint32_t bits, uint32_t lo, uint32_t span) {
    return (bits & 0x807fffffu) | ((lo + (bits >> 23) % span) << 23);
}

// Pair `id` of the stream `seed`.  Seven families: raw bit patterns (zeros, denormals,
// infinities and NaNs included); divisor inside the valid range; both inside; both near 1;
// divisors with extreme mantissas; signed zero numerators; quotients near 2^-10.
__device__ __forceinline__ void operand_pair(uint64_t id, uint32_t seed, float& x, float& y) {
    uint32_t yb = scramble(id * 2 + seed), xb = scramble(id * 2 + 1 + (uint64_t)seed * 77u);
    switch (id % 7) {
        case 1: yb = confine(yb, 67, 120); break;
        case 2: yb = confine(yb, 67, 120); xb = confine(xb, 67, 120); break;
        case 3: yb = confine(yb, 100, 50); xb = confine(xb, 100, 50); break;
        case 4:
            yb = (yb & 0xff800000u) | ((yb & 1u) ? 0x7fffffu : ((yb & 2u) ? 0u : 1u));
            yb = confine(yb, 67, 120);
            xb = confine(xb, 67, 120);
            break;
        case 5:
            if (xb & 3u) xb &= 0x80000000u;
            yb = confine(yb, 67, 120);
            break;
        case 6: yb = confine(yb, 120, 14); xb = confine(xb, 110, 20); break;
        default: break;
    }
    x = __uint_as_float(xb);
    y = __uint_as_float(yb);
}

__global__ void division_selftest_kernel(uint64_t pairs_per_thread, uint32_t seed, unsigned long long* mismatches,
                                         unsigned long long* short_path) {
    const uint64_t t = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    unsigned long long bad = 0, fast = 0;
    for (uint64_t i = 0; i < pairs_per_thread; ++i) {
        float x, y;
        operand_pair(t * pairs_per_thread + i, seed, x, y);
        const Divisor d = make_divisor(y);
        const float got = div_exact(x, d), want = __fdiv_rn(x, y);
        const bool both_nan = (got != got) && (want != want);
        if (__float_as_uint(got) != __float_as_uint(want) && !both_nan) ++bad;
        // the grouped form the solver uses: branch-free quotient, one fallback for the group
        // (a group of one here), in both numerator conventions
        bool redo = false, redo_nn = false;
        float g1 = div_fast(x, d, redo), g2 = div_fast<true>(x, d, redo_nn);
        if (redo) g1 = want;
        if (redo_nn) g2 = want;
        if (__float_as_uint(g1) != __float_as_uint(want) && !both_nan) ++bad;
        if (__float_as_uint(g2) != __float_as_uint(want) && !both_nan) ++bad;
        const uint32_t ax = __float_as_uint(x) & 0x7fffffffu;
        if (d.ok && (exactdiv_in_range(ax) || ax == 0u)) ++fast;
    }
    if (bad) atomicAdd(mismatches, bad);
    if (fast) atomicAdd(short_path, fast);
}

}  // namespace
}  // namespace p2b

extern "C" int p2b_selftest_division(uint64_t num_pairs, uint32_t seed, unsigned long long* mismatches,
                                     unsigned long long* short_path, void* stream) {
    using namespace p2b;
    if (!mismatches || !short_path) return set_error(P2B_ERR_ARG, "p2b_selftest_division: null pointer");
    constexpr int kBlocks = 148 * 8, kThreads = 256;
    const uint64_t threads = (uint64_t)kBlocks * kThreads;
    const uint64_t per_thread = (num_pairs + threads - 1) / threads;
    if (per_thread == 0) return P2B_OK;
    division_selftest_kernel<<<kBlocks, kThreads, 0, (cudaStream_t)stream>>>(per_thread, seed, mismatches, short_path);
    return check_cuda(cudaGetLastError(), "division_selftest_kernel");
}
