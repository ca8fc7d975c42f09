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
        // the form with the min/max guard (the iteration kernel); a non-negative numerator in its own convention
        DivGuard gd = guard_begin(d.ok);
        float g3 = div_g<false>(x, d.y, d.r, gd);
        if (guard_bad(gd)) g3 = want;
        if (__float_as_uint(g3) != __float_as_uint(want) && !both_nan) ++bad;
        if (__float_as_uint(x) < 0x80000000u) {  // +0 or positive (NaN patterns included: reported by the guard)
            DivGuard gn = guard_begin(d.ok);
            float g4 = div_g<true>(x, d.y, d.r, gn);
            if (guard_bad(gn)) g4 = want;
            if (__float_as_uint(g4) != __float_as_uint(want) && !both_nan) ++bad;
        }
        const uint32_t ax = __float_as_uint(x) & 0x7fffffffu;
        if (d.ok && (exactdiv_in_range(ax) || ax == 0u)) ++fast;
    }
    if (bad) atomicAdd(mismatches, bad);
    if (fast) atomicAdd(short_path, fast);
}

// Directed sweep: every one of the 2^23 divisor mantissas at a few exponents (the ends of the valid
// range, around 1, and two in between), each against numerators chosen to sit on rounding
// boundaries: 1, the largest mantissa, the divisor one ulp up and down, the divisor's mantissa
// mirrored, and pseudo-random ones.  All three forms of the short sequence must give the bits of the
// IEEE division.
__global__ void division_sweep_kernel(unsigned long long* mismatches, unsigned long long* checked) {
    const uint32_t exps[5] = {67u, 100u, 127u, 150u, 186u};
    unsigned long long bad = 0, n = 0;
    for (uint32_t m = blockIdx.x * blockDim.x + threadIdx.x; m < (1u << 23); m += gridDim.x * blockDim.x) {
#pragma unroll 1
        for (int ei = 0; ei < 5; ++ei) {
            const uint32_t yb = (exps[ei] << 23) | m;
            const float y = __uint_as_float(yb);
            const Divisor d = make_divisor(y);
#pragma unroll 1
            for (int k = 0; k < 16; ++k) {
                uint32_t xb;
                switch (k) {
                    case 0: xb = 127u << 23; break;
                    case 1: xb = (127u << 23) | 0x7fffffu; break;
                    case 2: xb = yb + 1u; break;
                    case 3: xb = yb - 1u; break;
                    case 4: xb = (exps[ei] << 23) | (0x7fffffu - m); break;
                    case 5: xb = (exps[(ei + 1) % 5] << 23) | m; break;
                    default: xb = confine(scramble(((uint64_t)m << 8) + ei * 16 + k), 67, 120) & 0x7fffffffu; break;
                }
                const float x = (k & 1) && k > 5 ? -__uint_as_float(xb) : __uint_as_float(xb);
                const float want = __fdiv_rn(x, y);
                const float g0 = div_exact(x, d);
                bool redo = false;
                float g1 = div_fast(x, d, redo);
                if (redo) g1 = want;
                DivGuard g = guard_begin(d.ok);
                float g2 = div_g<false>(x, d.y, d.r, g);
                if (guard_bad(g)) g2 = want;
                float g3 = want;
                if (x >= 0.0f) {
                    DivGuard gn = guard_begin(d.ok);
                    g3 = div_g<true>(x, d.y, d.r, gn);
                    if (guard_bad(gn)) g3 = want;
                }
                const uint32_t w = __float_as_uint(want);
                bad += (__float_as_uint(g0) != w) + (__float_as_uint(g1) != w) + (__float_as_uint(g2) != w) +
                       (__float_as_uint(g3) != w);
                ++n;
            }
        }
    }
    if (bad) atomicAdd(mismatches, bad);
    atomicAdd(checked, n);
}

}  // namespace
}  // namespace p2b

extern "C" int p2b_selftest_division_sweep(unsigned long long* mismatches, unsigned long long* checked, void* stream) {
    using namespace p2b;
    if (!mismatches || !checked) return set_error(P2B_ERR_ARG, "p2b_selftest_division_sweep: null pointer");
    division_sweep_kernel<<<148 * 8, 256, 0, (cudaStream_t)stream>>>(mismatches, checked);
    return check_cuda(cudaGetLastError(), "division_sweep_kernel");
}

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
