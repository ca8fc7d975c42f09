// Step-level kernels: one kernel per step of the CFR iteration, on caller-owned tensors in
// the upstream node order.  They mirror, one for one, the fused kernels of
// p2/search/fused_cfr_triton.py (cited per kernel) so that an evaluator written against
// that module can switch to this library step by step.  The whole-subgame kernel in
// cfr.cu is the fast path; these exist for drop-in compatibility.  Scalars that depend on
// the iteration number are read from device memory (as upstream's TScalars do).
#include "cfr_dev.cuh"
#include "common.cuh"
#include "exactdiv.cuh"

namespace p2b {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ double block_sum(double v, double* red) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double s = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[w];
    return s;
}

inline int blocks_for(long long n, int cap) {
    long long g = (n + kThreads - 1) / kThreads;
    if (g < 1) g = 1;
    if (g > cap) g = cap;
    return (int)g;
}

// fused_cfr_triton.py:72-121 (_fused_dcfr_update_kernel).  VEC: all arrays 16-byte aligned, four
// elements per thread and iteration (the tail is done one by one).
struct DcfrScalars {
    float an, bn;
    Divisor da, db;  // the two divisors are the same for every element (exactdiv.cuh)
};
__device__ __forceinline__ void dcfr_update_one(float& c, float& w, float reg, const DcfrScalars& k, int apply_dcfr,
                                                int cfr_plus) {
    if (apply_dcfr) {
        const bool pos = c > 0.0f;
        const float num = pos ? k.an : k.bn;
        Divisor d;
        d.y = pos ? k.da.y : k.db.y;
        d.r = pos ? k.da.r : k.db.r;
        d.ok = k.da.ok && k.db.ok;
        c = div_exact(__fmul_rn(c, num), d);
        w = div_exact(__fmul_rn(w, num), d);
    }
    w = __fadd_rn(w, 1.0f);
    c = __fadd_rn(c, reg);
    if (cfr_plus) c = fmaxf(c, 0.0f);
}

template <bool VEC>
__global__ void dcfr_update_kernel(const float* __restrict__ regrets, float* __restrict__ cumul,
                                   float* __restrict__ weights, float* __restrict__ pos_out,
                                   const float* __restrict__ scal /* a_num,b_num,a_den,b_den */, long long n,
                                   int apply_dcfr, int cfr_plus) {
    DcfrScalars k;
    k.an = scal[0];
    k.bn = scal[1];
    k.da = make_divisor(scal[2]);
    k.db = make_divisor(scal[3]);
    const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x, nthreads = (long long)gridDim.x * blockDim.x;
    long long done = 0;
    if (VEC) {
        const long long n4 = n >> 2;
        for (long long i = tid; i < n4; i += nthreads) {
            float4 c = reinterpret_cast<float4*>(cumul)[i], w = reinterpret_cast<float4*>(weights)[i];
            const float4 r = reinterpret_cast<const float4*>(regrets)[i];
            dcfr_update_one(c.x, w.x, r.x, k, apply_dcfr, cfr_plus);
            dcfr_update_one(c.y, w.y, r.y, k, apply_dcfr, cfr_plus);
            dcfr_update_one(c.z, w.z, r.z, k, apply_dcfr, cfr_plus);
            dcfr_update_one(c.w, w.w, r.w, k, apply_dcfr, cfr_plus);
            reinterpret_cast<float4*>(cumul)[i] = c;
            reinterpret_cast<float4*>(weights)[i] = w;
            if (pos_out)
                reinterpret_cast<float4*>(pos_out)[i] = make_float4(fmaxf(c.x, 0.0f), fmaxf(c.y, 0.0f), fmaxf(c.z, 0.0f), fmaxf(c.w, 0.0f));
        }
        done = n4 << 2;
    }
    for (long long i = done + tid; i < n; i += nthreads) {
        float c = cumul[i], w = weights[i];
        dcfr_update_one(c, w, regrets[i], k, apply_dcfr, cfr_plus);
        cumul[i] = c;
        weights[i] = w;
        if (pos_out) pos_out[i] = fmaxf(c, 0.0f);
    }
}

// fused_cfr_triton.py:246-284 (_fused_block_normalize_kernel): one block per row
__global__ void block_normalize_kernel(float* __restrict__ target, const unsigned char* __restrict__ allowed,
                                       const float* __restrict__ allowed_prob, long long rows, int outer_stride, int H,
                                       float eps) {
    __shared__ double red[kThreads / 32];
    __shared__ float srow[P2B_HPAD];
    __shared__ float s_total;
    constexpr int kPer = 6;  // 256 threads x 6 cover rows of up to 1536 entries in registers
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const long long outer = row / outer_stride;
        float* t = target + row * H;
        const unsigned char* m = allowed + outer * H;
        if (H <= kPer * kThreads) {
            float v[kPer];
            double s = 0.0;
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const int h = threadIdx.x + i * kThreads;
                v[i] = (h < H && m[h]) ? t[h] : 0.0f;
                s += (double)v[i];
            }
            float total;
            if (H == P2B_NUM_HANDS) {
                // a row of 1326 hands is summed in fp32 in the order of the upstream CPU reduction
                // (cfr_evaluator.py:263-273 through torch.sum), so the quotients carry its bits
#pragma unroll
                for (int i = 0; i < kPer; ++i) {
                    const int h = threadIdx.x + i * kThreads;
                    if (h < H) srow[h] = v[i];
                }
                __syncthreads();
                if (threadIdx.x < 32) {
                    const float r = row_sum_reference_order(srow);
                    if (threadIdx.x == 0) s_total = r;
                }
                __syncthreads();
                total = s_total;
            } else {
                total = (float)block_sum(s, red);
            }
            const Divisor d = make_divisor(total);
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const int h = threadIdx.x + i * kThreads;
                if (h < H) t[h] = total > eps ? div_exact(v[i], d) : allowed_prob[outer * H + h];
            }
            continue;
        }
        double s = 0.0;
        for (int h = threadIdx.x; h < H; h += blockDim.x) {
            const float v = m[h] ? t[h] : 0.0f;
            t[h] = v;
            s += (double)v;
        }
        const float total = (float)block_sum(s, red);
        for (int h = threadIdx.x; h < H; h += blockDim.x)
            t[h] = total > eps ? __fdiv_rn(t[h], total) : allowed_prob[outer * H + h];
    }
}

// fused_cfr_triton.py:346-367 (_fused_regret_matching_divide_kernel)
__global__ void regret_matching_divide_kernel(const float* __restrict__ pos, const float* __restrict__ den,
                                              const float* __restrict__ uniform, float* __restrict__ out, long long n,
                                              float eps) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float d = den[i];
        out[i] = d > eps ? __fdiv_rn(pos[i], fmaxf(d, eps)) : uniform[i];
    }
}

// fused_cfr_triton.py:410-436 (_fused_weight_child_values_kernel)
__global__ void weight_child_values_kernel(const float* __restrict__ values, const long long* __restrict__ prev_actor,
                                           const float* __restrict__ pol_hero, const float* __restrict__ pol_opp,
                                           float* __restrict__ out, long long M, int H) {
    const long long n = M * 2 * H;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / (2 * H);
        const int p = (int)((i / H) & 1), h = (int)(i % H);
        const float pol = (p == (int)prev_actor[m]) ? pol_hero[m * H + h] : pol_opp[m * H + h];
        out[i] = __fmul_rn(values[i], pol);
    }
}

// fused_cfr_triton.py:488-507 (_fused_update_average_values_kernel)
__global__ void update_average_values_kernel(float* __restrict__ avg, const float* __restrict__ latest,
                                             const float* __restrict__ old_p, const float* __restrict__ new_p,
                                             const float* __restrict__ inv_p, long long n) {
    const float o = *old_p, w = *new_p, inv = *inv_p;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        avg[i] = __fmul_rn(__fadd_rn(__fmul_rn(avg[i], o), __fmul_rn(latest[i], w)), inv);
}

// fused_cfr_triton.py:572-621 (_fused_avg_values_zs_kernel) and :1692-1737
// (_fused_model_values_mix_zs_kernel): out = a*ca (+|-) b*cb [* scale], then the zero-sum shift
// 0.5 * sum_p sum_h out_p * belief_p.  One block per row of [2,H].
__global__ void mix_zero_sum_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                    const float* __restrict__ beliefs, const unsigned char* __restrict__ ignore,
                                    const float* __restrict__ ca_p, const float* __restrict__ cb_p,
                                    const float* __restrict__ scale_p, float* __restrict__ out, long long rows, int H,
                                    int subtract_b, int enforce_zs) {
    __shared__ double red[kThreads / 32];
    // enforce_zs == 2 (H == 1326 only): the two sums over hands run in fp32 in the order of the CPU row
    // reduction the non-fused upstream code goes through (cfr_evaluator.py:973-976), then their mean
    __shared__ float prod[2][P2B_HPAD];
    __shared__ float rsum[2];
    const float ca = *ca_p, cb = *cb_p, sc = scale_p ? *scale_p : 1.0f;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const long long base = row * 2 * H;
        double s = 0.0;
        for (int i = threadIdx.x; i < 2 * H; i += blockDim.x) {
            const float x = __fmul_rn(a[base + i], ca), y = __fmul_rn(b[base + i], cb);
            float v = (subtract_b & 1) ? __fsub_rn(x, y) : __fadd_rn(x, y);
            if (scale_p) v = (subtract_b & 2) ? __fdiv_rn(v, sc) : __fmul_rn(v, sc);
            out[base + i] = v;
            if (enforce_zs == 1) s += (double)__fmul_rn(v, beliefs[base + i]);
            if (enforce_zs == 2) prod[i >= H][i >= H ? i - H : i] = __fmul_rn(v, beliefs[base + i]);
        }
        if (enforce_zs) {  // uniform branch: all threads take it
            float shift;
            if (enforce_zs == 2) {
                __syncthreads();
                const int warp = threadIdx.x >> 5;
                if (warp < 2) {
                    const float t = row_sum_reference_order(prod[warp]);
                    if ((threadIdx.x & 31) == 0) rsum[warp] = t;
                }
                __syncthreads();
                shift = __fmul_rn(__fadd_rn(rsum[0], rsum[1]), 0.5f);
            } else {
                shift = 0.5f * (float)block_sum(s, red);
            }
            if (ignore && ignore[row]) shift = 0.0f;
            for (int i = threadIdx.x; i < 2 * H; i += blockDim.x) out[base + i] = __fsub_rn(out[base + i], shift);
            __syncthreads();
        }
    }
}

// fused_cfr_triton.py:679-710 (_fused_regret_tail_kernel)
__global__ void regret_tail_kernel(const float* __restrict__ achieved, const float* __restrict__ actor_values,
                                   const float* __restrict__ src_weights, const long long* __restrict__ parent_index,
                                   const long long* __restrict__ prev_actor, float* __restrict__ regrets,
                                   long long bottom, long long total, int H) {
    const long long n = (total - bottom) * H;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long c = bottom + i / H;
        const int h = (int)(i % H);
        const long long par = parent_index[c];
        const float ach = achieved[(c * 2 + prev_actor[c]) * H + h];
        regrets[c * H + h] = __fmul_rn(src_weights[par * H + h], __fsub_rn(ach, actor_values[par * H + h]));
    }
}

// fused_cfr_triton.py:777-821 (_fused_average_policy_mix_kernel)
__global__ void average_policy_mix_kernel(const float* __restrict__ reach, const float* __restrict__ reach_avg,
                                          const float* __restrict__ policy, float* __restrict__ policy_avg,
                                          const long long* __restrict__ to_act, const long long* __restrict__ parent_index,
                                          const float* __restrict__ old_p, const float* __restrict__ new_p,
                                          const float* __restrict__ tot_p, long long bottom, long long total, int H,
                                          float eps) {
    const float o = *old_p, w = *new_p, tot = *tot_p;
    const long long n = (total - bottom) * H;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long c = bottom + i / H;
        const int h = (int)(i % H);
        const long long par = parent_index[c], row = (par * 2 + to_act[par]) * H + h;
        const float ra = __fmul_rn(reach_avg[row], o), rn = __fmul_rn(reach[row], w);
        const float avg = policy_avg[c * H + h], cur = policy[c * H + h];
        const float den = __fadd_rn(ra, rn);
        policy_avg[c * H + h] = den > eps ? __fdiv_rn(__fadd_rn(__fmul_rn(ra, avg), __fmul_rn(rn, cur)), den)
                                          : __fdiv_rn(__fadd_rn(__fmul_rn(o, avg), __fmul_rn(w, cur)), tot);
    }
}

// fused_cfr_triton.py:1210-1239 (_parent_sum_kernel) and :1168-1205 (_sibling_sum_kernel):
// broadcast = 0 writes one row per parent, = 1 one row per child (relative to out_offset).
__global__ void parent_sum_kernel(const float* __restrict__ values, const long long* __restrict__ child_offsets,
                                  const long long* __restrict__ child_count, float* __restrict__ out,
                                  long long num_parents, int H, int broadcast, long long out_offset) {
    const long long n = num_parents * H;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long p = i / H;
        const int h = (int)(i % H);
        const long long first = child_offsets[p], cnt = child_count[p];
        float acc = 0.0f;
        for (long long k = 0; k < cnt; ++k) acc = __fadd_rn(acc, values[(first + k) * H + h]);
        if (!broadcast) out[p * H + h] = acc;
        else
            for (long long k = 0; k < cnt; ++k) out[(first + k - out_offset) * H + h] = acc;
    }
}

// fused_cfr_triton.py:1241-1277 (_fused_divide_by_parent_sum_kernel)
__global__ void divide_by_parent_sum_kernel(const float* __restrict__ pos, const float* __restrict__ fallback,
                                            const float* __restrict__ parent_sum, const long long* __restrict__ parent_index,
                                            float* __restrict__ out, long long num_children, int H, float eps) {
    const long long n = num_children * H;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long c = i / H;
        const int h = (int)(i % H);
        const float d = parent_sum[parent_index[c] * H + h];
        const float f = fallback[i], pv = pos[i];
        out[i] = d > eps ? __fdiv_rn(pv, fmaxf(d, eps)) : f;
    }
}

// out = a*ca - b*cb (fused_cfr_triton.py:1613-1631, _fused_model_values_mix_kernel)
__global__ void scaled_difference_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                         const float* __restrict__ ca_p, const float* __restrict__ cb_p,
                                         float* __restrict__ out, long long n) {
    const float ca = *ca_p, cb = *cb_p;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = __fsub_rn(__fmul_rn(ca, a[i]), __fmul_rn(cb, b[i]));
}

// Hands holding each card, in combo order: nat[c*51 + i] = combo index of (c, i-th other card).
constexpr int kNatEntries = P2B_NUM_CARDS * 51;
__device__ __forceinline__ void fill_card_hand_table(uint16_t* nat) {
    for (int idx = threadIdx.x; idx < kNatEntries; idx += blockDim.x) {
        const int c = idx / 51, i = idx % 51, d = i < c ? i : i + 1;
        nat[idx] = (uint16_t)(c < d ? combo_index(c, d) : combo_index(d, c));
    }
}

constexpr int kRowRegs = (P2B_NUM_HANDS + kThreads - 1) / kThreads;  // 6 values per thread cover a row

// This thread's share of a 1326-combo row, from global memory into registers.
__device__ __forceinline__ void load_row_regs(const float* __restrict__ x, float (&v)[kRowRegs]) {
#pragma unroll
    for (int i = 0; i < kRowRegs; ++i) {
        const int h = threadIdx.x + i * kThreads;
        v[i] = h < P2B_NUM_HANDS ? x[h] : 0.0f;
    }
}

// Puts a row held in registers into shared memory, then computes its per-card sums (four
// threads per card, each a quarter of the 51 hands holding it) and its total, all in fp64; cs
// must hold 52 doubles, xs 1326 floats, nat the table above.  Returns the total.
__device__ __forceinline__ double row_card_sums(const float (&v)[kRowRegs], float* __restrict__ xs,
                                                const uint16_t* __restrict__ nat, double* cs, double* red) {
    __syncthreads();  // previous users of xs / cs are done
    double tot = 0.0;
#pragma unroll
    for (int i = 0; i < kRowRegs; ++i) {
        const int h = threadIdx.x + i * kThreads;
        if (h < P2B_NUM_HANDS) xs[h] = v[i];
        tot += (double)v[i];
    }
    const double S = block_sum(tot, red);  // contains the barriers that publish xs
    if (threadIdx.x < 224) {
        const int t = threadIdx.x < 208 ? threadIdx.x : 207, c = t >> 2, q = t & 3;
        // entries q, q+4, ..., q+48 of the card's list; only the last one can fall outside (q = 3)
        const uint16_t* idx = nat + c * 51 + q;
        float g[13];
#pragma unroll
        for (int i = 0; i < 12; ++i) g[i] = xs[idx[4 * i]];
        g[12] = q < 3 ? xs[idx[48]] : 0.0f;
        double s = 0.0;
#pragma unroll
        for (int i = 0; i < 13; ++i) s += (double)g[i];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if (threadIdx.x < 208 && q == 0) cs[c] = s;
    }
    __syncthreads();
    return S;
}

__device__ __forceinline__ float unblocked_value(const double* cs, double S, int c1, int c2, float x) {
    return fmaxf((float)(S - cs[c1] - cs[c2] + (double)x), 0.0f);
}

// unblocked mass of gathered rows: out[r] = U(src + row_index[r]*1326) (row_index null = r).
// fused_cfr_triton.py:929-960 with the S/card-sum preprocessing of :1008-1026 done in-kernel.
__global__ void unblocked_mass_kernel(const float* __restrict__ src, const long long* __restrict__ row_index,
                                      const ComboTable* __restrict__ combos, float* __restrict__ out, long long rows) {
    __shared__ double cs[P2B_NUM_CARDS];
    __shared__ double red[kThreads / 32];
    __shared__ float xs[P2B_NUM_HANDS];
    __shared__ uint16_t nat[kNatEntries];
    __shared__ unsigned char c1s[P2B_NUM_HANDS], c2s[P2B_NUM_HANDS];
    fill_card_hand_table(nat);
    for (int h = threadIdx.x; h < P2B_NUM_HANDS; h += blockDim.x) {
        c1s[h] = combos->c1[h];
        c2s[h] = combos->c2[h];
    }
    // the next row is fetched into registers while the current one is processed
    float cur[kRowRegs], nxt[kRowRegs];
    if (blockIdx.x < rows) load_row_regs(src + (row_index ? row_index[blockIdx.x] : (long long)blockIdx.x) * P2B_NUM_HANDS, cur);
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
        const long long rn = r + gridDim.x;
        if (rn < rows) load_row_regs(src + (row_index ? row_index[rn] : rn) * P2B_NUM_HANDS, nxt);
        const double S = row_card_sums(cur, xs, nat, cs, red);
#pragma unroll
        for (int i = 0; i < kRowRegs; ++i) {
            const int h = threadIdx.x + i * kThreads;
            if (h < P2B_NUM_HANDS) out[r * P2B_NUM_HANDS + h] = unblocked_value(cs, S, c1s[h], c2s[h], cur[i]);
        }
#pragma unroll
        for (int i = 0; i < kRowRegs; ++i) cur[i] = nxt[i];
    }
}

// ratio U(numer[c]) / U(denom[parent(c)]), 0 where the denominator is <= eps
// (fused_cfr_triton.py:1409-1497; parent_index null = denominator row c)
__global__ void unblocked_ratio_kernel(const float* __restrict__ numer, const float* __restrict__ denom,
                                       const long long* __restrict__ parent_index,
                                       const ComboTable* __restrict__ combos, float* __restrict__ out,
                                       long long rows, float eps) {
    __shared__ double cs_n[P2B_NUM_CARDS], cs_d[P2B_NUM_CARDS];
    __shared__ double red[kThreads / 32];
    __shared__ float xn_s[P2B_NUM_HANDS], xd_s[P2B_NUM_HANDS];
    __shared__ uint16_t nat[kNatEntries];
    __shared__ unsigned char c1s[P2B_NUM_HANDS], c2s[P2B_NUM_HANDS];
    fill_card_hand_table(nat);
    for (int h = threadIdx.x; h < P2B_NUM_HANDS; h += blockDim.x) {
        c1s[h] = combos->c1[h];
        c2s[h] = combos->c2[h];
    }
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xn = numer + r * P2B_NUM_HANDS;
        const float* xd = denom + (parent_index ? parent_index[r] : r) * P2B_NUM_HANDS;
        float vn[kRowRegs], vd[kRowRegs];
        load_row_regs(xn, vn);
        load_row_regs(xd, vd);
        const double Sn = row_card_sums(vn, xn_s, nat, cs_n, red);
        const double Sd = row_card_sums(vd, xd_s, nat, cs_d, red);
        for (int h = threadIdx.x; h < P2B_NUM_HANDS; h += blockDim.x) {
            const int c1 = c1s[h], c2 = c2s[h];
            const float n = unblocked_value(cs_n, Sn, c1, c2, xn_s[h]), d = unblocked_value(cs_d, Sd, c1, c2, xd_s[h]);
            out[r * P2B_NUM_HANDS + h] = d > eps ? __fdiv_rn(n, d) : 0.0f;
        }
    }
}

// fused_cfr_triton.py:1788-1836 (_fused_weighted_parent_sum_kernel)
__global__ void weighted_parent_sum_kernel(float* __restrict__ values, const long long* __restrict__ prev_actor,
                                           const float* __restrict__ pol_hero, const float* __restrict__ pol_opp,
                                           const long long* __restrict__ child_offsets,
                                           const long long* __restrict__ child_count, long long parent_base,
                                           long long num_parents, int H) {
    const long long n = num_parents * 2 * H;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long p = i / (2 * H);
        const int player = (int)((i / H) & 1), h = (int)(i % H);
        const long long first = child_offsets[p], cnt = child_count[p];
        if (cnt == 0) continue;
        float acc = 0.0f;
        for (long long k = 0; k < cnt; ++k) {
            const long long ch = first + k;
            const float pol = ((int)prev_actor[ch] == player) ? pol_hero[ch * H + h] : pol_opp[ch * H + h];
            acc = __fadd_rn(acc, __fmul_rn(values[(ch * 2 + player) * H + h], pol));
        }
        values[((parent_base + p) * 2 + player) * H + h] = acc;
    }
}

// fused_cfr_triton.py:1901-1942 (_fused_reach_weights_kernel)
__global__ void reach_weights_kernel(float* __restrict__ reach, const float* __restrict__ policy,
                                     const unsigned char* __restrict__ allowed, const long long* __restrict__ parent_index,
                                     const long long* __restrict__ prev_actor, long long start, long long end, int H) {
    const long long n = (end - start) * H;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long c = start + i / H;
        const int h = (int)(i % H);
        const long long par = parent_index[c];
        float v0 = reach[(par * 2 + 0) * H + h], v1 = reach[(par * 2 + 1) * H + h];
        const float pol = policy[c * H + h];
        if (prev_actor[c] == 0) v0 = __fmul_rn(v0, pol);
        else v1 = __fmul_rn(v1, pol);
        const bool ok = allowed[c * H + h] != 0;
        reach[(c * 2 + 0) * H + h] = ok ? v0 : 0.0f;
        reach[(c * 2 + 1) * H + h] = ok ? v1 : 0.0f;
    }
}

// fused_cfr_triton.py:1997-2037 (_fused_deep_beliefs_kernel): one block per (node, player)
__global__ void deep_beliefs_kernel(float* __restrict__ out, const float* __restrict__ root_beliefs,
                                    const float* __restrict__ reach, const float* __restrict__ allowed_prob,
                                    const long long* __restrict__ root_index, long long num_roots, long long total,
                                    int H, float eps) {
    __shared__ double red[kThreads / 32];
    __shared__ float srow[P2B_HPAD];
    __shared__ float s_total;
    const long long rows = (total - num_roots) * 2;
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
        const long long node = num_roots + r / 2;
        const int p = (int)(r & 1);
        const float* rb = root_beliefs + (root_index[node] * 2 + p) * H;
        const float* rw = reach + (node * 2 + p) * H;
        float* o = out + (node * 2 + p) * H;
        float tot;
        if (H == P2B_NUM_HANDS) {  // fp32 sum in the order of the upstream CPU reduction, as in block_normalize_kernel
            __syncthreads();       // the previous row's sum has been read
            for (int h = threadIdx.x; h < H; h += blockDim.x) srow[h] = __fmul_rn(rb[h], rw[h]);
            __syncthreads();
            if (threadIdx.x < 32) {
                const float v = row_sum_reference_order(srow);
                if (threadIdx.x == 0) s_total = v;
            }
            __syncthreads();
            tot = s_total;
        } else {
            double s = 0.0;
            for (int h = threadIdx.x; h < H; h += blockDim.x) s += (double)__fmul_rn(rb[h], rw[h]);
            tot = (float)block_sum(s, red);
        }
        for (int h = threadIdx.x; h < H; h += blockDim.x)
            o[h] = tot > eps ? __fdiv_rn(__fmul_rn(rb[h], rw[h]), tot) : allowed_prob[node * H + h];
    }
}

}  // namespace

int sm_count();

}  // namespace p2b

using namespace p2b;

#define STEP_CHECK(name) return check_cuda(cudaGetLastError(), name)
#define GRID_ELEMS(n) blocks_for((n), sm_count() * 16)
#define GRID_ROWS(r) ((int)((r) < (long long)sm_count() * 8 ? ((r) > 0 ? (r) : 1) : (long long)sm_count() * 8))

extern "C" {

int p2b_step_dcfr_update(const float* regrets, float* cumulative, float* weight_sums, float* positive_out,
                         const float* scalars4, int64_t n, int apply_dcfr, int cfr_plus, void* stream) {
    if (n <= 0) return P2B_OK;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(regrets) | reinterpret_cast<uintptr_t>(cumulative) |
                           reinterpret_cast<uintptr_t>(weight_sums) | reinterpret_cast<uintptr_t>(positive_out);
    if ((bits & 15) == 0)
        dcfr_update_kernel<true><<<GRID_ELEMS((n + 3) / 4), kThreads, 0, (cudaStream_t)stream>>>(
            regrets, cumulative, weight_sums, positive_out, scalars4, n, apply_dcfr, cfr_plus);
    else
        dcfr_update_kernel<false><<<GRID_ELEMS(n), kThreads, 0, (cudaStream_t)stream>>>(
            regrets, cumulative, weight_sums, positive_out, scalars4, n, apply_dcfr, cfr_plus);
    STEP_CHECK("dcfr_update_kernel");
}

int p2b_step_block_normalize(float* target, const uint8_t* allowed, const float* allowed_prob, int64_t rows,
                             int32_t rows_per_outer, int32_t H, float eps, void* stream) {
    if (rows <= 0) return P2B_OK;
    block_normalize_kernel<<<GRID_ROWS(rows), kThreads, 0, (cudaStream_t)stream>>>(target, allowed, allowed_prob, rows,
                                                                                  rows_per_outer, H, eps);
    STEP_CHECK("block_normalize_kernel");
}

int p2b_step_regret_matching_divide(const float* positive, const float* denom, const float* uniform, float* out,
                                    int64_t n, float eps, void* stream) {
    if (n <= 0) return P2B_OK;
    regret_matching_divide_kernel<<<GRID_ELEMS(n), kThreads, 0, (cudaStream_t)stream>>>(positive, denom, uniform, out, n, eps);
    STEP_CHECK("regret_matching_divide_kernel");
}

int p2b_step_weight_child_values(const float* values, const int64_t* prev_actor, const float* policy_hero,
                                 const float* policy_opp, float* out, int64_t M, int32_t H, void* stream) {
    if (M <= 0) return P2B_OK;
    weight_child_values_kernel<<<GRID_ELEMS(M * 2 * H), kThreads, 0, (cudaStream_t)stream>>>(
        values, (const long long*)prev_actor, policy_hero, policy_opp, out, M, H);
    STEP_CHECK("weight_child_values_kernel");
}

int p2b_step_update_average_values(float* values_avg, const float* latest, const float* old_w, const float* new_w,
                                   const float* inv_total, int64_t n, void* stream) {
    if (n <= 0) return P2B_OK;
    update_average_values_kernel<<<GRID_ELEMS(n), kThreads, 0, (cudaStream_t)stream>>>(values_avg, latest, old_w, new_w,
                                                                                      inv_total, n);
    STEP_CHECK("update_average_values_kernel");
}

int p2b_step_mix_zero_sum(const float* a, const float* b, const float* beliefs, const uint8_t* ignore,
                          const float* coef_a, const float* coef_b, const float* scale, float* out, int64_t rows,
                          int32_t H, int subtract_b, int enforce_zero_sum, void* stream) {
    if (rows <= 0) return P2B_OK;
    if (enforce_zero_sum == 2 && H != P2B_NUM_HANDS && H != P2B_HPAD)
        return set_error(P2B_ERR_ARG, "enforce_zero_sum = 2 (sums in the CPU row-reduction order) needs H = %d or rows padded to %d",
                         P2B_NUM_HANDS, P2B_HPAD);
    mix_zero_sum_kernel<<<GRID_ROWS(rows), kThreads, 0, (cudaStream_t)stream>>>(a, b, beliefs, ignore, coef_a, coef_b, scale,
                                                                               out, rows, H, subtract_b, enforce_zero_sum);
    STEP_CHECK("mix_zero_sum_kernel");
}

int p2b_step_scaled_difference(const float* a, const float* b, const float* coef_a, const float* coef_b, float* out,
                               int64_t n, void* stream) {
    if (n <= 0) return P2B_OK;
    scaled_difference_kernel<<<GRID_ELEMS(n), kThreads, 0, (cudaStream_t)stream>>>(a, b, coef_a, coef_b, out, n);
    STEP_CHECK("scaled_difference_kernel");
}

int p2b_step_regret_tail(const float* values_achieved, const float* actor_values, const float* src_weights,
                         const int64_t* parent_index, const int64_t* prev_actor, float* regrets, int64_t bottom,
                         int64_t total, int32_t H, void* stream) {
    if (total <= bottom) return P2B_OK;
    regret_tail_kernel<<<GRID_ELEMS((total - bottom) * H), kThreads, 0, (cudaStream_t)stream>>>(
        values_achieved, actor_values, src_weights, (const long long*)parent_index, (const long long*)prev_actor, regrets,
        bottom, total, H);
    STEP_CHECK("regret_tail_kernel");
}

int p2b_step_average_policy_mix(const float* reach, const float* reach_avg, const float* policy, float* policy_avg,
                                const int64_t* to_act, const int64_t* parent_index, const float* old_w,
                                const float* new_w, const float* total_w, int64_t bottom, int64_t total, int32_t H,
                                float eps, void* stream) {
    if (total <= bottom) return P2B_OK;
    average_policy_mix_kernel<<<GRID_ELEMS((total - bottom) * H), kThreads, 0, (cudaStream_t)stream>>>(
        reach, reach_avg, policy, policy_avg, (const long long*)to_act, (const long long*)parent_index, old_w, new_w,
        total_w, bottom, total, H, eps);
    STEP_CHECK("average_policy_mix_kernel");
}

int p2b_step_parent_sum(const float* values, const int64_t* child_offsets, const int64_t* child_count, float* out,
                        int64_t num_parents, int32_t H, int broadcast_to_children, int64_t out_offset, void* stream) {
    if (num_parents <= 0) return P2B_OK;
    parent_sum_kernel<<<GRID_ELEMS(num_parents * H), kThreads, 0, (cudaStream_t)stream>>>(
        values, (const long long*)child_offsets, (const long long*)child_count, out, num_parents, H, broadcast_to_children,
        out_offset);
    STEP_CHECK("parent_sum_kernel");
}

int p2b_step_divide_by_parent_sum(const float* pos, const float* fallback, const float* parent_sum,
                                  const int64_t* parent_index, float* out, int64_t num_children, int32_t H, float eps,
                                  void* stream) {
    if (num_children <= 0) return P2B_OK;
    divide_by_parent_sum_kernel<<<GRID_ELEMS(num_children * H), kThreads, 0, (cudaStream_t)stream>>>(
        pos, fallback, parent_sum, (const long long*)parent_index, out, num_children, H, eps);
    STEP_CHECK("divide_by_parent_sum_kernel");
}

int p2b_step_unblocked_mass(const float* src, const int64_t* row_index, float* out, int64_t rows, void* stream) {
    if (rows <= 0) return P2B_OK;
    int rc = ensure_tables();
    if (rc) return rc;
    unblocked_mass_kernel<<<GRID_ROWS(rows), kThreads, 0, (cudaStream_t)stream>>>(src, (const long long*)row_index,
                                                                                 device_combo_table(), out, rows);
    STEP_CHECK("unblocked_mass_kernel");
}

int p2b_step_unblocked_mass_ratio(const float* numer, const float* denom, const int64_t* parent_index, float* out,
                                  int64_t rows, float eps, void* stream) {
    if (rows <= 0) return P2B_OK;
    int rc = ensure_tables();
    if (rc) return rc;
    unblocked_ratio_kernel<<<GRID_ROWS(rows), kThreads, 0, (cudaStream_t)stream>>>(numer, denom, (const long long*)parent_index,
                                                                                  device_combo_table(), out, rows, eps);
    STEP_CHECK("unblocked_ratio_kernel");
}

int p2b_step_weighted_parent_sum(float* values, const int64_t* prev_actor, const float* policy_hero,
                                 const float* policy_opp, const int64_t* child_offsets, const int64_t* child_count,
                                 int64_t parent_base, int64_t num_parents, int32_t H, void* stream) {
    if (num_parents <= 0) return P2B_OK;
    weighted_parent_sum_kernel<<<GRID_ELEMS(num_parents * 2 * H), kThreads, 0, (cudaStream_t)stream>>>(
        values, (const long long*)prev_actor, policy_hero, policy_opp, (const long long*)child_offsets,
        (const long long*)child_count, parent_base, num_parents, H);
    STEP_CHECK("weighted_parent_sum_kernel");
}

int p2b_step_reach_weights(float* reach, const float* policy, const uint8_t* allowed, const int64_t* parent_index,
                           const int64_t* prev_actor, int64_t start, int64_t end, int32_t H, void* stream) {
    if (end <= start) return P2B_OK;
    reach_weights_kernel<<<GRID_ELEMS((end - start) * H), kThreads, 0, (cudaStream_t)stream>>>(
        reach, policy, allowed, (const long long*)parent_index, (const long long*)prev_actor, start, end, H);
    STEP_CHECK("reach_weights_kernel");
}

int p2b_step_deep_beliefs(float* out, const float* root_beliefs, const float* reach, const float* allowed_prob,
                          const int64_t* root_index, int64_t num_roots, int64_t total, int32_t H, float eps,
                          void* stream) {
    if (total <= num_roots) return P2B_OK;
    deep_beliefs_kernel<<<GRID_ROWS((total - num_roots) * 2), kThreads, 0, (cudaStream_t)stream>>>(
        out, root_beliefs, reach, allowed_prob, (const long long*)root_index, num_roots, total, H, eps);
    STEP_CHECK("deep_beliefs_kernel");
}

}  // extern "C"
