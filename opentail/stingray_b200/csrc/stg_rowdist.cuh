// The full-vocabulary pipeline for one row, run by one 1024-thread CTA:
//   bias -> history penalties -> 1/T -> softmax -> min-p -> top-p -> normalise -> inverse-CDF draw
// (Sampler.Sample's slow path, src/OpenTail.Stingray.Engine/Sampler.cs:41-95, and
// BuildFilteredDistribution, :118-163), plus GreedyWithHistoryPenalties (:421-437).
//
// The row is read from HBM once; later passes re-read it (or the exp values kept in a per-CTA
// scratch row) from L2.  Every sum the reference accumulates sequentially in fp32 is reproduced
// bit for bit by emul_scan; the one vectorised sum (Normalize's TensorPrimitives.Sum, whose order
// the reference does not pin) is accumulated in fp64 and rounded once.
//
// top-p is sort-free over the vocabulary: a histogram of the exp values bounds the nucleus, only
// the candidates above that bound are sorted (in shared memory), and the reference's sequential
// cumulative cut is then emulated over them.
#pragma once
#include <cuda_runtime.h>
#include <limits.h>
#include <math_constants.h>
#include <stdint.h>

#include "stg_emul.cuh"
#include "stg_select.cuh"
#include "stg_types.h"

namespace stg {

constexpr int kBins = 2048;  // exp-value histogram: 8 exponent + 4 mantissa bits of a float <= 1

struct RowCtl {
    EmulCtl em;
    double red_d[32];
    int red_i[32];
    u64 red_k[32];
    RowDist dist;
    int n_cand;       // candidates written by the compaction
    int n_surv;       // survivors of min-p over the whole row
    int c_lo;         // lowest histogram bin among the candidates
    int found;        // find_kth_match result
    int running;
};

// ---- sources of the row's adjusted, temperature-scaled logits ---------------------------------
template <bool BF16>
struct SrcLogits {
    const void *rowp;
    const uint32_t *mrow;
    int aligned;
    float inv_t;
    bool scale;
    __device__ __forceinline__ void get8(int base, int n, float x[8]) const
    {
        if (aligned && base + 8 <= n) {
            load_vec4<BF16, false>(rowp, base, x);
            load_vec4<BF16, false>(rowp, base + 4, x + 4);
            if (mrow) {
                uint32_t bits = __ldg(mrow + (base >> 5)) >> (base & 31);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (!((bits >> j) & 1u)) x[j] = -CUDART_INF_F;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                int i = base + j;
                float v = -CUDART_INF_F;
                if (i < n) {
                    v = load_one<BF16>(rowp, i);
                    if (mrow && !mask_bit(mrow, i)) v = -CUDART_INF_F;
                }
                x[j] = v;
            }
        }
        if (scale) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = __fmul_rn(x[j], inv_t);
        }
    }
};

struct SrcScratch {
    const float *p;
    float inv_t;
    bool scale;
    __device__ __forceinline__ void get8(int base, int n, float x[8]) const
    {
        if (base + 8 <= n) {
            float4 a = __ldcg((const float4 *)(p + base));
            float4 b = __ldcg((const float4 *)(p + base + 4));
            x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
            x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = (base + j < n) ? __ldcg(p + base + j) : -CUDART_INF_F;
        }
        if (scale) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = __fmul_rn(x[j], inv_t);
        }
    }
};

// ---- probability of an element from its exp value -----------------------------------------------
static __device__ __forceinline__ float eval_p2(float e, const RowDist &d)  // after softmax and min-p
{
    float p = (d.flags & kDistScale1) ? __fmul_rn(e, d.inv1) : e;
    if (d.flags & kDistTopK) {
        if (p < d.kth) return 0.f;
        if (d.flags & kDistScale2) p = __fmul_rn(p, d.inv2);
    }
    if ((d.flags & kDistMinP) && p < d.minp_thr) p = 0.f;
    return p;
}
static __device__ __forceinline__ float eval_p3(float e, int i, const RowDist &d)  // final probability
{
    float p = eval_p2(e, d);
    if (d.flags & kDistTopP) {
        if (p < d.tstar || (p == d.tstar && i > d.tie_idx_max)) p = 0.f;
    }
    if (d.flags & kDistScale3) p = __fmul_rn(p, d.inv3);
    return p;
}

// ---- emul_scan providers -------------------------------------------------------------------------
// exp pass: computes e_i = expf(x_i - max), stores it in the scratch row, feeds the histogram.
template <class Src>
struct ProvExp {
    Src src;
    float mx;
    float *scratch;
    unsigned *hcount;   // null: no histogram wanted
    u64 *hmass;
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
        if (base >= n) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = 0.f;
            return;
        }
        src.get8(base, n, x);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float e = (base + j < n) ? expf(__fsub_rn(x[j], mx)) : 0.f;
            x[j] = e;
            if (hcount && e > 0.f) {
                unsigned bin = __float_as_uint(e) >> 19;
                bin = bin < (unsigned)kBins ? bin : (unsigned)(kBins - 1);
                atomicAdd(&hcount[bin], 1u);
                atomicAdd(&hmass[bin], (u64)((double)e * 1099511627776.0));
            }
        }
        if (base + 8 <= n) {
            __stcg((float4 *)(scratch + base), make_float4(x[0], x[1], x[2], x[3]));
            __stcg((float4 *)(scratch + base + 4), make_float4(x[4], x[5], x[6], x[7]));
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (base + j < n) __stcg(scratch + base + j, x[j]);
        }
    }
};

struct ProvConstFill {  // every token has the same probability (no finite logit)
    float value;
    float *scratch;
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            x[j] = (base + j < n) ? value : 0.f;
            if (base + j < n) __stcg(scratch + base + j, value);
        }
    }
};

struct ProvFinal {  // final probabilities from the scratch row of exp values
    const float *scratch;
    const RowDist *d;
    float *dist_out;  // optional: materialise the distribution
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
        if (base >= n) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = 0.f;
            return;
        }
        SrcScratch s{scratch, 1.f, false};
        s.get8(base, n, x);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            x[j] = (base + j < n) ? eval_p3(x[j], base + j, *d) : 0.f;
            if (dist_out && base + j < n) dist_out[base + j] = x[j];
        }
    }
};

struct ProvKeys {  // descending sorted probability bit patterns
    const uint32_t *keys;
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
#pragma unroll
        for (int j = 0; j < 8; j++) x[j] = (base + j < n) ? __uint_as_float(keys[base + j]) : 0.f;
    }
};

// ---- block-wide helpers ----------------------------------------------------------------------------
template <class T>
static __device__ void bitonic_sort_desc_t(T *a, int p2)
{
    for (int k = 2; k <= p2; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < (p2 >> 1); t += kThreads) {
                int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                int l = i | j;
                bool desc = ((i & k) == 0);
                T x = a[i], y = a[l];
                if ((x < y) == desc) { a[i] = y; a[l] = x; }
            }
            __syncthreads();
        }
    }
}

static __device__ __forceinline__ u64 block_max_key_r(u64 k, u64 *scratch)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        u64 t = __shfl_xor_sync(0xFFFFFFFFu, k, o);
        k = t > k ? t : k;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = k;
    __syncthreads();
    if (threadIdx.x < 32) {
        k = scratch[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            u64 t = __shfl_xor_sync(0xFFFFFFFFu, k, o);
            k = t > k ? t : k;
        }
        if (threadIdx.x == 0) scratch[0] = k;
    }
    __syncthreads();
    k = scratch[0];
    __syncthreads();
    return k;
}

// (max value, lowest index of it) of the source as a key; 0 when nothing is > -infinity
template <class Src>
static __device__ u64 pass_max(const Src &src, int n, u64 *red)
{
    float best = -CUDART_INF_F;
    int best_i = -1;
    for (int base = threadIdx.x * 8; base < n; base += kThreads * 8) {
        float x[8];
        src.get8(base, n, x);
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (x[j] > best) { best = x[j]; best_i = base + j; }
    }
    // a thread's elements are not contiguous across tiles, but each thread keeps its own lowest
    // index per value and the key order (value, then lower index) resolves ties across threads
    u64 k = best_i >= 0 ? make_key(best, best_i) : 0ull;
    return block_max_key_r(k, red);
}

// index of the `kth` (1-based) element, in token order, whose post-min-p probability equals tstar
static __device__ int find_kth_match(RowCtl *rc, const float *scratch, int n, const RowDist &d, float tstar,
                              int kth)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __syncthreads();
    if (tid == 0) { rc->found = INT_MAX; rc->running = 0; }
    __syncthreads();
    for (int tile0 = 0; tile0 < n; tile0 += kEmulTile) {
        float x[8];
        const int base = tile0 + tid * 8;
        int m = 0;
        unsigned bits = 0;
        if (base < n) {
            SrcScratch s{scratch, 1.f, false};
            s.get8(base, n, x);
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (base + j < n && eval_p2(x[j], d) == tstar) { bits |= 1u << j; m++; }
        }
        int inc = m;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) rc->red_i[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            int w = rc->red_i[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int t = __shfl_up_sync(0xFFFFFFFFu, w, o);
                if (lane >= o) w += t;
            }
            rc->red_i[lane] = w;
        }
        __syncthreads();
        const int run0 = rc->running;
        int excl = run0 + (warp ? rc->red_i[warp - 1] : 0) + inc - m;
        const int tile_total = rc->red_i[31];
        if (m && excl < kth && kth <= excl + m) {
            int need = kth - excl;
#pragma unroll
            for (int j = 0; j < 8; j++)
                if ((bits >> j) & 1u) { if (--need == 0) rc->found = base + j; }
        }
        __syncthreads();
        if (tid == 0) rc->running = run0 + tile_total;
        const int f = rc->found;
        __syncthreads();
        if (f != INT_MAX) return f;
    }
    return INT_MAX;
}

// ---- history / bias overrides, applied to a raw copy of the row in the scratch row -----------------
// ApplyHistoryPenalties (Sampler.cs:367-419) after the logit bias (Sampler.cs:50-56): entries are
// sorted by token so that one thread owns each distinct token and applies, in the reference's
// order, the bias additions, the per-occurrence repetition penalty inside the window, and the
// presence/frequency penalty over the whole history.
static __device__ void apply_overrides(const SampleArgs &a, const RowPlan &rp, float *scratch, int n,
                                bool with_bias, u64 *keys /* arena */)
{
    const int tid = threadIdx.x;
    const int nh = rp.hist_len;
    const int nb = with_bias ? rp.bias_len : 0;
    const int ne = nh + nb;
    if (ne == 0) return;
    const int p2 = pow2_ceil(max(ne, 2));
    const int32_t *hist = a.hist_ids + rp.hist_off;
    for (int t = tid; t < p2; t += kThreads) {
        u64 k = 0ull;
        if (t < nb) {
            int id = __ldg(a.bias_ids + rp.bias_off + t);
            if ((unsigned)id < (unsigned)n) k = ~(((u64)(uint32_t)id << 32) | (u64)(uint32_t)t);
        } else if (t < ne) {
            int pos = t - nb;
            int id = __ldg(hist + pos);
            if ((unsigned)id < (unsigned)n) k = ~(((u64)(uint32_t)id << 32) | (u64)(0x80000000u | (uint32_t)pos));
        }
        keys[t] = k;
    }
    __syncthreads();
    bitonic_sort_desc(keys, p2);
    const bool has_hist_pen = nh > 0;
    for (int t = tid; t < ne; t += kThreads) {
        u64 kk = keys[t];
        if (kk == 0ull) continue;
        u64 k = ~kk;
        uint32_t id = (uint32_t)(k >> 32);
        if (t > 0 && keys[t - 1] != 0ull && (uint32_t)((~keys[t - 1]) >> 32) == id) continue;  // not a run start
        float x = __ldcg(scratch + id);
        int occ_all = 0, occ_w = 0;
        for (int r = t; r < ne; r++) {
            u64 rk = keys[r];
            if (rk == 0ull) break;
            u64 q = ~rk;
            if ((uint32_t)(q >> 32) != id) break;
            uint32_t sub = (uint32_t)q;
            if (sub & 0x80000000u) {
                occ_all++;
                if ((int)(sub & 0x7FFFFFFFu) >= rp.window_start) occ_w++;
            } else {
                x = __fadd_rn(x, __ldg(a.bias_vals + rp.bias_off + (int)sub));
            }
        }
        if (has_hist_pen && occ_all > 0) {
            if (rp.rep != 1.0f)
                for (int r = 0; r < occ_w; r++) x = x > 0.f ? __fdiv_rn(x, rp.rep) : __fmul_rn(x, rp.rep);
            if (!(rp.pres == 0.f && rp.freq == 0.f))
                x = __fsub_rn(x, __fadd_rn(rp.pres, __fmul_rn(rp.freq, (float)occ_all)));
        }
        __stcg(scratch + id, x);
    }
    __threadfence_block();
    __syncthreads();
}

// ---- the distribution of one row --------------------------------------------------------------------
// Leaves the exp values in `scratch` and the descriptor in rc->dist.  `src` yields the adjusted,
// temperature-scaled logits.
template <class Src>
static __device__ void build_dist(RowCtl *rc, SelCtl *sctl, const Src &src, const RowPlan &rp, int n,
                           float *scratch, unsigned char *arena, uint32_t *gkeys, int gkeys_cap,
                           uint32_t *flags_out)
{
    const int tid = threadIdx.x;
    uint32_t *skeys = (uint32_t *)arena;                       // kSortCap u32
    unsigned *hcount = (unsigned *)(arena + kSortCap * 4);     // kBins u32
    u64 *hmass = (u64 *)(arena + kSortCap * 4 + kBins * 4);    // kBins u64
    const bool want_topp = rp.top_p < 1.0f && rp.top_p > 0.f;
    const bool want_minp = rp.min_p > 0.f;
    const bool want_topk = rp.top_k > 0 && rp.top_k < n;

    u64 mk = pass_max(src, n, rc->red_k);
    RowDist d;
    d.flags = 0;
    d.inv_t = src.inv_t;
    d.tie_idx_max = INT_MAX;
    d.kth = 0.f; d.inv2 = 1.f; d.minp_thr = 0.f; d.tstar = 0.f; d.inv3 = 1.f; d.inv1 = 1.f;
    d.uniform_p = 0.f; d.sum_end = 0.f; d.argmax = 0;
    if (want_topp) {
        for (int t = tid; t < kBins; t += kThreads) { hcount[t] = 0u; hmass[t] = 0ull; }
    }
    __syncthreads();
    float sum = 0.f;
    if (mk == 0ull) {
        // Softmax's fully masked case (Sampler.cs:452-458): every token gets 1/V, no rescale
        d.flags |= kDistUniform;
        d.max_x = -CUDART_INF_F;
        d.uniform_p = __fdiv_rn(1.0f, (float)n);
        ProvConstFill pc{d.uniform_p, scratch};
        for (int base = tid * 8; base < n; base += kThreads * 8) { float x[8]; pc.load(base, n, x); }
        if (want_topp && tid == 0) {
            unsigned bin = __float_as_uint(d.uniform_p) >> 19;
            hcount[bin] = (unsigned)n;
            hmass[bin] = (u64)((double)d.uniform_p * 1099511627776.0) * (u64)n;
        }
        __syncthreads();
    } else {
        d.max_x = key_val(mk);
        ProvExp<Src> pe{src, d.max_x, scratch, want_topp ? hcount : nullptr, hmass};
        emul_scan<ProvExp<Src>, false>(&rc->em, pe, n, 0.f, false, &sum);
        if (sum > 0.f && sum != 1.0f) { d.flags |= kDistScale1; d.inv1 = __fdiv_rn(1.0f, sum); }
    }
    __syncthreads();
    if (want_topk) {
        // ApplyTopK + Normalize (Sampler.cs:477-488, :71-81): the k-th largest probability, counted
        // with multiplicity; everything below it is dropped, ties at it all survive.  Selected on
        // the exp values, of which the probabilities are a monotone image.
        Sel s;
        s.c = sctl;
        s.cap = 8192;
        s.buf[0] = (u64 *)arena;
        s.buf[1] = s.buf[0] + s.cap;
        s.n = rp.top_k;
        s.idx_off = 0;
        sel_reset(s);
        sel_stream<4, false>(s, scratch, nullptr, 0, n);
        const u64 *b = s.buf[sctl->cur];
        u64 inv_min = 0ull;
        for (int e = tid; e < sctl->cnt; e += kThreads) { u64 t = ~b[e]; inv_min = t > inv_min ? t : inv_min; }
        u64 mn = ~block_max_key_r(inv_min, rc->red_k);
        float kth_e = key_val(mn);
        d.kth = (d.flags & kDistScale1) ? __fmul_rn(kth_e, d.inv1) : kth_e;
        d.flags |= kDistTopK;
        double part = 0.0;
        for (int base = tid * 8; base < n; base += kThreads * 8) {
            float x[8];
            SrcScratch sc{scratch, 1.f, false};
            sc.get8(base, n, x);
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (base + j < n) part += (double)eval_p2(x[j], d);
        }
        float s2 = (float)block_sum_double(part, rc->red_d);
        if (s2 > 0.f && s2 != 1.0f) { d.flags |= kDistScale2; d.inv2 = __fdiv_rn(1.0f, s2); }
        __syncthreads();
    }
    if (want_minp) {
        // ApplyMinP (Sampler.cs:493-503): the largest probability belongs to exp value 1 (or 1/V)
        float emax = (d.flags & kDistUniform) ? d.uniform_p : 1.0f;
        float pmax = (d.flags & kDistScale1) ? __fmul_rn(emax, d.inv1) : emax;
        if (d.flags & kDistScale2) pmax = __fmul_rn(pmax, d.inv2);
        d.minp_thr = __fmul_rn(rp.min_p, pmax);
        d.flags |= kDistMinP;
    }

    double sum3 = 0.0;
    if (want_topp) {
        // bound the nucleus from the histogram (exact enough to be a superset; the cut itself is
        // decided below by the emulated sequential sum)
        for (int attempt = 0; attempt < 2; attempt++) {
            if (tid == 0) {
                int c_lo = 0;
                if (attempt == 0) {
                    double scale_p = ((d.flags & kDistScale1) ? (double)d.inv1 : 1.0) *
                                     ((d.flags & kDistScale2) ? (double)d.inv2 : 1.0) / 1099511627776.0;
                    u64 acc_m = 0ull;
                    unsigned acc_c = 0u;
                    for (int b = kBins - 1; b >= 0; --b) {
                        acc_c += hcount[b];
                        acc_m += hmass[b];
                        // estimate only: a bound that proves too tight is caught below (the
                        // emulated sum then never reaches top_p) and the cut is redone over all
                        double need = (double)rp.top_p * (1.0 + 1.0 / 65536.0) +
                                      16.0 * sqrt((double)acc_c) * 2.98e-8 + 1e-7;
                        if ((double)acc_m * scale_p >= need) { c_lo = b > 0 ? b - 1 : 0; break; }
                    }
                }
                rc->c_lo = c_lo;
                rc->n_cand = 0;
                rc->n_surv = 0;
            }
            __syncthreads();
            const uint32_t lo_bits = (uint32_t)rc->c_lo << 19;
            // how many candidates at most? decides shared vs global key storage
            int bound = 0;
            for (int b = rc->c_lo + tid; b < kBins; b += kThreads) bound += (int)hcount[b];
            bound = block_sum_int(bound, rc->red_i);
            uint32_t *keys = skeys;
            int cap = kSortCap;
            if (bound > kSortCap) { keys = gkeys; cap = gkeys_cap; *flags_out |= (1u << 7); }
            // compaction: probability bit patterns of the survivors above the bound
            int my_surv = 0;
            for (int base = tid * 8; base < n; base += kThreads * 8) {
                float x[8];
                SrcScratch s{scratch, 1.f, false};
                s.get8(base, n, x);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (base + j >= n) continue;
                    float p = eval_p2(x[j], d);
                    if (p > 0.f) {
                        my_surv++;
                        if (__float_as_uint(x[j]) >= lo_bits) {
                            int slot = atomicAdd(&rc->n_cand, 1);
                            if (slot < cap) keys[slot] = __float_as_uint(p);
                        }
                    }
                }
            }
            my_surv = block_sum_int(my_surv, rc->red_i);
            __syncthreads();
            const int nc = min(rc->n_cand, cap);
            if (nc == 0) break;
            const int p2 = pow2_ceil(max(nc, 2));
            for (int t = nc + tid; t < p2; t += kThreads) keys[t] = 0u;
            __syncthreads();
            if (!(d.flags & kDistUniform)) bitonic_sort_desc_t<uint32_t>(keys, p2);
            ProvKeys pk{keys};
            float cum = 0.f;
            int hit = emul_scan<ProvKeys, false>(&rc->em, pk, nc, rp.top_p, true, &cum);
            if (hit < 0 && nc < my_surv && attempt == 0) continue;  // bound was too tight: take all
            const int last = hit >= 0 ? hit : nc - 1;
            const float tstar = __uint_as_float(keys[last]);
            // ties at the cut: kept ones are a prefix (by token id) of the equal probabilities
            int keep = 0, all = 0;
            for (int t = tid; t < nc; t += kThreads) {
                if (keys[t] == __float_as_uint(tstar)) { all++; keep += (t <= last) ? 1 : 0; }
            }
            keep = block_sum_int(keep, rc->red_i);
            all = block_sum_int(all, rc->red_i);
            double part = 0.0;
            for (int t = tid; t <= last; t += kThreads) part += (double)__uint_as_float(keys[t]);
            sum3 = block_sum_double(part, rc->red_d);
            d.flags |= kDistTopP;
            d.tstar = tstar;
            d.tie_idx_max = INT_MAX;
            if (keep < all) {
                *flags_out |= (1u << 4);
                d.tie_idx_max = find_kth_match(rc, scratch, n, d, tstar, keep);
            }
            break;
        }
    } else {
        double part = 0.0;
        for (int base = tid * 8; base < n; base += kThreads * 8) {
            float x[8];
            SrcScratch s{scratch, 1.f, false};
            s.get8(base, n, x);
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (base + j < n) part += (double)eval_p2(x[j], d);
        }
        sum3 = block_sum_double(part, rc->red_d);
    }
    // Normalize (Sampler.cs:553-562)
    float s3 = (float)sum3;
    if (s3 > 0.f && s3 != 1.0f) { d.flags |= kDistScale3; d.inv3 = __fdiv_rn(1.0f, s3); }
    __syncthreads();
    if (tid == 0) rc->dist = d;
    __syncthreads();
}

template <bool BF16>
static __device__ void run_row(const SampleArgs &a, int row, SelCtl *sctl, unsigned char *arena)
{
    __shared__ RowCtl rc;
    const int tid = threadIdx.x;
    const RowPlan rp = a.plans[row];
    const int n = a.vocab;
    const int esz = BF16 ? 2 : 4;
    const void *rowp = (const char *)a.logits + (int64_t)row * a.row_stride * esz;
    const uint32_t *mrow = (rp.use_mask && a.mask) ? a.mask + (int64_t)row * a.mask_stride : nullptr;
    float *scratch = a.escratch + (int64_t)blockIdx.x * a.escratch_stride;
    uint32_t *gkeys = (uint32_t *)(a.keyscratch + (int64_t)blockIdx.x * a.key_stride);
    const int gkeys_cap = (int)(a.key_stride * 2);
    const bool greedy = rp.temperature <= 0.f;
    const bool with_bias = !greedy && rp.bias_len > 0;
    const bool overrides = (rp.has_penalty && rp.hist_len > 0) || with_bias;
    __shared__ uint32_t sh_flags;
    if (tid == 0) sh_flags = 0;
    __syncthreads();

    if (overrides) {
        // raw masked copy of the row, then the per-token adjustments
        SrcLogits<BF16> raw{rowp, mrow, a.vec == 4, 1.f, false};
        for (int base = tid * 8; base < n; base += kThreads * 8) {
            float x[8];
            raw.get8(base, n, x);
            if (base + 8 <= n) {
                __stcg((float4 *)(scratch + base), make_float4(x[0], x[1], x[2], x[3]));
                __stcg((float4 *)(scratch + base + 4), make_float4(x[4], x[5], x[6], x[7]));
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (base + j < n) __stcg(scratch + base + j, x[j]);
            }
        }
        __threadfence_block();
        __syncthreads();
        RowPlan eff = rp;
        if (!rp.has_penalty) eff.hist_len = 0;
        apply_overrides(a, eff, scratch, n, with_bias, (u64 *)arena);
    }

    if (greedy) {
        // Greedy / GreedyWithHistoryPenalties; in distribution mode a one-hot row
        u64 mk;
        if (overrides) { SrcScratch s{scratch, 1.f, false}; mk = pass_max(s, n, rc.red_k); }
        else { SrcLogits<BF16> s{rowp, mrow, a.vec == 4, 1.f, false}; mk = pass_max(s, n, rc.red_k); }
        int tok = mk ? key_idx(mk) : 0;
        if (a.mode == 2) {
            if (tid == 0) {
                RowDist d;
                memset(&d, 0, sizeof(d));
                d.flags = kDistOneHot;
                d.tie_idx_max = tok;
                d.argmax = tok;
                d.inv_t = 1.f; d.inv1 = 1.f; d.inv2 = 1.f; d.inv3 = 1.f;
                a.dists[row] = d;
            }
            __syncthreads();
            return;
        }
        if (a.mode == 1 && a.dist_out) {
            float *o = a.dist_out + (int64_t)row * n;
            for (int i = tid; i < n; i += kThreads) o[i] = (i == tok) ? 1.f : 0.f;
        }
        if (tid == 0) {
            if (a.tokens) a.tokens[row] = tok;
            if (a.token_probs) a.token_probs[row] = 1.f;
            if (a.row_flags) a.row_flags[row] = (uint32_t)rp.path | (mk ? 0u : (1u << 6));
        }
        __syncthreads();
        return;
    }

    const float inv_t = rp.temperature != 1.0f ? __fdiv_rn(1.0f, rp.temperature) : 1.0f;
    const bool scale = rp.temperature != 1.0f;
    if (overrides) {
        SrcScratch s{scratch, inv_t, scale};
        build_dist(&rc, sctl, s, rp, n, scratch, arena, gkeys, gkeys_cap, &sh_flags);
    } else {
        SrcLogits<BF16> s{rowp, mrow, a.vec == 4, inv_t, scale};
        build_dist(&rc, sctl, s, rp, n, scratch, arena, gkeys, gkeys_cap, &sh_flags);
    }
    if (a.mode == 2) {
        // descriptor only; the raw arg-max goes with it (the looser accept rule compares against it)
        SrcLogits<BF16> raw{rowp, mrow, a.vec == 4, 1.f, false};
        u64 mk = pass_max(raw, n, rc.red_k);
        if (tid == 0) {
            rc.dist.argmax = mk ? key_idx(mk) : 0;
            a.dists[row] = rc.dist;
        }
        __syncthreads();
        return;
    }

    // draw: SampleFromDistribution (Sampler.cs:564-576)
    float *dout = (a.mode == 1 && a.dist_out) ? a.dist_out + (int64_t)row * n : nullptr;
    ProvFinal pf{scratch, &rc.dist, dout};
    if (a.mode == 1) {
        for (int base = tid * 8; base < n; base += kThreads * 8) { float x[8]; pf.load(base, n, x); }
        if (tid == 0 && a.row_flags) a.row_flags[row] = kPathFull | sh_flags;
        __syncthreads();
        return;
    }
    const float u = a.uniforms ? __ldg(a.uniforms + row) : 0.5f;
    float cum = 0.f;
    int hit = emul_scan<ProvFinal, false>(&rc.em, pf, n, u, true, &cum);
    if (tid == 0) {
        uint32_t fl = kPathFull | sh_flags;
        if (rc.dist.flags & kDistUniform) fl |= (1u << 6);
        int tok = hit;
        if (hit < 0) { tok = n - 1; fl |= (1u << 5); }
        a.tokens[row] = tok;
        if (a.token_probs) a.token_probs[row] = eval_p3(__ldcg(scratch + tok), tok, rc.dist);
        if (a.row_flags) a.row_flags[row] = fl;
    }
    __syncthreads();
}

}  // namespace stg
