// Providers of speculative verification: a row's final probabilities recomputed from its logits and
// its distribution descriptor, and the positive part of p - q (shared by stg_spec_kernels.cu and the
// flat form in stg_flat_full.cu).
#pragma once
#include "stg_rowdist.cuh"

namespace stg {

template <bool BF16>
__device__ __forceinline__ float eval_point(const LogitRow rowp, int i, const RowDist &d)
{
    if (d.flags & kDistOneHot) return i == d.tie_idx_max ? 1.f : 0.f;
    float e;
    if (d.flags & kDistUniform) {
        e = d.uniform_p;
    } else {
        float x = load_one<BF16>(rowp, i);
        if (d.inv_t != 1.0f) x = __fmul_rn(x, d.inv_t);
        e = expf(__fsub_rn(x, d.max_x));
    }
    return eval_p3(e, i, d);
}

// final probabilities of a row, recomputed from its logits
template <bool BF16>
struct ProvRow {
    SrcLogits<BF16> src;
    RowDist d;  // by value: lives in registers
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
        if (base >= n) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = 0.f;
            return;
        }
        if (d.flags & kDistOneHot) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = (base + j == d.tie_idx_max) ? 1.f : 0.f;
            return;
        }
        src.get8(base, n, x);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float e = (d.flags & kDistUniform) ? d.uniform_p : expf(__fsub_rn(x[j], d.max_x));
            x[j] = (base + j < n) ? eval_p3(e, base + j, d) : 0.f;
        }
    }
    __device__ __forceinline__ void reload(int base, int n, float x[8]) const { load(base, n, x); }
};

// positive part of p - q (ResampleResidual's terms)
template <bool BF16>
struct ProvResidual {
    ProvRow<BF16> p, q;
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
        float y[8];
        p.load(base, n, x);
        q.load(base, n, y);
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float r = __fsub_rn(x[j], y[j]);
            x[j] = r > 0.f ? r : 0.f;
        }
    }
    __device__ __forceinline__ void reload(int base, int n, float x[8]) const { load(base, n, x); }
};

}  // namespace stg
