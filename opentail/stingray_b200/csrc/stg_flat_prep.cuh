// What a row of the flat step needs before it can be streamed (shared by k_flat_prep and k_full_prep).
#pragma once
#include <math_constants.h>

#include "stg_flat.cuh"
#include "stg_select.cuh"

namespace stg {

// One 1024-thread CTA for one chunked row.  Top-k rows: the filter bound.  Thread t takes elements
// 4t .. 4t+3 of the row's first 4096 (masked) logits and keeps their maximum; the 1024 maxima are cut
// into `flat_groups` equal groups of consecutive threads, and the bound is the smallest of the groups'
// maxima: at least flat_groups elements of the sample lie at or above it, about twice as many on
// average, and the planner picks flat_groups so that about 3 N elements of the whole row should.
template <bool BF16>
__device__ __forceinline__ void flat_prep_row(const SampleArgs &a, FlatRow *fr, int row, const RowPlan &rp, float softcap, uint32_t *red)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (rp.path != kPathTopK) {
        if (tid == 0) { fr[row].key = 0ull; fr[row].tau = 0.f; fr[row].cnt = 0; fr[row].cap = 0; }
        return;
    }
    const int esz = BF16 ? 2 : 4;
    const LogitRow rowp{(const char *)a.logits + (int64_t)row * a.row_stride * esz, softcap};
    const uint32_t *mrow = (rp.use_mask && a.mask) ? a.mask + (int64_t)row * a.mask_stride : nullptr;
    float v[4];
    int idx[4];
    load_items<4, BF16, false>(rowp, mrow, 0, 0, min(a.vocab, kFlatSample), v, idx);  // out of range reads -inf
    uint32_t m = ord32(fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3])));
    const int ng = rp.flat_groups;          // power of two, 1 .. 1024
    const int w = kThreads / ng;            // threads per group
    // maximum over the thread's group
    for (int o = 1; o < min(w, 32); o <<= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (w > 32) {
        if (lane == 0) red[warp] = m;
        __syncthreads();
        const int wpg = w / 32;             // warps per group
        const int g0 = (warp / wpg) * wpg;
        m = 0u;
        for (int k = 0; k < wpg; k++) m = max(m, red[g0 + k]);
        __syncthreads();
    }
    // minimum over all groups (every thread holds its group's maximum)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = min(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (warp == 0) {
        m = red[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = min(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
        if (lane == 0) { fr[row].key = 0ull; fr[row].tau = unord32(m); fr[row].cnt = 0; fr[row].cap = rp.sel + kFlatSlack; }
    }
}

}  // namespace stg
