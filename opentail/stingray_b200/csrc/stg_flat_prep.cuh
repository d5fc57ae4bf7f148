// What a row of the flat step needs before it can be streamed (shared by k_flat_prep and k_full_prep).
#pragma once
#include <math_constants.h>

#include "stg_flat.cuh"
#include "stg_select.cuh"

namespace stg {

// One 1024-thread CTA for one chunked row.  Top-k rows: the filter bound.  Thread t takes elements
// 4t .. 4t+3 of the row's first 4096 (masked) logits and keeps their maximum; the 1024 maxima are cut
// into `flat_groups` equal groups of consecutive threads, and the smallest of the groups' maxima is a
// first bound: at least flat_groups elements of the sample lie at or above it, two to five times as
// many on average.  With flat_rank set (the planner's choice whenever it applies) the bound proper is
// the sample's flat_rank-th largest logit, found among the elements above the first bound.
constexpr int kPrepList = 1024;  // sample elements the exact bound is ranked among at most (list[] holds two more words)

template <bool BF16>
__device__ __forceinline__ void flat_prep_row(const SampleArgs &a, FlatRow *fr, int row, const RowPlan &rp, float softcap, uint32_t *red,
                                              uint32_t *list)
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
    if (rp.flat_rank == 0) {
        if (warp == 0) {
            m = red[lane];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = min(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
            if (lane == 0) { fr[row].key = 0ull; fr[row].tau = unord32(m); fr[row].cnt = 0; fr[row].cap = rp.sel + kFlatSlack; }
        }
        return;
    }
    // The bound as the sample's flat_rank-th largest logit: the groups' bound tau0 fences off a short list
    // of sample elements, and the element of that list with exactly flat_rank - 1 others ahead of it is the
    // bound.  A list shorter than flat_rank, or one that does not fit (a sample full of equal values),
    // leaves tau0 as the bound; every bound is checked by the kernel that consumes the row's candidates.
    uint32_t t0 = red[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t0 = min(t0, __shfl_xor_sync(0xFFFFFFFFu, t0, o));
    __syncthreads();  // every warp has read red[]
    if (tid == 0) { list[kPrepList] = 0u; list[kPrepList + 1] = t0; }
    __syncthreads();
    unsigned n_mine = 0;
    uint32_t o4[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        o4[e] = ord32(v[e]);
        n_mine += (o4[e] >= t0 && !(isinf(v[e]) && v[e] < 0.f)) ? 1u : 0u;
    }
    if (n_mine) {
        unsigned slot = atomicAdd(&list[kPrepList], n_mine);
#pragma unroll
        for (int e = 0; e < 4; e++)
            if (o4[e] >= t0 && !(isinf(v[e]) && v[e] < 0.f)) {
                if (slot < (unsigned)kPrepList) list[slot] = o4[e];
                slot++;
            }
    }
    __syncthreads();
    const int n = (int)list[kPrepList];
    if (n >= rp.flat_rank && n <= kPrepList) {
        for (int t = tid; t < n; t += kThreads) {
            const uint32_t xv = list[t];
            int rank = 0;
            for (int j = 0; j < n; j++) {
                const uint32_t y = list[j];
                rank += (y > xv || (y == xv && j < t)) ? 1 : 0;
            }
            if (rank == rp.flat_rank - 1) list[kPrepList + 1] = xv;
        }
        __syncthreads();
    }
    if (tid == 0) { fr[row].key = 0ull; fr[row].tau = unord32(list[kPrepList + 1]); fr[row].cnt = 0; fr[row].cap = rp.sel + kFlatSlack; }
}

}  // namespace stg
