// The HBM pass of the flat step over the rows that are not full-vocabulary rows (top-k path and plain
// arg-max rows): the same work as those branches of k_flat_stream (stg_flat.cu), as a kernel of its
// own.  Without the full-vocabulary branch (overrides, stores, two running keys) and without a second
// register set for prefetched loads it needs 40 registers instead of 62, so more warps are resident to
// cover the load latency - measured on the arg-max form of this loop (stg_flat_greedy.cu), that is
// worth more than the prefetch.
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "stg_flat.cuh"
#include "stg_launch.h"
#include "stg_select.cuh"
#include "stg_types.h"

#ifndef STG_CHUNKS_MB
#define STG_CHUNKS_MB 5
#endif

namespace stg {

template <bool BF16>
__device__ __forceinline__ void chunk_load4(const LogitRow rowp, const uint32_t *mrow, int i, int end, float v[4])
{
    if (i + 3 < end) {
        load_vec4<BF16, true>(rowp, i, v);
    } else {
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = (i + e < end) ? load_one<BF16>(rowp, i + e) : -CUDART_INF_F;
    }
    if (mrow != nullptr && i < end) {
        const uint32_t bits = __ldg(mrow + (i >> 5)) >> (i & 31);
#pragma unroll
        for (int e = 0; e < 4; e++)
            if (!((bits >> e) & 1u)) v[e] = -CUDART_INF_F;
    }
}

// grid (pieces of kFlatPiece elements, rows of a.items); 256 threads; in step s thread t reads elements
// 4096 s + 1024 u + 4 t .. + 3 (u = 0..3) of the piece as four independent 16-byte loads
template <bool BF16, bool CAP>
__global__ void __launch_bounds__(kFlatThreads, STG_CHUNKS_MB) k_flat_stream_chunks(const __grid_constant__ SampleArgs a, FlatRow *fr)
{
    const int row = __ldg(&a.items[blockIdx.y].row), tid = threadIdx.x, lane = tid & 31;
    const RowPlan *rpp = a.plans + row;
    if (__ldg(&rpp->n_chunks) == 0) return;  // not a row of this pass
    const int begin = blockIdx.x * kFlatPiece;
    const int end = min(a.vocab, begin + kFlatPiece);
    if (begin >= end) return;
    const int esz = BF16 ? 2 : 4;
    const LogitRow rowp{(const char *)a.logits + (int64_t)row * a.row_stride * esz, CAP ? a.softcap : 0.f};
    const uint32_t *mrow = (__ldg(&rpp->use_mask) && a.mask) ? a.mask + (int64_t)row * a.mask_stride : nullptr;
    const int i0 = begin + tid * 4;

    if (__ldg(&rpp->path) == kPathGreedy) {
        __shared__ unsigned long long red[kFlatThreads / 32];
        float best = -CUDART_INF_F;
        int best_i = -1;
#pragma unroll 1
        for (int s = 0; s < kFlatSteps; s++) {
            float cur[4][4];
#pragma unroll
            for (int u = 0; u < 4; u++) chunk_load4<BF16>(rowp, mrow, i0 + (s * 4 + u) * 1024, end, cur[u]);
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (cur[u][e] > best) { best = cur[u][e]; best_i = i0 + (s * 4 + u) * 1024 + e; }
        }
        // a thread visits ascending indices, so it holds its lowest index of the value; the key
        // order (value, then lower index) settles ties between threads, pieces and CTAs
        unsigned long long k = best_i >= 0 ? make_key(best, best_i) : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long t = __shfl_xor_sync(0xFFFFFFFFu, k, o);
            k = t > k ? t : k;
        }
        if (lane == 0) red[tid >> 5] = k;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < kFlatThreads / 32; w++) k = red[w] > k ? red[w] : k;
            if (k != 0ull) atomicMax(&fr[row].key, k);
        }
        return;
    }

    // top-k path: every element above the row's bound becomes a candidate.  The CTA collects its
    // candidates in shared memory and hands them to the row's list with a single global atomicAdd at
    // the end; should a piece hold more than the staging area takes, the excess goes to the list
    // directly.
    __shared__ unsigned long long stage[kFlatStage];
    __shared__ int stage_cnt, list_first;
    if (tid == 0) stage_cnt = 0;
    __syncthreads();
    const float tau = fr[row].tau;
    const int cap = fr[row].cap;
    unsigned long long *cand = a.cand + __ldg(&rpp->cand_off);
    int *cnt_p = &fr[row].cnt;
    // The sweep itself only notes which of the thread's 64 elements pass (one bit each): keeping the
    // key construction and the appends out of the loop keeps it as tight as the arg-max loop.  The
    // few that pass (a fraction of a percent) are read again afterwards, from L2.
    unsigned long long passed = 0ull;
#pragma unroll 1
    for (int s = 0; s < kFlatSteps; s++) {
        float cur[4][4];
#pragma unroll
        for (int u = 0; u < 4; u++) chunk_load4<BF16>(rowp, mrow, i0 + (s * 4 + u) * 1024, end, cur[u]);
        unsigned pass = 0u;
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int e = 0; e < 4; e++) pass |= (cur[u][e] > tau) ? (1u << (u * 4 + e)) : 0u;  // out of range and masked read -inf
        passed |= (unsigned long long)pass << (16 * s);
    }
    static_assert(kFlatSteps * 16 <= 64, "one bit per element of a thread");
    while (passed != 0ull) {
        const int b = __ffsll((long long)passed) - 1;
        passed &= passed - 1ull;
        const int idx = i0 + (b >> 2) * 1024 + (b & 3);  // bit 16 s + 4 u + e: sub-step 4 s + u, element e
        const unsigned long long key = make_key(load_one<BF16>(rowp, idx), idx);
        const int slot = atomicAdd(&stage_cnt, 1);
        if (slot < kFlatStage) {
            stage[slot] = key;
        } else {
            const int g = atomicAdd(cnt_p, 1);
            if (g < cap) cand[g] = key;
        }
    }
    __syncthreads();
    const int staged = min(stage_cnt, kFlatStage);
    if (staged > 0) {
        if (tid == 0) list_first = atomicAdd(cnt_p, staged);
        __syncthreads();
        const int g0 = list_first;
        for (int t = tid; t < staged; t += kFlatThreads)
            if (g0 + t < cap) cand[g0 + t] = stage[t];
    }
}

cudaError_t launch_flat_stream_chunks(const SampleArgs &a, FlatRow *fr, cudaStream_t stream)
{
    const dim3 grid((unsigned)((a.vocab + kFlatPiece - 1) / kFlatPiece), (unsigned)a.n_items);
    const bool cap = a.softcap != 0.f;
    if (a.dtype == 1) { if (cap) k_flat_stream_chunks<true, true><<<grid, kFlatThreads, 0, stream>>>(a, fr); else k_flat_stream_chunks<true, false><<<grid, kFlatThreads, 0, stream>>>(a, fr); }
    else { if (cap) k_flat_stream_chunks<false, true><<<grid, kFlatThreads, 0, stream>>>(a, fr); else k_flat_stream_chunks<false, false><<<grid, kFlatThreads, 0, stream>>>(a, fr); }
    return cudaGetLastError();
}

}  // namespace stg
