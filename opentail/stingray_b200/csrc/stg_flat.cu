// Kernels of the flat form of a sampling step (see stg_flat.cuh): prep, the HBM streaming pass, and
// the per-row finish of the top-k path.
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "stg_flat.cuh"
#include "stg_flat_finish.cuh"
#include "stg_flat_prep.cuh"
#include "stg_launch.h"
#include "stg_select.cuh"
#include "stg_types.h"

namespace stg {

// ---- k_flat_prep --------------------------------------------------------------------------------------
// One 1024-thread CTA per row (flat_prep_row, stg_flat_prep.cuh).  Launched on its own only when the
// step has no full-vocabulary rows in the flat form; otherwise k_full_prep, which has a CTA per row
// anyway, does this for the rows that are not its own.
template <bool BF16, bool CAP>
__global__ void __launch_bounds__(kThreads) k_flat_prep(const __grid_constant__ SampleArgs a, FlatRow *fr)
{
    __shared__ uint32_t red[32];
    __shared__ uint32_t list[kPrepList + 2];
    const int row = blockIdx.x;
    const RowPlan rp = a.plans[row];
    if (rp.n_chunks == 0) return;  // not a row of the flat step
    flat_prep_row<BF16>(a, fr, row, rp, CAP ? a.softcap : 0.f, red, list);
}

// ---- k_flat_stream ------------------------------------------------------------------------------------
// Four masked elements of a 16-byte aligned row starting at element i (a multiple of 4); elements at
// or beyond `end` read as -infinity.
template <bool BF16>
__device__ __forceinline__ void flat_load4(const LogitRow rowp, const uint32_t *mrow, int i, int end, float v[4])
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

// One CTA of 256 threads per 16384-element piece of a row (grid.x pieces, grid.y rows).  Sub-step q
// (0..15) of a piece covers 1024 consecutive elements, thread t its elements 4t .. 4t+3; a thread
// keeps the loads of the next four sub-steps in flight while it works on the current four.  CAP: the
// batch has a soft cap (a build of its own, so that the common case carries no trace of it).
template <bool BF16, bool CAP>
__global__ void __launch_bounds__(kFlatThreads) k_flat_stream(const __grid_constant__ SampleArgs a, FlatRow *fr, const FullWs ws)
{
    __shared__ unsigned long long red[kFlatThreads / 32];
    // grid.y runs over the step's item list, which names the full-vocabulary rows first: their CTAs do
    // the most work per piece and so start first, and the light ones fill the tail of the grid
    const int row = __ldg(&a.items[blockIdx.y].row), tid = threadIdx.x, lane = tid & 31;
    const RowPlan *rpp = a.plans + row;
    const int fi = __ldg(&rpp->flat_full);
    if (__ldg(&rpp->n_chunks) == 0 && fi < 0) return;  // not a row of the flat step
    const int begin = blockIdx.x * kFlatPiece;
    const int end = min(a.vocab, begin + kFlatPiece);
    if (begin >= end) return;
    const int path = __ldg(&rpp->path);
    const int esz = BF16 ? 2 : 4;
    const LogitRow rowp{(const char *)a.logits + (int64_t)row * a.row_stride * esz, CAP ? a.softcap : 0.f};
    const uint32_t *mrow = (__ldg(&rpp->use_mask) && a.mask) ? a.mask + (int64_t)row * a.mask_stride : nullptr;
    const int i0 = begin + tid * 4;

    float cur[4][4], nxt[4][4];
#pragma unroll
    for (int u = 0; u < 4; u++) flat_load4<BF16>(rowp, mrow, i0 + u * 1024, end, cur[u]);

    if (fi >= 0) {
        // a full-vocabulary row (or greedy with penalties): x = overrides(masked logit) * 1/T goes to
        // the row's scratch, and the running (max, lowest index) key of x to the row's state
        __shared__ int s_id[kMaxOverride];
        __shared__ float s_adj[kMaxOverride];
        __shared__ unsigned s_bits[kFlatPiece / 32];
        FullRow *fw = ws.rows + fi;
        const float temperature = __ldg(&rpp->temperature);
        const bool greedy = !(temperature > 0.f);
        const bool scale = !greedy && temperature != 1.0f;
        const float inv_t = scale ? __fdiv_rn(1.0f, temperature) : 1.0f;
        const int ov_lo = fw->ov_piece[blockIdx.x], ov_n = fw->ov_piece[blockIdx.x + 1] - ov_lo;
        if (ov_n > 0) {
            for (int t = tid; t < kFlatPiece / 32; t += kFlatThreads) s_bits[t] = 0u;
            __syncthreads();
            const int32_t *gid = ws.ov_id + (size_t)fi * kMaxOverride + ov_lo;
            const float *gadj = ws.ov_adj + (size_t)fi * kMaxOverride + ov_lo;
            for (int t = tid; t < ov_n; t += kFlatThreads) {
                const int id = __ldg(gid + t);
                s_id[t] = id;
                s_adj[t] = __ldg(gadj + t);
                atomicOr(&s_bits[(id - begin) >> 5], 1u << ((id - begin) & 31));
            }
            __syncthreads();
        }
        float *e = ws.e + (size_t)fi * ws.e_stride;
        float best = -CUDART_INF_F, rbest = -CUDART_INF_F;
        int best_i = -1, rbest_i = -1;
        const bool want_raw = a.mode == 2;
#pragma unroll
        for (int s = 0; s < kFlatSteps; s++) {
            if (s + 1 < kFlatSteps) {
#pragma unroll
                for (int u = 0; u < 4; u++) flat_load4<BF16>(rowp, mrow, i0 + ((s + 1) * 4 + u) * 1024, end, nxt[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + (s * 4 + u) * 1024;
                if (i < end) {
                    if (want_raw) {
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            if (cur[u][k] > rbest) { rbest = cur[u][k]; rbest_i = i + k; }
                    }
                    if (ov_n > 0) {
                        const int rel = i - begin;
                        const unsigned nib = (s_bits[rel >> 5] >> (rel & 31)) & 0xFu;
                        if (nib) {
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                if ((nib >> k) & 1u) {
                                    int lo = 0, hi = ov_n - 1;  // the id is in the list: find it
                                    while (lo < hi) {
                                        const int mid = (lo + hi) >> 1;
                                        if (s_id[mid] < i + k) lo = mid + 1; else hi = mid;
                                    }
                                    cur[u][k] = s_adj[lo];
                                }
                            }
                        }
                    }
                    if (scale) {
#pragma unroll
                        for (int k = 0; k < 4; k++) cur[u][k] = __fmul_rn(cur[u][k], inv_t);
                    }
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        if (i + k < end && cur[u][k] > best) { best = cur[u][k]; best_i = i + k; }
                    if (!greedy) {
                        if (i + 3 < end) {
                            __stcg((float4 *)(e + i), make_float4(cur[u][0], cur[u][1], cur[u][2], cur[u][3]));
                        } else {
#pragma unroll
                            for (int k = 0; k < 4; k++)
                                if (i + k < end) __stcg(e + i + k, cur[u][k]);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int k = 0; k < 4; k++) cur[u][k] = nxt[u][k];
        }
        unsigned long long k = best_i >= 0 ? make_key(best, best_i) : 0ull;
        unsigned long long rk = rbest_i >= 0 ? make_key(rbest, rbest_i) : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long t = __shfl_xor_sync(0xFFFFFFFFu, k, o);
            k = t > k ? t : k;
            const unsigned long long rt = __shfl_xor_sync(0xFFFFFFFFu, rk, o);
            rk = rt > rk ? rt : rk;
        }
        __shared__ unsigned long long rred[kFlatThreads / 32];
        if (lane == 0) { red[tid >> 5] = k; rred[tid >> 5] = rk; }
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < kFlatThreads / 32; w++) { k = red[w] > k ? red[w] : k; rk = rred[w] > rk ? rred[w] : rk; }
            if (k != 0ull) atomicMax(&fw->maxkey, k);
            if (want_raw && rk != 0ull) atomicMax(&fw->rawkey, rk);
        }
        return;
    }

    if (path == kPathGreedy) {
        float best = -CUDART_INF_F;
        int best_i = -1;
#pragma unroll
        for (int s = 0; s < kFlatSteps; s++) {
            if (s + 1 < kFlatSteps) {
#pragma unroll
                for (int u = 0; u < 4; u++) flat_load4<BF16>(rowp, mrow, i0 + ((s + 1) * 4 + u) * 1024, end, nxt[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (cur[u][e] > best) { best = cur[u][e]; best_i = i0 + (s * 4 + u) * 1024 + e; }
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int e = 0; e < 4; e++) cur[u][e] = nxt[u][e];
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
#pragma unroll
    for (int s = 0; s < kFlatSteps; s++) {
        if (s + 1 < kFlatSteps) {
#pragma unroll
            for (int u = 0; u < 4; u++) flat_load4<BF16>(rowp, mrow, i0 + ((s + 1) * 4 + u) * 1024, end, nxt[u]);
        }
        unsigned pass = 0u;
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int e = 0; e < 4; e++) pass |= (cur[u][e] > tau) ? (1u << (u * 4 + e)) : 0u;  // out of range and masked read -inf
        passed |= (unsigned long long)pass << (16 * s);
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int e = 0; e < 4; e++) cur[u][e] = nxt[u][e];
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

// ---- k_flat_finish ------------------------------------------------------------------------------------
// The rows of a.items: one per CTA, or (SHARED) shared between the CTAs of a smaller grid, which
// leaves SMs to the kernels of the full-vocabulary rows it runs beside.
template <bool BF16, bool SHARED>
__global__ void __launch_bounds__(kThreads, 1) k_flat_finish(const __grid_constant__ SampleArgs a, FlatRow *fr)
{
    extern __shared__ __align__(16) unsigned char arena[];
    __shared__ SelCtl ctl;
    __shared__ FlatShared fs;
    if (!SHARED) {
        flat_finish_row<BF16>(a, fr, a.items[blockIdx.x].row, blockIdx.x, a.cap, arena, ctl, fs);
        return;
    }
    for (int i = blockIdx.x; i < a.n_items; i += gridDim.x) {
        flat_finish_row<BF16>(a, fr, a.items[i].row, i, a.cap, arena, ctl, fs);
        __syncthreads();
    }
}

cudaError_t launch_flat_prep(const SampleArgs &a, FlatRow *fr, cudaStream_t stream)
{
    const bool cap = a.softcap != 0.f;
    if (a.dtype == 1) { if (cap) k_flat_prep<true, true><<<a.rows, kThreads, 0, stream>>>(a, fr); else k_flat_prep<true, false><<<a.rows, kThreads, 0, stream>>>(a, fr); }
    else { if (cap) k_flat_prep<false, true><<<a.rows, kThreads, 0, stream>>>(a, fr); else k_flat_prep<false, false><<<a.rows, kThreads, 0, stream>>>(a, fr); }
    return cudaGetLastError();
}

cudaError_t launch_flat_stream(const SampleArgs &a, FlatRow *fr, const FullWs &ws, cudaStream_t stream)
{
    const dim3 grid((unsigned)((a.vocab + kFlatPiece - 1) / kFlatPiece), (unsigned)a.n_items);
    const bool cap = a.softcap != 0.f;
    if (a.dtype == 1) { if (cap) k_flat_stream<true, true><<<grid, kFlatThreads, 0, stream>>>(a, fr, ws); else k_flat_stream<true, false><<<grid, kFlatThreads, 0, stream>>>(a, fr, ws); }
    else { if (cap) k_flat_stream<false, true><<<grid, kFlatThreads, 0, stream>>>(a, fr, ws); else k_flat_stream<false, false><<<grid, kFlatThreads, 0, stream>>>(a, fr, ws); }
    return cudaGetLastError();
}

cudaError_t launch_flat_finish(const SampleArgs &a, FlatRow *fr, int grid, size_t smem, cudaStream_t stream)
{
    const bool shared = grid < a.n_items;
    void (*fn)(const SampleArgs, FlatRow *) = a.dtype == 1 ? (shared ? k_flat_finish<true, true> : k_flat_finish<true, false>)
                                                           : (shared ? k_flat_finish<false, true> : k_flat_finish<false, false>);
    cudaError_t e = ensure_dynamic_smem((const void *)fn, smem);
    if (e != cudaSuccess) return e;
    fn<<<grid, kThreads, smem, stream>>>(a, fr);
    return cudaGetLastError();
}

}  // namespace stg
