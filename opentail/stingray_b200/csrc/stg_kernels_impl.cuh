// Kernels of the sampling library (sm_100a); the launchers that instantiate them are spread over
// several translation units (stg_kernels.cu, stg_chunks_*.cu, stg_rows_*.cu) so that they compile
// in parallel.
//
// k_sample is one persistent launch per sampling step: 1024-thread CTAs (one per SM) pull work
// items from a global counter.  A chunk item streams part of a row once from HBM through the
// exact top-N selection (or the arg-max); the last chunk of a row to finish merges the row's
// candidates and runs the sequential finish.  A row item runs the full-vocabulary pipeline for one
// row (stg_rowdist.cuh).
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "stg_launch.h"
#include "stg_rowdist.cuh"
#include "stg_select.cuh"
#include "stg_types.h"

namespace stg {

static_assert(kRowArenaEnd == (int)kRowArenaBytes, "row arena layout and its launch size disagree");

struct ItemShared {
    int item;
    int last;
    FinishOut fout;
    u64 best;
};

__device__ __forceinline__ u64 block_max_key(u64 k, u64 *scratch /* 32 entries */)
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

// Arg-max of elements [begin, end) as a key (0 when no element is > -infinity).
template <int VEC, bool BF16>
__device__ u64 greedy_stream(const LogitRow rowp, const uint32_t *mrow, int begin, int end, int idx_off,
                             u64 *scratch)
{
    constexpr int U = 4;
    float best = -CUDART_INF_F;
    int best_i = -1;
    for (int base = begin; base < end; base += kThreads * 4 * U) {
        float v[U][4];
        int idx[U][4];
#pragma unroll
        for (int u = 0; u < U; u++) load_items<VEC, BF16, true>(rowp, mrow, base, u, end, v[u], idx[u]);
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (v[u][e] > best) { best = v[u][e]; best_i = idx[u][e]; }
    }
    u64 k = best_i >= 0 ? make_key(best, best_i + idx_off) : 0ull;
    return block_max_key(k, scratch);
}

__device__ __forceinline__ void write_greedy(const SampleArgs &a, int row, u64 key, const LogitRow rowp)
{
    if (threadIdx.x != 0) return;
    int tok = 0;
    float val;
    uint32_t fl = kPathGreedy;
    if (key != 0ull) {
        tok = key_idx(key);
        val = key_val(key);
    } else {
        val = load_one_dyn(rowp, a.dtype, 0);  // Greedy of a row without a finite value: token 0
        fl |= (1u << 6);
    }
    if (a.pairs_out) {
        ((int32_t *)a.pairs_out)[2 * row] = tok;
        ((float *)a.pairs_out)[2 * row + 1] = val;
    }
    if (a.tokens) a.tokens[row] = tok;
    if (a.token_probs) a.token_probs[row] = 1.0f;
    if (a.row_flags) a.row_flags[row] = fl;
}

template <int VEC, bool BF16>
__device__ void run_chunk(const SampleArgs &a, int row, int chunk, int item, SelCtl *ctl, ItemShared *ish,
                          unsigned char *arena)
{
    u64 *tk = a.phase_ticks ? a.phase_ticks + (int64_t)item * 32 : nullptr;
    tick(tk, 0);
    const RowPlan rp = a.plans[row];
    const int esz = BF16 ? 2 : 4;
    const LogitRow rowp{(const char *)a.logits + (int64_t)row * a.row_stride * esz, a.softcap};
    const uint32_t *mrow = (rp.use_mask && a.mask) ? a.mask + (int64_t)row * a.mask_stride : nullptr;
    const int begin = chunk * a.chunk_len;
    const int end = min(a.vocab, begin + a.chunk_len);
    u64 *scratch = (u64 *)arena;  // 32 entries, only used by the greedy path

    if (rp.path == kPathGreedy) {
        u64 k = greedy_stream<VEC, BF16>(rowp, mrow, begin, end, a.vocab_offset, scratch);
        if (rp.n_chunks > 1) {
            if (threadIdx.x == 0) {
                a.cand[rp.cand_off + chunk] = k;
                __threadfence();
                unsigned old = atomicAdd(&a.tickets[row], 1u);
                ish->last = (old == (unsigned)(rp.n_chunks - 1));
                if (ish->last) {
                    a.tickets[row] = 0;
                    __threadfence();
                    u64 best = 0ull;
                    for (int c = 0; c < rp.n_chunks; c++) {
                        u64 t = __ldcg(a.cand + rp.cand_off + c);
                        best = t > best ? t : best;
                    }
                    k = best;
                    ish->best = best;
                }
            }
            __syncthreads();
            if (!ish->last) return;
            k = ish->best;
        }
        if (a.shard_mode == 1) {
            if (threadIdx.x == 0) {
                a.xchg_local[(int64_t)row * a.xchg_stride] = k;
                a.xchg_count[row] = k ? 1 : 0;
            }
            return;
        }
        write_greedy(a, row, k, rowp);
        return;
    }

    // top-k path
    Sel s;
    s.c = ctl;
    s.buf[0] = (u64 *)arena;
    s.buf[1] = s.buf[0] + a.cap;
    s.cap = a.cap;
    s.n = rp.sel;
    s.idx_off = a.vocab_offset;
    sel_reset(s);
    sel_stream<VEC, BF16>(s, rowp, mrow, begin, end);
    tick(tk, 1);
    if (rp.n_chunks > 1) {
        const int cnt = ctl->cnt;
        u64 *dst = a.cand + rp.cand_off + (int64_t)chunk * 2 * rp.sel;
        const u64 *src = s.buf[ctl->cur];
        for (int e = threadIdx.x; e < cnt; e += kThreads) dst[e] = src[e];
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            a.cand_count[rp.slot + chunk] = cnt;
            __threadfence();
            unsigned old = atomicAdd(&a.tickets[row], 1u);
            ish->last = (old == (unsigned)(rp.n_chunks - 1));
            if (ish->last) a.tickets[row] = 0;
        }
        __syncthreads();
        if (!ish->last) return;
        __threadfence();
        sel_reset(s);
        for (int c = 0; c < rp.n_chunks; c++) {
            int m = __ldcg(a.cand_count + rp.slot + c);
            sel_append_keys(s, a.cand + rp.cand_off + (int64_t)c * 2 * rp.sel, m);
        }
    }
    if (a.shard_mode == 1) {
        // vocabulary-sharded mode: hand this rank's best `sel` survivors to the exchange buffer
        if (ctl->cnt > rp.sel) sel_compact(s);
        const int cnt = ctl->cnt;
        const u64 *src = s.buf[ctl->cur];
        u64 *dst = a.xchg_local + (int64_t)row * a.xchg_stride;
        for (int e = threadIdx.x; e < cnt; e += kThreads) dst[e] = src[e];
        if (threadIdx.x == 0) a.xchg_count[row] = cnt;
        __syncthreads();
        return;
    }
    tick(tk, 2);
    const int32_t *hist = a.hist_ids ? a.hist_ids + rp.hist_off : nullptr;
    const float *ptab = (a.pow_tab && rp.pow_off >= 0) ? a.pow_tab + rp.pow_off : nullptr;
    float u = a.uniforms ? __ldg(a.uniforms + row) : 0.5f;
    int64_t o = (int64_t)row * a.topk_stride;
    finish_topk(s, rp, hist, ptab, u, &ish->fout, a.topk_ids ? a.topk_ids + o : nullptr,
                a.topk_logits ? a.topk_logits + o : nullptr, a.topk_probs ? a.topk_probs + o : nullptr);
    if (threadIdx.x == 0) {
        a.tokens[row] = ish->fout.token;
        if (a.token_probs) a.token_probs[row] = ish->fout.prob;
        if (a.row_flags) a.row_flags[row] = ish->fout.flags;
        count_row_flags(a.counters, ish->fout.flags);
    }
    tick(tk, 3);
    __syncthreads();
}

// Chunk items: the streaming arg-max / top-N selection (HBM-bound).
template <int VEC, bool BF16>
__global__ void __launch_bounds__(kThreads, 1) k_sample_chunks(const __grid_constant__ SampleArgs a)
{
    extern __shared__ __align__(16) unsigned char arena[];
    __shared__ SelCtl ctl;
    __shared__ ItemShared ish;
    for (;;) {
        if (threadIdx.x == 0) ish.item = (int)(atomicAdd(a.work_counter, 1u) - a.work_base);
        __syncthreads();
        const int item = ish.item;
        __syncthreads();
        if ((unsigned)item >= (unsigned)a.n_items) break;
        const WorkItem w = a.items[item];
        run_chunk<VEC, BF16>(a, w.row, w.chunk, a.item_base + item, &ctl, &ish, arena);
        __syncthreads();
    }
}

// Row items: the full-vocabulary pipeline, one row per CTA at a time.
template <bool BF16>
__global__ void __launch_bounds__(kThreads, 1) k_sample_rows(const __grid_constant__ SampleArgs a)
{
    extern __shared__ __align__(16) unsigned char arena[];
    __shared__ SelCtl ctl;
    __shared__ int sh_item;
    int next = blockIdx.x;
    for (;;) {
        int item;
        if (a.static_items) {
            item = next;
            next += gridDim.x;
        } else {
            if (threadIdx.x == 0) sh_item = (int)(atomicAdd(a.work_counter, 1u) - a.work_base);
            __syncthreads();
            item = sh_item;
            __syncthreads();
        }
        if ((unsigned)item >= (unsigned)a.n_items) break;
        const WorkItem w = a.items[item];
        run_row<BF16>(a, w.row, a.item_base + item, &ctl, arena);
        __syncthreads();
    }
}

}  // namespace stg
