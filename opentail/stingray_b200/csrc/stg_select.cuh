// Streaming exact top-N selection over a row (or a chunk of one), the block-wide sort that orders
// the survivors, and the sequential finish of the top-k sampling path.
//
// Selection semantics follow SampleTopK's insertion select
// (src/OpenTail.Stingray.Engine/Sampler.cs:240-249): the N largest raw logits, descending, equal
// values in ascending token order, the earlier token kept on a tie at the boundary, -infinity never
// selected.  A candidate is the 64-bit key (order-preserving float bits << 32) | ~token, so
// "larger key" is exactly that order and keys are distinct.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "stg_types.h"

namespace stg {

typedef unsigned long long u64;

static __device__ __forceinline__ uint32_t ord32(float v)
{
    v = v + 0.0f;  // -0 -> +0: the reference compares floats, for which the two are equal
    uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
static __device__ __forceinline__ float unord32(uint32_t k)
{
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}
static __device__ __forceinline__ u64 make_key(float v, int idx)
{
    return ((u64)ord32(v) << 32) | (u64)(0xFFFFFFFFu - (uint32_t)idx);
}
static __device__ __forceinline__ float key_val(u64 k) { return unord32((uint32_t)(k >> 32)); }
static __device__ __forceinline__ int key_idx(u64 k) { return (int)(0xFFFFFFFFu - (uint32_t)k); }

// elements one load_items call of the CTA covers (4 per thread): the sample the streaming select draws its first bound from
constexpr int kSelTile = 4 * kThreads;

// ---- element access --------------------------------------------------------------------------
static __device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
static __device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// A row of logits as the kernels read it.  cap != 0: the final-logit soft cap
// x <- tanh(x / cap) * cap (llm_softcap_inplace, src/OpenTail.Stingray.Cuda/CudaTextKernels.cs:374-383,
// which the reference runs as a pass of its own over the logits before sampling) is applied to every
// element as it is loaded, with that kernel's own operations in its order, so the row is never
// rewritten in device memory.
struct LogitRow {
    const void *p;
    float cap;
};
static __device__ __forceinline__ float soft_cap(float x, float cap) { return __fmul_rn(tanhf(__fdiv_rn(x, cap)), cap); }

template <bool BF16, bool STREAM>
static __device__ __forceinline__ void load_vec4(const LogitRow rowp, int i, float v[4])
{
    if (BF16) {
        const uint2 *p = (const uint2 *)((const uint16_t *)rowp.p + i);
        uint2 t = STREAM ? __ldcs(p) : __ldg(p);
        v[0] = bf16_lo(t.x); v[1] = bf16_hi(t.x); v[2] = bf16_lo(t.y); v[3] = bf16_hi(t.y);
    } else {
        const float4 *p = (const float4 *)((const float *)rowp.p + i);
        float4 t = STREAM ? __ldcs(p) : __ldg(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    if (rowp.cap != 0.f) {
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = soft_cap(v[e], rowp.cap);
    }
}
template <bool BF16>
static __device__ __forceinline__ float load_one(const LogitRow rowp, int i)
{
    float x;
    if (BF16) x = __uint_as_float((uint32_t)__ldg((const uint16_t *)rowp.p + i) << 16);
    else x = __ldg((const float *)rowp.p + i);
    return rowp.cap != 0.f ? soft_cap(x, rowp.cap) : x;
}
static __device__ __forceinline__ float load_one_dyn(const LogitRow rowp, int dtype, int i)
{
    return dtype ? load_one<true>(rowp, i) : load_one<false>(rowp, i);
}
static __device__ __forceinline__ bool mask_bit(const uint32_t *mrow, int i)
{
    return (__ldg(mrow + (i >> 5)) >> (i & 31)) & 1u;
}

// Loads the 4 elements a thread owns in sub-step `u` of a 16384-element iteration starting at
// `base`, applying the allowed-token mask; out-of-range elements read as -infinity.
// VEC == 4: elements base + (u*1024 + tid)*4 + e (one 128-bit / 64-bit load);
// VEC == 1: elements base + (u*4 + e)*1024 + tid (scalar loads, any alignment).
template <int VEC, bool BF16, bool STREAM>
static __device__ __forceinline__ void load_items(const LogitRow rowp, const uint32_t *mrow, int base, int u,
                                           int end, float v[4], int idx[4])
{
    const int tid = threadIdx.x;
    if (VEC == 4) {
        int i = base + (u * kThreads + tid) * 4;
#pragma unroll
        for (int e = 0; e < 4; e++) idx[e] = i + e;
        if (i + 3 < end) {
            load_vec4<BF16, STREAM>(rowp, i, v);
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++) v[e] = (i + e < end) ? load_one<BF16>(rowp, i + e) : -CUDART_INF_F;
        }
        if (mrow != nullptr && i < end) {
            uint32_t bits = __ldg(mrow + (i >> 5)) >> (i & 31);
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (!((bits >> e) & 1u)) v[e] = -CUDART_INF_F;
        }
    } else {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            int i = base + (u * 4 + e) * kThreads + tid;
            idx[e] = i;
            float x = -CUDART_INF_F;
            if (i < end) {
                x = load_one<BF16>(rowp, i);
                if (mrow != nullptr && !mask_bit(mrow, i)) x = -CUDART_INF_F;
            }
            v[e] = x;
        }
    }
}

// ---- block utilities ---------------------------------------------------------------------------
static __device__ __forceinline__ int warp_sum(int v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// Control block of one selection, in shared memory.
struct SelCtl {
    int cnt;          // entries in the active buffer
    int cnt2;         // entries written to the other buffer during a compaction
    int overflow;     // an optimistic append ran out of room
    int cur;          // active buffer (0/1)
    int tmp;          // block-wide counter scratch
    float tau;        // a later element can only be selected if it is > tau
    int want;
    int stop;
    u64 prefix;
    u64 thr;
    u64 minkey;
    unsigned hist[256];
    unsigned red[32];     // block reductions
    unsigned ord_lo;      // lower end and shift of the coarse histogram of an approximate compaction
    int shift;
    int cut;              // its boundary bin
};

struct Sel {
    SelCtl *c;
    u64 *buf[2];
    int cap;
    int n;        // selection count N
    int idx_off;  // added to a column index to form the token id stored in a key
};

static __device__ __forceinline__ void sel_reset(Sel &s)
{
    if (threadIdx.x == 0) {
        s.c->cnt = 0; s.c->cnt2 = 0; s.c->overflow = 0; s.c->cur = 0; s.c->tmp = 0;
        s.c->tau = -CUDART_INF_F;
    }
    __syncthreads();
}

// Keeps the N largest keys of the active buffer (block-wide radix select on the 64-bit keys, most
// significant byte first), moves them to the other buffer and raises tau to the N-th value.
// Requires cnt > N.  All threads call it.
static __device__ void sel_compact(Sel &s)
{
    SelCtl *c = s.c;
    const int tid = threadIdx.x;
    const int cnt = c->cnt;
    const u64 *src = s.buf[c->cur];
    u64 *dst = s.buf[c->cur ^ 1];
    __syncthreads();
    if (tid == 0) { c->want = s.n; c->prefix = 0; c->stop = 0; c->cnt2 = 0; c->minkey = ~0ull; }
    for (int pass = 7; pass >= 0; --pass) {
        if (tid < 256) c->hist[tid] = 0;
        __syncthreads();
        const u64 prefix = c->prefix;
        const int sh = 8 * pass;
        for (int e = tid; e < cnt; e += kThreads) {
            u64 k = src[e];
            if (pass == 7 || (k >> (sh + 8)) == prefix) atomicAdd(&c->hist[(unsigned)(k >> sh) & 255u], 1u);
        }
        __syncthreads();
        if (tid < 32) {
            // lane l owns bins 8l..8l+7; suffix sums locate the bin holding the want-th largest key
            unsigned h[8];
            unsigned local = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) { h[j] = c->hist[tid * 8 + j]; local += h[j]; }
            const unsigned want = (unsigned)c->want;  // read before the shuffles order the lanes
            unsigned above = 0;  // keys in bins of higher lanes
            unsigned run = local;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                unsigned t = __shfl_down_sync(0xFFFFFFFFu, run, o);
                if (tid + o < 32) run += t;
            }
            above = run - local;
            bool mine = above < want && want <= above + local;
            if (mine) {
                unsigned acc = above;
#pragma unroll
                for (int j = 7; j >= 0; --j) {
                    if (want <= acc + h[j]) {
                        c->prefix = (prefix << 8) | (u64)(tid * 8 + j);
                        c->want = (int)(want - acc);
                        if (h[j] == want - acc || pass == 0) {
                            c->stop = 1;
                            c->thr = ((prefix << 8) | (u64)(tid * 8 + j)) << sh;
                        }
                        break;
                    }
                    acc += h[j];
                }
            }
        }
        __syncthreads();
        if (c->stop) break;
    }
    const u64 thr = c->thr;
    u64 mymin = ~0ull;
    for (int e = tid; e < cnt; e += kThreads) {
        u64 k = src[e];
        if (k >= thr) {
            int slot = atomicAdd(&c->cnt2, 1);
            dst[slot] = k;
            if (k < mymin) mymin = k;
        }
    }
    if (mymin != ~0ull) atomicMin(&c->minkey, mymin);
    __syncthreads();
    if (tid == 0) {
        c->cnt = c->cnt2;
        c->cur ^= 1;
        c->tau = key_val(c->minkey);
    }
    __syncthreads();
}

// Cheap compaction: raises tau without finding the exact N-th key.  The keys are binned by value
// into 256 bins covering the top 4 binades below the buffer's maximum; the highest boundary that
// still keeps at least N keys becomes the cut, the keys below it are dropped, and tau becomes the
// smallest surviving value (at least N better-or-earlier keys are held, so the strict `> tau`
// test stays exact).  Leaves between N and N + (one bin) keys.  Falls back to the exact
// selection when the binning cannot separate the keys (heavy ties, or the N-th key far below the
// maximum).  Requires cnt > N.  All threads call it.
static __device__ void sel_compact(Sel &s);
static __device__ void sel_raise(Sel &s)
{
    SelCtl *c = s.c;
    const int tid = threadIdx.x;
    const int cnt = c->cnt;
    const u64 *src = s.buf[c->cur];
    u64 *dst = s.buf[c->cur ^ 1];
    __syncthreads();
    // maximum value (as ordered bits) in the buffer
    unsigned mx = 0u;
    for (int e = tid; e < cnt; e += kThreads) mx = max(mx, (unsigned)(src[e] >> 32));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if ((tid & 31) == 0) c->red[tid >> 5] = mx;
    if (tid < 256) c->hist[tid] = 0;
    __syncthreads();
    if (tid < 32) {
        mx = tid < kThreads / 32 ? c->red[tid] : 0u;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        if (tid == 0) {
            // 256 bins of 2^18 ordered-bit units (1/32 of a binade) below the maximum
            const unsigned span = 256u << 18;
            c->ord_lo = mx >= span ? mx - span + 1u : 0u;
            c->shift = 18;
            c->cnt2 = 0;
            c->minkey = ~0ull;
            c->cut = 0;   // no lane finds a boundary bin (fewer keys than wanted): the exact selection decides
            c->want = 0;
        }
    }
    __syncthreads();
    const unsigned lo = c->ord_lo;
    const int sh = c->shift;
    for (int e = tid; e < cnt; e += kThreads) {
        const unsigned o = (unsigned)(src[e] >> 32);
        const unsigned b = o >= lo ? min((o - lo) >> sh, 255u) : 0u;
        atomicAdd(&c->hist[b], 1u);
    }
    __syncthreads();
    if (tid < 32) {
        unsigned h[8];
        unsigned local = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) { h[j] = c->hist[tid * 8 + j]; local += h[j]; }
        unsigned run = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            unsigned t = __shfl_down_sync(0xFFFFFFFFu, run, o);
            if (tid + o < 32) run += t;
        }
        const unsigned above = run - local;
        const unsigned want = (unsigned)s.n;
        if (above < want && want <= above + local) {
            unsigned acc = above;
            bool found = false;
#pragma unroll
            for (int j = 7; j >= 0; --j) {
                if (!found && want <= acc + h[j]) { c->cut = tid * 8 + j; c->want = (int)(acc + h[j]); found = true; }
                acc += h[j];
            }
        }
    }
    __syncthreads();
    const int cut = c->cut;
    const int kept = c->want;  // keys in bins >= cut
    if (cut == 0 || kept > s.n + ((s.cap - s.n) >> 2)) {
        // bin 0 collects everything below the window, and a crowded boundary bin means ties:
        // let the exact selection handle those
        sel_compact(s);
        return;
    }
    u64 mymin = ~0ull;
    for (int e = tid; e < cnt; e += kThreads) {
        const u64 k = src[e];
        const unsigned o = (unsigned)(k >> 32);
        const unsigned b = o >= lo ? min((o - lo) >> sh, 255u) : 0u;
        if ((int)b >= cut) {
            int slot = atomicAdd(&c->cnt2, 1);
            dst[slot] = k;
            if (k < mymin) mymin = k;
        }
    }
    if (mymin != ~0ull) atomicMin(&c->minkey, mymin);
    __syncthreads();
    if (tid == 0) {
        c->cnt = c->cnt2;
        c->cur ^= 1;
        c->tau = key_val(c->minkey);
    }
    __syncthreads();
}

// Appends the caller's up-to-4 passing elements; exact (counted) form used when room is short.
static __device__ __forceinline__ void sel_append_exact(Sel &s, const float v[4], const int idx[4], int end)
{
    SelCtl *c = s.c;
    for (int attempt = 0;; attempt++) {
        const float tau = c->tau;
        int n = 0;
#pragma unroll
        for (int e = 0; e < 4; e++) n += (idx[e] < end && v[e] > tau) ? 1 : 0;
        int w = warp_sum(n);
        if ((threadIdx.x & 31) == 0 && w) atomicAdd(&c->tmp, w);
        __syncthreads();
        const int total = c->tmp;
        const int cnt = c->cnt;
        __syncthreads();
        if (threadIdx.x == 0) c->tmp = 0;
        if (cnt + total > s.cap) {
            // cnt > N here because cap >= N + kSubTile >= N + total; the exact selection leaves
            // exactly N keys, after which a sub-tile always fits
            if (attempt == 0) sel_raise(s); else sel_compact(s);
            continue;
        }
        if (n) {
            int slot = atomicAdd(&c->cnt, n);
            u64 *b = s.buf[c->cur];
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (idx[e] < end && v[e] > tau) b[slot++] = make_key(v[e], idx[e] + s.idx_off);
        }
        __syncthreads();
        return;
    }
}

// token index of element e of sub-step u in the iteration starting at base (see load_items)
template <int VEC>
static __device__ __forceinline__ int item_index(int base, int u, int e)
{
    return VEC == 4 ? base + (u * kThreads + (int)threadIdx.x) * 4 + e
                    : base + (u * 4 + e) * kThreads + (int)threadIdx.x;
}

template <int VEC, bool BF16>
static __device__ __forceinline__ void sel_load_iter(const LogitRow rowp, const uint32_t *mrow, int base, int end,
                                                     float v[4][4])
{
    int idx[4];
#pragma unroll
    for (int u = 0; u < 4; u++) load_items<VEC, BF16, true>(rowp, mrow, base, u, end, v[u], idx);
}

// filters one 16384-element iteration into the buffer; returns with the block in step
template <int VEC>
static __device__ __forceinline__ void sel_process_iter(Sel &s, const float v[4][4], int base, int end, int &cnt0)
{
    SelCtl *c = s.c;
    const float tau = c->tau;
    int n = 0;
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
        for (int e = 0; e < 4; e++) n += (v[u][e] > tau) ? 1 : 0;  // out of range reads -inf
    if (n) {
        int slot = atomicAdd(&c->cnt, n);
        if (slot + n > s.cap) {
            c->overflow = 1;
        } else {
            u64 *b = s.buf[c->cur];
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (v[u][e] > tau) b[slot++] = make_key(v[u][e], item_index<VEC>(base, u, e) + s.idx_off);
        }
    }
    __syncthreads();
    if (c->overflow) {
        __syncthreads();
        if (threadIdx.x == 0) { c->cnt = cnt0; c->overflow = 0; }
        __syncthreads();
        if (c->cnt > s.n) sel_raise(s);
#pragma unroll
        for (int u = 0; u < 4; u++) {
            int idx[4];
#pragma unroll
            for (int e = 0; e < 4; e++) idx[e] = item_index<VEC>(base, u, e);
            sel_append_exact(s, v[u], idx, end);
        }
    } else if (c->cnt > s.n + ((s.cap - s.n) >> 1)) {
        // keep head-room so that the optimistic append rarely has to be rolled back
        sel_raise(s);
    }
    cnt0 = c->cnt;
    __syncthreads();
}

// Streams elements [begin, end) of one row through the selection.  Elements are visited in
// ascending token order per 16384-element iteration, which is what makes the strict `> tau` test
// exact: an element equal to the N-th best value arrives after N better-or-earlier ones.
// The first 4096 elements are appended exactly and tau raised from them, so that it is a real
// bound before the bulk arrives; after that the loads of the next iteration are issued before the
// current one is filtered (two iterations, 128 KB, in flight per CTA).  On return the buffer
// holds a superset of the best N keys of the range, at most 2N of them.
template <int VEC, bool BF16>
static __device__ void sel_stream_pass(Sel &s, const LogitRow rowp, const uint32_t *mrow, int begin, int end,
                                       bool optimistic)
{
    SelCtl *c = s.c;
    constexpr int STEP = kThreads * 16;
    const int first_end = min(end, begin + kSelTile);
    {
        float v[4];
        int idx[4];
        load_items<VEC, BF16, true>(rowp, mrow, begin, 0, first_end, v, idx);
        sel_append_exact(s, v, idx, first_end);
        if (c->cnt > s.n) {
            // optimistic bound: the first sub-tile taken as a sample of the range, tau is set where
            // about 2.5 N elements of the whole range should pass (the caller checks the outcome)
            const int n_saved = s.n;
            if (optimistic) {
                const long long m = (5ll * s.n * kSelTile) / (2ll * (long long)(end - begin));
                const int target = (int)max(32ll, min((long long)s.n, m));
                // the floor of 32 may exceed N: a sample with fewer keys than that (a sparse mask) keeps N,
                // which it is known to exceed - the selection needs more keys than it is asked for
                if (target < c->cnt) s.n = target;
            }
            sel_raise(s);
            s.n = n_saved;
        }
    }
    int cnt0 = c->cnt;
    int base = first_end;
    if (base < end) {
        float va[4][4], vb[4][4];
        sel_load_iter<VEC, BF16>(rowp, mrow, base, end, va);
        for (;;) {
            int nb = base + STEP;
            bool more = nb < end;
            if (more) sel_load_iter<VEC, BF16>(rowp, mrow, nb, end, vb);
            sel_process_iter<VEC>(s, va, base, end, cnt0);
            if (!more) break;
            base = nb;
            nb = base + STEP;
            more = nb < end;
            if (more) sel_load_iter<VEC, BF16>(rowp, mrow, nb, end, va);
            sel_process_iter<VEC>(s, vb, base, end, cnt0);
            if (!more) break;
            base = nb;
        }
    }
}

template <int VEC, bool BF16>
static __device__ void sel_stream(Sel &s, const LogitRow rowp, const uint32_t *mrow, int begin, int end)
{
    SelCtl *c = s.c;
    // With a bound guessed from the first sub-tile the buffer rarely fills and tau is rarely raised
    // again.  The guess is checked: the survivors are exactly the elements above the final tau, so
    // N or more of them contain the best N; fewer (the first sub-tile was not representative) and
    // the range is streamed again with the safe bound, the N-th best seen so far.
    const bool try_optimistic = end - begin >= 4 * kSelTile;
    sel_stream_pass<VEC, BF16>(s, rowp, mrow, begin, end, try_optimistic);
    if (try_optimistic) {
        __syncthreads();
        const bool short_of = c->cnt < s.n && !(c->tau == -CUDART_INF_F);  // any bound but "none" may have been too high
        __syncthreads();
        if (short_of) {
            sel_reset(s);
            sel_stream_pass<VEC, BF16>(s, rowp, mrow, begin, end, false);
        }
    }
    if (c->cnt > 2 * s.n) sel_raise(s);
    if (c->cnt > 2 * s.n) sel_compact(s);
}

// A whole row by one CTA when time matters more than certainty (the second chance of a row of the
// flat step, stg_flat.cu): the bound is set from the first sub-tile as in sel_stream_pass, but
// generously - about `over` / 2 times N elements of the row should pass - and the rest of the row is
// filtered against it without any block-wide step: a thread that finds an element above the bound
// appends it by itself.  The outcome is checked like every optimistic bound here (N or more
// survivors, none dropped for lack of room); on failure the exact, self-correcting sel_stream runs.
// `preset`: the caller knows a bound below which no element of the best N lies (tau_preset); the
// sample is skipped and the whole range filtered against it.
template <int VEC, bool BF16>
static __device__ void sel_stream_generous(Sel &s, const LogitRow rowp, const uint32_t *mrow, int begin, int end, int over,
                                           bool preset, float tau_preset)
{
    SelCtl *c = s.c;
    constexpr int STEP = kThreads * 16;
    int first_end = min(end, begin + kSelTile);
    bool ok = preset || end - begin >= 4 * kSelTile;
    if (preset) {
        if (threadIdx.x == 0) c->tau = tau_preset;
        __syncthreads();
        first_end = begin;
    } else if (ok) {
        float v[4];
        int idx[4];
        load_items<VEC, BF16, true>(rowp, mrow, begin, 0, first_end, v, idx);
        sel_append_exact(s, v, idx, first_end);
        ok = c->cnt > s.n;
        if (ok) {
            const int n_saved = s.n;
            const long long m = ((long long)over * s.n * kSelTile) / (2ll * (long long)(end - begin));
            const int target = (int)max(32ll, min((long long)s.n, m));
            if (target < c->cnt) s.n = target;  // as in sel_stream_pass: never more keys wanted than the sample holds
            sel_raise(s);
            s.n = n_saved;
        }
    }
    if (ok) {
        const float tau = c->tau;
        u64 *b = s.buf[c->cur];
        float va[4][4], vb[4][4];
        int base = first_end;
        auto filter = [&](const float (&v)[4][4], int at) {
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (v[u][e] > tau) {  // out of range and masked elements read -inf
                        const int slot = atomicAdd(&c->cnt, 1);
                        if (slot < s.cap) b[slot] = make_key(v[u][e], item_index<VEC>(at, u, e) + s.idx_off);
                    }
        };
        if (base < end) {
            sel_load_iter<VEC, BF16>(rowp, mrow, base, end, va);
            for (;;) {
                int nb = base + STEP;
                bool more = nb < end;
                if (more) sel_load_iter<VEC, BF16>(rowp, mrow, nb, end, vb);
                filter(va, base);
                if (!more) break;
                base = nb;
                nb = base + STEP;
                more = nb < end;
                if (more) sel_load_iter<VEC, BF16>(rowp, mrow, nb, end, va);
                filter(vb, base);
                if (!more) break;
                base = nb;
            }
        }
        __syncthreads();
        ok = c->cnt >= s.n && c->cnt <= s.cap;
        __syncthreads();
    }
    if (!ok) {
        sel_reset(s);
        sel_stream<VEC, BF16>(s, rowp, mrow, begin, end);
        return;
    }
    if (c->cnt > 2 * s.n) sel_raise(s);
    if (c->cnt > 2 * s.n) sel_compact(s);
}

// Appends `count` keys from global memory (another chunk's survivors).
static __device__ void sel_append_keys(Sel &s, const u64 *keys, int count, bool reduce = true)
{
    SelCtl *c = s.c;
    for (int base = 0; base < count; base += kSelTile) {
        int m = min(kSelTile, count - base);
        __syncthreads();
        if (c->cnt + m > s.cap) sel_raise(s);
        u64 *b = s.buf[c->cur];
        const int cnt = c->cnt;
        __syncthreads();
        for (int e = threadIdx.x; e < m; e += kThreads) b[cnt + e] = __ldcg(keys + base + e);
        __syncthreads();
        if (threadIdx.x == 0) c->cnt = cnt + m;
        __syncthreads();
    }
    if (reduce && c->cnt > 2 * s.n) sel_raise(s);
    if (reduce && c->cnt > 2 * s.n) sel_compact(s);
}

// ---- block-wide bitonic sort, descending, of `p2` (power of two) 64-bit keys in shared memory --
static __device__ void bitonic_sort_desc(u64 *a, int p2)
{
    for (int k = 2; k <= p2; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = threadIdx.x; t < (p2 >> 1); t += kThreads) {
                int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                int l = i | j;
                bool desc = ((i & k) == 0);
                u64 x = a[i], y = a[l];
                if ((x < y) == desc) { a[i] = y; a[l] = x; }
            }
            __syncthreads();
        }
    }
}

// descending rank sort of `cnt` distinct keys from src into dst (quadratic work, two barriers):
// cheaper than the bitonic network for the few hundred candidates of a typical row
static __device__ void rank_sort_desc(const u64 *src, u64 *dst, int cnt)
{
    for (int t = threadIdx.x; t < cnt; t += kThreads) {
        const u64 k = src[t];
        int rank = 0;
        for (int j = 0; j < cnt; j++) rank += (src[j] > k) ? 1 : 0;
        dst[rank] = k;
    }
    __syncthreads();
}

static __device__ __forceinline__ int pow2_ceil(int n)
{
    int p = 1;
    while (p < n) p <<= 1;
    return p;
}

// ---- history lookups of the top-k path ---------------------------------------------------------
// occurrences of `id` in the whole history and inside the repetition window
// (Sampler.cs:271-279).  All threads scan the same addresses, so the loads broadcast.
static __device__ __forceinline__ void count_occurrences(const int32_t *hist, int hlen, int wstart, int id,
                                                  int &occ_all, int &occ_w)
{
    int a = 0, w = 0;
    for (int h = 0; h < hlen; h++) {
        int x = __ldg(hist + h);
        if (x == id) { a++; w += (h >= wstart) ? 1 : 0; }
    }
    occ_all = a;
    occ_w = w;
}

// powf(rep, occ) as the host's libm gives it (table built by the planner), falling back to a
// correctly rounded double evaluation beyond the table.
static __device__ __forceinline__ float pow_rep(const float *tab, float rep, int occ)
{
    if (tab != nullptr && occ <= kPowTab) return __ldg(tab + occ - 1);
    return (float)pow((double)rep, (double)occ);
}

// Threshold of the `want` largest values of P[0..cnt) (block-wide radix select, most significant
// byte first).  On return every P > *thr belongs to the `want` largest, and *need of the entries
// equal to *thr complete them (which ones is the caller's tie rule).  All threads call it;
// 1 <= want <= cnt.
static __device__ void select_thr32(SelCtl *c, const uint32_t *P, int cnt, int want_in, uint32_t *thr, int *need)
{
    const int tid = threadIdx.x;
    __syncthreads();
    if (tid == 0) { c->want = want_in; c->prefix = 0; c->stop = 0; }
    for (int pass = 3; pass >= 0; --pass) {
        if (tid < 256) c->hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = (uint32_t)c->prefix;
        const int sh = 8 * pass;
        for (int e = tid; e < cnt; e += kThreads) {
            const uint32_t k = P[e];
            if (pass == 3 || (k >> (sh + 8)) == prefix) atomicAdd(&c->hist[(k >> sh) & 255u], 1u);
        }
        __syncthreads();
        if (tid < 32) {
            unsigned h[8];
            unsigned local = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) { h[j] = c->hist[tid * 8 + j]; local += h[j]; }
            const unsigned want = (unsigned)c->want;  // read before the shuffles order the lanes
            unsigned run = local;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                unsigned t = __shfl_down_sync(0xFFFFFFFFu, run, o);
                if (tid + o < 32) run += t;
            }
            const unsigned above = run - local;
            if (above < want && want <= above + local) {
                unsigned acc = above;
#pragma unroll
                for (int j = 7; j >= 0; --j) {
                    if (want <= acc + h[j]) {
                        const uint32_t np = (prefix << 8) | (uint32_t)(tid * 8 + j);
                        c->prefix = np;
                        c->want = (int)(want - acc);
                        if (pass == 0) {
                            c->stop = 1;  // np is the exact threshold value
                            c->cut = (int)h[j];  // entries equal to it
                        } else if (h[j] == want - acc) {
                            c->stop = 2;  // the whole bucket is taken: no ties to resolve
                            c->thr = (u64)np << sh;
                        }
                        break;
                    }
                    acc += h[j];
                }
            }
        }
        __syncthreads();
        if (c->stop) break;
    }
    if (c->stop == 2) {
        const uint32_t lo = (uint32_t)c->thr;  // everything >= lo is taken
        *thr = lo ? lo - 1u : 0u;
        *need = lo ? 0 : 0x7FFFFFFF;           // lo == 0: every entry, also those equal to 0
    } else {
        *thr = (uint32_t)c->prefix;
        // all the entries equal to the threshold are wanted: nothing to rank, they are taken like the ones above
        const uint32_t at = (uint32_t)c->prefix;
        if (c->want >= c->cut && at != 0u) { *thr = at - 1u; *need = 0; }
        else *need = c->want;
    }
    __syncthreads();
}

struct FinishOut {
    int token;
    float prob;
    uint32_t flags;
};

constexpr int kFastFinishK = 256;  // up to this top_k the candidates are selected, not sorted

static __device__ void finish_topk_sort(Sel &s, const RowPlan &rp, const int32_t *hist, const float *pow_tab);
static __device__ void finish_topk_draw(Sel &s, const RowPlan &rp, float uniform, FinishOut *out_sh, int32_t *o_ids,
                                        float *o_vals, float *o_probs);

// Candidate order for a small k without sorting the candidates: the exact candidate set by radix
// select on the raw keys (Sampler.cs:225, :242-249), their penalised values (Sampler.cs:263-287),
// the k best of those by a second radix select, and a rank sort of just these k in the stable
// order of Sampler.cs:289-294 (penalised value descending, raw order among equals).  Leaves vals /
// ids of the first k at the start of the buffer that is not active.
static __device__ __forceinline__ bool penalties_only_demote(const RowPlan &rp)
{
    return !rp.has_penalty || (rp.rep >= 1.0f && rp.pres >= 0.f && rp.freq >= 0.f);
}

static __device__ void finish_topk_select(Sel &s, const RowPlan &rp, const int32_t *hist, const float *pow_tab)
{
    SelCtl *c = s.c;
    const int tid = threadIdx.x;
    const int k = rp.top_k;
    const int keep = rp.has_penalty ? rp.sel : k;
    // The reference penalises the `sel` best raw logits and takes the k best penalised ones.  When
    // no penalty can raise a logit (repetition >= 1, presence and frequency >= 0) any superset of
    // those `sel` gives the same k candidates in the same order: a logit outside the raw top-`sel`
    // has at least k unpenalised logits above it and penalties only move others further down.  So
    // the exact raw selection is skipped then, and it runs only when a penalty may promote.
    if (!penalties_only_demote(rp) && c->cnt > keep) {
        if (c->cnt <= 512) {
            // few candidates: rank them directly (fewer barriers than the radix passes)
            const int m = c->cnt;
            const u64 *src = s.buf[c->cur];
            u64 *dst = s.buf[c->cur ^ 1];
            __syncthreads();
            for (int t = tid; t < m; t += kThreads) {
                const u64 key = src[t];
                int rank = 0;
                for (int j = 0; j < m; j++) rank += (src[j] > key) ? 1 : 0;
                if (rank < keep) dst[rank] = key;
            }
            __syncthreads();
            if (tid == 0) { c->cnt = keep; c->cur ^= 1; }
            __syncthreads();
        } else {
            const int n_saved = s.n;
            s.n = keep;
            sel_compact(s);
            s.n = n_saved;
        }
    }
    const int cnt = c->cnt;
    const u64 *a = s.buf[c->cur];
    unsigned char *bb = (unsigned char *)s.buf[c->cur ^ 1];
    float *vals = (float *)bb;
    int *ids = (int *)(vals + k);
    const int ke = min(k, cnt);
    if (!rp.has_penalty && cnt <= 256) {
        for (int t = tid; t < k; t += kThreads)
            if (t >= ke) { vals[t] = -CUDART_INF_F; ids[t] = -1; }
        for (int t = tid; t < cnt; t += kThreads) {
            const u64 key = a[t];
            int rank = 0;
            for (int j = 0; j < cnt; j++) rank += (a[j] > key) ? 1 : 0;
            if (rank < ke) { vals[rank] = key_val(key); ids[rank] = key_idx(key); }
        }
        __syncthreads();
        return;
    }
    // scratch behind vals / ids / probs
    uint32_t *P = (uint32_t *)(bb + (((size_t)3 * k * 4 + 15) & ~(size_t)15));  // penalised values, ordered bits
    uint32_t *SP = P + ((cnt + 3) & ~3);                                        // ... of the k selected
    u64 *SK = (u64 *)(SP + ((k + 3) & ~3));                                     // their raw keys
    int hslots = 64;
    while (hslots < 2 * rp.hist_len) hslots <<= 1;
    int *hkey = (int *)(SK + k);
    int *hall = hkey + hslots, *hwin = hall + hslots;
    const bool use_hash = rp.has_penalty && (char *)(hwin + hslots) <= (char *)(s.buf[c->cur ^ 1] + s.cap);
    if (use_hash) {
        for (int t = tid; t < hslots; t += kThreads) { hkey[t] = -1; hall[t] = 0; hwin[t] = 0; }
        __syncthreads();
        for (int t = tid; t < rp.hist_len; t += kThreads) {
            const int id = __ldg(hist + t);
            if (id < 0) continue;  // never a candidate, and -1 marks an empty slot
            int h = (int)(((unsigned)id * 2654435761u) >> 7) & (hslots - 1);
            for (;;) {
                int old = atomicCAS(&hkey[h], -1, id);
                if (old == -1 || old == id) break;
                h = (h + 1) & (hslots - 1);
            }
            atomicAdd(&hall[h], 1);
            if (t >= rp.window_start) atomicAdd(&hwin[h], 1);
        }
        __syncthreads();
    }
    for (int t = tid; t < cnt; t += kThreads) {
        float v = key_val(a[t]);
        const int id = key_idx(a[t]);
        int occ_all = 0, occ_w = 0;
        if (!rp.has_penalty) {
            // no penalties: the candidates compete with their raw values
        } else if (use_hash) {
            int h = (int)(((unsigned)id * 2654435761u) >> 7) & (hslots - 1);
            for (;;) {
                const int kx = hkey[h];
                if (kx == id) { occ_all = hall[h]; occ_w = hwin[h]; break; }
                if (kx == -1) break;
                h = (h + 1) & (hslots - 1);
            }
        } else {
            count_occurrences(hist, rp.hist_len, rp.window_start, id, occ_all, occ_w);
        }
        if (occ_all > 0) {
            if (rp.rep != 1.0f && occ_w > 0) {
                float pw = pow_rep(pow_tab, rp.rep, occ_w);
                v = v > 0.f ? __fdiv_rn(v, pw) : __fmul_rn(v, pw);
            }
            float add = __fadd_rn(rp.pres, __fmul_rn(rp.freq, (float)occ_all));
            v = __fsub_rn(v, add);
        }
        P[t] = ord32(v);
    }
    __syncthreads();
    if (cnt <= 256) {
        // few candidates: the rank in the stable order is the position
        for (int t = tid; t < k; t += kThreads) {
            if (t >= ke) { vals[t] = -CUDART_INF_F; ids[t] = -1; }
        }
        for (int t = tid; t < cnt; t += kThreads) {
            const uint32_t pv = P[t];
            const u64 key = a[t];
            int rank = 0;
            for (int j = 0; j < cnt; j++) {
                const uint32_t pj = P[j];
                rank += (pj > pv || (pj == pv && a[j] > key)) ? 1 : 0;
            }
            if (rank < ke) { vals[rank] = unord32(pv); ids[rank] = key_idx(key); }
        }
        __syncthreads();
        return;
    }
    uint32_t thr;
    int need;
    select_thr32(c, P, cnt, ke, &thr, &need);
    if (tid == 0) c->cnt2 = 0;
    __syncthreads();
    for (int t = tid; t < cnt; t += kThreads) {
        const uint32_t pv = P[t];
        bool take = pv > thr;
        if (pv == thr && need > 0) {
            // ties at the k-th penalised value: the earlier ones in raw order complete the k
            const u64 key = a[t];
            int r = 0;
            for (int j = 0; j < cnt; j++) r += (P[j] == thr && a[j] > key) ? 1 : 0;
            take = r < need;
        }
        if (take) {
            const int slot = atomicAdd(&c->cnt2, 1);
            if (slot < k) { SP[slot] = pv; SK[slot] = a[t]; }
        }
    }
    __syncthreads();
    const int got = min(c->cnt2, k);
    for (int t = tid; t < k; t += kThreads) {
        if (t >= got) { vals[t] = -CUDART_INF_F; ids[t] = -1; continue; }
        const uint32_t pv = SP[t];
        const u64 key = SK[t];
        int rank = 0;
        for (int j = 0; j < got; j++) {
            const uint32_t pj = SP[j];
            rank += (pj > pv || (pj == pv && SK[j] > key)) ? 1 : 0;
        }
        vals[rank] = unord32(pv);
        ids[rank] = key_idx(key);
    }
    __syncthreads();
}

// Finishes the top-k path for one row whose candidates - the exact top-`sel` raw logits, possibly
// with some extra ones below them - sit (unsorted) in the active buffer: order the k best by
// penalised value, softmax over them, min-p, top-p, draw.
// Every fp32 operation is issued separately (no fused multiply-add), in the order of
// Sampler.cs:257-349.  `vals`/`ids`/`probs` views alias the inactive buffer.
static __device__ void finish_topk(Sel &s, const RowPlan &rp, const int32_t *hist, const float *pow_tab,
                            float uniform, FinishOut *out_sh, int32_t *o_ids, float *o_vals,
                            float *o_probs, unsigned long long *tk = nullptr)
{
    SelCtl *c = s.c;
    const int tid = threadIdx.x;
    const int cnt = c->cnt;
    const int k = rp.top_k;
    if (cnt == 0) {  // Sampler.cs:254-255: no finite logit -> Greedy(raw) == token 0
        if (tid == 0) { out_sh->token = 0; out_sh->prob = 0.f; out_sh->flags = kPathTopKNoFinite | (1u << 6); }
        for (int t = tid; t < k; t += kThreads) {
            if (o_ids) o_ids[t] = -1;
            if (o_vals) o_vals[t] = -CUDART_INF_F;
            if (o_probs) o_probs[t] = 0.f;
        }
        __syncthreads();
        return;
    }
    tick(tk, 20);
    if (k <= kFastFinishK) {
        finish_topk_select(s, rp, hist, pow_tab);
    } else {
        finish_topk_sort(s, rp, hist, pow_tab);
    }
    tick(tk, 21);  // diagnostic stamps 20 .. 22: order the k best | softmax, filters, draw
    finish_topk_draw(s, rp, uniform, out_sh, o_ids, o_vals, o_probs);
    tick(tk, 22);
}

// Candidate order by sorting everything (any k): leaves vals / ids of the first k in the buffer
// that is not active.
static __device__ void finish_topk_sort(Sel &s, const RowPlan &rp, const int32_t *hist, const float *pow_tab)
{
    SelCtl *c = s.c;
    const int tid = threadIdx.x;
    int cnt = c->cnt;
    u64 *a = s.buf[c->cur];
    u64 *b = s.buf[c->cur ^ 1];
    const int k = rp.top_k;
    const int sel = rp.sel;
    // raw order (Sampler.cs:242-249): descending value, ascending token on ties
    const bool small = cnt <= 192;  // the quadratic rank sort only wins for a handful of keys
    const int p2 = pow2_ceil(max(cnt, 2));
    u64 *raw;    // sorted raw candidates
    u64 *work;   // the other buffer
    if (small) {
        rank_sort_desc(a, b, cnt);
        raw = b; work = a;
    } else {
        for (int t = cnt + tid; t < p2; t += kThreads) a[t] = 0ull;
        __syncthreads();
        bitonic_sort_desc(a, p2);
        raw = a; work = b;
    }
    u64 *pen = work;  // sorted penalised keys when has_penalty
    const int m_all = cnt;
    cnt = min(cnt, sel);  // the reference's candidates: the best `sel` raw logits (Sampler.cs:225)

    if (rp.has_penalty) {
        // penalise each candidate (Sampler.cs:263-287), then stable re-sort by penalised value
        // (Sampler.cs:289-294): key = (penalised value, raw rank).  Occurrence counts come from a
        // hash of the history built once (token -> count, count inside the window) when it fits
        // behind the keys, else from a scan of the history per candidate.
        u64 *unsorted = small ? raw + m_all : work;
        const int m = small ? cnt : p2;
        int hslots = 64;
        while (hslots < 2 * rp.hist_len) hslots <<= 1;
        int *hkey = (int *)(unsorted + m);
        int *hall = hkey + hslots, *hwin = hall + hslots;
        const bool use_hash = (char *)(hwin + hslots) <= (char *)(s.buf[unsorted >= s.buf[1] ? 1 : 0] + s.cap);
        if (use_hash) {
            for (int t = tid; t < hslots; t += kThreads) { hkey[t] = -1; hall[t] = 0; hwin[t] = 0; }
            __syncthreads();
            for (int t = tid; t < rp.hist_len; t += kThreads) {
                const int id = __ldg(hist + t);
                if (id < 0) continue;  // never a candidate, and -1 marks an empty slot
                int h = (int)(((unsigned)id * 2654435761u) >> 7) & (hslots - 1);
                for (;;) {
                    int old = atomicCAS(&hkey[h], -1, id);
                    if (old == -1 || old == id) break;
                    h = (h + 1) & (hslots - 1);
                }
                atomicAdd(&hall[h], 1);
                if (t >= rp.window_start) atomicAdd(&hwin[h], 1);
            }
            __syncthreads();
        }
        for (int t = tid; t < m; t += kThreads) {
            u64 key2 = 0ull;
            if (t < cnt) {
                float v = key_val(raw[t]);
                int id = key_idx(raw[t]);
                int occ_all = 0, occ_w = 0;
                if (use_hash) {
                    int h = (int)(((unsigned)id * 2654435761u) >> 7) & (hslots - 1);
                    for (;;) {
                        const int kx = hkey[h];
                        if (kx == id) { occ_all = hall[h]; occ_w = hwin[h]; break; }
                        if (kx == -1) break;
                        h = (h + 1) & (hslots - 1);
                    }
                } else {
                    count_occurrences(hist, rp.hist_len, rp.window_start, id, occ_all, occ_w);
                }
                if (occ_all > 0) {
                    if (rp.rep != 1.0f && occ_w > 0) {
                        float pw = pow_rep(pow_tab, rp.rep, occ_w);
                        v = v > 0.f ? __fdiv_rn(v, pw) : __fmul_rn(v, pw);
                    }
                    float add = __fadd_rn(rp.pres, __fmul_rn(rp.freq, (float)occ_all));
                    v = __fsub_rn(v, add);
                }
                key2 = ((u64)ord32(v) << 32) | (u64)(0xFFFFFFFFu - (uint32_t)t);
            }
            unsorted[t] = key2;
        }
        __syncthreads();
        if (small) rank_sort_desc(unsorted, work, cnt);
        else bitonic_sort_desc(work, p2);
    }

    // first k candidates -> registers -> compact arrays over the buffer that is no longer needed
    constexpr int R = kMaxSel / kThreads;
    float rv[R];
    int ri[R];
#pragma unroll
    for (int j = 0; j < R; j++) {
        int t = tid + j * kThreads;
        rv[j] = -CUDART_INF_F;
        ri[j] = -1;
        if (t < k && t < cnt) {
            if (rp.has_penalty) {
                u64 k2 = pen[t];
                int raw_rank = (int)(0xFFFFFFFFu - (uint32_t)k2);
                rv[j] = unord32((uint32_t)(k2 >> 32));
                ri[j] = key_idx(raw[raw_rank]);
            } else {
                rv[j] = key_val(raw[t]);
                ri[j] = key_idx(raw[t]);
            }
        }
    }
    __syncthreads();
    // the draw reads vals / ids from the buffer that is not active
    if (tid == 0 && work != b) c->cur ^= 1;
    __syncthreads();
    float *vals = (float *)work;
    int *ids = (int *)(vals + k);
#pragma unroll
    for (int j = 0; j < R; j++) {
        int t = tid + j * kThreads;
        if (t < k) { vals[t] = rv[j]; ids[t] = ri[j]; }
    }
    __syncthreads();
}

// Softmax over the k ordered candidates, min-p, top-p and the draw (Sampler.cs:296-349).  vals / ids
// sit at the start of the buffer that is not active.
static __device__ void finish_topk_draw(Sel &s, const RowPlan &rp, float uniform, FinishOut *out_sh, int32_t *o_ids,
                                        float *o_vals, float *o_probs)
{
    SelCtl *c = s.c;
    const int tid = threadIdx.x;
    const int k = rp.top_k;
    float *vals = (float *)s.buf[c->cur ^ 1];
    int *ids = (int *)(vals + k);
    float *probs = (float *)(ids + k);
    const float inv_t = rp.temperature == 1.0f ? 1.0f : __fdiv_rn(1.0f, rp.temperature);
    const float mx = __fmul_rn(vals[0], inv_t);
    for (int t = tid; t < k; t += kThreads) {
        float v = vals[t];
        float e = 0.f;
        if (!(isinf(v) && v < 0.f)) e = (float)exp((double)__fsub_rn(__fmul_rn(v, inv_t), mx));
        probs[t] = e;
    }
    __syncthreads();
    __shared__ float sh_inv_sum;
    if (tid == 0) {
        float sum = 0.f;
        for (int t = 0; t < k; t++) sum = __fadd_rn(sum, probs[t]);
        sh_inv_sum = sum > 0.f ? __fdiv_rn(1.0f, sum) : 0.f;
    }
    __syncthreads();
    const float inv_sum = sh_inv_sum;
    for (int t = tid; t < k; t += kThreads) probs[t] = __fmul_rn(probs[t], inv_sum);
    __syncthreads();
    if (tid == 0) {
        int count = k;
        if (rp.min_p > 0.f) {
            float thr = __fmul_rn(rp.min_p, probs[0]);
            for (int t = 0; t < count; t++)
                if (probs[t] < thr) { count = t; break; }
        }
        // The reference runs three sequential sums over the surviving probabilities - the top-p running
        // sum, the kept mass, the CDF of the draw (Sampler.cs:318-349) - and all three add the same values
        // in the same order from 0, so their partial sums are the same floats: one chain of additions,
        // kept in `pre`, serves all three.
        float *pre = (float *)s.buf[c->cur];  // the candidates' buffer: the selection is over, nobody reads it again
        const bool cut = rp.top_p < 1.0f && rp.top_p > 0.f;
        float acc = 0.f;
        for (int t = 0; t < count; t++) {
            acc = __fadd_rn(acc, probs[t]);
            pre[t] = acc;
            if (cut && acc >= rp.top_p) { count = t + 1; break; }
        }
        const float kept = count > 0 ? pre[count - 1] : 0.f;
        float r = __fmul_rn(uniform, kept);
        int tok = ids[0];
        float pr = probs[0];
        uint32_t fl = kPathTopK | (1u << 5);
        for (int t = 0; t < count; t++) {
            const float cacc = pre[t];
            if (r <= cacc && ids[t] >= 0) {
                const float prev = t > 0 ? pre[t - 1] : 0.f;
                tok = ids[t]; pr = probs[t]; fl = kPathTopK;
                // the draw within 1e-6 (of the kept mass) of the step below or above the token
                if (r - prev <= kNearTol * kept || cacc - r <= kNearTol * kept) fl |= kFlagNearBoundary;
                break;
            }
        }
        out_sh->token = tok;
        out_sh->prob = kept > 0.f ? pr / kept : 0.f;
        out_sh->flags = fl;
    }
    for (int t = tid; t < k; t += kThreads) {
        if (o_ids) o_ids[t] = ids[t];
        if (o_vals) o_vals[t] = vals[t];
        if (o_probs) o_probs[t] = probs[t];
    }
    __syncthreads();
}

}  // namespace stg
