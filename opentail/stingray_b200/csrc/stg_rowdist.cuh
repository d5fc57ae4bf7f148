// The full-vocabulary pipeline for one row, run by one 1024-thread CTA:
//   bias -> history penalties -> 1/T -> softmax -> [top-k] -> min-p -> top-p -> normalise -> draw
// (Sampler.Sample's slow path, src/OpenTail.Stingray.Engine/Sampler.cs:41-95, and
// BuildFilteredDistribution, :118-163), plus GreedyWithHistoryPenalties (:421-437).
//
// The row is read from HBM once; later passes re-read it (or the exp values kept in a per-CTA
// scratch row) from L2.  Every sum the reference accumulates sequentially in fp32 is reproduced
// bit for bit (stg_emul2.cuh); the one vectorised sum (Normalize's TensorPrimitives.Sum, whose
// order the reference does not pin) is accumulated in fp64 and rounded once.
//
// History and bias adjustments touch a few hundred tokens: they are gathered into a shared-memory
// hash table (token -> adjusted logit) that the first pass consults through a folded bitmap.
//
// top-p is sort-free over the vocabulary.  A histogram of the exp values (4096 bins: exponent and
// 5 mantissa bits) bounds the nucleus; the candidates above the bound are scattered into bin order
// (largest bin first, arbitrary order inside a bin); only the bins in which the reference's
// sequential cumulative sum can change binade or reach top_p are sorted; the emulated sum then
// runs over that partially ordered sequence and refuses to replay an unsorted stretch element by
// element - in that case the stretch is sorted and the sum run again.
#pragma once
#include <cuda_runtime.h>
#include <limits.h>
#include <math_constants.h>
#include <stdint.h>
#include <string.h>

#include "stg_emul.cuh"
#include "stg_emul2.cuh"
#include "stg_select.cuh"
#include "stg_types.h"

namespace stg {

constexpr int kBins = 4096;        // exp-value histogram: 32 binades below 2.0, 7 mantissa bits each
constexpr int kBinExp0 = 96;       // biased exponent of the lowest binade with bins of its own
constexpr int kMaxDirty = 1024;    // bins sorted individually before giving up on the partial order
constexpr int kDirtyRound = 2048;  // elements rank-sorted per round
constexpr int kMaxOvSlots = 4096;  // hash slots => at most 2048 history + bias entries per row
static_assert(kSortCap * 4 >= kStageBytes, "the staged loops borrow the key region");
static_assert(kBins == 4 * kThreads, "the bin scans assign 4 bins to a thread");

// shared-memory arena of a row item
constexpr int kOffKeys = 0;                                      // u32[kSortCap] | hash table | Sel buffers
constexpr int kOffCount = kSortCap * 4;                          // u32[kBins]
constexpr int kOffMass = kOffCount + kBins * 4;                  // float[kBins]
constexpr int kOffBinOff = kOffMass + kBins * 4;                 // u32[kBins]: start of each bin in the list
constexpr int kOffEmul = kOffBinOff + kBins * 4;                 // Emul2Work
constexpr int kOffReplayOk = kOffEmul + (int)sizeof(Emul2Work);  // u8[kMaxSubTiles]
constexpr int kOffBinExp = kOffReplayOk + kMaxSubTiles;          // u8[kBins]: binade of the running sum at each bin
constexpr int kOffSubSrc = kOffBinExp + kBins;                   // int[kMaxSubTiles]: list offset of each list sub-tile
constexpr int kOffSubCnt = kOffSubSrc + kMaxSubTiles * 4;        // u16[kMaxSubTiles]: entries in it
constexpr int kRowArenaEnd = kOffSubCnt + kMaxSubTiles * 2;

// histogram bin of an exp value (0 < e <= 1): values below 2^-31 share bin 0
__device__ __forceinline__ unsigned bin_of(uint32_t ebits)
{
    const int b = (int)(ebits >> 16) - (kBinExp0 << 7);
    return (unsigned)min(max(b, 0), kBins - 1);
}
// smallest bit pattern that falls into bin b or above
__device__ __forceinline__ uint32_t bin_floor_bits(int b)
{
    return b > 0 ? (uint32_t)(b + (kBinExp0 << 7)) << 16 : 0u;
}

struct RowCtl {
    EmulCtl em;
    Emul2Ctl em2;
    double red_d[32];
    int red_i[32];
    u64 red_k[32];
    float red_f[32];
    RowDist dist;
    int n_cand;       // candidates in the bin-ordered list
    int bound;        // their number as the histogram counted them
    int c_lo;         // lowest histogram bin among the candidates
    int found;        // find_kth_match result
    int running;
    int n_dirty;      // bins waiting to be sorted
    int give_up;      // partial order abandoned: sort everything
    int n_list;       // candidates in the token-ordered list (-1: no list)
    unsigned flag_bits[kBins / 32];    // bins in which the sum may change binade, meet top_p or hit a tie
    unsigned short dirty[kMaxDirty];
    int dirty_cum[kMaxDirty + 1];
    unsigned sorted_bits[kBins / 32];  // bins already sorted
};

// ---- hash table of adjusted logits ---------------------------------------------------------------
struct OvTable {
    int *key;          // token id or -1
    int *cnt_all;      // occurrences in the whole history
    int *cnt_w;        // occurrences inside the repetition window
    int *n_bias;       // bias entries for this token
    float *bias;       // their sum
    float *adj;        // adjusted (unscaled) logit
    unsigned char *bitmap;  // 65536 folded bits: bit (id & 0xFFFF) set when id may be in the table
    int mask;          // slots - 1
    __device__ __forceinline__ int find(int id) const
    {
        int h = (int)(((unsigned)id * 2654435761u) >> 7) & mask;
        for (;;) {
            int k = key[h];
            if (k == id) return h;
            if (k == -1) return -1;
            h = (h + 1) & mask;
        }
    }
    __device__ __forceinline__ int insert(int id)
    {
        int h = (int)(((unsigned)id * 2654435761u) >> 7) & mask;
        for (;;) {
            int old = atomicCAS(&key[h], -1, id);
            if (old == -1 || old == id) return h;
            h = (h + 1) & mask;
        }
    }
};

// What the streaming passes need of the table, in three registers: the arrays follow one another
// (key, cnt_all, cnt_w, n_bias, bias, adj: `slots` words each, then the bitmap).
struct OvView {
    const int *key;
    int mask;  // slots - 1
    __device__ __forceinline__ int find(int id) const
    {
        int h = (int)(((unsigned)id * 2654435761u) >> 7) & mask;
        for (;;) {
            int k = key[h];
            if (k == id) return h;
            if (k == -1) return -1;
            h = (h + 1) & mask;
        }
    }
    __device__ __forceinline__ float adj(int slot) const { return ((const float *)key)[5 * (mask + 1) + slot]; }
    __device__ __forceinline__ unsigned bitmap_byte(int i) const
    {
        return ((const unsigned char *)(key + 6 * (mask + 1)))[(i & 0xFFFF) >> 3];
    }
};

// ---- sources of the row's adjusted, temperature-scaled logits ---------------------------------
template <bool BF16>
struct SrcLogits {
    LogitRow rowp;
    const uint32_t *mrow;
    int aligned;
    float inv_t;
    bool scale;
    __device__ __forceinline__ void get8raw(int base, int n, float x[8]) const
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
    }
    __device__ __forceinline__ void get8(int base, int n, float x[8]) const
    {
        get8raw(base, n, x);
        if (scale) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = __fmul_rn(x[j], inv_t);
        }
    }
    // staged reads (stg_emul2.cuh): the thread's 8 elements as 16-byte quads copied to shared memory
    static constexpr int kQuads = BF16 ? 1 : 2;
    __device__ __forceinline__ bool stage_ok() const { return aligned != 0; }
    __device__ __forceinline__ const char *stage_src(int base) const
    {
        return (const char *)rowp.p + (size_t)base * (BF16 ? 2 : 4);
    }
    __device__ __forceinline__ void decode(int base, const float4 *q, float x[8]) const
    {
        if (BF16) {
            const uint4 t = *(const uint4 *)q;
            x[0] = bf16_lo(t.x); x[1] = bf16_hi(t.x); x[2] = bf16_lo(t.y); x[3] = bf16_hi(t.y);
            x[4] = bf16_lo(t.z); x[5] = bf16_hi(t.z); x[6] = bf16_lo(t.w); x[7] = bf16_hi(t.w);
        } else {
            x[0] = q[0].x; x[1] = q[0].y; x[2] = q[0].z; x[3] = q[0].w;
            x[4] = q[1].x; x[5] = q[1].y; x[6] = q[1].z; x[7] = q[1].w;
        }
        if (rowp.cap != 0.f) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = soft_cap(x[j], rowp.cap);
        }
        if (mrow) {
            uint32_t bits = __ldg(mrow + (base >> 5)) >> (base & 31);
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (!((bits >> j) & 1u)) x[j] = -CUDART_INF_F;
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
    static constexpr int kQuads = 2;
    __device__ __forceinline__ bool stage_ok() const { return true; }
    __device__ __forceinline__ const char *stage_src(int base) const { return (const char *)(p + base); }
    __device__ __forceinline__ void decode(int base, const float4 *q, float x[8]) const
    {
        x[0] = q[0].x; x[1] = q[0].y; x[2] = q[0].z; x[3] = q[0].w;
        x[4] = q[1].x; x[5] = q[1].y; x[6] = q[1].z; x[7] = q[1].w;
        if (scale) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = __fmul_rn(x[j], inv_t);
        }
    }
};

// the row's logits with the history / bias overrides applied on the fly (then temperature-scaled)
template <bool BF16>
struct SrcLogitsOv {
    SrcLogits<BF16> raw;  // unscaled
    OvView ov;
    float inv_t;
    bool scale;
    __device__ __forceinline__ void adjust(int base, int n, float x[8]) const
    {
        const unsigned m = ov.bitmap_byte(base);
        if (m) {
            // static indices only: a runtime index would push the whole array into local memory
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (((m >> j) & 1u) && base + j < n) {
                    int slot = ov.find(base + j);
                    if (slot >= 0) x[j] = ov.adj(slot);
                }
            }
        }
        if (scale) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = __fmul_rn(x[j], inv_t);
        }
    }
    __device__ __forceinline__ void get8(int base, int n, float x[8]) const
    {
        raw.get8raw(base, n, x);
        adjust(base, n, x);
    }
    static constexpr int kQuads = SrcLogits<BF16>::kQuads;
    __device__ __forceinline__ bool stage_ok() const { return raw.stage_ok(); }
    __device__ __forceinline__ const char *stage_src(int base) const { return raw.stage_src(base); }
    __device__ __forceinline__ void decode(int base, const float4 *q, float x[8]) const
    {
        raw.decode(base, q, x);
        adjust(base, base + 8, x);
    }
};

__device__ __forceinline__ void store8(float *p, int base, int n, const float x[8])
{
    if (base + 8 <= n) {
        __stcg((float4 *)(p + base), make_float4(x[0], x[1], x[2], x[3]));
        __stcg((float4 *)(p + base + 4), make_float4(x[4], x[5], x[6], x[7]));
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (base + j < n) __stcg(p + base + j, x[j]);
    }
}

// ---- probability of an element from its exp value -----------------------------------------------
__device__ __forceinline__ float eval_p2(float e, const RowDist &d)  // softmax, top-k, min-p
{
    float p = (d.flags & kDistScale1) ? __fmul_rn(e, d.inv1) : e;
    if (d.flags & kDistTopK) {
        if (p < d.kth) return 0.f;
        if (d.flags & kDistScale2) p = __fmul_rn(p, d.inv2);
    }
    if ((d.flags & kDistMinP) && p < d.minp_thr) p = 0.f;
    return p;
}
__device__ __forceinline__ float eval_p3(float e, int i, const RowDist &d)  // final probability
{
    float p = eval_p2(e, d);
    if (d.flags & kDistTopP) {
        if (p < d.tstar || (p == d.tstar && i > d.tie_idx_max)) p = 0.f;
    }
    if (d.flags & kDistScale3) p = __fmul_rn(p, d.inv3);
    return p;
}

// ---- providers of the emulated sums ----------------------------------------------------------------
// exp pass: computes e_i = expf(x_i - max), stores it in the scratch row, feeds the histogram.
// `load` is called by whole warps (the histogram update of bin 0 is aggregated over the warp:
// a peaked row sends nearly every value there).
template <class Src>
struct ProvExp {
    Src src;
    float mx;
    float *scratch;
    unsigned long long *hist;  // null: no histogram wanted.  Per bin: count << 40 | sum of the top 12
                               // mantissa bits (all values in a bin share the exponent)
    __device__ __forceinline__ void finish(int base, int n, float x[8]) const
    {
        int low = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float e = (base + j < n) ? expf(__fsub_rn(x[j], mx)) : 0.f;
            x[j] = e;
            if (hist && e > 0.f) {
                const uint32_t eb = __float_as_uint(e);
                const unsigned bin = bin_of(eb);
                if (bin == 0u) low++;
                else atomicAdd(&hist[bin], (1ull << 40) | (unsigned long long)(((eb & 0x7FFFFFu) | 0x800000u) >> 12));
            }
        }
        if (hist) {
            low = __reduce_add_sync(0xFFFFFFFFu, low);
            if (low && (threadIdx.x & 31) == 0)
                atomicAdd(&hist[0], ((unsigned long long)low << 40) | ((unsigned long long)low * 0xFFFull));
        }
        if (base < n) store8(scratch, base, n, x);
    }
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
        if (base < n) src.get8(base, n, x);
        finish(base, n, x);
    }
    __device__ __forceinline__ void reload(int base, int n, float x[8]) const
    {
        if (base >= n) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = 0.f;
            return;
        }
        SrcScratch s{scratch, 1.f, false};
        s.get8(base, n, x);
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (base + j >= n) x[j] = 0.f;
    }
    // staged reads
    static constexpr int kQuadsLoad = Src::kQuads, kQuadsReload = 2;
    __device__ __forceinline__ bool stage_ok() const { return src.stage_ok(); }
    __device__ __forceinline__ const char *stage_src(int base, bool re) const
    {
        return re ? (const char *)(scratch + base) : src.stage_src(base);
    }
    __device__ __forceinline__ void load_from(int base, int n, const float4 *q, float x[8]) const
    {
        src.decode(base, q, x);
        finish(base, n, x);
    }
    __device__ __forceinline__ void reload_from(int base, int n, const float4 *q, float x[8]) const
    {
        x[0] = q[0].x; x[1] = q[0].y; x[2] = q[0].z; x[3] = q[0].w;
        x[4] = q[1].x; x[5] = q[1].y; x[6] = q[1].z; x[7] = q[1].w;
    }
};

struct ProvFinal {  // final probabilities from the scratch row of exp values
    const float *scratch;
    RowDist d;        // by value: lives in registers
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
            x[j] = (base + j < n) ? eval_p3(x[j], base + j, d) : 0.f;
            if (dist_out && base + j < n) dist_out[base + j] = x[j];
        }
    }
    __device__ __forceinline__ void reload(int base, int n, float x[8]) const
    {
        if (base >= n) {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = 0.f;
            return;
        }
        SrcScratch s{scratch, 1.f, false};
        s.get8(base, n, x);
#pragma unroll
        for (int j = 0; j < 8; j++) x[j] = (base + j < n) ? eval_p3(x[j], base + j, d) : 0.f;
    }
};

struct ProvList {  // final probabilities of the top-p candidates, in token order (id << 32 | exp bits).
    // The sequence is made of sub-tiles of kSub entries: sub-tile t starts at list[sub_src[t]] and
    // holds sub_cnt[t] entries; the rest of it counts as zeros.
    const u64 *list;
    const int *sub_src;
    const unsigned short *sub_cnt;
    RowDist d;
    __device__ __forceinline__ const u64 *at(int pos) const { return list + sub_src[pos >> 8] + (pos & (kSub - 1)); }
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
        const int t = base >> 8, off = base & (kSub - 1);
        const int cnt = base < n ? (int)sub_cnt[t] : 0;
        const u64 *p = list + (base < n ? sub_src[t] : 0) + off;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float v = 0.f;
            if (off + j < cnt) {
                const u64 c = __ldcg(p + j);
                v = eval_p3(__uint_as_float((uint32_t)c), (int)(c >> 32), d);
            }
            x[j] = v;
        }
    }
    __device__ __forceinline__ void reload(int base, int n, float x[8]) const { load(base, n, x); }
    // staged reads: 8 entries of 8 bytes
    static constexpr int kQuadsLoad = 4, kQuadsReload = 4;
    __device__ __forceinline__ bool stage_ok() const { return true; }
    __device__ __forceinline__ const char *stage_src(int base, bool) const { return (const char *)at(base); }
    __device__ __forceinline__ void load_from(int base, int n, const float4 *q, float x[8]) const
    {
        const int off = base & (kSub - 1);
        const int cnt = (int)sub_cnt[base >> 8];
#pragma unroll
        for (int h = 0; h < 4; h++) {
            const uint4 v = *(const uint4 *)&q[h];
            x[2 * h] = (off + 2 * h < cnt) ? eval_p3(__uint_as_float(v.x), (int)v.y, d) : 0.f;
            x[2 * h + 1] = (off + 2 * h + 1 < cnt) ? eval_p3(__uint_as_float(v.z), (int)v.w, d) : 0.f;
        }
    }
    __device__ __forceinline__ void reload_from(int base, int n, const float4 *q, float x[8]) const
    {
        load_from(base, n, q, x);
    }
};

struct ProvKeys {  // probability bit patterns in (partial) descending order
    const uint32_t *keys;
    bool global;  // the list sits in global memory (a nucleus too wide for shared memory): staged reads pay
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
#pragma unroll
        for (int j = 0; j < 8; j++) x[j] = (base + j < n) ? __uint_as_float(keys[base + j]) : 0.f;
    }
    __device__ __forceinline__ void reload(int base, int n, float x[8]) const { load(base, n, x); }
    static constexpr int kQuadsLoad = 2, kQuadsReload = 2;
    __device__ __forceinline__ bool stage_ok() const { return global; }
    __device__ __forceinline__ const char *stage_src(int base, bool) const { return (const char *)(keys + base); }
    __device__ __forceinline__ void load_from(int base, int n, const float4 *q, float x[8]) const
    {
        x[0] = q[0].x; x[1] = q[0].y; x[2] = q[0].z; x[3] = q[0].w;
        x[4] = q[1].x; x[5] = q[1].y; x[6] = q[1].z; x[7] = q[1].w;
    }
    __device__ __forceinline__ void reload_from(int base, int n, const float4 *q, float x[8]) const
    {
        load_from(base, n, q, x);
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

__device__ __forceinline__ u64 block_max_key_r(u64 k, u64 *scratch)
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

__device__ __forceinline__ float block_max_float(float v, float *scratch)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    v = scratch[threadIdx.x & 31];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    __syncthreads();
    return v;
}

// (max value, lowest index of it) of the source as a key; 0 when nothing is > -infinity
template <class Src>
static __device__ u64 pass_max(const Src &src, int n, u64 *red)
{
    float best = -CUDART_INF_F;
    int best_i = -1;
    for (int base = threadIdx.x * 8; base < n; base += kThreads * 8 * 2) {
        float x[2][8];
        const int b1 = base + kThreads * 8;
        src.get8(base, n, x[0]);
        if (b1 < n) src.get8(b1, n, x[1]);
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (x[0][j] > best) { best = x[0][j]; best_i = base + j; }
        if (b1 < n) {
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (x[1][j] > best) { best = x[1][j]; best_i = b1 + j; }
        }
    }
    // each thread keeps its own lowest index per value (it visits ascending indices), and the key
    // order (value, then lower index) resolves ties across threads
    u64 k = best_i >= 0 ? make_key(best, best_i) : 0ull;
    return block_max_key_r(k, red);
}

// index of the `kth` (1-based) element, in token order, whose pre-top-p probability equals tstar
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

// ---- history / bias overrides ------------------------------------------------------------------------
// ApplyHistoryPenalties (Sampler.cs:367-419) after the logit bias (Sampler.cs:50-56).  One hash
// slot per distinct token: its bias sum, its occurrence counts, then - by the slot's owner thread,
// in the reference's order - bias additions, the per-occurrence repetition penalty inside the
// window, and the presence/frequency penalty over the whole history.  Requires
// 2 * (history + bias entries) <= slots <= kMaxOvSlots.
template <bool BF16>
static __device__ void build_overrides(const SampleArgs &a, const RowPlan &rp, const LogitRow rowp,
                                       const uint32_t *mrow, int n, bool with_hist, bool with_bias, OvTable &ov,
                                       unsigned char *arena, int slots)
{
    const int tid = threadIdx.x;
    ov.key = (int *)arena;
    ov.cnt_all = ov.key + slots;
    ov.cnt_w = ov.cnt_all + slots;
    ov.n_bias = ov.cnt_w + slots;
    ov.bias = (float *)(ov.n_bias + slots);
    ov.adj = ov.bias + slots;
    ov.bitmap = (unsigned char *)(ov.adj + slots);
    ov.mask = slots - 1;
    for (int t = tid; t < slots; t += kThreads) {
        ov.key[t] = -1; ov.cnt_all[t] = 0; ov.cnt_w[t] = 0; ov.n_bias[t] = 0; ov.bias[t] = 0.f;
    }
    for (int t = tid; t < 2048; t += kThreads) ((uint32_t *)ov.bitmap)[t] = 0u;
    __syncthreads();
    const int nh = with_hist ? rp.hist_len : 0;
    const int nb = with_bias ? rp.bias_len : 0;
    for (int t = tid; t < nh + nb; t += kThreads) {
        if (t < nh) {
            int id = __ldg(a.hist_ids + rp.hist_off + t);
            if ((unsigned)id >= (unsigned)n) continue;
            int h = ov.insert(id);
            atomicAdd(&ov.cnt_all[h], 1);
            if (t >= rp.window_start) atomicAdd(&ov.cnt_w[h], 1);
        } else {
            int b = t - nh;
            int id = __ldg(a.bias_ids + rp.bias_off + b);
            if ((unsigned)id >= (unsigned)n) continue;
            int h = ov.insert(id);
            atomicAdd(&ov.n_bias[h], 1);
            atomicAdd(&ov.bias[h], __ldg(a.bias_vals + rp.bias_off + b));
        }
    }
    __syncthreads();
    for (int h = tid; h < slots; h += kThreads) {
        int id = ov.key[h];
        if (id < 0) continue;
        float x = load_one<BF16>(rowp, id);
        if (mrow && !mask_bit(mrow, id)) x = -CUDART_INF_F;
        if (ov.n_bias[h] > 0) x = __fadd_rn(x, ov.bias[h]);
        const int occ_all = ov.cnt_all[h], occ_w = ov.cnt_w[h];
        if (occ_all > 0) {
            if (rp.rep != 1.0f)
                for (int r = 0; r < occ_w; r++) x = x > 0.f ? __fdiv_rn(x, rp.rep) : __fmul_rn(x, rp.rep);
            if (!(rp.pres == 0.f && rp.freq == 0.f))
                x = __fsub_rn(x, __fadd_rn(rp.pres, __fmul_rn(rp.freq, (float)occ_all)));
        }
        ov.adj[h] = x;
        atomicOr((unsigned *)ov.bitmap + ((id & 0xFFFF) >> 5), 1u << (id & 31));
    }
    __syncthreads();
}

// First pass of a row: (maximum, lowest index of it) of the (adjusted,) scaled logits as
// a key; 0 when nothing is > -infinity.  `stage` is shared memory for cp.async reads ahead.
template <class Src>
static __device__ __noinline__ u64 pass_max_staged(const Src &src_in, int n, u64 *red, unsigned char *stage,
                                                   int stage_bytes)
{
    const Src src = src_in;
    float best = -CUDART_INF_F;
    int best_i = -1;
    constexpr int NQ = Src::kQuads;
    constexpr int step = kThreads * 8;
    const int depth = stage_depth(stage_bytes, NQ);
    if (stage != nullptr && depth >= 2 && src.stage_ok()) {
        int bq = threadIdx.x * 8;
        for (int sidx = 0; sidx < depth; sidx++, bq += step) {
            if (bq + 8 <= n) {
                const char *g = src.stage_src(bq);
#pragma unroll
                for (int q = 0; q < NQ; q++) cp_async16(stage_slot<NQ>(stage, sidx, q), g + q * 16);
            }
            cp_async_commit();
        }
        int sidx = 0;
        for (int base = threadIdx.x * 8; base < n; base += step) {
            cp_async_wait_dyn(depth - 1);
            float x[8];
            if (base + 8 <= n) {
                float4 qd[NQ];
#pragma unroll
                for (int q = 0; q < NQ; q++) qd[q] = *stage_slot<NQ>(stage, sidx, q);
                src.decode(base, qd, x);
            } else {
                src.get8(base, n, x);
            }
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (base + j < n && x[j] > best) { best = x[j]; best_i = base + j; }
            if (bq + 8 <= n) {
                const char *g = src.stage_src(bq);
#pragma unroll
                for (int q = 0; q < NQ; q++) cp_async16(stage_slot<NQ>(stage, sidx, q), g + q * 16);
            }
            cp_async_commit();
            bq += step;
            sidx = sidx + 1 == depth ? 0 : sidx + 1;
        }
        cp_async_wait<0>();
    } else {
        for (int base = threadIdx.x * 8; base < n; base += step) {
            float x[8];
            src.get8(base, n, x);
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (base + j < n && x[j] > best) { best = x[j]; best_i = base + j; }
        }
    }
    u64 k = best_i >= 0 ? make_key(best, best_i) : 0ull;
    return block_max_key_r(k, red);
}

// mass of a histogram bin in exp-value units: every value in bin b >= 1 has the biased exponent
// kBinExp0 + (b >> 7), and hmass holds the sum of the top 12 bits of their 24-bit mantissas (the
// smaller values gathered in bin 0 are overestimated, which only widens the nucleus bound)
__device__ __forceinline__ double bin_mass(const unsigned *hmass, int b)
{
    return ldexp((double)hmass[b], kBinExp0 + (b >> 7) - 127 - 11);  // truncation makes it up to 2^-12 low
}

// ---- top-p over a partially ordered candidate list ---------------------------------------------------
// rank-sorts (descending) every bin on the dirty list.  The bins are taken in rounds of whole bins
// holding at most kDirtyRound keys together (the sort is in place, so a bin must not be split over
// rounds); a single bin larger than that makes the caller give the partial order up.
static __device__ void sort_dirty_bins(RowCtl *rc, uint32_t *keys, const unsigned *bstart, const unsigned *hcount,
                                       uint32_t *tmp_key, int *tmp_dst)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nd = min(rc->n_dirty, kMaxDirty);
    static_assert(kMaxDirty <= kThreads, "one dirty bin per thread in the prefix sum");
    __syncthreads();
    // exclusive prefix of the dirty bins' key counts
    {
        const int c = tid < nd ? (int)hcount[rc->dirty[tid]] : 0;
        int inc = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int v = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += v;
        }
        if (lane == 31) rc->red_i[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            int w = rc->red_i[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int v = __shfl_up_sync(0xFFFFFFFFu, w, o);
                if (lane >= o) w += v;
            }
            rc->red_i[lane] = w;
        }
        __syncthreads();
        const int excl = inc - c + (warp ? rc->red_i[warp - 1] : 0);
        if (tid < nd) rc->dirty_cum[tid] = excl;
        if (tid == nd - 1) rc->dirty_cum[nd] = excl + c;
        __syncthreads();
    }
    int first = 0;
    while (first < nd) {
        // round: the longest run of bins first .. last-1 holding at most kDirtyRound keys
        const int base_cum = rc->dirty_cum[first];
        int lo = first, hi = nd + 1;  // largest i with dirty_cum[i] - base_cum <= kDirtyRound
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (rc->dirty_cum[mid] - base_cum <= kDirtyRound) lo = mid; else hi = mid;
        }
        const int last = lo;
        if (last == first) {  // one bin alone is too large for the in-place sort
            __syncthreads();
            if (tid == 0) rc->give_up = 1;
            __syncthreads();
            return;
        }
        const int m = rc->dirty_cum[last] - base_cum;
        for (int e = tid; e < m; e += kThreads) {
            int l2 = first, h2 = last;  // last i in [first, last) with dirty_cum[i] - base_cum <= e
            while (h2 - l2 > 1) {
                int mid = (l2 + h2) >> 1;
                if (rc->dirty_cum[mid] - base_cum <= e) l2 = mid; else h2 = mid;
            }
            const int b = rc->dirty[l2];
            const int off = (int)bstart[b], cnt = (int)hcount[b];
            const int pos = e - (rc->dirty_cum[l2] - base_cum);
            const uint32_t k = keys[off + pos];
            int rank = 0;
            for (int j = 0; j < cnt; j++) {
                const uint32_t o = keys[off + j];
                rank += (o > k || (o == k && j < pos)) ? 1 : 0;
            }
            tmp_key[e] = k;
            tmp_dst[e] = off + rank;
        }
        __syncthreads();
        for (int e = tid; e < m; e += kThreads) keys[tmp_dst[e]] = tmp_key[e];
        __syncthreads();
        first = last;
    }
}

__device__ __forceinline__ double scan4_double(double tot, RowCtl *rc)  // inclusive block scan of per-thread totals
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    double run = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        double t = __shfl_up_sync(0xFFFFFFFFu, run, o);
        if (lane >= o) run += t;
    }
    __syncthreads();
    if (lane == 31) rc->red_d[warp] = run;
    __syncthreads();
    if (warp == 0) {
        double w = rc->red_d[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            double t = __shfl_up_sync(0xFFFFFFFFu, w, o);
            if (lane >= o) w += t;
        }
        rc->red_d[lane] = w;
    }
    __syncthreads();
    return run + (warp ? rc->red_d[warp - 1] : 0.0);
}

// top-k of the full-vocabulary pipeline (ApplyTopK + Normalize); updates rc->dist.  Out of line
// for the same reason as topp_cut.
static __device__ __noinline__ void topk_cut(RowCtl *rc, SelCtl *sctl, const RowPlan &rp, int n, const float *scratch,
                                             unsigned char *arena)
{
    const int tid = threadIdx.x;
    RowDist d = rc->dist;
    {
        // ApplyTopK + Normalize (Sampler.cs:477-488, :71-81): the k-th largest probability, counted
        // with multiplicity; everything below it is dropped, ties at it all survive.  Selected on
        // the exp values, of which the probabilities are a monotone image.
        Sel s;
        s.c = sctl;
        s.cap = 8192;
        s.buf[0] = (u64 *)(arena + kOffKeys);
        s.buf[1] = s.buf[0] + s.cap;
        s.n = rp.top_k;
        s.idx_off = 0;
        sel_reset(s);
        sel_stream<4, false>(s, LogitRow{scratch, 0.f}, nullptr, 0, n);
        if (sctl->cnt > s.n) sel_compact(s);  // exactly the best k: their minimum is the k-th largest
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
    __syncthreads();
    if (tid == 0) rc->dist = d;
    __syncthreads();
}

// top-p (ApplyTopP, Sampler.cs:516-551): finds the cut of the reference's sorted sequential
// cumulative sum without sorting the vocabulary; updates rc->dist (tstar, tie_idx_max) and
// returns the fp64 sum of the kept probabilities.  Kept out of line: it is long, runs once per
// row, and would otherwise dominate the register allocation of the streaming phases around it.
static __device__ __noinline__ double topp_cut(RowCtl *rc, const RowPlan &rp, int n, const float *scratch,
                                               unsigned char *arena, uint32_t *gkeys, int gkeys_cap, u64 *list,
                                               uint32_t *flags_out, u64 *tk)
{
    const int tid = threadIdx.x;
    uint32_t *skeys = (uint32_t *)(arena + kOffKeys);
    unsigned *hcount = (unsigned *)(arena + kOffCount);
    unsigned *hmass = (unsigned *)(arena + kOffMass);
    unsigned *bstart = (unsigned *)(arena + kOffBinOff);
    Emul2Work *wk2 = (Emul2Work *)(arena + kOffEmul);
    unsigned char *replay_ok = arena + kOffReplayOk;
    unsigned char *bin_exp = arena + kOffBinExp;
    int *sub_src = (int *)(arena + kOffSubSrc);
    unsigned short *sub_cnt = (unsigned short *)(arena + kOffSubCnt);
    RowDist d = rc->dist;
    const bool uniform = (d.flags & kDistUniform) != 0;
    double sum3 = 0.0;
    {
        const double scale_p = ((d.flags & kDistScale1) ? (double)d.inv1 : 1.0) *
                               ((d.flags & kDistScale2) ? (double)d.inv2 : 1.0);
        for (int attempt = 0; attempt < 2; attempt++) {
            // (1) bound the nucleus: bins from the top until the estimated mass clears top_p.  An
            // estimate suffices: a bound that proves too tight is caught below (the emulated sum
            // then never reaches top_p although survivors remain) and everything is taken.
            if (tid == 0) { rc->c_lo = 0; rc->give_up = 0; rc->n_dirty = 0; }
            __syncthreads();
            if (attempt == 0) {
                // mass and count of the bins above each bin (4 bins per thread, highest bins first)
                double lm[4], tm = 0.0, tc = 0.0;
                unsigned lc[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int b = kBins - 1 - (tid * 4 + j);
                    lc[j] = hcount[b];
                    lm[j] = lc[j] ? bin_mass(hmass, b) : 0.0;
                    tm += lm[j];
                    tc += (double)lc[j];
                }
                double am = scan4_double(tm, rc) - tm;
                double ac = scan4_double(tc, rc) - tc;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int b = kBins - 1 - (tid * 4 + j);
                    am += lm[j];
                    ac += (double)lc[j];
                    if (lc[j]) {
                        const double need = (double)rp.top_p * (1.0 + 1.0 / 65536.0) + 16.0 * sqrt(ac) * 2.98e-8 + 1e-7;
                        if (am * scale_p >= need) atomicMax(&rc->c_lo, b > 0 ? b - 1 : 0);
                    }
                }
                __syncthreads();
            }
            for (int t = tid; t < kBins / 32; t += kThreads) rc->sorted_bits[t] = 0u;
            __syncthreads();
            tick(tk, 5);
            const int c_lo = rc->c_lo;
            // (2) start of every candidate bin in the bin-ordered list (largest bin first)
            unsigned *cursor = (unsigned *)wk2;  // kBins u32 = 16 KB over Emul2Work's sums + comp, free here
            {
                unsigned loc[4], tot = 0;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    int b = kBins - 1 - (tid * 4 + j);
                    loc[j] = b >= c_lo ? hcount[b] : 0u;
                    cursor[b] = 0u;
                    tot += loc[j];
                }
                const double incl = scan4_double((double)tot, rc);
                unsigned run = (unsigned)(incl - (double)tot);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    int b = kBins - 1 - (tid * 4 + j);
                    bstart[b] = run;
                    run += loc[j];
                }
                if (tid == kThreads - 1) rc->bound = (int)run;
                __syncthreads();
            }
            const int bound = rc->bound;
            uint32_t *keys = skeys;
            int cap = kSortCap;
            if (bound > kSortCap) { keys = gkeys; cap = gkeys_cap; *flags_out |= (1u << 7); }
            // (3) per bin, from the estimated mass before and after it: the binade the sequential sum
            // is in when it reaches the bin, and whether it may change binade or meet top_p inside
            // the bin.  Such bins - and the head of the list, where the sum changes binade every few
            // keys - must be in exact order before the sum is emulated.
            for (int t = tid; t < kBins / 32; t += kThreads) rc->flag_bits[t] = 0u;
            __syncthreads();
            {
                double loc[4], tot = 0.0;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    int b = kBins - 1 - (tid * 4 + j);
                    loc[j] = (b >= c_lo && hcount[b]) ? bin_mass(hmass, b) * scale_p : 0.0;
                    tot += loc[j];
                }
                double before = scan4_double(tot, rc) - tot;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    int b = kBins - 1 - (tid * 4 + j);
                    // the estimate is low by at most 2^-12 (mantissa truncation) and the emulated
                    // sum drifts by ~1e-5; a miss is caught by the scan itself
                    const double lo = before * (1.0 - 1.0 / 32768.0), hi = (before + loc[j]) * (1.0 + 1.0 / 2048.0);
                    const int e_lo = exp_of_double(lo);
                    bin_exp[b] = (unsigned char)e_lo;
                    if (b >= c_lo && hcount[b]) {
                        const bool crosses = e_lo != exp_of_double(hi);
                        const bool cut = lo <= (double)rp.top_p && hi >= (double)rp.top_p;
                        const bool head = bstart[b] < 2048u;
                        if (crosses || cut || head) atomicOr(&rc->flag_bits[b >> 5], 1u << (b & 31));
                    }
                    before += loc[j];
                }
                __syncthreads();
            }
            // (4) scatter the survivors above the bound into bin order, and - in token order - into
            // the candidate list the draw later walks; count all survivors.  A key whose addition
            // would be an exact tie (where the parity of the running sum decides the rounding, so
            // the order inside its bin matters) flags its bin.
            int my_surv = 0;
            const uint32_t lo_bits = bin_floor_bits(c_lo);
            // every warp owns a contiguous run of sub-tiles and compacts its candidates to the front
            // of the same stretch of the list: token order is kept without a block-wide scan
            const int lane = tid & 31, warp = tid >> 5;
            const int nsub_v = (n + kSub - 1) / kSub;
            const int per_warp = (nsub_v + (kThreads / 32) - 1) / (kThreads / 32);
            const int t_begin = warp * per_warp, t_end = min(t_begin + per_warp, nsub_v);
            u64 *seg = list + (size_t)t_begin * kSub;
            int seg_cnt = 0;
            for (int t = t_begin; t < t_end; t += 2) {
                float x[2][8];
                const int base = t * kSub + lane * 8;
                const int b1 = base + kSub;
                const bool has1 = t + 1 < t_end;
                SrcScratch sc{scratch, 1.f, false};
                if (base < n) sc.get8(base, n, x[0]);
                if (has1 && b1 < n) sc.get8(b1, n, x[1]);
                unsigned take[2] = {0u, 0u};
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int bb = h ? b1 : base;
                    if ((h && !has1) || bb >= n) continue;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        if (bb + j >= n) continue;
                        const float e = x[h][j];
                        const float p = eval_p2(e, d);
                        if (p > 0.f) {
                            my_surv++;
                            const uint32_t ebits = __float_as_uint(e);
                            if (ebits >= lo_bits) {
                                take[h] |= 1u << j;
                                const unsigned bin = bin_of(ebits);
                                unsigned pos = bstart[bin] + atomicAdd(&cursor[bin], 1u);
                                const uint32_t pbits = __float_as_uint(p);
                                if (pos < (unsigned)cap) keys[pos] = pbits;
                                const int k = (int)bin_exp[bin] - (int)((pbits >> 23) & 255u);
                                if (k >= 1 && k <= 24) {
                                    const uint32_t m = (pbits & 0x7FFFFFu) | 0x800000u;
                                    if ((m & ((1u << k) - 1u)) == (1u << (k - 1)))
                                        atomicOr(&rc->flag_bits[bin >> 5], 1u << (bin & 31));
                                }
                            }
                        }
                    }
                }
                const int mine = __popc(take[0]) | (__popc(take[1]) << 16);
                int inc = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    int v = __shfl_up_sync(0xFFFFFFFFu, inc, o);
                    if (lane >= o) inc += v;
                }
                const int total = __shfl_sync(0xFFFFFFFFu, inc, 31);
                const int excl = inc - mine;
                int pos0 = seg_cnt + (excl & 0xFFFF);
                int pos1 = seg_cnt + (total & 0xFFFF) + (excl >> 16);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if ((take[0] >> j) & 1u)
                        seg[pos0++] = ((u64)(uint32_t)(base + j) << 32) | __float_as_uint(x[0][j]);
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if ((take[1] >> j) & 1u)
                        seg[pos1++] = ((u64)(uint32_t)(b1 + j) << 32) | __float_as_uint(x[1][j]);
                }
                seg_cnt += (total & 0xFFFF) + (total >> 16);
            }
            // the list as a sequence of sub-tiles: each warp's stretch, padded to whole sub-tiles
            __syncthreads();
            if (lane == 0) rc->red_i[warp] = (seg_cnt + kSub - 1) / kSub;
            __syncthreads();
            {
                int first = 0, all = 0;
                for (int w = 0; w < kThreads / 32; w++) {
                    const int c = rc->red_i[w];
                    if (w < warp) first += c;
                    all += c;
                }
                const int mine_tiles = (seg_cnt + kSub - 1) / kSub;
                for (int k = lane; k < mine_tiles && first + k < kMaxSubTiles; k += 32) {
                    sub_src[first + k] = (t_begin + k) * kSub;
                    sub_cnt[first + k] = (unsigned short)min(kSub, seg_cnt - k * kSub);
                }
                __syncthreads();
                if (tid == 0) rc->n_list = all <= kMaxSubTiles ? all * kSub : -1;  // -1: the draw walks the row instead
            }
            my_surv = block_sum_int(my_surv, rc->red_i);
            // The filters before top-p drop the smallest values only, so the bins that lost
            // elements are the last ones of the list: it stays dense.  From here on the histogram
            // describes the list.
            int mine = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                int b = kBins - 1 - (tid * 4 + j);
                unsigned have = b >= c_lo ? cursor[b] : 0u;
                if (b >= c_lo) hcount[b] = have;  // the bins below keep their counts for a second attempt
                mine += (int)have;
            }
            const int nc = min(block_sum_int(mine, rc->red_i), cap);
            __syncthreads();
            tick(tk, 6);
            if (nc == 0) { if (tid == 0) rc->n_list = -1; __syncthreads(); break; }
            // (5) a sub-tile of the emulated sum is replayed whole, so every bin that shares a
            // sub-tile with a flagged bin has to be sorted with it
            for (int t = tid; t < kMaxSubTiles; t += kThreads) replay_ok[t] = 0;
            __syncthreads();
            for (int b = c_lo + tid; b < kBins; b += kThreads) {
                const unsigned cnt = hcount[b];
                if (cnt && ((rc->flag_bits[b >> 5] >> (b & 31)) & 1u)) {
                    const int t0 = (int)bstart[b] >> 8, t1 = (int)(bstart[b] + cnt - 1) >> 8;
                    for (int t = t0; t <= t1 && t < kMaxSubTiles; t++) replay_ok[t] = 1;
                }
            }
            __syncthreads();
            for (int b = c_lo + tid; b < kBins; b += kThreads) {
                const unsigned cnt = hcount[b];
                if (cnt >= 2u) {
                    const int t0 = (int)bstart[b] >> 8, t1 = (int)(bstart[b] + cnt - 1) >> 8;
                    bool need = false;
                    for (int t = t0; t <= t1 && t < kMaxSubTiles; t++) need |= replay_ok[t] != 0;
                    if (need) {
                        int slot = atomicAdd(&rc->n_dirty, 1);
                        if (slot < kMaxDirty) rc->dirty[slot] = (unsigned short)b; else rc->give_up = 1;
                    }
                }
            }
            __syncthreads();
            int hit = -1;
            float cum = 0.f;
            bool sorted_all = uniform;  // all keys equal: any order is sorted
            if (tk && tid == 0) { tk[28] = (u64)rc->n_dirty; tk[29] = (u64)nc; tk[30] = 0; tk[31] = 0; }
            for (int pass = 0; pass < 64; pass++) {
                if (tk && tid == 0) tk[30] = (u64)(pass + 1);
                if (!sorted_all && (rc->give_up || pass == 63)) {
                    // partial order abandoned: sort the whole list
                    const int p2 = pow2_ceil(max(nc, 2));
                    for (int t = nc + tid; t < p2; t += kThreads) keys[t] = 0u;
                    __syncthreads();
                    bitonic_sort_desc_t<uint32_t>(keys, p2);
                    sorted_all = true;
                } else if (!sorted_all && rc->n_dirty > 0) {
                    if (tk && tid == 0) tk[31] += 1;
                    sort_dirty_bins(rc, keys, bstart, hcount, (uint32_t *)wk2, (int *)wk2 + kDirtyRound);
                    __syncthreads();
                    if (rc->give_up) continue;  // a bin was too large for the in-place sort: sort everything
                    for (int i = tid; i < min(rc->n_dirty, kMaxDirty); i += kThreads)
                        atomicOr(&rc->sorted_bits[rc->dirty[i] >> 5], 1u << (rc->dirty[i] & 31));
                    __syncthreads();
                    if (tid == 0) rc->n_dirty = 0;
                }
                __syncthreads();
                if (!sorted_all) {
                    // a sub-tile that overlaps an unsorted bin of two or more keys may not be replayed
                    for (int t = tid; t < kMaxSubTiles; t += kThreads) replay_ok[t] = 1;
                    __syncthreads();
                    for (int b = c_lo + tid; b < kBins; b += kThreads) {
                        const unsigned cnt = hcount[b];
                        if (cnt >= 2u && !((rc->sorted_bits[b >> 5] >> (b & 31)) & 1u)) {
                            const int t0 = (int)bstart[b] >> 8, t1 = (int)(bstart[b] + cnt - 1) >> 8;
                            for (int t = t0; t <= t1 && t < kMaxSubTiles; t++) replay_ok[t] = 0;
                        }
                    }
                    __syncthreads();
                }
                ProvKeys pk{keys, keys != skeys};
                if (nc <= kSub * kMaxSubTiles) {
                    hit = emul_scan2<ProvKeys, false, true, 4>(&rc->em2, wk2, pk, nc, rp.top_p, true, &cum,
                                                            sorted_all ? nullptr : replay_ok, nullptr,
                                                            keys != skeys ? arena + kOffKeys : nullptr, kSortCap * 4);
                } else {
                    if (!sorted_all) { if (tid == 0) rc->give_up = 1; __syncthreads(); continue; }
                    hit = emul_scan<ProvKeys, false>(&rc->em, pk, nc, rp.top_p, true, &cum);
                }
                if (hit != -2) break;
                // the sum needed the internal order of an unsorted stretch: sort its bins and rerun
                const int t_abort = rc->em2.abort_at;
                for (int b = c_lo + tid; b < kBins; b += kThreads) {
                    const unsigned cnt = hcount[b];
                    if (cnt >= 2u && !((rc->sorted_bits[b >> 5] >> (b & 31)) & 1u)) {
                        const int t0 = (int)bstart[b] >> 8, t1 = (int)(bstart[b] + cnt - 1) >> 8;
                        if (t0 <= t_abort && t_abort <= t1) {
                            int slot = atomicAdd(&rc->n_dirty, 1);
                            if (slot < kMaxDirty) rc->dirty[slot] = (unsigned short)b; else rc->give_up = 1;
                        }
                    }
                }
                __syncthreads();
            }
            tick(tk, 8);
            if (hit < 0 && nc < my_surv && attempt == 0) continue;  // bound was too tight: take all
            // no hit: the running sum never reaches top_p (min-p or top-k removed too much mass), and
            // ApplyTopP then cuts nothing (Sampler.cs:536-549).  The list is only partially ordered,
            // so its last key is not its smallest: the threshold is simply zero.
            const int last = hit >= 0 ? hit : nc - 1;
            const float tstar = hit >= 0 ? __uint_as_float(keys[last]) : 0.f;
            if (hit >= 0 && nc <= kSub * kMaxSubTiles && tid == 0 &&
                (cum - rp.top_p <= kNearTol || rp.top_p - rc->em2.hit_before <= kNearTol))
                *flags_out |= kFlagNearCut;  // a last-bit difference in exp could move the cut by a token
            // ties at the cut: the kept ones are a prefix (by token id) of the equal probabilities
            int keep = 0, all = 0;
            double part = 0.0;
            for (int t = tid; t < nc; t += kThreads) {
                const uint32_t kb = keys[t];
                if (kb == __float_as_uint(tstar)) { all++; keep += (t <= last) ? 1 : 0; }
                if (t <= last) part += (double)__uint_as_float(kb);
            }
            keep = block_sum_int(keep, rc->red_i);
            all = block_sum_int(all, rc->red_i);
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
    }
    __syncthreads();
    if (tid == 0) rc->dist = d;
    __syncthreads();
    return sum3;
}

// ---- the distribution of one row --------------------------------------------------------------------
// Leaves the exp values in `scratch` and the descriptor in rc->dist.  `src` yields the adjusted,
// temperature-scaled logits; `mx_known` is their maximum when the caller already has it.
template <class Src>
static __device__ void build_dist(RowCtl *rc, SelCtl *sctl, const Src &src, const RowPlan &rp, int n,
                                  float *scratch, unsigned char *arena, uint32_t *gkeys, int gkeys_cap, u64 *list,
                                  uint32_t *flags_out, u64 *tk, bool have_max, float mx_known,
                                  unsigned char *stage, int stage_bytes)
{
    const int tid = threadIdx.x;
    unsigned *hcount = (unsigned *)(arena + kOffCount);
    unsigned *hmass = (unsigned *)(arena + kOffMass);
    Emul2Work *wk2 = (Emul2Work *)(arena + kOffEmul);
    const bool want_topp = rp.top_p < 1.0f && rp.top_p > 0.f;
    const bool want_minp = rp.min_p > 0.f;
    const bool want_topk = rp.top_k > 0 && rp.top_k < n;

    float mx;
    if (have_max) {
        mx = mx_known;
    } else {
        u64 mk = pass_max_staged(src, n, rc->red_k, stage, stage_bytes);
        mx = mk ? key_val(mk) : -CUDART_INF_F;
    }
    tick(tk, 2);
    RowDist d;
    d.flags = 0;
    d.inv_t = src.inv_t;
    d.tie_idx_max = INT_MAX;
    d.kth = 0.f; d.inv2 = 1.f; d.minp_thr = 0.f; d.tstar = 0.f; d.inv3 = 1.f; d.inv1 = 1.f;
    d.uniform_p = 0.f; d.sum_end = 0.f; d.argmax = 0;
    if (want_topp) {
        for (int t = tid; t < kBins; t += kThreads) { hcount[t] = 0u; hmass[t] = 0u; }
    }
    __syncthreads();
    float sum = 0.f;
    const bool uniform = !(mx > -CUDART_INF_F);  // also covers NaN
    if (uniform) {
        // Softmax's fully masked case (Sampler.cs:452-458): every token gets 1/V, no rescale
        d.flags |= kDistUniform;
        d.max_x = -CUDART_INF_F;
        d.uniform_p = __fdiv_rn(1.0f, (float)n);
        for (int i = tid; i < n; i += kThreads) __stcg(scratch + i, d.uniform_p);
        if (want_topp && tid == 0) {
            unsigned bin = bin_of(__float_as_uint(d.uniform_p));
            hcount[bin] = (unsigned)n;
            hmass[bin] = (unsigned)min((unsigned long long)n * ((((unsigned long long)__float_as_uint(d.uniform_p) & 0x7FFFFFu) | 0x800000u) >> 12), 0xFFFFFFFFull);
        }
        __syncthreads();
    } else {
        d.max_x = mx;
        // the histogram is accumulated as one packed 64-bit word per bin (count << 40 | mass) over
        // the two 32-bit arrays, which are adjacent, and unpacked afterwards
        static_assert(kOffMass == kOffCount + kBins * 4, "count and mass arrays must be adjacent");
        unsigned long long *hist = (unsigned long long *)hcount;
        ProvExp<Src> pe{src, mx, scratch, want_topp ? hist : nullptr};
        emul_any<ProvExp<Src>, false>(&rc->em, &rc->em2, wk2, pe, n, 0.f, false, &sum, tk ? tk + 12 : nullptr,
                                      stage, stage_bytes);
        if (sum > 0.f && sum != 1.0f) { d.flags |= kDistScale1; d.inv1 = __fdiv_rn(1.0f, sum); }
        if (want_topp) {
            unsigned long long v[4];
#pragma unroll
            for (int j = 0; j < 4; j++) v[j] = hist[tid * 4 + j];
            __syncthreads();
#pragma unroll
            for (int j = 0; j < 4; j++) {
                hcount[tid * 4 + j] = (unsigned)(v[j] >> 40);
                hmass[tid * 4 + j] = (unsigned)(v[j] & 0xFFFFFFFFull);
            }
        }
    }
    __syncthreads();
    tick(tk, 3);
    if (want_topk) {
        __syncthreads();
        if (tid == 0) rc->dist = d;
        __syncthreads();
        topk_cut(rc, sctl, rp, n, scratch, arena);
        d = rc->dist;
    }
    tick(tk, 4);
    if (want_minp) {
        // ApplyMinP (Sampler.cs:493-503): the largest probability belongs to exp value 1 (or 1/V)
        float emax = uniform ? d.uniform_p : 1.0f;
        float pmax = (d.flags & kDistScale1) ? __fmul_rn(emax, d.inv1) : emax;
        if (d.flags & kDistScale2) pmax = __fmul_rn(pmax, d.inv2);
        d.minp_thr = __fmul_rn(rp.min_p, pmax);
        d.flags |= kDistMinP;
    }

    double sum3 = 0.0;
    if (want_topp) {
        __syncthreads();
        if (tid == 0) rc->dist = d;
        __syncthreads();
        sum3 = topp_cut(rc, rp, n, scratch, arena, gkeys, gkeys_cap, list, flags_out, tk);
        d = rc->dist;
    } else
    {
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
    tick(tk, 9);
    // Normalize (Sampler.cs:553-562)
    float s3 = (float)sum3;
    if (s3 > 0.f && s3 != 1.0f) { d.flags |= kDistScale3; d.inv3 = __fdiv_rn(1.0f, s3); }
    __syncthreads();
    if (tid == 0) rc->dist = d;
    __syncthreads();
}

template <bool BF16>
static __device__ void run_row(const SampleArgs &a, int row, int item, SelCtl *sctl, unsigned char *arena)
{
    u64 *tk = a.phase_ticks ? a.phase_ticks + (int64_t)item * 32 : nullptr;
    tick(tk, 0);
    __shared__ RowCtl rc;
    __shared__ RowPlan sh_rp;  // kept in shared memory: the row's parameters are read rarely
    const int tid = threadIdx.x;
    __syncthreads();
    if (tid == 0) sh_rp = a.plans[row];
    __syncthreads();
    const RowPlan &rp = sh_rp;
    // second chance of the flat step: only the rows it flagged are run
    if (a.redo_flags != nullptr && (rp.flat_full < 0 || a.redo_flags[(size_t)rp.flat_full * a.redo_stride] == 0)) return;
    const int n = a.vocab;
    const int esz = BF16 ? 2 : 4;
    const LogitRow rowp{(const char *)a.logits + (int64_t)row * a.row_stride * esz, a.softcap};
    const uint32_t *mrow = (rp.use_mask && a.mask) ? a.mask + (int64_t)row * a.mask_stride : nullptr;
    float *scratch = a.escratch + (int64_t)blockIdx.x * a.escratch_stride;
    uint32_t *gkeys = (uint32_t *)(a.keyscratch + (int64_t)blockIdx.x * a.key_stride);
    const int gkeys_cap = (int)(a.key_stride * 2);
    u64 *list = a.listscratch + (int64_t)blockIdx.x * (a.key_stride + 2 * kSub);
    const bool greedy = rp.temperature <= 0.f;
    const bool with_bias = !greedy && rp.bias_len > 0;
    const bool with_hist = rp.has_penalty && rp.hist_len > 0;
    const bool overrides = with_hist || with_bias;
    __shared__ uint32_t sh_flags;
    if (tid == 0) { sh_flags = 0; rc.n_list = -1; }
    __syncthreads();

    const float inv_t = (!greedy && rp.temperature != 1.0f) ? __fdiv_rn(1.0f, rp.temperature) : 1.0f;
    const bool scale = !greedy && rp.temperature != 1.0f;
    SrcLogits<BF16> raw{rowp, mrow, a.vec == 4, 1.f, false};
    // rows with history penalties or logit bias: the adjusted logits of the few tokens concerned
    // go into a hash table at the bottom of the key region; every later read of the row applies
    // them on the fly.  What is left of the region stages the reads.
    SrcLogitsOv<BF16> adj;
    adj.raw = raw;
    adj.inv_t = inv_t;
    adj.scale = scale;
    int table_bytes = 0;
    u64 mk_adj = 0ull;
    if (overrides) {
        const int entries = (with_hist ? rp.hist_len : 0) + (with_bias ? rp.bias_len : 0);
        int slots = 64;
        while (slots < 2 * entries) slots <<= 1;
        OvTable table;
        build_overrides<BF16>(a, rp, rowp, mrow, n, with_hist, with_bias, table, arena, slots);
        adj.ov.key = table.key;
        adj.ov.mask = table.mask;
        table_bytes = (slots * 24 + 8192 + 1023) & ~1023;
        tick(tk, 11);
        mk_adj = pass_max_staged(adj, n, rc.red_k, arena + table_bytes, kSortCap * 4 - table_bytes);
    }
    tick(tk, 1);

    if (greedy) {
        // Greedy / GreedyWithHistoryPenalties; in distribution mode a one-hot row
        const u64 mk = overrides ? mk_adj : pass_max(raw, n, rc.red_k);
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
        if ((a.mode == 1 || a.mode == 3) && a.dist_out) {
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

    if (overrides) {
        build_dist(&rc, sctl, adj, rp, n, scratch, arena, gkeys, gkeys_cap, list, &sh_flags, tk, true,
                   mk_adj ? key_val(mk_adj) : -CUDART_INF_F, arena + table_bytes, kSortCap * 4 - table_bytes);
    } else {
        SrcLogits<BF16> s{rowp, mrow, a.vec == 4, inv_t, scale};
        build_dist(&rc, sctl, s, rp, n, scratch, arena, gkeys, gkeys_cap, list, &sh_flags, tk, false, 0.f,
                   arena + kOffKeys, kSortCap * 4);
    }
    if (a.mode == 2) {
        // descriptor only; the raw arg-max goes with it (the looser accept rule compares against it)
        u64 mk = pass_max(raw, n, rc.red_k);
        if (tid == 0) {
            rc.dist.argmax = mk ? key_idx(mk) : 0;
            a.dists[row] = rc.dist;
        }
        __syncthreads();
        return;
    }

    // draw: SampleFromDistribution (Sampler.cs:564-576)
    float *dout = ((a.mode == 1 || a.mode == 3) && a.dist_out) ? a.dist_out + (int64_t)row * n : nullptr;
    ProvFinal pf{scratch, rc.dist, dout};
    if (a.mode == 1 || (a.mode == 3 && dout != nullptr)) {
        for (int base = tid * 8; base < n; base += kThreads * 8) { float x[8]; pf.load(base, n, x); }
        if (a.mode == 1) {
            if (tid == 0 && a.row_flags) a.row_flags[row] = kPathFull | sh_flags;
            __syncthreads();
            return;
        }
        pf.dist_out = nullptr;  // mode 3 goes on to the draw
        __syncthreads();
    }
    const float u = a.uniforms ? __ldg(a.uniforms + row) : 0.5f;
    float cum = 0.f;
    Emul2Work *wk2 = (Emul2Work *)(arena + kOffEmul);
    int hit;
    const int n_list = rc.n_list;
    if (n_list >= 0) {
        // after top-p only the listed candidates can be non-zero, and adding a zero neither changes
        // the running sum nor can be the first element to reach the target (unless the target is
        // not positive, which the first token meets whatever its probability)
        ProvList pl{list, (const int *)(arena + kOffSubSrc), (const unsigned short *)(arena + kOffSubCnt), rc.dist};
        hit = emul_any<ProvList, false>(&rc.em, &rc.em2, wk2, pl, n_list, u, true, &cum, tk ? tk + 20 : nullptr,
                                        arena + kOffKeys);
        if (hit >= 0) hit = (int)(__ldcg(pl.at(hit)) >> 32);
        if (!(u > 0.f)) hit = 0;
    } else {
        hit = emul_any<ProvFinal, false>(&rc.em, &rc.em2, wk2, pf, n, u, true, &cum, tk ? tk + 20 : nullptr);
    }
    if (tid == 0) {
        uint32_t fl = kPathFull | sh_flags | (a.redo_flags ? kFlagFlatRedo : 0u);  // redone after the flat step gave up
        if (rc.dist.flags & kDistUniform) fl |= (1u << 6);
        int tok = hit;
        if (hit < 0) { tok = n - 1; fl |= (1u << 5); }
        else if (n <= kSub * kMaxSubTiles && u > 0.f && (u - rc.em2.hit_before <= kNearTol || cum - u <= kNearTol)) fl |= kFlagNearBoundary;
        a.tokens[row] = tok;
        if (a.token_probs) a.token_probs[row] = eval_p3(__ldcg(scratch + tok), tok, rc.dist);
        if (a.row_flags) a.row_flags[row] = fl;
        count_row_flags(a.counters, fl);
    }
    tick(tk, 10);
    __syncthreads();
}

}  // namespace stg
