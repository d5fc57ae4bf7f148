// Full-vocabulary rows of the flat step (see stg_flat.cuh): the per-row and per-piece kernels behind
// the HBM pass.  The arithmetic is that of stg_rowdist.cuh, whose device functions are reused; what
// differs is where the work runs - every pass over V as small CTAs over pieces of all rows at once,
// every serial part as one CTA per row over summaries or candidates.
#include <cuda_runtime.h>
#include <limits.h>
#include <math_constants.h>
#include <stdint.h>

#include "stg_flat.cuh"
#include "stg_flat_prep.cuh"
#include "stg_spec_prov.cuh"
#include "stg_launch.h"
#include "stg_rowdist.cuh"

namespace stg {

constexpr int kFullThreads = 256;              // threads of a per-piece kernel: 8 warps, one sub-tile each at a time
constexpr int kPhasePiece = 8192;                  // elements of a row one CTA of a per-piece phase kernel covers
constexpr int kPieceSubTiles = kPhasePiece / kSub;  // 32 sub-tiles of 256 elements: 4 per warp, two in flight at a time
static_assert(kSub * kMaxSubTiles / kPhasePiece <= kFullMaxParts, "FullRow::part has one entry per phase piece");

__device__ __forceinline__ bool row_wants_topp(const RowPlan &rp) { return rp.top_p < 1.0f && rp.top_p > 0.f; }

// ---- prep: the override list ---------------------------------------------------------------------------
// One 1024-thread CTA per row of the batch; rows outside the full flat pipeline leave at once.
// ApplyHistoryPenalties after the logit bias (Sampler.cs:50-56, :367-419) through build_overrides,
// then the distinct tokens sorted by id with their adjusted logits, and where every piece starts
// in that list.  Also clears the row's histogram and bin cursors.
// `flat`: the step's chunked rows are in the flat form too; their CTAs of this kernel do k_flat_prep's work.
template <bool BF16>
__global__ void __launch_bounds__(kThreads, 1) k_full_prep(const __grid_constant__ SampleArgs a, const FullWs ws, FlatRow *flat)
{
    extern __shared__ __align__(16) unsigned char arena[];
    __shared__ int n_ent;
    __shared__ uint32_t red[32];
    // grid over the step's item list: it names the full rows first, whose CTAs take longest
    const int row = a.items[blockIdx.x].row, tid = threadIdx.x;
    const RowPlan rp = a.plans[row];
    const int fi = rp.flat_full;
    if (fi < 0) {
        if (flat != nullptr && rp.n_chunks != 0) flat_prep_row<BF16>(a, flat, row, rp, a.softcap, red, (uint32_t *)arena);
        return;
    }
    FullRow *fr = ws.rows + fi;
    const int n = a.vocab;
    const bool greedy = rp.temperature <= 0.f;
    const bool with_bias = !greedy && rp.bias_len > 0;
    const bool with_hist = rp.has_penalty && rp.hist_len > 0;
    if (tid == 0) {
        fr->maxkey = 0ull; fr->rawkey = 0ull; fr->sum = 0.f; fr->surv = 0; fr->redo = 0; fr->flags = 0u;
        fr->c_lo = 0; fr->bound = 0; fr->n_ov = 0;
        for (int p = 0; p <= kFullMaxPieces; p++) fr->ov_piece[p] = 0;
        fr->n_cross[0] = 0; fr->n_cross[1] = 0;
    }
    if (tid < 2 * kFullMaxParts) fr->pflag[tid / kFullMaxParts][tid % kFullMaxParts] = 0u;
    if (row_wants_topp(rp) && !greedy) {
        unsigned long long *hist = ws.hist + (size_t)fi * kHistBins;
        uint32_t *cursor = ws.cursor + (size_t)fi * kHistBins;
        for (int b = tid; b < kHistBins; b += kThreads) { hist[b] = 0ull; cursor[b] = 0u; }
    }
    if (!(with_hist || with_bias)) return;
    const int esz = BF16 ? 2 : 4;
    const LogitRow rowp{(const char *)a.logits + (int64_t)row * a.row_stride * esz, a.softcap};
    const uint32_t *mrow = (rp.use_mask && a.mask) ? a.mask + (int64_t)row * a.mask_stride : nullptr;
    const int entries = (with_hist ? rp.hist_len : 0) + (with_bias ? rp.bias_len : 0);
    int slots = 64;
    while (slots < 2 * entries) slots <<= 1;
    OvTable table;
    build_overrides<BF16>(a, rp, rowp, mrow, n, with_hist, with_bias, table, arena, slots);
    const int table_bytes = (slots * 24 + 8192 + 1023) & ~1023;
    int *cid = (int *)(arena + table_bytes);
    float *cadj = (float *)(cid + kMaxOverride);
    int *sid = (int *)(cadj + kMaxOverride);
    float *sadj = (float *)(sid + kMaxOverride);
    if (tid == 0) n_ent = 0;
    __syncthreads();
    for (int h = tid; h < slots; h += kThreads) {
        const int id = table.key[h];
        if (id >= 0) {
            const int k = atomicAdd(&n_ent, 1);
            if (k < kMaxOverride) { cid[k] = id; cadj[k] = table.adj[h]; }
        }
    }
    __syncthreads();
    const int cnt = min(n_ent, kMaxOverride);
    for (int t = tid; t < cnt; t += kThreads) {
        const int id = cid[t];
        int rank = 0;
        for (int j = 0; j < cnt; j++) rank += (cid[j] < id) ? 1 : 0;  // ids are distinct
        sid[rank] = id;
        sadj[rank] = cadj[t];
    }
    __syncthreads();
    int32_t *gid = ws.ov_id + (size_t)fi * kMaxOverride;
    float *gadj = ws.ov_adj + (size_t)fi * kMaxOverride;
    for (int t = tid; t < cnt; t += kThreads) { gid[t] = sid[t]; gadj[t] = sadj[t]; }
    for (int p = tid; p <= kFullMaxPieces; p += kThreads) {
        const long long first = (long long)p * kFlatPiece;  // first token id of piece p
        int lo = 0, hi = cnt;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if ((long long)sid[mid] < first) lo = mid + 1; else hi = mid;
        }
        fr->ov_piece[p] = lo;
    }
    if (tid == 0) fr->n_ov = cnt;
}

// ---- look-back over the pieces of a row; guesses and composites of a piece --------------------------------
// A per-piece phase kernel needs, for every sub-tile, the binade the sequential running sum is in
// when it gets there - a guess from the fp64 prefix of the sub-tile sums (stg_emul2.cuh, phase B).
// Inside a piece that is a warp scan; across pieces every CTA publishes the total of its piece
// (FullRow::ptotal, then the flag, release order) and collects the totals of the pieces before it.
// Those belong to CTAs with a lower linear block index, which the hardware has dispatched before this
// one, so they are running or done and none of them waits for a later piece.  The wait is bounded all
// the same: when it runs out the row is flagged `redo` (the self-contained row kernel takes it) and
// the CTA leaves.
constexpr int kLookbackSpins = 100000;  // x 40 ns: a few milliseconds at most

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Warp 0 of the CTA of piece `p` (k: 0 exp values, 1 final probabilities), given the sums of the
// piece's sub-tiles in shared memory (s_sum[0..nloc)): publishes the piece total, looks back, and
// leaves the guessed binade and the crossing slot of every sub-tile of the piece in shared memory
// and in the row's Emul2Work.  Returns false (to every lane) when the look-back timed out.
// `drill`: the wait-runs-out drill (SampleArgs::lookback_drill): piece 0 of the drilled pass keeps its flag
// to itself and the wait gives up after 64 polls, so every other piece of every row times out.
__device__ __forceinline__ bool piece_guesses(FullRow *fr, Emul2Work *ew, int k, int p, int t0, int nloc, int nsub,
                                              const float *s_sum, unsigned char *s_guess, unsigned char *s_xslot, bool drill)
{
    const int lane = threadIdx.x & 31;
    const double mine = lane < nloc ? (double)s_sum[lane] : 0.0;
    double tot = mine;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xFFFFFFFFu, tot, o);
    if (lane == 0 && !(drill && p == 0)) {
        __stcg(&fr->ptotal[k][p], tot);
        __threadfence();
        atomicExch(&fr->pflag[k][p], 1u);
    }
    const int spins = drill ? 64 : kLookbackSpins;
    bool ok = true;
    double before = 0.0;
    if (lane < p) {
        int it = 0;
        while (ld_acquire_u32(&fr->pflag[k][lane]) == 0u) {
            if (++it > spins) { ok = false; break; }
            __nanosleep(40);
        }
        if (ok) before = __ldcg(&fr->ptotal[k][lane]);
    }
    ok = __all_sync(0xFFFFFFFFu, ok);
    // sum of the earlier pieces' totals in piece order (lane 0 adds them: a guess needs no more, but
    // every CTA of the row must see the same prefix at a piece boundary whoever computes it)
    double base = 0.0;
    for (int q = 0; q < p; q++) base += __shfl_sync(0xFFFFFFFFu, before, q);
    double inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += t;
    }
    const int g = exp_of_double(base + (inc - mine));
    const int gnext = exp_of_double(base + inc);  // the guess at the sub-tile behind this one
    int xs = 0;
    if (ok && lane < nloc && t0 + lane + 1 < nsub && gnext == g + 1 && s_sum[lane] > 0.f) {
        // the sum should pass into the next binade inside this sub-tile: it gets a CrossSlot
        const int slot = atomicAdd(&fr->n_cross[k], 1);
        if (slot < kMaxCross) xs = slot + 1;
    }
    if (lane < nloc) {
        s_guess[lane] = (unsigned char)g;
        s_xslot[lane] = (unsigned char)xs;
        ew->guess[t0 + lane] = (unsigned char)g;
        ew->xslot[t0 + lane] = (unsigned char)xs;
    }
    if (!ok && lane == 0) fr->redo = 1;
    return ok;
}

// Composite increment of every sub-tile of the piece under its guess (phase C), CrossSlots included.
// FINAL: over the final probabilities, else over the exp values.  All threads of the CTA.
// The values come in registers: xs[i] holds the warp's i-th sub-tile of the piece (sub-tile warp + 8 i,
// this lane's 8 elements, zeros beyond the row's end) as the first stage of the kernel left them.
constexpr int kWarpSubTiles = kPieceSubTiles / (kFullThreads / 32);  // 4
__device__ __forceinline__ void piece_composites(Emul2Work *ew, const float (&xs)[kWarpSubTiles][8], int begin, int n,
                                                 const float *s_sum, const unsigned char *s_guess, const unsigned char *s_xslot)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int W = kFullThreads / 32;
#pragma unroll
    for (int i = 0; i < kWarpSubTiles; i++) {
        const int st = warp + i * W;
        const int t = (begin >> 8) + st;
        if (t * kSub >= n) continue;
        int a0 = 0, a1 = 0;
        if (!(s_sum[st] == 0.f)) {  // else nothing to add: composite 0
            const int g = s_guess[st];
            subtile_composite<false>(xs[i], g, a0, a1);
            const int xsl = s_xslot[st];
            if (xsl) {
                CrossSlot &cs = ew->xs[xsl - 1];
                int l0, l1, h0, h1;
                lane_composite(xs[i], g, l0, l1);
                lane_composite(xs[i], g + 1, h0, h1);
                cs.lo[lane][0] = l0; cs.lo[lane][1] = l1;
                cs.hi[lane][0] = h0; cs.hi[lane][1] = h1;
            }
        }
        if (lane == 0) { ew->comp[t][0] = a0; ew->comp[t][1] = a1; }
    }
}

// the tail both per-piece kernels share: look-back and guesses by warp 0, composites by everyone
template <bool FINAL>
__device__ __forceinline__ void piece_tail(FullRow *fr, Emul2Work *ew, const float (&xs)[kWarpSubTiles][8], int begin, int n,
                                           float *s_sum, unsigned char *s_guess, unsigned char *s_xslot, int *s_ok,
                                           bool drill = false)
{
    const int t0 = begin >> 8, nsub = (n + kSub - 1) / kSub;
    const int nloc = min(kPieceSubTiles, nsub - t0);
    __syncthreads();  // s_sum is complete
    if (threadIdx.x < 32) {
        const bool ok = piece_guesses(fr, ew, FINAL ? 1 : 0, begin / kPhasePiece, t0, nloc, nsub, s_sum, s_guess, s_xslot, drill);
        if (threadIdx.x == 0) *s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (!*s_ok) return;
    piece_composites(ew, xs, begin, n, s_sum, s_guess, s_xslot);
}

// ---- exp: e = exp(x - max), sub-tile sums, histogram ----------------------------------------------------
// grid (pieces, full rows), 256 threads: warp w takes sub-tiles w, w + 8, ... of the piece, lane l the
// 8 consecutive elements 8l .. 8l+7 of a sub-tile (the element order the sequential-sum emulation
// is defined on, stg_emul2.cuh).
__global__ void __launch_bounds__(kFullThreads) k_full_exp(const __grid_constant__ SampleArgs a, const FullWs ws,
                                                           const WorkItem *full_items)
{
    __shared__ unsigned hcnt[kHistBins];
    __shared__ unsigned hmass[kHistBins];
    __shared__ float s_sum[kPieceSubTiles];
    __shared__ unsigned char s_guess[kPieceSubTiles], s_xslot[kPieceSubTiles];
    __shared__ int s_ok;
    const int fi = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = full_items[fi].row;
    const RowPlan *rpp = a.plans + row;
    if (!(__ldg(&rpp->temperature) > 0.f)) return;  // greedy with penalties: the stream pass found the token
    const int n = a.vocab;
    const int begin = blockIdx.x * kPhasePiece;
    if (begin >= n) return;
    FullRow *fr = ws.rows + fi;
    const float top_p = __ldg(&rpp->top_p);
    const bool want_hist = top_p < 1.0f && top_p > 0.f;
    const unsigned long long mk = fr->maxkey;
    const bool uniform = mk == 0ull;  // nothing finite: Softmax's 1/V case (Sampler.cs:452-458)
    const float mx = uniform ? -CUDART_INF_F : key_val(mk);
    const float up = __fdiv_rn(1.0f, (float)n);
    float *e = ws.e + (size_t)fi * ws.e_stride;
    Emul2Work *ew = ws.ew + fi;
    if (want_hist) {
        for (int b = tid; b < kHistBins; b += kFullThreads) { hcnt[b] = 0u; hmass[b] = 0u; }
        __syncthreads();
    }
    constexpr int W = kFullThreads / 32;
    float xs[kWarpSubTiles][8];
#pragma unroll
    for (int it = 0; it < kWarpSubTiles / 2; it++) {
        const int st0 = warp + it * 2 * W;
        float (&x)[2][8] = *reinterpret_cast<float (*)[2][8]>(&xs[it * 2]);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int st = st0 + h * W;
            const int base = begin + st * kSub + lane * 8;
            if (st < kPieceSubTiles && base + 8 <= n) {
                const float4 q0 = __ldcg((const float4 *)(e + base)), q1 = __ldcg((const float4 *)(e + base + 4));
                x[h][0] = q0.x; x[h][1] = q0.y; x[h][2] = q0.z; x[h][3] = q0.w;
                x[h][4] = q1.x; x[h][5] = q1.y; x[h][6] = q1.z; x[h][7] = q1.w;
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) x[h][j] = (st < kPieceSubTiles && base + j < n) ? __ldcg(e + base + j) : -CUDART_INF_F;
            }
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int st = st0 + h * W;
            const int base = begin + st * kSub + lane * 8;
            if (st >= kPieceSubTiles || begin + st * kSub >= n) {  // the same for the whole warp
#pragma unroll
                for (int j = 0; j < 8; j++) x[h][j] = 0.f;
                continue;
            }
            float acc = 0.f;
            int low = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float v = 0.f;
                if (base + j < n) v = uniform ? up : expf(__fsub_rn(x[h][j], mx));
                x[h][j] = v;
                acc += v > 0.f ? v : 0.f;
                if (want_hist && v > 0.f) {
                    const uint32_t eb = __float_as_uint(v);
                    const unsigned bin = bin_of(eb);
                    if (bin == 0u) low++;
                    else { atomicAdd(&hcnt[bin], 1u); atomicAdd(&hmass[bin], ((eb & 0x7FFFFFu) | 0x800000u) >> 12); }
                }
            }
            if (want_hist) {
                low = __reduce_add_sync(0xFFFFFFFFu, low);
                if (low && lane == 0) { atomicAdd(&hcnt[0], (unsigned)low); atomicAdd(&hmass[0], (unsigned)low * 0xFFFu); }
            }
            if (base < n) store8(e, base, n, x[h]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
            if (lane == 0) { ew->sums[(begin >> 8) + st] = acc; s_sum[st] = acc; }
        }
    }
    if (want_hist) {
        __syncthreads();
        unsigned long long *hist = ws.hist + (size_t)fi * kHistBins;
        for (int b = tid; b < kHistBins; b += kFullThreads) {
            const unsigned c = hcnt[b];
            if (c) atomicAdd(&hist[b], ((unsigned long long)c << 40) | (unsigned long long)hmass[b]);
        }
    }
    // phases B and C of the softmax sum for this piece, on the exp values still in registers
    piece_tail<false>(fr, ew, xs, begin, n, s_sum, s_guess, s_xslot, &s_ok, a.lookback_drill == 1);
}

// ---- sums of the final probabilities (the draw's phase A) ------------------------------------------------
__global__ void __launch_bounds__(kFullThreads) k_full_psums(const __grid_constant__ SampleArgs a, const FullWs ws,
                                                             const WorkItem *full_items)
{
    __shared__ float s_sum[kPieceSubTiles];
    __shared__ unsigned char s_guess[kPieceSubTiles], s_xslot[kPieceSubTiles];
    __shared__ int s_ok;
    const int fi = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = full_items[fi].row;
    const RowPlan *rpp = a.plans + row;
    if (!(__ldg(&rpp->temperature) > 0.f)) return;
    const int n = a.vocab;
    const int begin = blockIdx.x * kPhasePiece;
    if (begin >= n) return;
    FullRow *fr = ws.rows + fi;
    if (fr->redo) return;
    const ProvFinal pf{ws.e + (size_t)fi * ws.e_stride, fr->dist, nullptr};
    Emul2Work *ew = ws.ew + fi;
    constexpr int W = kFullThreads / 32;
    float xs[kWarpSubTiles][8];
#pragma unroll
    for (int it = 0; it < kWarpSubTiles / 2; it++) {
        const int st0 = warp + it * 2 * W;
        float (&x)[2][8] = *reinterpret_cast<float (*)[2][8]>(&xs[it * 2]);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int st = st0 + h * W;
            pf.reload(st < kPieceSubTiles ? begin + st * kSub + lane * 8 : n, n, x[h]);  // zeros beyond the row
        }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int st = st0 + h * W;
            if (st >= kPieceSubTiles || begin + st * kSub >= n) continue;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) acc += x[h][j] > 0.f ? x[h][j] : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
            if (lane == 0) { ew->sums[(begin >> 8) + st] = acc; s_sum[st] = acc; }
        }
    }
    piece_tail<true>(fr, ew, xs, begin, n, s_sum, s_guess, s_xslot, &s_ok, a.lookback_drill == 2);
}

// copies a row's sub-tile summaries from device memory into the shared-memory work area of the walk
__device__ __forceinline__ void load_work(Emul2Work *dst, const Emul2Work *src)
{
    const uint4 *s = (const uint4 *)src;
    uint4 *d = (uint4 *)dst;
    for (int i = threadIdx.x; i < (int)(sizeof(Emul2Work) / 16); i += kThreads) d[i] = __ldcg(s + i);
    __syncthreads();
}
static_assert(sizeof(Emul2Work) % 16 == 0, "Emul2Work is copied in 16-byte words");

// exp values of a row as the walk replays them (ProvExp's reload without its load side)
struct ProvE {
    const float *scratch;
    __device__ __forceinline__ void load(int base, int n, float x[8]) const { reload(base, n, x); }
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
};

// ---- a shared-memory cache of the sub-tiles a walk will replay ------------------------------------------
// The walk (emul2_walk) consumes most sub-tiles by their composites and touches elements only where
// the running sum changes binade, where a guess was off by one sub-tile, or where the target is met.
// Those places are known in advance from the fp64 prefix of the sub-tile sums: the sub-tiles with a
// crossing slot and their neighbours, the first sub-tiles (the sum climbs through many binades
// there), and the sub-tile in which the prefix reaches the target.  All warps copy them into shared
// memory before the one walking warp starts, so that its replays do not wait on L2.
constexpr int kXcEntries = 64;
struct XCache {
    int of[kMaxSubTiles];      // 0: not cached, else 1 + entry
    int tile[kXcEntries];
    int n;
    int hit_tile;
    double wsum[32];
};

template <class P>
struct ProvCached {
    P base;
    const float *xc;
    const int *of;
    __device__ __forceinline__ void load(int b, int n, float x[8]) const { reload(b, n, x); }
    __device__ __forceinline__ void reload(int b, int n, float x[8]) const
    {
        const int idx = of[b >> 8];
        if (idx > 0) {
            const float4 *q = (const float4 *)(xc + (size_t)(idx - 1) * kSub + (b & (kSub - 1)));
            const float4 q0 = q[0], q1 = q[1];
            x[0] = q0.x; x[1] = q0.y; x[2] = q0.z; x[3] = q0.w; x[4] = q1.x; x[5] = q1.y; x[6] = q1.z; x[7] = q1.w;
        } else {
            base.reload(b, n, x);
        }
    }
};

// Fills the cache for the sequence behind `pv` (n elements, nsub sub-tiles, summaries in wk).  With
// has_target the sub-tile in which the fp64 prefix of the sums reaches `target` is cached too.
// All kThreads threads call it.
template <class P>
__device__ void build_xcache(XCache *xc, float *xdata, const Emul2Work *wk, const P &pv, int n, int nsub, float target,
                             bool has_target)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int t = tid; t < kMaxSubTiles; t += kThreads) xc->of[t] = 0;
    if (tid == 0) { xc->n = 0; xc->hit_tile = INT_MAX; }
    __syncthreads();
    if (has_target) {
        double v = tid < nsub ? (double)wk->sums[tid] : 0.0, inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) xc->wsum[warp] = inc;
        __syncthreads();
        double before = 0.0;
        for (int w = 0; w < warp; w++) before += xc->wsum[w];
        if (tid < nsub && before + inc >= (double)target * (1.0 - 1e-5)) atomicMin(&xc->hit_tile, tid);
        __syncthreads();
    }
    auto mark = [&](int t) {
        if (t >= 0 && t < nsub && atomicCAS(&xc->of[t], 0, -1) == 0) {
            const int e = atomicAdd(&xc->n, 1);
            if (e < kXcEntries) { xc->tile[e] = t; xc->of[t] = e + 1; } else { xc->of[t] = 0; }
        }
    };
    if (tid < 4) mark(tid);
    if (tid < nsub && wk->xslot[tid]) { mark(tid - 1); mark(tid); mark(tid + 1); mark(tid + 2); }
    if (has_target && tid == 0 && xc->hit_tile != INT_MAX) { mark(xc->hit_tile - 1); mark(xc->hit_tile); mark(xc->hit_tile + 1); }
    __syncthreads();
    const int ne = min(xc->n, kXcEntries);
    for (int e = warp; e < ne; e += kThreads / 32) {
        float x[8];
        pv.reload(xc->tile[e] * kSub + lane * 8, n, x);
        float4 *q = (float4 *)(xdata + (size_t)e * kSub + lane * 8);
        q[0] = make_float4(x[0], x[1], x[2], x[3]);
        q[1] = make_float4(x[4], x[5], x[6], x[7]);
    }
    __syncthreads();
}

// ---- walk: exact softmax sum, min-p, top-p plan ----------------------------------------------------------
// One 1024-thread CTA per full row.  The top-p plan is steps (1)-(3) of topp_cut (stg_rowdist.cuh):
// the bins that bound the nucleus, where every bin starts in the bin-ordered candidate list, the
// binade the sorted running sum is in at every bin, and the bins that must be in exact order.
__global__ void __launch_bounds__(kThreads, 1) k_full_walk(const __grid_constant__ SampleArgs a, const FullWs ws,
                                                           const WorkItem *full_items)
{
    extern __shared__ __align__(16) unsigned char arena[];
    __shared__ RowCtl rc;
    __shared__ XCache xcache;
    const int fi = blockIdx.x, tid = threadIdx.x;
    const int row = full_items[fi].row;
    const RowPlan rp = a.plans[row];
    FullRow *fr = ws.rows + fi;
    const int n = a.vocab;
    const unsigned long long mk = fr->maxkey;
    unsigned long long *tk = a.phase_ticks ? a.phase_ticks + (int64_t)fi * 32 : nullptr;
    tick(tk, 0);
    if (!(rp.temperature > 0.f)) {
        // GreedyWithHistoryPenalties (Sampler.cs:421-437): the arg-max of the adjusted logits
        if (tid == 0) {
            const int tok = mk ? key_idx(mk) : 0;
            if (a.mode == 2) {
                RowDist d;
                memset(&d, 0, sizeof(d));
                d.flags = kDistOneHot;
                d.tie_idx_max = tok;
                d.argmax = tok;
                d.inv_t = 1.f; d.inv1 = 1.f; d.inv2 = 1.f; d.inv3 = 1.f;
                a.dists[row] = d;
            } else {
                if (a.tokens) a.tokens[row] = tok;
                if (a.token_probs) a.token_probs[row] = 1.f;
                if (a.row_flags) a.row_flags[row] = (uint32_t)rp.path | (mk ? 0u : (1u << 6));
            }
        }
        return;
    }
    Emul2Work *wk2 = (Emul2Work *)(arena + kOffEmul);
    const float *e = ws.e + (size_t)fi * ws.e_stride;
    const bool uniform = mk == 0ull;
    const float inv_t = rp.temperature != 1.0f ? __fdiv_rn(1.0f, rp.temperature) : 1.0f;
    RowDist d;
    d.flags = 0;
    d.inv_t = inv_t;
    d.tie_idx_max = INT_MAX;
    d.kth = 0.f; d.inv2 = 1.f; d.minp_thr = 0.f; d.tstar = 0.f; d.inv3 = 1.f; d.inv1 = 1.f;
    d.uniform_p = 0.f; d.sum_end = 0.f; d.argmax = 0;
    float sum = 0.f;
    if (uniform) {
        d.flags |= kDistUniform;
        d.max_x = -CUDART_INF_F;
        d.uniform_p = __fdiv_rn(1.0f, (float)n);
    } else {
        d.max_x = key_val(mk);
        load_work(wk2, ws.ew + fi);
        tick(tk, 1);
        const int nsub = (n + kSub - 1) / kSub;
        const ProvE pe{e};
        float *xdata = (float *)(arena + kOffKeys);  // the key region is free in this kernel
        build_xcache(&xcache, xdata, wk2, pe, n, nsub, 0.f, false);
        tick(tk, 2);
        if (tid < 32) {
            const ProvCached<ProvE> pc{pe, xdata, xcache.of};
            emul2_walk<ProvCached<ProvE>, false, false>(&rc.em2, wk2, pc, n, nsub, 0.f, false, nullptr, tk ? tk + 24 : nullptr);
        }
        __syncthreads();
        tick(tk, 3);
        sum = rc.em2.s;
        if (sum > 0.f && sum != 1.0f) { d.flags |= kDistScale1; d.inv1 = __fdiv_rn(1.0f, sum); }
    }
    if (rp.min_p > 0.f) {
        // ApplyMinP (Sampler.cs:493-503): the largest probability belongs to exp value 1 (or 1/V)
        const float emax = uniform ? d.uniform_p : 1.0f;
        const float pmax = (d.flags & kDistScale1) ? __fmul_rn(emax, d.inv1) : emax;
        d.minp_thr = __fmul_rn(rp.min_p, pmax);
        d.flags |= kDistMinP;
    }
    tick(tk, 4);
    if (tid == 0) { fr->dist = d; fr->sum = sum; }
}

// ---- plan: where the nucleus ends in the histogram, where every bin starts in the candidate list ----------
// Steps (1) to (3) of topp_cut.  They need the softmax sum only to turn histogram masses into
// probabilities, and every use carries a margin (the bound of step 1, the binade guesses and flags of
// step 3), so the fp64 sum of the sub-tile sums stands in for the exact sequential sum, which
// k_full_walk is computing at the same time on another stream.  Should the bound come out too tight
// all the same, k_full_cut notices (the sum never reaches top_p although survivors remain) and the
// row is redone.
__global__ void __launch_bounds__(kThreads, 1) k_full_plan(const __grid_constant__ SampleArgs a, const FullWs ws,
                                                           const WorkItem *full_items)
{
    extern __shared__ __align__(16) unsigned char arena[];
    __shared__ RowCtl rc;
    const int fi = blockIdx.x, tid = threadIdx.x;
    const int row = full_items[fi].row;
    const RowPlan rp = a.plans[row];
    if (!(rp.temperature > 0.f) || !row_wants_topp(rp)) return;
    FullRow *fr = ws.rows + fi;
    const int n = a.vocab;
    const bool uniform = fr->maxkey == 0ull;
    unsigned *hcount = (unsigned *)(arena + kOffCount);
    unsigned *hmass = (unsigned *)(arena + kOffMass);
    unsigned *bstart = (unsigned *)(arena + kOffBinOff);
    unsigned char *bin_exp = arena + kOffBinExp;
    struct { int flags; float inv1; float uniform_p; } d;
    d.flags = 0; d.inv1 = 1.f; d.uniform_p = 0.f;
    if (uniform) {
        d.flags |= kDistUniform;
        d.uniform_p = __fdiv_rn(1.0f, (float)n);
    } else {
        const int nsub = (n + kSub - 1) / kSub;
        const float *sums = (ws.ew + fi)->sums;
        double part = 0.0;
        for (int t = tid; t < nsub; t += kThreads) part += (double)__ldcg(sums + t);
        const double total = block_sum_double(part, rc.red_d);
        if (total > 0.0 && total != 1.0) { d.flags |= kDistScale1; d.inv1 = (float)(1.0 / total); }
    }
    const bool want_topp = true;
    if (want_topp) {
        // histogram of the exp values as the exp pass left it
        const unsigned long long *hist = ws.hist + (size_t)fi * kHistBins;
        if (uniform) {
            for (int b = tid; b < kHistBins; b += kThreads) { hcount[b] = 0u; hmass[b] = 0u; }
            __syncthreads();
            if (tid == 0) {
                const unsigned bin = bin_of(__float_as_uint(d.uniform_p));
                hcount[bin] = (unsigned)n;
                hmass[bin] = (unsigned)min((unsigned long long)n * ((((unsigned long long)__float_as_uint(d.uniform_p) & 0x7FFFFFu) | 0x800000u) >> 12), 0xFFFFFFFFull);
            }
        } else {
            for (int b = tid; b < kHistBins; b += kThreads) {
                const unsigned long long v = __ldcg(hist + b);
                hcount[b] = (unsigned)(v >> 40);
                hmass[b] = (unsigned)(v & 0xFFFFFFFFull);
            }
        }
        __syncthreads();
        const double scale_p = (d.flags & kDistScale1) ? (double)d.inv1 : 1.0;
        if (tid == 0) rc.c_lo = 0;
        __syncthreads();
        {
            // (1) bound the nucleus: bins from the top until the estimated mass clears top_p
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
            double am = scan4_double(tm, &rc) - tm;
            double ac = scan4_double(tc, &rc) - tc;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int b = kBins - 1 - (tid * 4 + j);
                am += lm[j];
                ac += (double)lc[j];
                if (lc[j]) {
                    const double need = (double)rp.top_p * (1.0 + 1.0 / 65536.0) + 16.0 * sqrt(ac) * 2.98e-8 + 1e-7;
                    if (am * scale_p >= need) atomicMax(&rc.c_lo, b > 0 ? b - 1 : 0);
                }
            }
            __syncthreads();
        }
        const int c_lo = rc.c_lo;
        {
            // (2) start of every candidate bin in the bin-ordered list (largest bin first)
            unsigned loc[4], tot = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int b = kBins - 1 - (tid * 4 + j);
                loc[j] = b >= c_lo ? hcount[b] : 0u;
                tot += loc[j];
            }
            const double incl = scan4_double((double)tot, &rc);
            unsigned run = (unsigned)(incl - (double)tot);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int b = kBins - 1 - (tid * 4 + j);
                bstart[b] = run;
                run += loc[j];
            }
            if (tid == kThreads - 1) rc.bound = (int)run;
            __syncthreads();
        }
        for (int t = tid; t < kBins / 32; t += kThreads) rc.flag_bits[t] = 0u;
        __syncthreads();
        {
            // (3) the binade the sorted running sum is in at every bin; bins in which it may change
            // binade or meet top_p, and the head of the list, must be in exact order
            double loc[4], tot = 0.0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int b = kBins - 1 - (tid * 4 + j);
                loc[j] = (b >= c_lo && hcount[b]) ? bin_mass(hmass, b) * scale_p : 0.0;
                tot += loc[j];
            }
            double before = scan4_double(tot, &rc) - tot;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int b = kBins - 1 - (tid * 4 + j);
                const double lo = before * (1.0 - 1.0 / 32768.0), hi = (before + loc[j]) * (1.0 + 1.0 / 2048.0);
                const int e_lo = exp_of_double(lo);
                bin_exp[b] = (unsigned char)e_lo;
                if (b >= c_lo && hcount[b]) {
                    const bool crosses = e_lo != exp_of_double(hi);
                    const bool cut = lo <= (double)rp.top_p && hi >= (double)rp.top_p;
                    const bool head = bstart[b] < 2048u;
                    if (crosses || cut || head) atomicOr(&rc.flag_bits[b >> 5], 1u << (b & 31));
                }
                before += loc[j];
            }
            __syncthreads();
        }
        // the plan, for the scatter pass and the cut
        uint32_t *g_bstart = ws.bstart + (size_t)fi * kHistBins;
        unsigned char *g_binexp = ws.bin_exp + (size_t)fi * kHistBins;
        uint32_t *g_flags = ws.flag_bits + (size_t)fi * (kHistBins / 32);
        for (int b = tid; b < kHistBins; b += kThreads) { g_bstart[b] = bstart[b]; g_binexp[b] = bin_exp[b]; }
        for (int t = tid; t < kHistBins / 32; t += kThreads) g_flags[t] = rc.flag_bits[t];
        if (tid == 0) { fr->c_lo = c_lo; fr->bound = rc.bound; }
    }
}

// ---- scatter: candidates into bin order, survivors counted ---------------------------------------------
// Step (4) of topp_cut over a piece: every exp value at or above the plan's lowest bin goes to its
// bin's range of the row's candidate list, AS AN EXP VALUE - the list is ordered by bins of exp
// values, and the probability of a candidate (exp value times 1 / sum, then the min-p filter) is a
// non-decreasing function of it, so k_full_cut turns the list into probabilities once the exact sum
// is known.  That leaves this pass independent of the walk that computes the sum: the two run side by
// side.  Rows without top-p are not touched (k_full_nosum).
__global__ void __launch_bounds__(kFullThreads) k_full_scatter(const __grid_constant__ SampleArgs a, const FullWs ws,
                                                               const WorkItem *full_items)
{
    // Positions are handed out in two levels: the CTA counts its candidates per bin in shared memory
    // (a candidate's count at that moment is its rank inside the CTA's share of the bin), reserves the
    // CTA's share of every bin it touched with ONE global atomicAdd per bin, and then writes.  The
    // per-element global atomic with a returned value that this replaces cost a round trip to L2 each.
    __shared__ unsigned s_cnt[kBins];
    __shared__ int red_i[kFullThreads / 32];
    const int fi = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = full_items[fi].row;
    const RowPlan *rpp = a.plans + row;
    if (!(__ldg(&rpp->temperature) > 0.f)) return;
    const float top_p = __ldg(&rpp->top_p);
    if (!(top_p < 1.0f && top_p > 0.f)) return;
    const int n = a.vocab;
    const int begin = blockIdx.x * kPhasePiece;
    if (begin >= n) return;
    FullRow *fr = ws.rows + fi;
    const float *e = ws.e + (size_t)fi * ws.e_stride;
    const int c_lo = fr->c_lo;
    const uint32_t lo_bits = bin_floor_bits(c_lo);
    const unsigned cap = (unsigned)ws.key_stride;
    const uint32_t *bstart = ws.bstart + (size_t)fi * kHistBins;
    uint32_t *cursor = ws.cursor + (size_t)fi * kHistBins;
    uint32_t *keys = ws.keys + (size_t)fi * ws.key_stride;
    constexpr int R = kPhasePiece / (kFullThreads * 8);  // rounds of 8 consecutive elements per thread
    float x[R][8];
    unsigned short rank[R][8];
    for (int b = tid; b < kBins; b += kFullThreads) s_cnt[b] = 0u;
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int base = begin + (r * kFullThreads + tid) * 8;
        if (base < n) {
            SrcScratch sc{e, 1.f, false};
            sc.get8(base, n, x[r]);
        }
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (base + j >= n) x[r][j] = 0.f;
    }
    __syncthreads();
    int my_surv = 0;
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float ev = x[r][j];
            rank[r][j] = 0xFFFFu;  // not a candidate
            if (ev > 0.f) {
                my_surv++;  // survives softmax; min-p may still drop it (k_full_cut errs on the safe side)
                const uint32_t ebits = __float_as_uint(ev);
                if (ebits >= lo_bits) rank[r][j] = (unsigned short)atomicAdd(&s_cnt[bin_of(ebits)], 1u);
            }
        }
    __syncthreads();
    // the CTA's share of every bin it touched: s_cnt turns from a count into the first position
    for (int b = tid; b < kBins; b += kFullThreads) {
        const unsigned c = s_cnt[b];
        if (c) s_cnt[b] = __ldg(bstart + b) + atomicAdd(&cursor[b], c);
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (rank[r][j] != 0xFFFFu) {
                const uint32_t ebits = __float_as_uint(x[r][j]);
                const unsigned pos = s_cnt[bin_of(ebits)] + rank[r][j];
                if (pos < cap) keys[pos] = ebits;
            }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) my_surv += __shfl_xor_sync(0xFFFFFFFFu, my_surv, o);
    if (lane == 0) red_i[warp] = my_surv;
    __syncthreads();
    if (tid == 0) {
        int t = 0;
        for (int w = 0; w < kFullThreads / 32; w++) t += red_i[w];
        if (t) atomicAdd(&fr->surv, t);
    }
}

// ---- rows without top-p: the fp64 sum of their probabilities for Normalize (Sampler.cs:553-562) ----------
// Needs the exact distribution descriptor, so it runs behind k_full_walk; launched only when the step
// has such rows.
__global__ void __launch_bounds__(kFullThreads) k_full_nosum(const __grid_constant__ SampleArgs a, const FullWs ws,
                                                             const WorkItem *full_items)
{
    __shared__ double red_d[kFullThreads / 32];
    const int fi = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = full_items[fi].row;
    const RowPlan *rpp = a.plans + row;
    if (!(__ldg(&rpp->temperature) > 0.f)) return;
    const float top_p = __ldg(&rpp->top_p);
    if (top_p < 1.0f && top_p > 0.f) return;
    const int n = a.vocab;
    const int begin = blockIdx.x * kPhasePiece;
    if (begin >= n) return;
    FullRow *fr = ws.rows + fi;
    const RowDist d = fr->dist;
    const float *e = ws.e + (size_t)fi * ws.e_stride;
    const int end = min(n, begin + kPhasePiece);
    double part = 0.0;
    for (int base = begin + tid * 8; base < end; base += kFullThreads * 8) {
        float x[8];
        SrcScratch sc{e, 1.f, false};
        sc.get8(base, n, x);
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (base + j < n) part += (double)eval_p2(x[j], d);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, o);
    if (lane == 0) red_d[warp] = part;
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int w = 0; w < kFullThreads / 32; w++) t += red_d[w];
        fr->part[blockIdx.x] = t;
    }
}

// ---- ties: candidates whose addition would be an exact tie flag their bin --------------------------------
// With the exact sum known (k_full_walk) and the candidates in place (k_full_scatter): a candidate
// whose probability falls exactly between two floats at the binade the sorted running sum has at its
// bin makes the rounding depend on the parity of the sum, so the order inside that bin matters and
// k_full_cut has to sort it.  One pass over the candidate lists, all SMs: grid (pieces of 8192
// candidates, full rows).
__global__ void __launch_bounds__(kFullThreads) k_full_ties(const __grid_constant__ SampleArgs a, const FullWs ws,
                                                            const WorkItem *full_items)
{
    const int fi = blockIdx.y, tid = threadIdx.x;
    const int row = full_items[fi].row;
    const RowPlan *rpp = a.plans + row;
    const float top_p = __ldg(&rpp->top_p);
    if (!(__ldg(&rpp->temperature) > 0.f) || !(top_p < 1.0f && top_p > 0.f)) return;
    const FullRow *fr = ws.rows + fi;
    const int nc = min(fr->bound, (int)ws.key_stride);
    const int begin = blockIdx.x * kPhasePiece;
    if (begin >= nc) return;
    const RowDist d = fr->dist;
    const int scale = (d.flags & kDistScale1) ? 1 : 0, minp = (d.flags & kDistMinP) ? 1 : 0;
    const unsigned char *bin_exp = ws.bin_exp + (size_t)fi * kHistBins;
    uint32_t *flag_bits = ws.flag_bits + (size_t)fi * (kHistBins / 32);
    const uint4 *g16 = (const uint4 *)(ws.keys + (size_t)fi * ws.key_stride);
    const int q_end = (min(nc, begin + kPhasePiece) + 3) >> 2;
    constexpr int U = kPhasePiece / (4 * kFullThreads);  // quads per thread
    uint4 eb[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
        const int q = (begin >> 2) + u * kFullThreads + tid;
        eb[u] = q < q_end ? __ldcg(g16 + q) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
        const int q = (begin >> 2) + u * kFullThreads + tid;
        const uint32_t four[4] = {eb[u].x, eb[u].y, eb[u].z, eb[u].w};
#pragma unroll
        for (int c4 = 0; c4 < 4; c4++) {
            if (q >= q_end || q * 4 + c4 >= nc) continue;
            const uint32_t ebits = four[c4];
            float p = __uint_as_float(ebits);
            if (scale) p = __fmul_rn(p, d.inv1);
            if (minp && p < d.minp_thr) p = 0.f;
            const uint32_t pbits = __float_as_uint(p);
            const unsigned bin = bin_of(ebits);
            const int k = (int)__ldg(bin_exp + bin) - (int)((pbits >> 23) & 255u);
            if (k >= 1 && k <= 24) {
                const uint32_t m = (pbits & 0x7FFFFFu) | 0x800000u;
                if ((m & ((1u << k) - 1u)) == (1u << (k - 1))) atomicOr(&flag_bits[bin >> 5], 1u << (bin & 31));
            }
        }
    }
}

// The candidate list of the flat step holds exp values (k_full_scatter); every reader turns them into
// the probabilities the reference sorts and sums - softmax scale, then the min-p filter (eval_p2; the
// flat step has no rows with top-k on this path) - as it loads them.  The conversion is monotonic, so
// the list's order by exp value is an order by probability.
struct KeyConv {
    int scale;        // multiply by inv1
    float inv1;
    int minp;         // apply the min-p threshold
    float minp_thr;
    __device__ __forceinline__ float operator()(uint32_t ebits) const
    {
        float p = __uint_as_float(ebits);
        if (scale) p = __fmul_rn(p, inv1);
        if (minp && p < minp_thr) p = 0.f;
        return p;
    }
};
struct ProvKeysE {
    const uint32_t *keys;
    bool global;  // the list sits in global memory (a nucleus too wide for shared memory): staged reads pay
    KeyConv conv;
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
#pragma unroll
        for (int j = 0; j < 8; j++) x[j] = (base + j < n) ? conv(keys[base + j]) : 0.f;
    }
    __device__ __forceinline__ void reload(int base, int n, float x[8]) const { load(base, n, x); }
    static constexpr int kQuadsLoad = 2, kQuadsReload = 2;
    __device__ __forceinline__ bool stage_ok() const { return global; }
    __device__ __forceinline__ const char *stage_src(int base, bool) const { return (const char *)(keys + base); }
    __device__ __forceinline__ void load_from(int base, int n, const float4 *q, float x[8]) const
    {
        const uint32_t *u = (const uint32_t *)q;
#pragma unroll
        for (int j = 0; j < 8; j++) x[j] = conv(u[j]);
    }
    __device__ __forceinline__ void reload_from(int base, int n, const float4 *q, float x[8]) const
    {
        load_from(base, n, q, x);
    }
};

// ---- cut: the top-p threshold from the bin-ordered candidates; Normalize ---------------------------------
// Steps (5) onwards of topp_cut for a row whose candidates the scatter pass left in device memory.
__global__ void __launch_bounds__(kThreads, 1) k_full_cut(const __grid_constant__ SampleArgs a, const FullWs ws,
                                                          const WorkItem *full_items)
{
    extern __shared__ __align__(16) unsigned char arena[];
    __shared__ RowCtl rc_s;
    __shared__ uint32_t sh_flags;
    RowCtl *rc = &rc_s;
    const int fi = blockIdx.x, tid = threadIdx.x;
    const int row = full_items[fi].row;
    const RowPlan rp = a.plans[row];
    if (!(rp.temperature > 0.f)) return;
    FullRow *fr = ws.rows + fi;
    const int n = a.vocab;
    RowDist d = fr->dist;
    const float *scratch = ws.e + (size_t)fi * ws.e_stride;
    const bool want_topp = row_wants_topp(rp);
    double sum3 = 0.0;
    unsigned long long *tk = a.phase_ticks ? a.phase_ticks + (int64_t)fi * 32 : nullptr;
    tick(tk, 8);
    if (tid == 0) sh_flags = 0u;
    __syncthreads();
    if (!want_topp) {
        const int pieces = (n + kPhasePiece - 1) / kPhasePiece;
        for (int p = 0; p < pieces; p++) sum3 += fr->part[p];  // fixed order: deterministic
    } else {
        uint32_t *skeys = (uint32_t *)(arena + kOffKeys);
        unsigned *hcount = (unsigned *)(arena + kOffCount);
        unsigned *bstart = (unsigned *)(arena + kOffBinOff);
        Emul2Work *wk2 = (Emul2Work *)(arena + kOffEmul);
        unsigned char *replay_ok = arena + kOffReplayOk;
        const bool uniform = (d.flags & kDistUniform) != 0;
        const int c_lo = fr->c_lo;
        const int bound = fr->bound;
        const int my_surv = fr->surv;
        const uint32_t *g_cursor = ws.cursor + (size_t)fi * kHistBins;
        const uint32_t *g_bstart = ws.bstart + (size_t)fi * kHistBins;
        const uint32_t *g_flags = ws.flag_bits + (size_t)fi * (kHistBins / 32);
        uint32_t *gkeys = ws.keys + (size_t)fi * ws.key_stride;
        if (tid == 0) { rc->c_lo = c_lo; rc->give_up = 0; rc->n_dirty = 0; rc->bound = bound; }
        // from here on the histogram describes the list: the filters before top-p drop the smallest
        // values only, so the bins that lost elements are the last ones of the list and it stays dense
        int mine = 0;
        for (int b = tid; b < kHistBins; b += kThreads) {
            const unsigned have = b >= c_lo ? __ldcg(g_cursor + b) : 0u;
            hcount[b] = have;
            bstart[b] = __ldcg(g_bstart + b);
            mine += (int)have;
        }
        for (int t = tid; t < kHistBins / 32; t += kThreads) { rc->flag_bits[t] = __ldcg(g_flags + t); rc->sorted_bits[t] = 0u; }
        uint32_t *keys = skeys;
        int cap = kSortCap;
        if (bound > kSortCap) { keys = gkeys; cap = (int)ws.key_stride; if (tid == 0) sh_flags |= (1u << 7); }
        const int nc = min(block_sum_int(mine, rc->red_i), cap);
        __syncthreads();
        // The list holds exp values (k_full_scatter): a short one is copied to shared memory, a wide one
        // stays where it is; every reader turns them into probabilities as it loads them (KeyConv).
        const KeyConv conv{(d.flags & kDistScale1) ? 1 : 0, d.inv1, (d.flags & kDistMinP) ? 1 : 0, d.minp_thr};
        if (keys == skeys) {
            // 16-byte loads (the list starts on a 16-byte boundary and is read in whole quads: what lies
            // behind its end is never used)
            const uint4 *g16 = (const uint4 *)gkeys;
            const int nq = (nc + 3) >> 2;
            __syncthreads();
            for (int q = tid; q < nq; q += kThreads) ((uint4 *)skeys)[q] = __ldcg(g16 + q);
            __syncthreads();
        }
        tick(tk, 9);
        if (tk && tid == 0) { tk[20] = (unsigned long long)nc; tk[21] = 0; }
        if (nc > 0) {
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
                        const int slot = atomicAdd(&rc->n_dirty, 1);
                        if (slot < kMaxDirty) rc->dirty[slot] = (unsigned short)b; else rc->give_up = 1;
                    }
                }
            }
            __syncthreads();
            int hit = -1;
            float cum = 0.f;
            bool sorted_all = uniform;  // all keys equal: any order is sorted
            tick(tk, 10);
            if (tk && tid == 0) tk[22] = (unsigned long long)rc->n_dirty;
            for (int pass = 0; pass < 64; pass++) {
                if (tk && tid == 0) tk[21] = (unsigned long long)(pass + 1);
                if (!sorted_all && (rc->give_up || pass == 63)) {
                    const int p2 = pow2_ceil(max(nc, 2));
                    for (int t = nc + tid; t < p2; t += kThreads) keys[t] = 0u;
                    __syncthreads();
                    bitonic_sort_desc_t<uint32_t>(keys, p2);
                    sorted_all = true;
                } else if (!sorted_all && rc->n_dirty > 0) {
                    sort_dirty_bins(rc, keys, bstart, hcount, (uint32_t *)wk2, (int *)wk2 + kDirtyRound);
                    __syncthreads();
                    if (rc->give_up) continue;
                    for (int i = tid; i < min(rc->n_dirty, kMaxDirty); i += kThreads)
                        atomicOr(&rc->sorted_bits[rc->dirty[i] >> 5], 1u << (rc->dirty[i] & 31));
                    __syncthreads();
                    if (tid == 0) rc->n_dirty = 0;
                }
                __syncthreads();
                if (pass == 0) tick(tk, 11);
                if (!sorted_all) {
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
                ProvKeysE pk{keys, keys != skeys, conv};
                if (nc <= kSub * kMaxSubTiles) {
                    hit = emul_scan2<ProvKeysE, false, true, 4>(&rc->em2, wk2, pk, nc, rp.top_p, true, &cum,
                                                            sorted_all ? nullptr : replay_ok, tk ? tk + 24 : nullptr,
                                                            keys != skeys ? arena + kOffKeys : nullptr, kSortCap * 4);
                } else {
                    if (!sorted_all) { if (tid == 0) rc->give_up = 1; __syncthreads(); continue; }
                    hit = emul_scan<ProvKeysE, false>(&rc->em, pk, nc, rp.top_p, true, &cum);
                }
                if (hit != -2) break;
                const int t_abort = rc->em2.abort_at;
                for (int b = c_lo + tid; b < kBins; b += kThreads) {
                    const unsigned cnt = hcount[b];
                    if (cnt >= 2u && !((rc->sorted_bits[b >> 5] >> (b & 31)) & 1u)) {
                        const int t0 = (int)bstart[b] >> 8, t1 = (int)(bstart[b] + cnt - 1) >> 8;
                        if (t0 <= t_abort && t_abort <= t1) {
                            const int slot = atomicAdd(&rc->n_dirty, 1);
                            if (slot < kMaxDirty) rc->dirty[slot] = (unsigned short)b; else rc->give_up = 1;
                        }
                    }
                }
                __syncthreads();
            }
            tick(tk, 12);
            if (hit < 0 && nc < my_surv) {
                // the bound was too tight (the sum never reached top_p although survivors remain
                // below it): the self-contained row kernel redoes the row
                if (tid == 0) fr->redo = 1;
                return;
            }
            const int last = hit >= 0 ? hit : nc - 1;
            const float tstar = hit >= 0 ? conv(keys[last]) : 0.f;
            if (hit >= 0 && nc <= kSub * kMaxSubTiles && tid == 0 &&
                (cum - rp.top_p <= kNearTol || rp.top_p - rc->em2.hit_before <= kNearTol))
                sh_flags |= kFlagNearCut;  // a last-bit difference in exp could move the cut by a token
            int keep = 0, all = 0;
            double part = 0.0;
            for (int t = tid; t < nc; t += kThreads) {
                const float p = conv(keys[t]);
                if (p == tstar) { all++; keep += (t <= last) ? 1 : 0; }
                if (t <= last) part += (double)p;
            }
            keep = block_sum_int(keep, rc->red_i);
            all = block_sum_int(all, rc->red_i);
            sum3 = block_sum_double(part, rc->red_d);
            d.flags |= kDistTopP;
            d.tstar = tstar;
            d.tie_idx_max = INT_MAX;
            if (keep < all) {
                if (tid == 0) sh_flags |= (1u << 4);
                d.tie_idx_max = find_kth_match(rc, scratch, n, d, tstar, keep);
            }
        }
    }
    // Normalize (Sampler.cs:553-562)
    const float s3 = (float)sum3;
    if (s3 > 0.f && s3 != 1.0f) { d.flags |= kDistScale3; d.inv3 = __fdiv_rn(1.0f, s3); }
    __syncthreads();
    tick(tk, 13);
    if (tid == 0) {
        fr->dist = d;
        fr->flags |= sh_flags;
        if (a.mode == 2) {
            const unsigned long long rk = fr->rawkey;
            d.argmax = rk ? key_idx(rk) : 0;
            a.dists[row] = d;
        }
    }
}

// ---- draw: SampleFromDistribution (Sampler.cs:564-576) ----------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1) k_full_draw(const __grid_constant__ SampleArgs a, const FullWs ws,
                                                           const WorkItem *full_items)
{
    extern __shared__ __align__(16) unsigned char arena[];
    __shared__ Emul2Ctl ctl;
    __shared__ XCache xcache;
    const int fi = blockIdx.x, tid = threadIdx.x;
    const int row = full_items[fi].row;
    const RowPlan rp = a.plans[row];
    if (!(rp.temperature > 0.f)) return;
    const FullRow *fr = ws.rows + fi;
    if (fr->redo) return;
    const int n = a.vocab;
    Emul2Work *wk2 = (Emul2Work *)arena;
    float *xdata = (float *)(arena + sizeof(Emul2Work));
    unsigned long long *tk = a.phase_ticks ? a.phase_ticks + (int64_t)fi * 32 : nullptr;
    tick(tk, 16);
    load_work(wk2, ws.ew + fi);
    tick(tk, 17);
    const float *e = ws.e + (size_t)fi * ws.e_stride;
    const RowDist d = fr->dist;
    const float u = a.uniforms ? __ldg(a.uniforms + row) : 0.5f;
    const int nsub = (n + kSub - 1) / kSub;
    const ProvFinal pf{e, d, nullptr};
    build_xcache(&xcache, xdata, wk2, pf, n, nsub, u, true);
    tick(tk, 18);
    if (tid < 32) {
        const ProvCached<ProvFinal> pc{pf, xdata, xcache.of};
        emul2_walk<ProvCached<ProvFinal>, false, false>(&ctl, wk2, pc, n, nsub, u, true, nullptr, nullptr);
    }
    __syncthreads();
    tick(tk, 19);
    if (tid == 0) {
        uint32_t fl = kPathFull | fr->flags;
        if (d.flags & kDistUniform) fl |= (1u << 6);
        int tok = ctl.hit;
        if (tok < 0) { tok = n - 1; fl |= (1u << 5); }
        else if (u > 0.f && (u - ctl.hit_before <= kNearTol || ctl.s - u <= kNearTol)) fl |= kFlagNearBoundary;
        a.tokens[row] = tok;
        if (a.token_probs) a.token_probs[row] = eval_p3(__ldcg(e + tok), tok, d);
        if (a.row_flags) a.row_flags[row] = fl;
        count_row_flags(a.counters, fl);
    }
}

constexpr size_t kDrawSmem = sizeof(Emul2Work) + (size_t)kXcEntries * kSub * 4;

// ---- launchers ---------------------------------------------------------------------------------------------
// ---- speculative verification in the flat form ---------------------------------------------------------
// What k_spec_finish (stg_spec_kernels.cu) does with one CTA per sequence - the accept chain, then one
// or two emulated sums over V whose every phase recomputes p (and q) from the logits - as three
// kernels: the accept chain (one warp per sequence, the draft positions evaluated side by side), ONE
// flat pass that writes the values the draw runs over - the final probabilities of the target row
// (bonus draw, or the looser rule's draw from p) or the residual max(p - q, 0) - into the sequence's
// scratch row with their sub-tile sums, guesses and composites (the tail k_full_psums has), and a
// per-sequence walk: for the residual first without a target (its sum), then to u * sum with the same
// composites.  Sequences whose draw needs one of the rare fall-backs (an empty residual, a walk that
// runs off the end, a look-back that ran out) are flagged, and k_spec_finish redoes exactly those.
struct SpecSeq {
    int32_t acc;       // accepted draft tokens
    int32_t kind;      // 0: done (greedy), 1: draw from the target row `acc`, 2: residual of position `acc`
    uint32_t flags;    // STG_SEQ_* gathered so far
    int32_t pad;
};

template <bool BF16>
__global__ void __launch_bounds__(256) k_spec_accept(const __grid_constant__ SpecArgs a, const FullWs ws, SpecSeq *seq,
                                                     int32_t *fallback)
{
    const int lane = threadIdx.x & 31;
    const int s = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (s >= a.n_seq) return;
    const int L = a.n_draft, V = a.vocab;
    const int esz = BF16 ? 2 : 4;
    const RowDist *td = a.tdist + (int64_t)s * (L + 1);
    const RowDist *dd = a.ddist ? a.ddist + (int64_t)s * L : nullptr;
    const char *trows = (const char *)a.target + (int64_t)s * (L + 1) * V * esz;
    const char *drows = a.draft ? (const char *)a.draft + (int64_t)s * L * V * esz : nullptr;
    const double *u = a.uniforms + (int64_t)s * (L + 2);
    const bool greedy = (td[0].flags & kDistOneHot) != 0;
    bool ok = true, bad = false;
    float shown = 0.f;
    if (lane < L) {
        const int i = lane;
        const int tok = a.draft_tokens[(int64_t)s * L + i];
        if ((unsigned)tok >= (unsigned)V) {
            // a draft token outside the vocabulary (the reference's pDist[tokens[i]] throws,
            // SpeculativeDecoder.cs:534): never read, rejected, and reported in the flags
            ok = false;
            bad = true;
        } else if (greedy) {
            ok = (tok == td[i].tie_idx_max);  // SpeculativeDecoder.Step, SpeculativeDecoder.cs:400-405
            shown = ok ? 1.f : 0.f;
        } else {
            const float px = eval_point<BF16>(LogitRow{trows + (int64_t)i * V * esz, a.target_cap}, tok, td[i]);
            if (a.mode == 0) {
                const float qx = eval_point<BF16>(LogitRow{drows + (int64_t)i * V * esz, a.draft_cap}, tok, dd[i]);
                const float r = qx > 0.f ? fminf(1.f, __fdiv_rn(px, qx)) : (px > 0.f ? 1.f : 0.f);
                ok = u[i] < (double)r;
                shown = r;
            } else {
                ok = px >= a.p_min || tok == td[i].argmax;
                shown = px;
            }
        }
    }
    const unsigned rej = __ballot_sync(0xFFFFFFFFu, lane < L && !ok);
    const int acc = rej ? __ffs(rej) - 1 : L;
    // positions after the first rejection are not tested
    if (a.accept_probs && lane < L) a.accept_probs[(int64_t)s * L + lane] = lane <= acc ? shown : 0.f;
    const bool bad_draft = acc < L && __shfl_sync(0xFFFFFFFFu, bad ? 1 : 0, acc) != 0;
    if (lane == 0) {
        const uint32_t fl = bad_draft ? (1u << 9) : 0u;
        SpecSeq q;
        q.acc = acc;
        q.flags = fl;
        q.pad = 0;
        q.kind = greedy ? 0 : ((acc == L || a.mode == 1) ? 1 : 2);
        seq[s] = q;
        fallback[s] = 0;
        a.accepted[s] = acc;
        if (greedy) {
            a.correction[s] = td[acc].tie_idx_max;
            if (a.seq_flags) a.seq_flags[s] = fl;
        }
        FullRow *fr = ws.rows + s;
        fr->redo = 0;
        fr->n_cross[1] = 0;
    }
    FullRow *fr = ws.rows + s;
    for (int p = lane; p < kFullMaxParts; p += 32) fr->pflag[1][p] = 0u;
}

template <bool BF16>
__global__ void __launch_bounds__(kFullThreads) k_spec_values(const __grid_constant__ SpecArgs a, const FullWs ws,
                                                              const SpecSeq *seq)
{
    __shared__ float s_sum[kPieceSubTiles];
    __shared__ unsigned char s_guess[kPieceSubTiles], s_xslot[kPieceSubTiles];
    __shared__ int s_ok;
    const int s = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const SpecSeq q = seq[s];
    if (q.kind == 0) return;
    const int L = a.n_draft, n = a.vocab;
    const int begin = blockIdx.x * kPhasePiece;
    if (begin >= n) return;
    const int esz = BF16 ? 2 : 4;
    const bool al = a.vec == 4;
    const RowDist td = a.tdist[(int64_t)s * (L + 1) + q.acc];
    const LogitRow prow{(const char *)a.target + ((int64_t)s * (L + 1) + q.acc) * n * esz, a.target_cap};
    const ProvRow<BF16> pp{SrcLogits<BF16>{prow, nullptr, al, td.inv_t, td.inv_t != 1.0f}, td};
    FullRow *fr = ws.rows + s;
    Emul2Work *ew = ws.ew + s;
    float *e = ws.e + (size_t)s * ws.e_stride;
    constexpr int W = kFullThreads / 32;
    float xs[kWarpSubTiles][8];
    if (q.kind == 2) {
        const RowDist dq = a.ddist[(int64_t)s * L + q.acc];
        const LogitRow qrow{(const char *)a.draft + ((int64_t)s * L + q.acc) * n * esz, a.draft_cap};
        const ProvRow<BF16> qq{SrcLogits<BF16>{qrow, nullptr, al, dq.inv_t, dq.inv_t != 1.0f}, dq};
        const ProvResidual<BF16> rr{pp, qq};
#pragma unroll
        for (int i = 0; i < kWarpSubTiles; i++) {
            const int st = warp + i * W;
            rr.load(begin + st * kSub + lane * 8, n, xs[i]);  // zeros beyond the row
        }
    } else {
#pragma unroll
        for (int i = 0; i < kWarpSubTiles; i++) {
            const int st = warp + i * W;
            pp.load(begin + st * kSub + lane * 8, n, xs[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < kWarpSubTiles; i++) {
        const int st = warp + i * W;
        const int base = begin + st * kSub + lane * 8;
        if (begin + st * kSub >= n) continue;  // the same for the whole warp
        if (base < n) store8(e, base, n, xs[i]);
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) acc += xs[i][j] > 0.f ? xs[i][j] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
        if (lane == 0) { ew->sums[(begin >> 8) + st] = acc; s_sum[st] = acc; }
    }
    piece_tail<true>(fr, ew, xs, begin, n, s_sum, s_guess, s_xslot, &s_ok);
}

__global__ void __launch_bounds__(kThreads, 1) k_spec_draw(const __grid_constant__ SpecArgs a, const FullWs ws,
                                                           const SpecSeq *seq, int32_t *fallback)
{
    extern __shared__ __align__(16) unsigned char arena[];
    __shared__ Emul2Ctl ctl;
    __shared__ XCache xcache;
    const int s = blockIdx.x, tid = threadIdx.x;
    const SpecSeq q = seq[s];
    if (q.kind == 0) return;
    const FullRow *fr = ws.rows + s;
    if (fr->redo) {
        if (tid == 0) fallback[s] = 1;
        return;
    }
    const int L = a.n_draft, n = a.vocab;
    const int nsub = (n + kSub - 1) / kSub;
    Emul2Work *wk2 = (Emul2Work *)arena;
    float *xdata = (float *)(arena + sizeof(Emul2Work));
    load_work(wk2, ws.ew + s);
    const ProvE pe{ws.e + (size_t)s * ws.e_stride};
    const float u0 = __double2float_rn(a.uniforms[(int64_t)s * (L + 2) + L]);
    float target = u0;
    if (q.kind == 2) {
        // ResampleResidual (Sampler.cs:587-618): the sum of the residual, then the draw to u * sum
        build_xcache(&xcache, xdata, wk2, pe, n, nsub, 0.f, false);
        if (tid < 32) {
            const ProvCached<ProvE> pc{pe, xdata, xcache.of};
            emul2_walk<ProvCached<ProvE>, false, false>(&ctl, wk2, pc, n, nsub, 0.f, false, nullptr, nullptr);
        }
        __syncthreads();
        const float sum = ctl.s;
        __syncthreads();
        if (!(sum > 0.f)) {  // nothing left of p - q (or NaN): the draw from p with the spare uniform
            if (tid == 0) fallback[s] = 1;
            return;
        }
        target = __fmul_rn(u0, sum);
    }
    build_xcache(&xcache, xdata, wk2, pe, n, nsub, target, true);
    if (tid < 32) {
        const ProvCached<ProvE> pc{pe, xdata, xcache.of};
        emul2_walk<ProvCached<ProvE>, false, false>(&ctl, wk2, pc, n, nsub, target, true, nullptr, nullptr);
    }
    __syncthreads();
    if (tid == 0) {
        int corr = ctl.hit;
        uint32_t fl = q.flags;
        if (corr < 0) {
            if (q.kind == 2) { fallback[s] = 1; return; }  // the rounding fall-back of the residual draw
            corr = n - 1;
            fl |= (1u << 5);
        }
        a.correction[s] = corr;
        if (a.seq_flags) a.seq_flags[s] = fl;
    }
}

cudaError_t launch_spec_flat(const SpecArgs &a, const FullWs &ws, void *seq_ctl, int32_t *fallback, cudaStream_t stream)
{
    SpecSeq *seq = (SpecSeq *)seq_ctl;
    cudaError_t e = ensure_dynamic_smem((const void *)k_spec_draw, kDrawSmem);
    if (e != cudaSuccess) return e;
    const dim3 pg((unsigned)((a.vocab + kPhasePiece - 1) / kPhasePiece), (unsigned)a.n_seq);
    if (a.dtype == 1) {
        k_spec_accept<true><<<(a.n_seq + 7) / 8, 256, 0, stream>>>(a, ws, seq, fallback);
        k_spec_values<true><<<pg, kFullThreads, 0, stream>>>(a, ws, seq);
    } else {
        k_spec_accept<false><<<(a.n_seq + 7) / 8, 256, 0, stream>>>(a, ws, seq, fallback);
        k_spec_values<false><<<pg, kFullThreads, 0, stream>>>(a, ws, seq);
    }
    k_spec_draw<<<a.n_seq, kThreads, kDrawSmem, stream>>>(a, ws, seq, fallback);
    return cudaGetLastError();
}

static dim3 piece_grid(const SampleArgs &a, int n_full) { return dim3((unsigned)((a.vocab + kPhasePiece - 1) / kPhasePiece), (unsigned)n_full); }

cudaError_t launch_full_prep(const SampleArgs &a, const FullWs &ws, FlatRow *flat, cudaStream_t stream)
{
    const size_t smem = (size_t)kMaxOvSlots * 24 + 8192 + 1024 + (size_t)kMaxOverride * 16;
    void (*fn)(const SampleArgs, const FullWs, FlatRow *) = a.dtype == 1 ? k_full_prep<true> : k_full_prep<false>;
    cudaError_t e = ensure_dynamic_smem((const void *)fn, smem);
    if (e != cudaSuccess) return e;
    fn<<<a.n_items, kThreads, smem, stream>>>(a, ws, flat);
    return cudaGetLastError();
}

// everything behind the HBM pass for the `n_full` full rows listed in `full_rows` (device array)
// part 0: exp .. cut; part 1: the draw's partial sums (the last kernel that can give a row up: its
// look-back is a bounded wait too), after which the rows to redo are known; part 2: the draw
cudaError_t launch_full_rest(const SampleArgs &a, const FullWs &ws, const WorkItem *full_items, int n_full, int *launches,
                             KernelTimer *kt, cudaStream_t stream, int part, const FullSide &side)
{
    const dim3 pg = piece_grid(a, n_full);
    if (part == 1) {
        if (a.mode != 0) return cudaSuccess;
        k_full_psums<<<pg, kFullThreads, 0, stream>>>(a, ws, full_items);
        kt->mark("full_psums", stream);
        *launches += 1;
        return cudaGetLastError();
    }
    if (part == 2) {
        if (a.mode != 0) return cudaSuccess;
        k_full_draw<<<n_full, kThreads, kDrawSmem, stream>>>(a, ws, full_items);
        kt->mark("full_draw", stream);
        *launches += 1;
        return cudaGetLastError();
    }
    cudaError_t e = ensure_dynamic_smem((const void *)k_full_walk, kRowArenaBytes);
    if (e == cudaSuccess) e = ensure_dynamic_smem((const void *)k_full_cut, kRowArenaBytes);
    if (e == cudaSuccess) e = ensure_dynamic_smem((const void *)k_full_draw, kDrawSmem);
    if (e != cudaSuccess) return e;
    e = ensure_dynamic_smem((const void *)k_full_plan, kRowArenaBytes);
    if (e != cudaSuccess) return e;
    k_full_exp<<<pg, kFullThreads, 0, stream>>>(a, ws, full_items);
    kt->mark("full_exp", stream);
    // the plan and the scatter pass need the histogram and the sub-tile sums, not the exact sum: they
    // run on the side stream beside the walk (and have nothing to do when no row has top-p on)
    if (side.any_with_top_p) {
        e = cudaEventRecord(side.after_exp, stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(side.stream, side.after_exp, 0);
        if (e != cudaSuccess) return e;
        k_full_plan<<<n_full, kThreads, kRowArenaBytes, side.stream>>>(a, ws, full_items);
        k_full_scatter<<<pg, kFullThreads, 0, side.stream>>>(a, ws, full_items);
        e = cudaEventRecord(side.after_scatter, side.stream);
        if (e != cudaSuccess) return e;
        *launches += 2;
    }
    k_full_walk<<<n_full, kThreads, kRowArenaBytes, stream>>>(a, ws, full_items);
    kt->mark("full_walk", stream);
    *launches += 2;
    if (side.any_without_top_p) {
        k_full_nosum<<<pg, kFullThreads, 0, stream>>>(a, ws, full_items);
        kt->mark("full_nosum", stream);
        *launches += 1;
    }
    if (side.any_with_top_p) {
        e = cudaStreamWaitEvent(stream, side.after_scatter, 0);
        if (e != cudaSuccess) return e;
        kt->mark("wait_scatter", stream);
        k_full_ties<<<pg, kFullThreads, 0, stream>>>(a, ws, full_items);
        kt->mark("full_ties", stream);
        *launches += 1;
    }
    k_full_cut<<<n_full, kThreads, kRowArenaBytes, stream>>>(a, ws, full_items);
    kt->mark("full_cut", stream);
    *launches += 1;
    return cudaGetLastError();
}

}  // namespace stg
