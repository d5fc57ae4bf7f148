// C ABI of the sampling library: argument checks, the per-step host planner, staging of host
// arrays, and the launches.  Everything behind this file is CUDA; there is no CPU code path.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "stg_emul2.cuh"
#include "stg_flat.cuh"
#include "stg_handle.h"
#include "stg_launch.h"
#include "stg_types.h"

using namespace stg;

namespace stg {

static std::string g_create_error;

int fail(StgHandle h, int code, const std::string &msg)
{
    if (h) h->err = msg; else g_create_error = msg;
    return code;
}

int cuda_fail(StgHandle h, cudaError_t e, const char *what)
{
    return fail(h, STG_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

int dev_alloc(StgHandle h, DevBuf &b, size_t bytes)
{
    bytes = std::max<size_t>(bytes, 256);
    const bool guard = h != nullptr && h->checked;
    if (guard) bytes = round_up(bytes, 256);
    cudaError_t e = cudaMalloc(&b.p, bytes + (guard ? kGuardBytes : 0));
    if (e != cudaSuccess) return cuda_fail(h, e, "cudaMalloc");
    b.bytes = bytes;
    b.guarded = guard;
    if (guard) {
        e = cudaMemset((char *)b.p + bytes, kGuardByte, kGuardBytes);
        if (e != cudaSuccess) return cuda_fail(h, e, "cudaMemset");
    }
    return STG_OK;
}

void dev_free(DevBuf &b)
{
    if (b.p) cudaFree(b.p);
    b.p = nullptr;
    b.bytes = 0;
    b.guarded = false;
}

}  // namespace stg

namespace {

// RepeatWindowStart, src/OpenTail.Stingray.Engine/Sampler.cs:364-365
int repeat_window_start(int count, int last_n) { return (last_n <= 0 || last_n >= count) ? 0 : count - last_n; }


// Resolves every row's path exactly as Sampler.Sample dispatches (Sampler.cs:19-39) and lays out
// the work items: whole-row items first (they run longest), then the chunk items row by row.
int make_plan(StgHandle h, const StgSampleBatch *b, int mode, bool shard, int global_vocab, bool flat_ok, bool full_ok,
              Plan &pl)
{
    const int rows = b->rows, V = b->vocab;
    const int GV = global_vocab > 0 ? global_vocab : V;  // the vocabulary the reference's rules see
    pl.rows.resize(rows);
    std::vector<std::pair<uint32_t, int>> reps;  // distinct repetition penalties -> table offset
    int n_chunk_rows = 0, max_sel = 1;
    for (int r = 0; r < rows; r++) {
        const StgRowParams &p = b->params[r];
        RowPlan &rp = pl.rows[r];
        memset(&rp, 0, sizeof(rp));
        rp.flat_full = -1;
        rp.temperature = p.temperature; rp.top_p = p.top_p; rp.min_p = p.min_p;
        rp.rep = p.repetition_penalty; rp.pres = p.presence_penalty; rp.freq = p.frequency_penalty;
        rp.top_k = p.top_k;
        int hoff = 0, hlen = 0, boff = 0, blen = 0;
        if (b->mem_flags & STG_MEM_HISTORY_RING) {
            hoff = r * std::max(h->cfg.max_history, 1);
            hlen = h->ring_len[r];
            const bool pen = p.repetition_penalty != 1.0f || p.presence_penalty != 0.f || p.frequency_penalty != 0.f;
            if (h->ring_dropped[r] && pen &&
                (p.presence_penalty != 0.f || p.frequency_penalty != 0.f || p.repeat_last_n <= 0 || p.repeat_last_n > hlen))
                return fail(h, STG_ERR_CAPACITY, "the device-resident history has dropped tokens this row's penalties would count");
        } else if (b->history_offsets && b->history_ids) {
            hoff = b->history_offsets[r];
            hlen = b->history_offsets[r + 1] - hoff;
        }
        if (b->bias_offsets && b->bias_ids && b->bias_values) {
            boff = b->bias_offsets[r];
            blen = b->bias_offsets[r + 1] - boff;
        }
        if (hlen < 0 || blen < 0) return fail(h, STG_ERR_INVALID_ARGUMENT, "CSR offsets must be non-decreasing");
        if (hlen > h->cfg.max_history) return fail(h, STG_ERR_CAPACITY, "history longer than max_history");
        if (blen > h->cfg.max_bias) return fail(h, STG_ERR_CAPACITY, "more bias entries than max_bias");
        rp.hist_off = hoff; rp.hist_len = hlen; rp.bias_off = boff; rp.bias_len = blen;
        rp.window_start = repeat_window_start(hlen, p.repeat_last_n);
        rp.use_mask = b->mask != nullptr && (b->row_uses_mask == nullptr || b->row_uses_mask[r] != 0);
        rp.pow_off = -1;
        const bool pen_set = p.repetition_penalty != 1.0f || p.presence_penalty != 0.f || p.frequency_penalty != 0.f;
        rp.has_penalty = pen_set && hlen > 0;
        rp.sel = 1;
        if (mode != 0) {
            rp.path = p.temperature <= 0.f ? (rp.has_penalty ? kPathGreedyPen : kPathGreedy) : kPathFull;
            rp.n_chunks = 0;
        } else if (p.temperature <= 0.f) {
            rp.path = rp.has_penalty ? kPathGreedyPen : kPathGreedy;
        } else if (p.top_k > 0 && p.top_k < GV && blen == 0) {
            rp.path = kPathTopK;
            pl.max_topk_path_k = std::max(pl.max_topk_path_k, (int)p.top_k);
            int64_t want = (int64_t)p.top_k + (rp.has_penalty ? hlen : 0);
            rp.sel = (int)std::min<int64_t>(want, GV);
            if (p.top_k > h->cfg.max_top_k) return fail(h, STG_ERR_CAPACITY, "top_k larger than max_top_k");
            if (rp.sel > kMaxSel) return fail(h, STG_ERR_CAPACITY, "top_k + history length exceeds 8192");
            if (rp.has_penalty && p.repetition_penalty != 1.0f) {
                uint32_t bits;
                memcpy(&bits, &p.repetition_penalty, 4);
                int off = -1;
                for (auto &e : reps) if (e.first == bits) off = e.second;
                if (off < 0) {
                    off = (int)pl.pow_tab.size();
                    reps.push_back({bits, off});
                    // MathF.Pow(RepetitionPenalty, occWindow), Sampler.cs:283, through the host's libm
                    for (int o = 1; o <= kPowTab; o++) pl.pow_tab.push_back(powf(p.repetition_penalty, (float)o));
                }
                rp.pow_off = off;
            }
        } else {
            rp.path = kPathFull;
        }
        if (rp.path == kPathFull || rp.path == kPathGreedyPen) {
            if (p.top_k > 4096 && p.top_k < GV)
                return fail(h, STG_ERR_UNSUPPORTED, "top_k above 4096 on the full-vocabulary path");
            if (hlen + blen > kMaxOverride) return fail(h, STG_ERR_CAPACITY, "history + bias entries exceed 2048 on the full-vocabulary path");
        }
        if (shard && !(rp.path == kPathTopK || rp.path == kPathGreedy))
            return fail(h, STG_ERR_UNSUPPORTED, "vocabulary-sharded mode supports top-k and plain greedy rows only");
        const bool chunked = mode == 0 && (rp.path == kPathGreedy || rp.path == kPathTopK);
        if (chunked) { n_chunk_rows++; max_sel = std::max(max_sel, rp.sel); }
        else pl.any_row_item = true;
        if (rp.path == kPathTopK) pl.n_topk++; else if (rp.path == kPathFull) pl.n_full++; else pl.n_greedy++;
        if (rp.path == kPathFull && !(p.top_p < 1.0f && p.top_p > 0.f)) pl.n_full_without_top_p++;
        if (rp.path == kPathFull && p.top_p < 1.0f && p.top_p > 0.f) pl.n_full_with_top_p++;
    }
    pl.n_chunk_rows = n_chunk_rows;
    // The flat step needs long, aligned rows and a candidate list (N + kFlatSlack entries) that about 3 N
    // expected survivors fit well inside.
    pl.flat = flat_ok && n_chunk_rows > 0 && V >= 4 * kFlatSample && 3 * (size_t)max_sel + 256 <= (size_t)max_sel + kFlatSlack;
    if (pl.flat) {
        size_t need = 0;
        for (auto &rp : pl.rows)
            if (rp.path == kPathTopK) need += (size_t)rp.sel + kFlatSlack;
        if (need > h->cand_entries) pl.flat = false;
    }
    // chunking: enough chunk items to balance the SMs, whole 4096-element sub-tiles per chunk
    int S = 1;
    if (n_chunk_rows > 0 && !pl.flat) {
        int want = (2 * h->sm_count + n_chunk_rows - 1) / n_chunk_rows;  // about two items per SM
        int max_s = std::max(1, (V + 16383) / 16384);
        S = std::max(1, std::min({want, max_s, 64}));
        if (shard) S = std::min(S, 16);
    }
    for (; !pl.flat;) {
        pl.chunk_len = (int)round_up((size_t)((V + S - 1) / S), kSubTile);
        int n_chunks = (V + pl.chunk_len - 1) / pl.chunk_len;
        size_t need = 0;
        for (auto &rp : pl.rows)
            if (mode == 0 && (rp.path == kPathGreedy || rp.path == kPathTopK)) need += (size_t)n_chunks * 2 * (size_t)rp.sel;
        if (n_chunks == 1 || need <= h->cand_entries) { S = n_chunks; break; }
        S = std::max(1, S / 2);
    }
    int cand_off = 0, slot = 0;
    struct Memo { int sel = -1, groups = 0, rank = 0; } memo[64];
    for (int r = 0; r < rows; r++) {
        RowPlan &rp = pl.rows[r];
        if (mode == 0 && (rp.path == kPathGreedy || rp.path == kPathTopK)) {
            if (pl.flat) {
                rp.n_chunks = 1;  // one finishing item per row
                rp.cand_off = cand_off;
                rp.slot = slot++;
                if (rp.path == kPathTopK) {
                    cand_off += rp.sel + kFlatSlack;
                    // the choice below depends on the row's N alone (V is the step's): most rows of a step share it
                    Memo &mm = memo[rp.sel & 63];
                    if (rp.sel == mm.sel) { rp.flat_groups = mm.groups; rp.flat_rank = mm.rank; continue; }
                    // groups of the 4096-element sample: about 3 N survivors (at least 256) over the row
                    // The bound is the smallest of ng group maxima of the sample, above which about
                    // ng * H(ng) of the sample's elements lie (H the harmonic number), so about
                    // E(ng) = ng * H(ng) * V / sample of the row's.  Wanted: E between 2.5 N (at least
                    // 400: small group counts scatter widely) and 0.6 of the list's capacity; the
                    // smallest power of two that gets there, else the one that comes closest.
                    const double lo = std::max(2.5 * rp.sel, 400.0), hi = 0.6 * (rp.sel + (double)kFlatSlack);
                    const double per = (double)V / std::min<double>(kFlatSample, V);
                    int ng = 8, best_ng = 8;
                    double best_fit = -1.0, hn = 0.0;
                    for (int i = 1; i <= 8; i++) hn += 1.0 / i;
                    for (int g = 8; g <= 1024; g *= 2) {
                        const double ex = g * hn * per;
                        const double fit = std::min(ex / lo, hi / ex);
                        if (fit > best_fit) { best_fit = fit; best_ng = g; }
                        if (ex >= lo && ex <= hi) { best_ng = g; break; }
                        for (int i = g + 1; i <= 2 * g; i++) hn += 1.0 / i;
                    }
                    ng = best_ng;
                    // The smallest of ng group maxima can also come out too high: the row then has fewer than
                    // N logits above it and must be read again.  With x = N * sample / V (N counted in sample
                    // elements) that happens with probability (1 - exp(-x / ng))^ng per row; more groups
                    // until it is below 1e-7, the list's capacity permitting.
                    const double x = (double)rp.sel / per;
                    auto p_short = [&](int g) { return std::pow(1.0 - std::exp(-x / g), (double)g); };
                    while (ng < 1024 && p_short(ng) > 1e-7) {
                        double h2 = 0.0;
                        for (int i = 1; i <= 2 * ng; i++) h2 += 1.0 / i;
                        if (2 * ng * h2 * per > hi) break;
                        ng *= 2;
                    }
                    rp.flat_groups = ng;
                    rp.flat_rank = 0;
                    // Sharper, and what is used whenever it applies: the bound as an exact order statistic of
                    // the sample.  The row's count above the sample's r-th largest logit is V / sample times a
                    // Gamma(r) variable - mean r, spread sqrt(r), thin tails - where the smallest of g group
                    // maxima scatters over a factor of three and comes in powers of two.  r: about `lo` logits
                    // of the row above the bound, and large enough that fewer than N is a 1e-7 event
                    // (P[Poisson(x) >= r]).  The groups' bound, with g >= r / 2 groups, then only fences off the
                    // few dozen to few hundred sample elements among which the r-th largest is found by
                    // ranking (flat_prep_row); should fewer than r lie above it, it stays the bound.
                    static const bool no_rank = getenv("STG_NO_FLAT_RANK") != nullptr;
                    int r = std::max(8, (int)std::ceil(lo / per));
                    for (;; r++) {
                        double term = std::exp(-x), cdf = 0.0;  // P[Poisson(x) <= r - 1]
                        for (int i = 0; i < r; i++) { cdf += term; term *= x / (i + 1); }
                        if (1.0 - cdf <= 1e-7 || r > 128) break;
                    }
                    if (!no_rank && r <= 128 && r * per <= hi) {
                        int g = 8;
                        while (2 * g < r) g *= 2;
                        rp.flat_groups = g;
                        rp.flat_rank = r;
                    }
                    mm.sel = rp.sel; mm.groups = rp.flat_groups; mm.rank = rp.flat_rank;
                }
                continue;
            }
            rp.n_chunks = S;
            rp.cand_off = cand_off;
            rp.slot = slot;
            cand_off += S * 2 * rp.sel;
            slot += S;
        }
    }
    for (int r = 0; r < rows; r++)
        if (pl.rows[r].n_chunks == 0) pl.items.push_back({r, -1});
    pl.n_row_items = (int)pl.items.size();
    // The full-vocabulary rows join the flat step when every one of them can: no top-k on this path
    // (it only arises together with a logit bias), a vocabulary the segment-parallel sum emulation
    // covers, and room in the workspace.
    pl.flat_full = full_ok && pl.n_row_items > 0 && pl.n_row_items <= h->full_cap && V <= kSub * kMaxSubTiles;
    for (int i = 0; i < pl.n_row_items && pl.flat_full; i++) {
        const RowPlan &rp = pl.rows[pl.items[i].row];
        if (rp.top_k > 0 && rp.top_k < GV && rp.temperature > 0.f) pl.flat_full = false;
    }
    if (pl.flat_full)
        for (int i = 0; i < pl.n_row_items; i++) pl.rows[pl.items[i].row].flat_full = i;
    for (int r = 0; r < rows; r++)
        for (int c = 0; c < pl.rows[r].n_chunks; c++) pl.items.push_back({r, c});
    // room for two 4096-element sub-tiles beyond the selection when shared memory allows it: fewer compactions
    pl.max_sel = max_sel;
    pl.cap = max_sel + 2 * kSubTile;
    if ((size_t)pl.cap * 16 > h->smem_optin) pl.cap = max_sel + kSubTile;
    pl.smem = std::max<size_t>((size_t)pl.cap * 16, 1024);  // chunk kernel; the row kernel has a fixed arena
    return STG_OK;
}

// Uploads the plan unless it is byte-identical to the one already resident on the device.
int upload_plan(StgHandle h, const Plan &pl, cudaStream_t stream, const RowPlan **d_rows,
                const WorkItem **d_items, const float **d_pow)
{
    const size_t b_rows = round_up(pl.rows.size() * sizeof(RowPlan), 256);
    const size_t b_items = round_up(pl.items.size() * sizeof(WorkItem), 256);
    const size_t b_pow = round_up(pl.pow_tab.size() * sizeof(float), 256);
    const size_t total = b_rows + b_items + b_pow;
    if (total > h->plan_bytes_cap) return fail(h, STG_ERR_CAPACITY, "plan exceeds the workspace");
    std::vector<unsigned char> bytes(total, 0);
    memcpy(bytes.data(), pl.rows.data(), pl.rows.size() * sizeof(RowPlan));
    memcpy(bytes.data() + b_rows, pl.items.data(), pl.items.size() * sizeof(WorkItem));
    if (!pl.pow_tab.empty()) memcpy(bytes.data() + b_rows + b_items, pl.pow_tab.data(), pl.pow_tab.size() * sizeof(float));
    unsigned char *dev = (unsigned char *)h->plan_dev.p;
    *d_rows = (const RowPlan *)dev;
    *d_items = (const WorkItem *)(dev + b_rows);
    *d_pow = pl.pow_tab.empty() ? nullptr : (const float *)(dev + b_rows + b_items);
    if (bytes == h->plan_cache) return STG_OK;
    const int slot = h->plan_slot;
    h->plan_slot = (slot + 1) & 3;
    CK(cudaEventSynchronize(h->plan_ev[slot]));
    unsigned char *pin = h->plan_host + (size_t)slot * h->plan_bytes_cap;
    memcpy(pin, bytes.data(), total);
    CK(cudaMemcpyAsync(dev, pin, total, cudaMemcpyHostToDevice, stream));
    CK(cudaEventRecord(h->plan_ev[slot], stream));
    h->plan_cache.swap(bytes);
    h->stats.plan_uploads++;
    return STG_OK;
}

}  // namespace

namespace stg {
// Returns the device address of a caller array, copying it into `stage` first when it is host memory.
int stage_in(StgHandle h, const void *src, size_t bytes, bool on_host, DevBuf &stage, cudaStream_t stream,
             const void **out)
{
    if (src == nullptr || bytes == 0) { *out = src; return STG_OK; }
    if (!on_host) { *out = src; return STG_OK; }
    if (bytes > stage.bytes) {
        // staging for host arrays is sized at creation from the handle's capacities; the logits and
        // mask staging (the large ones) are sized there too with STG_CFG_HOST_LOGITS, and otherwise
        // grown on first use
        if (&stage != &h->st_logits && &stage != &h->st_mask)
            return fail(h, STG_ERR_CAPACITY, "host array larger than the staging buffer");
        CK(cudaStreamSynchronize(stream));
        dev_free(stage);
        int rc = dev_alloc(h, stage, bytes);
        if (rc) return rc;
    }
    CK(cudaMemcpyAsync(stage.p, src, bytes, cudaMemcpyHostToDevice, stream));
    *out = stage.p;
    return STG_OK;
}

}  // namespace stg

namespace {

int check_batch(StgHandle h, const StgSampleBatch *b, bool no_logits)
{
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (!b || b->struct_size != (int32_t)sizeof(StgSampleBatch)) return fail(h, STG_ERR_INVALID_ARGUMENT, "bad StgSampleBatch");
    if (!(b->logit_softcap >= 0.f) || b->logit_softcap > 3.0e38f)
        return fail(h, STG_ERR_INVALID_ARGUMENT, "logit_softcap must be 0 (off) or a finite positive cap");
    if (b->rows < 0 || b->vocab <= 0) return fail(h, STG_ERR_INVALID_ARGUMENT, "rows must be >= 0 and vocab > 0");
    if (b->rows > h->cfg.max_rows) return fail(h, STG_ERR_CAPACITY, "rows exceed max_rows");
    if (b->vocab > h->cfg.max_vocab) return fail(h, STG_ERR_CAPACITY, "vocab exceeds max_vocab");
    if (b->rows > 0 && ((!b->logits && !no_logits) || !b->params)) return fail(h, STG_ERR_INVALID_ARGUMENT, "logits and params are required");
    if (b->row_stride < b->vocab) return fail(h, STG_ERR_INVALID_ARGUMENT, "row_stride smaller than vocab");
    if (b->logits_dtype != STG_DTYPE_F32 && b->logits_dtype != STG_DTYPE_BF16) return fail(h, STG_ERR_INVALID_ARGUMENT, "unknown logits_dtype");
    if (b->mask && b->mask_row_stride < (b->vocab + 31) / 32) return fail(h, STG_ERR_INVALID_ARGUMENT, "mask_row_stride too small");
    return STG_OK;
}

bool rows_aligned(const void *p, int64_t row_stride, int dtype)
{
    const size_t esz = dtype == STG_DTYPE_BF16 ? 2 : 4;
    const size_t need = dtype == STG_DTYPE_BF16 ? 8 : 16;
    return ((uintptr_t)p % need) == 0 && ((size_t)row_stride * esz) % need == 0;
}

}  // namespace

namespace stg {

int run_batch(StgHandle h, const StgSampleBatch *b, const BatchExtra &x, void *stream_)
{
    const int mode = x.mode;
    float *dist_out = x.dist_out;
    void *pairs_out = x.pairs_out;
    cudaStream_t stream = (cudaStream_t)stream_;
    int rc = check_batch(h, b, x.shard_mode == 2);
    if (rc) return rc;
    if (b->rows == 0) return STG_OK;
    CK(cudaSetDevice(h->cfg.device));
    // The workspace, the plan and the work counters belong to the handle, so consecutive calls must
    // not overlap on the device.  On one stream they cannot; when the stream changes, this call is
    // put behind everything enqueued so far on the previous one.
    if (h->last_stream_valid && stream != h->last_stream) {
        CK(cudaEventRecord(h->ev_order, h->last_stream));
        CK(cudaStreamWaitEvent(stream, h->ev_order, 0));
    }
    h->last_stream = stream;
    h->last_stream_valid = true;
    const uint32_t mf = b->mem_flags;
    const int rows = b->rows, V = b->vocab;
    if ((mode == 0 || mode == 3) && !pairs_out && !b->tokens && !x.shard_mode) return fail(h, STG_ERR_INVALID_ARGUMENT, "tokens is required");
    if (x.shard_mode && (!h->xchg_local.p || b->rows > h->shard_rows)) return fail(h, STG_ERR_CAPACITY, "exchange buffers are missing or too small");

    const size_t esz0 = b->logits_dtype == STG_DTYPE_BF16 ? 2 : 4, need0 = b->logits_dtype == STG_DTYPE_BF16 ? 8 : 16;
    const bool aligned = ((size_t)b->row_stride * esz0) % need0 == 0 &&
                         ((b->mem_flags & STG_MEM_HOST_LOGITS) || ((uintptr_t)b->logits % need0) == 0);
    const bool flat_ok = mode == 0 && x.shard_mode != 2 && aligned && !getenv("STG_NO_FLAT") &&
                         !(x.shard_mode == 1 && getenv("STG_NO_FLAT_SHARD"));
    const bool full_ok = (mode == 0 || mode == 2) && x.shard_mode == 0 && aligned && !getenv("STG_NO_FLAT") && !getenv("STG_NO_FLAT_FULL");
    // The plan depends on the batch description only (never on the logits): a decode loop that
    // repeats a description byte for byte reuses the plan of the previous call as it is.
    std::vector<unsigned char> &key = h->plan_key_scratch;
    key.clear();
    auto put = [&key](const void *p, size_t n) { const unsigned char *c = (const unsigned char *)p; key.insert(key.end(), c, c + n); };
    const int32_t head[11] = {rows, V, b->logits_dtype, mode, x.shard_mode, x.global_vocab, (int32_t)flat_ok, (int32_t)full_ok,
                              (int32_t)(b->mask != nullptr), (b->mem_flags & STG_MEM_HISTORY_RING) ? 2 : (int32_t)(b->history_ids != nullptr), (int32_t)(b->bias_ids != nullptr && b->bias_values != nullptr)};
    put(head, sizeof(head));
    put(b->params, (size_t)rows * sizeof(StgRowParams));
    const bool ring = (b->mem_flags & STG_MEM_HISTORY_RING) != 0;
    if (ring) {
        put(h->ring_len.data(), (size_t)rows * 4);
        put(h->ring_dropped.data(), (size_t)rows);
    } else if (b->history_offsets) put(b->history_offsets, (size_t)(rows + 1) * 4);
    if (b->bias_offsets) put(b->bias_offsets, (size_t)(rows + 1) * 4);
    if (b->row_uses_mask) put(b->row_uses_mask, (size_t)rows);
    Plan &pl = h->plan;
    if (!h->plan_valid || key != h->plan_key) {
        h->plan_valid = false;
        pl = Plan();
        rc = make_plan(h, b, mode, x.shard_mode != 0, x.global_vocab, flat_ok, full_ok, pl);
        if (rc) return rc;
        if (pl.smem > h->smem_optin || kRowArenaBytes > h->smem_optin) return fail(h, STG_ERR_CAPACITY, "shared memory needed exceeds the device limit");
        rc = upload_plan(h, pl, stream, &h->d_rows, &h->d_items, &h->d_pow);
        if (rc) return rc;
        h->plan_key = key;
        h->plan_valid = true;
        h->plan_version++;
    }
    const RowPlan *d_rows = h->d_rows; const WorkItem *d_items = h->d_items; const float *d_pow = h->d_pow;

    SampleArgs a;
    memset(&a, 0, sizeof(a));
    const size_t esz = b->logits_dtype == STG_DTYPE_BF16 ? 2 : 4;
    const void *p;
    p = nullptr;
    if (x.shard_mode != 2) {
        rc = stage_in(h, b->logits, ((size_t)(rows - 1) * b->row_stride + V) * esz, mf & STG_MEM_HOST_LOGITS, h->st_logits, stream, &p);
        if (rc) return rc;
    }
    a.logits = p;
    if (ring) {
        p = h->ring_ids.p;
    } else {
        const int hist_total = (b->history_offsets && b->history_ids) ? b->history_offsets[rows] : 0;
        rc = stage_in(h, b->history_ids, (size_t)hist_total * 4, mf & STG_MEM_HOST_HISTORY, h->st_hist, stream, &p);
        if (rc) return rc;
    }
    a.hist_ids = (const int32_t *)p;
    const int bias_total = (b->bias_offsets && b->bias_ids) ? b->bias_offsets[rows] : 0;
    rc = stage_in(h, b->bias_ids, (size_t)bias_total * 4, mf & STG_MEM_HOST_BIAS, h->st_bias_ids, stream, &p);
    if (rc) return rc;
    a.bias_ids = (const int32_t *)p;
    rc = stage_in(h, b->bias_values, (size_t)bias_total * 4, mf & STG_MEM_HOST_BIAS, h->st_bias_vals, stream, &p);
    if (rc) return rc;
    a.bias_vals = (const float *)p;
    rc = stage_in(h, b->mask, b->mask ? ((size_t)(rows - 1) * b->mask_row_stride + (V + 31) / 32) * 4 : 0, mf & STG_MEM_HOST_MASK, h->st_mask, stream, &p);
    if (rc) return rc;
    a.mask = (const uint32_t *)p;
    rc = stage_in(h, b->uniforms, (size_t)rows * 4, mf & STG_MEM_HOST_UNIFORMS, h->st_uniforms, stream, &p);
    if (rc) return rc;
    a.uniforms = (const float *)p;

    const bool host_out = mf & STG_MEM_HOST_OUTPUTS;
    const int ts = b->topk_stride;
    if ((b->topk_ids || b->topk_logits || b->topk_probs) && ts < 1) return fail(h, STG_ERR_INVALID_ARGUMENT, "topk_stride must be positive");
    // every top-k-path row writes top_k entries of each requested top-k output at row * topk_stride
    if ((b->topk_ids || b->topk_logits || b->topk_probs) && pl.max_topk_path_k > ts)
        return fail(h, STG_ERR_INVALID_ARGUMENT, "topk_stride is smaller than a row's top_k");
    if (host_out && (b->topk_ids || b->topk_logits || b->topk_probs) && (size_t)rows * ts * 4 > h->o_topk_ids.bytes)
        return fail(h, STG_ERR_CAPACITY, "topk outputs exceed max_rows * max_top_k");
    a.tokens = host_out ? (int32_t *)h->o_tokens.p : b->tokens;
    a.token_probs = b->token_probs ? (host_out ? (float *)h->o_probs.p : b->token_probs) : nullptr;
    a.row_flags = b->row_flags ? (host_out ? (uint32_t *)h->o_flags.p : b->row_flags) : nullptr;
    a.topk_ids = b->topk_ids ? (host_out ? (int32_t *)h->o_topk_ids.p : b->topk_ids) : nullptr;
    a.topk_logits = b->topk_logits ? (host_out ? (float *)h->o_topk_vals.p : b->topk_logits) : nullptr;
    a.topk_probs = b->topk_probs ? (host_out ? (float *)h->o_topk_probs.p : b->topk_probs) : nullptr;
    a.topk_stride = ts;
    a.pairs_out = pairs_out;
    if (mode == 1) {
        if (!dist_out) return fail(h, STG_ERR_INVALID_ARGUMENT, "probs is required");
        if (host_out) {
            // distribution rows land in a device buffer first when the caller wants them on the host
            const size_t bytes = (size_t)rows * V * 4;
            if (bytes > h->o_pairs.bytes) {
                CK(cudaStreamSynchronize(stream));
                dev_free(h->o_pairs);
                rc = dev_alloc(h, h->o_pairs, bytes);
                if (rc) return rc;
            }
            a.dist_out = (float *)h->o_pairs.p;
        } else {
            a.dist_out = dist_out;
        }
        if (a.tokens == nullptr) a.tokens = (int32_t *)h->o_tokens.p;
    }
    if (mode == 3) a.dist_out = dist_out;  // sample and materialise: device memory, may be null
    a.plans = d_rows; a.items = d_items; a.pow_tab = d_pow;
    a.cand = (unsigned long long *)h->cand.p;
    a.cand_count = (int32_t *)h->cand_count.p;
    a.tickets = (uint32_t *)h->tickets.p;
    a.work_counter = (uint32_t *)h->work_counter.p;
    a.counters = (unsigned long long *)h->work_counter.p + 16;  // bytes 128..191 of the same small buffer
    a.softcap = b->logit_softcap;
    a.lookback_drill = h->lookback_drill;
    a.phase_ticks = (unsigned long long *)h->ticks.p;
    h->ticks_items = (int)pl.items.size();
    a.escratch = (float *)h->escratch.p;
    a.keyscratch = (unsigned long long *)h->keyscratch.p;
    a.listscratch = (unsigned long long *)h->listscratch.p;
    a.dists = x.dists_out;
    // vocabulary-sharded mode: one block per rank, [rows, stride] keys followed by [rows] counts,
    // with the stride of this step (its largest selection count), so that one all-gather of
    // exactly the bytes in use moves both
    const int xstride = pl.max_sel;
    const size_t xblock = round_up((size_t)rows * xstride * 8 + (size_t)rows * 4, 16);
    a.xchg_local = (unsigned long long *)h->xchg_local.p;
    a.xchg_count = (int32_t *)((char *)h->xchg_local.p + (size_t)rows * xstride * 8);
    a.xchg_stride = xstride;
    a.row_stride = b->row_stride;
    a.mask_stride = b->mask_row_stride;
    a.escratch_stride = h->escratch_stride;
    a.key_stride = h->key_stride;
    a.work_base = h->work_base;
    a.n_items = (int)pl.items.size();
    a.rows = rows; a.vocab = V; a.dtype = b->logits_dtype;
    a.chunk_len = pl.chunk_len;
    a.cap = pl.cap;
    a.vec = rows_aligned(a.logits, b->row_stride, b->logits_dtype) ? 4 : 1;
    a.mode = mode;
    a.vocab_offset = x.vocab_offset; a.shard_mode = x.shard_mode; a.n_ranks = h->n_ranks;

    if (x.shard_mode && xblock > h->xchg_local.bytes) return fail(h, STG_ERR_CAPACITY, "exchange buffers are too small");
    if (x.shard_mode == 1) { h->shard_rows_used = rows; h->shard_stride_used = xstride; h->shard_block_bytes = xblock; }
    if (x.shard_mode == 2) {
        if (rows != h->shard_rows_used || xstride != h->shard_stride_used)
            return fail(h, STG_ERR_INVALID_ARGUMENT, "batch differs from the one selected");
        cudaError_t e2 = launch_shard_finish(a, h->xchg_gather.p, xblock, (size_t)pl.cap * 16, stream);
        if (e2 != cudaSuccess) return cuda_fail(h, e2, "k_shard_finish launch");
        h->stats.kernel_launches++;
        if (host_out) {
            if (b->tokens) CK(cudaMemcpyAsync(b->tokens, a.tokens, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream));
            if (b->token_probs) CK(cudaMemcpyAsync(b->token_probs, a.token_probs, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream));
            if (b->row_flags) CK(cudaMemcpyAsync(b->row_flags, a.row_flags, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream));
            CK(cudaStreamSynchronize(stream));
        }
        return STG_OK;
    }
    // Row items are the full-vocabulary rows (and greedy rows with penalties), chunk items the rows
    // of the top-k path and plain greedy rows.  In the flat form (stg_flat.cuh) ONE streaming kernel
    // reads every row of both kinds from HBM; after it the per-row finish of the chunked rows runs on
    // a side stream beside the phases of the full rows.  Rows the flat form does not take run in the
    // two persistent kernels of the first design, again side by side.
    const int n_rows_items = pl.n_row_items, n_chunk_items = (int)pl.items.size() - pl.n_row_items;
    cudaError_t e = cudaSuccess;
    const bool both = n_rows_items > 0 && n_chunk_items > 0;
    int launches = 0;
    int row_grid = 0;
    FlatRow *fr = (FlatRow *)h->flat_rows.p;
    FullWs ws;
    memset(&ws, 0, sizeof(ws));
    ws.rows = (FullRow *)h->fw_rows.p; ws.e = (float *)h->fw_e.p; ws.e_stride = h->escratch_stride;
    ws.ov_id = (int32_t *)h->fw_ov_id.p; ws.ov_adj = (float *)h->fw_ov_adj.p; ws.ew = (Emul2Work *)h->fw_ew.p;
    ws.hist = (unsigned long long *)h->fw_hist.p; ws.bstart = (uint32_t *)h->fw_bstart.p;
    ws.bin_exp = (unsigned char *)h->fw_binexp.p; ws.flag_bits = (uint32_t *)h->fw_flagbits.p;
    ws.cursor = (uint32_t *)h->fw_cursor.p; ws.keys = (uint32_t *)h->fw_keys.p; ws.key_stride = h->key_stride;
    const bool flat_chunks = pl.flat && n_chunk_items > 0, flat_full = pl.flat_full && n_rows_items > 0;
    auto launch_rows_kernel = [&](bool redo_only, cudaStream_t on) {
        SampleArgs r = a;
        r.n_items = n_rows_items;
        r.item_base = 0;
        r.work_counter = (uint32_t *)h->work_counter.p + 1;
        r.work_base = h->work_base_rows;
        if (redo_only) { r.redo_flags = &ws.rows[0].redo; r.redo_stride = (int32_t)(sizeof(FullRow) / 4); r.static_items = 1; }
        row_grid = std::min(n_rows_items, h->sm_count);
        cudaError_t er = launch_sample_rows(r, row_grid, on);
        if (er == cudaSuccess) { if (!redo_only) h->work_base_rows += (uint32_t)n_rows_items + (uint32_t)row_grid; launches++; }
        return er;
    };
    SampleArgs c = a;  // the chunked rows' view of the step
    c.items = a.items + n_rows_items;
    c.n_items = n_chunk_items;
    // The launches of the step.  When this plan and these arguments (every pointer included) have been
    // launched before, the whole sequence - three streams, their events - is captured once into a CUDA
    // graph and replayed from then on: one submission instead of a dozen, and no host time between the
    // kernels of the chain.  Only steps made of replayable launches qualify: the flat form (the
    // persistent kernels of the first design draw work from counters whose base the host advances),
    // inputs already on the device, no diagnostics.
    // every row a plain arg-max row of the flat form: one launch does the whole step (stg_flat_greedy.cu)
    static const bool no_greedy_step = getenv("STG_NO_GREEDY_STEP") != nullptr;
    const bool greedy_step = flat_chunks && n_rows_items == 0 && pl.n_greedy == (uint64_t)rows && n_chunk_items == rows &&
                             x.shard_mode == 0 && a.phase_ticks == nullptr && !no_greedy_step;
    auto issue = [&]() {
    if (greedy_step) {
        e = launch_greedy_step(a, fr, stream);
        launches++;
        h->kt.mark("greedy_step", stream);
        return;
    }
    if (flat_chunks || flat_full) {
        if (flat_chunks && !flat_full) { e = launch_flat_prep(c, fr, stream); launches++; h->kt.mark("flat_prep", stream); }
        if (e == cudaSuccess && flat_full) { e = launch_full_prep(a, ws, flat_chunks ? fr : nullptr, stream); launches++; h->kt.mark("full_prep", stream); }
        // The HBM pass: the full-vocabulary rows (first in the item list) by the general kernel, the
        // others by a kernel of their own that needs fewer registers and keeps more warps resident.
        static const bool one_stream_pass = getenv("STG_ONE_STREAM_PASS") != nullptr;
        if (one_stream_pass) {
            if (e == cudaSuccess) { e = launch_flat_stream(a, fr, ws, stream); launches++; h->kt.mark("flat_stream", stream); }
        } else if (flat_full && flat_chunks) {
            // both kinds: the full rows' pass on the caller's stream, where their phases follow at once; the
            // others' pass on the side stream beside the first of those phases (the exp pass is bound by
            // arithmetic, this one by HBM, and the full rows' chain is the longer one)
            static const bool serial_passes = getenv("STG_SERIAL_PASSES") != nullptr;
            cudaStream_t cs = serial_passes ? stream : h->aux_stream;
            SampleArgs af = a;
            af.n_items = n_rows_items;
            if (e == cudaSuccess && !serial_passes) e = cudaEventRecord(h->ev_fork, stream);
            if (e == cudaSuccess && !serial_passes) e = cudaStreamWaitEvent(h->aux_stream, h->ev_fork, 0);
            if (e == cudaSuccess) { e = launch_flat_stream(af, fr, ws, stream); launches++; h->kt.mark("flat_stream_full_rows", stream); }
            if (e == cudaSuccess) { e = launch_flat_stream_chunks(c, fr, cs); launches++; if (serial_passes) h->kt.mark("flat_stream_chunks", stream); }
        } else if (flat_full) {
            if (e == cudaSuccess) { e = launch_flat_stream(a, fr, ws, stream); launches++; h->kt.mark("flat_stream", stream); }
        } else {
            if (e == cudaSuccess) { e = launch_flat_stream_chunks(c, fr, stream); launches++; h->kt.mark("flat_stream_chunks", stream); }
        }
    }
    const bool flat_rows = flat_full && n_rows_items > 0;
    const bool fork = both || flat_rows;  // the redo pass of the flat full rows runs on the side stream too
    if (e == cudaSuccess && fork) {
        e = cudaEventRecord(h->ev_fork, stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(h->aux_stream, h->ev_fork, 0);
    }
    // the chunked rows: on the side stream when the step also has full rows
    auto launch_chunked = [&]() {
        if (e != cudaSuccess || n_chunk_items == 0) return;
        cudaStream_t cs = fork ? h->aux_stream : stream;
        if (flat_chunks) {
            // beside the full rows' one-SM-per-row kernels the finish must not take every SM
            const int sms = flat_rows ? std::max(8, h->sm_count - std::min(n_rows_items, h->sm_count) - 4) : h->sm_count;
            c.item_base = n_rows_items;  // diagnostic stamps: behind the full rows' slots
            static const bool no_small = getenv("STG_NO_SMALL_FINISH") != nullptr;
            // Smaller CTAs, several per SM, shorten the finish as long as all rows are in flight at once: the
            // phases of a row are short and barrier-separated, so a 1024-thread CTA leaves most of its SM
            // idle, but per row the smaller forms do more work (measured on 2048 rows: 577 us with 256
            // threads against 304 us with 1024).  So: 512 threads, two per SM, up to 2 rows per SM; 256
            // threads, four per SM, up to 4 rows per SM (not beside the one-SM CTAs of full rows, which
            // need whole SMs to come free); beyond that one full-size CTA per row.  The smaller forms also
            // need their shorter buffers to hold a row's N best and one batch of its list.
            constexpr int kHalfCap = 6912, kQuarterCap = 3456;  // 2 x 110,592 B, 4 x 55,296 B (+ static) fit an SM
            if (!no_small && n_chunk_items <= 2 * sms && pl.max_sel + 2048 + 512 <= kHalfCap) {
                c.finish_cap = kHalfCap;
                e = launch_flat_finish_half(c, fr, n_chunk_items, cs);
            } else if (!no_small && !flat_rows && n_chunk_items <= 4 * sms && pl.max_sel + 1024 + 512 <= kQuarterCap) {
                c.finish_cap = kQuarterCap;
                e = launch_flat_finish_quarter(c, fr, n_chunk_items, cs);
            } else {
                e = launch_flat_finish(c, fr, std::min(n_chunk_items, flat_rows ? sms : n_chunk_items), pl.smem, cs);
            }
            if (e == cudaSuccess) launches++;
            if (!fork) h->kt.mark("flat_finish", cs);
        } else {
            c.item_base = n_rows_items;
            const int room = h->sm_count - row_grid >= 16 ? h->sm_count - row_grid : h->sm_count;
            const int grid = std::min(n_chunk_items, room);
            e = launch_sample_chunks(c, grid, pl.smem, cs);
            if (e == cudaSuccess) { h->work_base += (uint32_t)n_chunk_items + (uint32_t)grid; launches++; }
        }
    };
    if (flat_rows) {
        // Main stream: the phases of the full rows (their plan and scatter kernels on a stream of their
        // own beside the walk).  Side stream: the finish of the chunked rows - held back until the scatter
        // pass is through, because its one-SM CTAs would otherwise sit on the SMs that pass needs while
        // the walk holds the others, whereas the cut that follows leaves two thirds of the GPU idle -
        // and behind it, once the last kernel that can give a row up (the draw's partial sums) is through,
        // the row kernel for exactly the rows the flat form gave up (every other CTA of it leaves at
        // once), beside the draw.
        if (!flat_chunks) launch_chunked();
        const FullSide side{h->plan_stream, h->ev_exp, h->ev_scatter, pl.n_full_without_top_p > 0, pl.n_full_with_top_p > 0};
        if (e == cudaSuccess) e = launch_full_rest(a, ws, a.items, n_rows_items, &launches, &h->kt, stream, 0, side);
        if (flat_chunks) {
            if (e == cudaSuccess && side.any_with_top_p) e = cudaStreamWaitEvent(h->aux_stream, h->ev_scatter, 0);
            launch_chunked();
        }
        if (e == cudaSuccess) e = launch_full_rest(a, ws, a.items, n_rows_items, &launches, &h->kt, stream, 1, side);
        if (e == cudaSuccess) e = cudaEventRecord(h->ev_cut, stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(h->aux_stream, h->ev_cut, 0);
        if (e == cudaSuccess) e = launch_rows_kernel(true, h->aux_stream);
        if (e == cudaSuccess) e = launch_full_rest(a, ws, a.items, n_rows_items, &launches, &h->kt, stream, 2, side);
    } else {
        if (e == cudaSuccess && n_rows_items > 0) {
            e = launch_rows_kernel(false, stream);
            h->kt.mark("rows_kernel", stream);
        }
        launch_chunked();
    }
    if (e == cudaSuccess && fork) e = cudaEventRecord(h->ev_join, h->aux_stream);
    if (e == cudaSuccess && fork) e = cudaStreamWaitEvent(stream, h->ev_join, 0);
    h->kt.mark("join_side_stream", stream);
    };
    const uint32_t host_in = STG_MEM_HOST_LOGITS | STG_MEM_HOST_HISTORY | STG_MEM_HOST_MASK | STG_MEM_HOST_BIAS | STG_MEM_HOST_UNIFORMS;
    const bool all_flat = (flat_chunks || n_chunk_items == 0) && (flat_full || n_rows_items == 0);
    bool replayed = false;
    cudaStreamCaptureStatus cap_status = cudaStreamCaptureStatusNone;
    if (!h->graphs_off) cudaStreamIsCapturing(stream, &cap_status);  // never a capture inside a caller's capture
    if (!h->graphs_off && cap_status == cudaStreamCaptureStatusNone && all_flat && x.shard_mode == 0 && (mf & host_in) == 0 &&
        !h->kt.on && a.phase_ticks == nullptr) {
        std::vector<unsigned char> &gk = h->plan_key_scratch;  // free again: the plan key has been compared
        gk.assign((const unsigned char *)&a, (const unsigned char *)&a + sizeof(a));
        const uint64_t extra[3] = {h->plan_version, (uint64_t)(uintptr_t)stream, (uint64_t)mode};
        gk.insert(gk.end(), (const unsigned char *)extra, (const unsigned char *)extra + sizeof(extra));
        uint64_t hash = 1469598103934665603ull;
        for (unsigned char ch : gk) hash = (hash ^ ch) * 1099511628211ull;
        StgSampler_::StepGraph *hit = nullptr;
        for (auto &g : h->graphs)
            if (g.exec && g.key == gk) hit = &g;
        if (hit == nullptr && std::find(h->seen_keys.begin(), h->seen_keys.end(), hash) != h->seen_keys.end()) {
            // second sighting: capture.  Nothing runs during a capture; a failed one is abandoned and the
            // step launched directly, with graphs off for this handle from then on.
            cudaGraph_t graph = nullptr;
            cudaGraphExec_t exec = nullptr;
            cudaError_t ce = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
            if (ce == cudaSuccess) {
                issue();
                const cudaError_t launch_e = e;
                ce = cudaStreamEndCapture(stream, &graph);
                if (ce == cudaSuccess && launch_e != cudaSuccess) ce = launch_e;
            }
            if (ce == cudaSuccess) ce = cudaGraphInstantiate(&exec, graph, 0);
            if (graph) cudaGraphDestroy(graph);
            if (ce == cudaSuccess) {
                StgSampler_::StepGraph *slot = nullptr;
                if (h->graphs.size() < 16) { h->graphs.emplace_back(); slot = &h->graphs.back(); }
                else {
                    slot = &h->graphs[0];
                    for (auto &g : h->graphs) if (g.used < slot->used) slot = &g;
                    if (slot->exec) cudaGraphExecDestroy(slot->exec);
                }
                slot->key = gk;
                slot->exec = exec;
                slot->launches = launches;
                hit = slot;
            } else {
                cudaGetLastError();  // clear
                h->graphs_off = true;
                e = cudaSuccess;
                launches = 0;
            }
        } else if (hit == nullptr) {
            if (h->seen_keys.size() >= 8) h->seen_keys.erase(h->seen_keys.begin());
            h->seen_keys.push_back(hash);
        }
        if (hit != nullptr) {
            hit->used = ++h->graph_tick;
            e = cudaGraphLaunch(hit->exec, stream);
            replayed = true;
            h->stats.graph_replays++;
            launches = hit->launches;
        }
    }
    if (!replayed) {
        h->kt.begin(stream);
        launches = 0;
        e = cudaSuccess;
        issue();
    }
    if (e != cudaSuccess) {
        cudaMemsetAsync(h->work_counter.p, 0, 8, stream);
        cudaMemsetAsync(h->tickets.p, 0, h->tickets.bytes, stream);
        cudaMemsetAsync(h->flat_rows.p, 0, h->flat_rows.bytes, stream);
        h->work_base = 0;
        h->work_base_rows = 0;
        return cuda_fail(h, e, "sampling kernel launch");
    }
    h->stats.kernel_launches += launches - 1;  // the call below counts one
    h->stats.calls++;
    h->stats.kernel_launches++;
    h->stats.rows_sampled += rows;
    h->stats.rows_greedy += pl.n_greedy; h->stats.rows_topk_path += pl.n_topk; h->stats.rows_full_path += pl.n_full;

    if (host_out) {
        if ((mode == 0 || mode == 3) && b->tokens) CK(cudaMemcpyAsync(b->tokens, a.tokens, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream));
        if (b->token_probs) CK(cudaMemcpyAsync(b->token_probs, a.token_probs, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream));
        if (b->row_flags) CK(cudaMemcpyAsync(b->row_flags, a.row_flags, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream));
        if (b->topk_ids) CK(cudaMemcpyAsync(b->topk_ids, a.topk_ids, (size_t)rows * ts * 4, cudaMemcpyDeviceToHost, stream));
        if (b->topk_logits) CK(cudaMemcpyAsync(b->topk_logits, a.topk_logits, (size_t)rows * ts * 4, cudaMemcpyDeviceToHost, stream));
        if (b->topk_probs) CK(cudaMemcpyAsync(b->topk_probs, a.topk_probs, (size_t)rows * ts * 4, cudaMemcpyDeviceToHost, stream));
        if (mode == 1) CK(cudaMemcpyAsync(dist_out, a.dist_out, (size_t)rows * V * 4, cudaMemcpyDeviceToHost, stream));
        CK(cudaStreamSynchronize(stream));
    }
    return STG_OK;
}

// every device buffer a handle owns
std::vector<DevBuf *> all_buffers(StgHandle h)
{
    return {&h->plan_dev, &h->flat_rows, &h->fw_rows, &h->fw_e, &h->fw_keys, &h->fw_ov_id, &h->fw_ov_adj, &h->fw_ew, &h->fw_hist,
            &h->fw_bstart, &h->fw_binexp, &h->fw_flagbits, &h->fw_cursor, &h->cand, &h->cand_count, &h->tickets, &h->work_counter,
            &h->escratch, &h->keyscratch, &h->listscratch, &h->dists, &h->st_hist, &h->st_bias_ids, &h->st_bias_vals, &h->st_uniforms,
            &h->st_mask, &h->st_logits, &h->o_tokens, &h->o_probs, &h->o_flags, &h->o_topk_ids, &h->o_topk_vals, &h->o_topk_probs,
            &h->o_pairs, &h->ticks, &h->ring_ids, &h->ring_len_dev, &h->mc_words, &h->mc_slots, &h->sp_draft, &h->sp_uniforms,
            &h->sp_accepted, &h->sp_correction, &h->sp_aprobs, &h->sp_flags, &h->sp_rowstats, &h->xchg_local, &h->xchg_gather};
}

}  // namespace stg

extern "C" {

int stg_abi_version(void) { return STG_ABI_VERSION; }

int stg_create(const StgConfig *cfg, StgHandle *out)
{
    StgHandle h = nullptr;
    if (!cfg || !out || cfg->struct_size != (int32_t)sizeof(StgConfig))
        return fail(nullptr, STG_ERR_INVALID_ARGUMENT, "bad StgConfig");
    *out = nullptr;
    if (cfg->max_rows <= 0 || cfg->max_vocab <= 0 || cfg->max_history < 0 || cfg->max_top_k < 0 || cfg->max_bias < 0 ||
        cfg->max_cached_masks < 0)
        return fail(nullptr, STG_ERR_INVALID_ARGUMENT, "capacities must be positive");
    if ((int64_t)cfg->max_top_k + cfg->max_history > kMaxSel)
        return fail(nullptr, STG_ERR_CAPACITY, "max_top_k + max_history must not exceed 8192");
    int n_dev = 0;
    cudaError_t e = cudaGetDeviceCount(&n_dev);
    if (e != cudaSuccess || n_dev <= 0 || cfg->device < 0 || cfg->device >= n_dev)
        return fail(nullptr, STG_ERR_NO_DEVICE, std::string("no usable CUDA device (there is no CPU fallback): ") + cudaGetErrorString(e));
    e = cudaSetDevice(cfg->device);
    if (e != cudaSuccess) return fail(nullptr, STG_ERR_NO_DEVICE, cudaGetErrorString(e));
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, cfg->device);
    if (e != cudaSuccess) return fail(nullptr, STG_ERR_CUDA, cudaGetErrorString(e));
    if (prop.major < 10) return fail(nullptr, STG_ERR_NO_DEVICE, "this library is built for sm_100a (B200) only");

    h = new StgSampler_();
    h->cfg = *cfg;
    h->checked = getenv("STG_CHECKED") != nullptr && getenv("STG_CHECKED")[0] == '1';
    if (const char *drill = getenv("STG_LOOKBACK_DRILL")) h->lookback_drill = drill[0] == '1' ? 1 : drill[0] == '2' ? 2 : 0;
    h->graphs_off = getenv("STG_NO_GRAPH") != nullptr;
    h->sm_count = prop.multiProcessorCount;
    h->smem_optin = prop.sharedMemPerBlockOptin > 4096 ? prop.sharedMemPerBlockOptin - 4096 : 0;
    const size_t R = (size_t)cfg->max_rows, V = (size_t)cfg->max_vocab;
    const size_t sel_max = std::max<size_t>(1, (size_t)cfg->max_top_k + cfg->max_history);
    h->cand_entries = R * std::max<size_t>({8 * sel_max, sel_max + (size_t)kFlatSlack, (size_t)64});
    h->escratch_stride = (int64_t)round_up(V + 8, 64);
    h->key_stride = (int64_t)round_up(V + 8, 64);
    h->plan_bytes_cap = round_up(R * sizeof(RowPlan), 256) + round_up((R * 65) * sizeof(WorkItem), 256) +
                        round_up(R * kPowTab * sizeof(float), 256) + 1024;
    int rc = STG_OK;
    auto A = [&](DevBuf &b, size_t bytes) { if (rc == STG_OK) rc = dev_alloc(h, b, bytes); };
    A(h->plan_dev, h->plan_bytes_cap);
    A(h->cand, h->cand_entries * 8);
    A(h->cand_count, R * 64 * 4);
    A(h->tickets, R * 4);
    A(h->flat_rows, R * sizeof(FlatRow));
    {
        // full-vocabulary rows of the flat step (FullWs): per row the exp values and the candidate keys
        // (4 bytes per token each), the histogram and its plan, the override list, the sub-tile summaries
        h->full_cap = (int)std::min<size_t>(R, 1024);
        const size_t F = (size_t)h->full_cap;
        A(h->fw_rows, F * sizeof(FullRow));
        A(h->fw_e, F * (size_t)h->escratch_stride * 4);
        A(h->fw_keys, F * (size_t)h->key_stride * 4);
        A(h->fw_ov_id, F * kMaxOverride * 4);
        A(h->fw_ov_adj, F * kMaxOverride * 4);
        A(h->fw_ew, F * sizeof(Emul2Work));
        A(h->fw_hist, F * kHistBins * 8);
        A(h->fw_bstart, F * kHistBins * 4);
        A(h->fw_binexp, F * kHistBins);
        A(h->fw_flagbits, F * (kHistBins / 32) * 4);
        A(h->fw_cursor, F * kHistBins * 4);
    }
    A(h->work_counter, 256);
    A(h->escratch, (size_t)h->sm_count * h->escratch_stride * 4);
    A(h->keyscratch, (size_t)h->sm_count * h->key_stride * 8);
    A(h->listscratch, (size_t)h->sm_count * (h->key_stride + 512) * 8);  // + 2 sub-tiles: padded reads
    A(h->st_hist, R * std::max<size_t>(cfg->max_history, 1) * 4);
    A(h->ring_ids, R * std::max<size_t>(cfg->max_history, 1) * 4);
    A(h->ring_len_dev, R * 4);
    h->ring_len.assign(R, 0);
    h->ring_dropped.assign(R, 0);
    if (cfg->max_cached_masks > 0) {
        h->mc_stride = (int64_t)round_up(((size_t)V + 31) / 32, 4);  // rows start on 16-byte boundaries
        A(h->mc_words, (size_t)cfg->max_cached_masks * h->mc_stride * 4);
        A(h->mc_slots, R * 32 * 4);
        h->mc_key.assign(cfg->max_cached_masks, 0);
        h->mc_used.assign(cfg->max_cached_masks, 0);
    }
    A(h->st_bias_ids, R * std::max<size_t>(cfg->max_bias, 1) * 4);
    A(h->st_bias_vals, R * std::max<size_t>(cfg->max_bias, 1) * 4);
    A(h->st_uniforms, R * 8);
    if (cfg->flags & STG_CFG_HOST_LOGITS) {
        A(h->st_mask, R * ((V + 31) / 32) * 4);
        A(h->st_logits, R * V * 4);
    } else {
        A(h->st_mask, 256);
        A(h->st_logits, 256);
    }
    A(h->o_tokens, R * 4); A(h->o_probs, R * 4); A(h->o_flags, R * 4);
    const size_t tk = R * std::max<size_t>(cfg->max_top_k, 1) * 4;
    A(h->o_topk_ids, tk); A(h->o_topk_vals, tk); A(h->o_topk_probs, tk);
    if (getenv("STG_PHASE_TICKS") && getenv("STG_PHASE_TICKS")[0] == '1') A(h->ticks, R * 65 * 32 * 8);
    if (getenv("STG_KERNEL_TIMES") && getenv("STG_KERNEL_TIMES")[0] == '1') {
        h->kt.on = true;
        for (int i = 0; i <= KernelTimer::kMax; i++) cudaEventCreate(&h->kt.ev[i]);
    }
    if (cfg->max_spec_draft > 0) {
        const size_t L = (size_t)cfg->max_spec_draft;
        A(h->sp_draft, R * L * 4); A(h->sp_uniforms, R * (L + 2) * 8);
        A(h->sp_accepted, R * 4); A(h->sp_correction, R * 4); A(h->sp_aprobs, R * L * 4); A(h->sp_flags, R * 4);
        A(h->dists, R * (2 * L + 1) * sizeof(RowDist));
        A(h->sp_rowstats, R * 20);  // flat verification: 16 bytes of control and a fall-back flag per sequence
    }
    if (rc == STG_OK) {
        e = cudaHostAlloc((void **)&h->plan_host, h->plan_bytes_cap * 4, cudaHostAllocDefault);
        if (e != cudaSuccess) rc = cuda_fail(nullptr, e, "cudaHostAlloc");
    }
    if (rc == STG_OK) {
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        e = cudaStreamCreateWithPriority(&h->aux_stream, cudaStreamNonBlocking, lo);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_fork, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_join, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_order, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_cut, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_exp, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_scatter, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&h->plan_stream, cudaStreamNonBlocking, hi);
        if (e != cudaSuccess) rc = cuda_fail(nullptr, e, "side stream");
    }
    for (int i = 0; i < 4 && rc == STG_OK; i++) {
        e = cudaEventCreateWithFlags(&h->plan_ev[i], cudaEventDisableTiming);
        if (e != cudaSuccess) rc = cuda_fail(nullptr, e, "cudaEventCreate");
    }
    if (rc == STG_OK) {
        e = cudaMemset(h->work_counter.p, 0, 256);
        if (e == cudaSuccess) e = cudaMemset(h->tickets.p, 0, h->tickets.bytes);
        if (e == cudaSuccess) e = cudaMemset(h->ring_len_dev.p, 0, h->ring_len_dev.bytes);
        if (e == cudaSuccess) e = cudaMemset(h->flat_rows.p, 0, h->flat_rows.bytes);  // keys and tickets are zero between steps
        if (e != cudaSuccess) rc = cuda_fail(nullptr, e, "cudaMemset");
    }
    if (rc != STG_OK) {
        stg::g_create_error = h->err.empty() ? stg::g_create_error : h->err;
        stg_destroy(h);
        return rc;
    }
    *out = h;
    return STG_OK;
}

int stg_destroy(StgHandle h)
{
    if (!h) return STG_OK;
    cudaSetDevice(h->cfg.device);
    cudaDeviceSynchronize();
    stg_comm_destroy(h);
    for (auto &g : h->graphs) if (g.exec) cudaGraphExecDestroy(g.exec);
    for (DevBuf *b : all_buffers(h)) dev_free(*b);
    if (h->plan_host) cudaFreeHost(h->plan_host);
    for (auto &ev : h->plan_ev) if (ev) cudaEventDestroy(ev);
    if (h->ev_fork) cudaEventDestroy(h->ev_fork);
    if (h->ev_join) cudaEventDestroy(h->ev_join);
    if (h->ev_order) cudaEventDestroy(h->ev_order);
    if (h->ev_cut) cudaEventDestroy(h->ev_cut);
    if (h->ev_exp) cudaEventDestroy(h->ev_exp);
    if (h->ev_scatter) cudaEventDestroy(h->ev_scatter);
    if (h->plan_stream) cudaStreamDestroy(h->plan_stream);
    if (h->aux_stream) cudaStreamDestroy(h->aux_stream);
    delete h;
    return STG_OK;
}

int stg_debug_check_guards(StgHandle h, int32_t *n_guarded, int32_t *first_bad)
{
    if (!h || !n_guarded || !first_bad) return STG_ERR_INVALID_ARGUMENT;
    *n_guarded = 0;
    *first_bad = -1;
    CK(cudaSetDevice(h->cfg.device));
    CK(cudaDeviceSynchronize());
    std::vector<unsigned char> tail(kGuardBytes);
    int index = 0;
    for (DevBuf *b : all_buffers(h)) {
        if (b->p && b->guarded) {
            CK(cudaMemcpy(tail.data(), (char *)b->p + b->bytes, kGuardBytes, cudaMemcpyDeviceToHost));
            ++*n_guarded;
            for (unsigned char c : tail)
                if (c != kGuardByte && *first_bad < 0) *first_bad = index;
        }
        index++;
    }
    return STG_OK;
}

size_t stg_last_error(StgHandle h, char *buf, size_t len)
{
    const std::string &s = h ? h->err : stg::g_create_error;
    if (buf && len) {
        size_t n = std::min(len - 1, s.size());
        memcpy(buf, s.data(), n);
        buf[n] = 0;
    }
    return s.size() + 1;
}

int stg_debug_phase_ticks(StgHandle h, uint64_t *out, int32_t max_items, int32_t *n_items)
{
    if (!h || !out || !n_items) return STG_ERR_INVALID_ARGUMENT;
    if (!h->ticks.p) return fail(h, STG_ERR_UNSUPPORTED, "create the handle with STG_PHASE_TICKS=1 in the environment");
    CK(cudaSetDevice(h->cfg.device));
    CK(cudaDeviceSynchronize());
    const int n = std::min(max_items, h->ticks_items);
    CK(cudaMemcpy(out, h->ticks.p, (size_t)n * 32 * 8, cudaMemcpyDeviceToHost));
    *n_items = n;
    return STG_OK;
}

int stg_debug_kernel_times(StgHandle h, float *out_us, char *names, int32_t name_len, int32_t max_items, int32_t *n_items)
{
    if (!h || !out_us || !n_items) return STG_ERR_INVALID_ARGUMENT;
    if (!h->kt.on) return fail(h, STG_ERR_UNSUPPORTED, "create the handle with STG_KERNEL_TIMES=1 in the environment");
    CK(cudaSetDevice(h->cfg.device));
    CK(cudaDeviceSynchronize());
    const int n = std::min<int>(max_items, h->kt.n);
    for (int i = 0; i < n; i++) {
        float ms = 0.f;
        CK(cudaEventElapsedTime(&ms, h->kt.ev[i], h->kt.ev[i + 1]));
        out_us[i] = ms * 1000.f;
        if (names && name_len > 0) {
            strncpy(names + (size_t)i * name_len, h->kt.name[i] ? h->kt.name[i] : "", (size_t)name_len - 1);
            names[(size_t)i * name_len + name_len - 1] = 0;
        }
    }
    *n_items = n;
    return STG_OK;
}

int stg_get_stats(StgHandle h, StgStats *out)
{
    if (!h || !out) return STG_ERR_INVALID_ARGUMENT;
    // the event counters live on the device (the kernels bump them where they write a row's flags):
    // this call waits for the work enqueued so far
    unsigned long long ctr[kCtrCount] = {0};
    CK(cudaSetDevice(h->cfg.device));
    CK(cudaMemcpy(ctr, (unsigned long long *)h->work_counter.p + 16, sizeof(ctr), cudaMemcpyDeviceToHost));
    h->stats.boundary_draws = ctr[kCtrBoundary]; h->stats.tie_rows = ctr[kCtrTie]; h->stats.cdf_fallbacks = ctr[kCtrFallback];
    h->stats.wide_nucleus_rows = ctr[kCtrWide]; h->stats.reread_rows = ctr[kCtrReread]; h->stats.near_cut_rows = ctr[kCtrNearCut];
    h->stats.fully_masked_rows = ctr[kCtrMasked];
    *out = h->stats;
    return STG_OK;
}

int stg_sample_rows(StgHandle h, const StgSampleBatch *b, void *stream)
{
    BatchExtra x;
    return run_batch(h, b, x, stream);
}

int stg_sample_with_distribution(StgHandle h, const StgSampleBatch *b, float *probs, void *stream)
{
    BatchExtra x;
    x.mode = 3;
    x.dist_out = probs;
    return run_batch(h, b, x, stream);
}

int stg_build_distribution(StgHandle h, const StgSampleBatch *b, float *probs, void *stream)
{
    BatchExtra x;
    x.mode = 1;
    x.dist_out = probs;
    return run_batch(h, b, x, stream);
}

int stg_argmax_rows(StgHandle h, const void *logits, int32_t dtype, int32_t rows, int32_t vocab, int64_t row_stride,
                    void *out_pairs, void *stream)
{
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (!out_pairs) return fail(h, STG_ERR_INVALID_ARGUMENT, "out_pairs is required");
    if (rows < 0 || rows > h->cfg.max_rows) return fail(h, STG_ERR_CAPACITY, "rows exceed max_rows");
    std::vector<StgRowParams> params((size_t)std::max(rows, 1));
    for (auto &p : params) { memset(&p, 0, sizeof(p)); p.temperature = 0.f; p.top_p = 1.f; p.repetition_penalty = 1.f; }
    StgSampleBatch b;
    memset(&b, 0, sizeof(b));
    b.struct_size = sizeof(b);
    b.rows = rows; b.vocab = vocab; b.logits_dtype = dtype; b.logits = logits; b.row_stride = row_stride;
    b.params = params.data();
    b.tokens = (int32_t *)h->o_tokens.p;
    BatchExtra x;
    x.pairs_out = out_pairs;
    return run_batch(h, &b, x, stream);
}

}  // extern "C"
