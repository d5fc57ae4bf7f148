// Plain structs shared by the host planner and the kernels.
#pragma once
#include <stdint.h>

namespace stg {

#ifndef STG_KTHREADS
#define STG_KTHREADS 1024
#endif
constexpr int kThreads = STG_KTHREADS;  // threads per CTA of the row-level kernels (one translation unit builds the
                                        // top-k finish with 512, two CTAs per SM: stg_flat_finish_half.cu)
constexpr int kSubTile = 4096;          // elements one CTA filters per exact-append step
constexpr int kMaxSel = 8192;           // largest selection count (top_k + history length)
constexpr int kPowTab = 32;             // host-computed powf(rep, occ) entries per distinct rep
constexpr int kEmulItems = 8;           // consecutive elements per thread in the sequential-sum scan
constexpr int kEmulTile = kThreads * kEmulItems;
constexpr int kSortCap = 32768;         // top-p candidate keys sorted in shared memory
constexpr int kHistBins = 4096;         // probability histogram bins (exponent + 4 mantissa bits)
constexpr int kMaxOverride = 2048;      // history + bias entries per row on the full-vocabulary path

constexpr uint32_t kFlagFlatRedo = 1u << 8;       // row flag: an optimistic bound failed, the row was processed twice
constexpr uint32_t kFlagNearBoundary = 1u << 3;   // row flag: the draw lies within kNearTol of a CDF step at the token
constexpr uint32_t kFlagNearCut = 1u << 10;       // row flag: the top-p running sum passes top_p within kNearTol
constexpr float kNearTol = 1e-6f;

// device event counters of a handle (read by stg_get_stats)
enum { kCtrBoundary = 0, kCtrTie, kCtrFallback, kCtrWide, kCtrReread, kCtrNearCut, kCtrMasked, kCtrCount = 8 };

enum Path : int32_t {
    kPathGreedy = 0,        // Sampler.Greedy
    kPathGreedyPen = 1,     // GreedyWithHistoryPenalties
    kPathTopK = 2,          // SampleTopK
    kPathFull = 3,          // full-vocabulary pipeline
    kPathTopKNoFinite = 4,  // SampleTopK fell back to Greedy
};

// One row of a sampling step, resolved by the host planner from StgRowParams and the CSR arrays.
struct RowPlan {
    float temperature, top_p, min_p, rep, pres, freq;
    int32_t top_k, window_start;
    int32_t hist_off, hist_len, bias_off, bias_len;
    int32_t path;       // Path
    int32_t sel;        // selection count of the streaming select (1 for plain greedy)
    int32_t n_chunks;   // chunk work items of this row (0 for row-type rows)
    int32_t cand_off;   // first entry of this row's candidate scratch (entries of 8 bytes)
    int32_t use_mask, has_penalty, pow_off, slot;
    int32_t flat_groups; // flat step, top-k rows: groups of the sample whose maxima bound the filter (power of two)
    int32_t flat_full;   // flat step: index of a full-vocabulary row in the step's FullWs, -1 otherwise
    int32_t flat_rank;   // flat step, top-k rows: the bound is the sample's flat_rank-th largest logit (0: the groups' bound itself)
};

struct WorkItem {
    int32_t row;
    int32_t chunk;  // -1: the whole row is one work item
};

// Distribution descriptor of one row on the full-vocabulary pipeline: everything needed to
// evaluate p[i] from the row's logit i without any per-row scratch.
struct RowDist {
    float max_x;      // maximum of the adjusted, temperature-scaled logits
    float inv_t;      // 1/T (1 when T == 1)
    float inv1;       // softmax: 1/sum (multiplied in when scale1)
    float kth;        // top-k: smallest surviving probability (before its normalise)
    float inv2;       // top-k normalise
    float minp_thr;   // min-p threshold
    float tstar;      // top-p: smallest surviving probability
    float inv3;       // final normalise
    int32_t tie_idx_max;  // top-p: ties at tstar survive up to this token id
    uint32_t flags;       // kDist*
    float uniform_p;      // probability of every token when no logit is finite
    int32_t argmax;       // arg-max of the raw row (distribution-only mode)
    float sum_end;        // last value of the sequential CDF (diagnostic)
};
enum : uint32_t {
    kDistScale1 = 1u, kDistTopK = 2u, kDistScale2 = 4u, kDistMinP = 8u, kDistTopP = 16u,
    kDistScale3 = 32u, kDistUniform = 64u, kDistOneHot = 128u,
};

struct SampleArgs {
    const void *logits;
    const RowPlan *plans;
    const WorkItem *items;
    const int32_t *hist_ids;
    const int32_t *bias_ids;
    const float *bias_vals;
    const uint32_t *mask;
    const float *uniforms;
    const float *pow_tab;
    int32_t *tokens;
    float *token_probs;
    uint32_t *row_flags;
    int32_t *topk_ids;
    float *topk_logits;
    float *topk_probs;
    float *dist_out;                 // build_distribution: [rows, vocab] probabilities or null
    void *pairs_out;                 // argmax_rows: rows x {int32 index, float value} or null
    unsigned long long *cand;        // candidate scratch
    int32_t *cand_count;             // per (row, chunk) entry counts
    uint32_t *tickets;               // per-row arrival counters (self-resetting)
    uint32_t *work_counter;
    unsigned long long *phase_ticks; // diagnostic: 32 globaltimer stamps per work item, or null
    float *escratch;                 // per-CTA exp scratch rows [grid, escratch_stride]
    unsigned long long *keyscratch;  // per-CTA wide-nucleus key scratch [grid, key_stride]
    unsigned long long *listscratch; // per-CTA top-p candidates in token order [grid, key_stride]: id << 32 | exp bits
    RowDist *dists;                  // per-row distribution descriptors (optional output)
    unsigned long long *xchg_local;  // vocabulary-sharded mode: this rank's candidates [rows, xchg_stride]
    int32_t *xchg_count;             // ... and how many each row has
    int32_t xchg_stride;
    int64_t row_stride;
    int64_t mask_stride;
    int64_t escratch_stride;
    int64_t key_stride;
    uint32_t work_base;
    int32_t n_items;
    int32_t item_base;               // index of this launch's first item in the step's item list
    int32_t rows, vocab, dtype, topk_stride;
    int32_t chunk_len;               // elements per chunk work item (multiple of kSubTile)
    int32_t cap;                     // entries per candidate buffer in shared memory
    int32_t vec;                     // 4: rows are 16-byte (fp32) / 8-byte (bf16) aligned
    int32_t mode;                    // 0 sample, 1 materialise distributions, 2 distribution descriptors only
    int32_t vocab_offset;            // vocabulary-sharded mode: global id of local column 0
    int32_t shard_mode;              // 0 off, 1 select only (write candidates), 2 finish from gather
    int32_t n_ranks;
    unsigned long long *counters;    // kCtr* event counters, never null
    float softcap;                   // != 0: every logit is read as tanh(x / softcap) * softcap
    int32_t finish_cap;              // candidates per buffer of the half-size finish (stg_flat_finish_half.cu)
    int32_t static_items;            // row kernel: CTA b takes items b, b + grid, ... (no work counter: the launch can be replayed)
    int32_t lookback_drill;          // STG_LOOKBACK_DRILL at stg_create: 1 makes the exp pass's look-back run out, 2 that of the draw's partial sums
    const int32_t *redo_flags;       // row kernel as the flat step's second chance: only rows whose flag
    int32_t redo_stride;             // redo_flags[flat_full * redo_stride] is set are run; null: every row item
};

#ifdef __CUDACC__
// counts the reportable events of a finished row (called by the one thread that writes its flags)
__device__ __forceinline__ void count_row_flags(unsigned long long *ctr, uint32_t fl)
{
    if (ctr == nullptr || (fl & ~7u) == 0u) return;
    if (fl & kFlagNearBoundary) atomicAdd(ctr + kCtrBoundary, 1ull);
    if (fl & (1u << 4)) atomicAdd(ctr + kCtrTie, 1ull);
    if (fl & (1u << 5)) atomicAdd(ctr + kCtrFallback, 1ull);
    if (fl & (1u << 6)) atomicAdd(ctr + kCtrMasked, 1ull);
    if (fl & (1u << 7)) atomicAdd(ctr + kCtrWide, 1ull);
    if (fl & kFlagFlatRedo) atomicAdd(ctr + kCtrReread, 1ull);
    if (fl & kFlagNearCut) atomicAdd(ctr + kCtrNearCut, 1ull);
}

// diagnostic time stamp (nanoseconds) of phase k of the current work item; a no-op when disabled
__device__ __forceinline__ void tick(unsigned long long *t, int k)
{
    if (t != nullptr && threadIdx.x == 0) {
        unsigned long long v;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
        t[k] = v;
    }
}
#endif

}  // namespace stg
