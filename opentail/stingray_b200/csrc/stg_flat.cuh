// The flat form of a sampling step: instead of a few fat persistent CTAs that each own a row (or a
// large piece of one) from the first load to the last draw, the step is a short sequence of kernels
//
//   k_flat_prep    one CTA per row   what a row needs before it can be streamed: the filter bound of
//                                    a top-k row (an order statistic of its first 4096 logits), zeroed
//                                    counters (done by k_full_prep when the step has full rows too)
//   k_flat_stream, k_flat_stream_chunks
//                  one small CTA per 16384-element piece of a row: the only kernels that read the
//                  logits from HBM, each row once - the first over the full-vocabulary rows
//                  (stg_flat.cu), the second over all others (stg_flat_chunks.cu: fewer registers,
//                  more resident warps).  Greedy rows keep a running arg-max key (64-bit atomicMax),
//                  top-k rows append every logit above the row's bound to the row's candidate list
//                  (staged in shared memory, one global atomicAdd per CTA)
//   k_flat_finish  one CTA per row   candidates only: the exact top-N selection, penalties, softmax
//                                    over k, min-p, top-p and the draw of SampleTopK
//                                    (src/OpenTail.Stingray.Engine/Sampler.cs:216-357); built for 1024,
//                                    512 and 256 threads (one, two, four CTAs per SM)
//   k_greedy_step  a step whose rows are all plain arg-max rows: the HBM pass with prep and finish
//                  folded in, one launch (stg_flat_greedy.cu)
//
// so that the HBM pass runs on all SMs whatever the mix of rows - thousands of 256-thread CTAs that
// the hardware scheduler balances - and everything serial touches a few hundred candidates per row.
//
// The bound of a top-k row is optimistic, and checked: k_flat_finish accepts the candidate list only
// when it holds between N = top_k + history length and its capacity entries - they are then exactly
// the logits above the bound, hence a superset of the N best.  Otherwise (the first 4096 logits were
// not representative: ties, masks, sorted rows) the finishing CTA streams the row again itself with
// the exact selection of stg_select.cuh.  No CTA of these kernels waits on another.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "stg_types.h"

namespace stg {

constexpr int kFlatThreads = 256;                  // threads of a k_flat_stream CTA
constexpr int kFlatPiece = 16384;                  // elements of a row one such CTA reads
constexpr int kFlatSteps = kFlatPiece / 4096;      // steps of 4 sub-steps of 1024 elements each
constexpr int kFlatSample = 4096;                  // leading elements of a row the bound is guessed from
constexpr int kFlatSlack = 8192;                   // candidate capacity of a top-k row beyond N (the bound scatters: up to ~3x the expected count was seen)
constexpr int kFlatStage = 1024;                   // candidates a k_flat_stream CTA collects in shared memory

// per-row state of the flat step (device memory, 32 bytes)
struct FlatRow {
    unsigned long long key;  // greedy: running (value, lowest index) arg-max key; 0: nothing finite yet
    float tau;               // top-k: every logit > tau is a candidate
    int32_t cnt;             // top-k: candidates appended (may exceed the capacity: the excess was dropped)
    int32_t cap;             // top-k: capacity of the row's candidate list
    int32_t ticket;          // all-greedy step (stg_flat_greedy.cu): pieces of the row that have arrived; 0 between steps
    int32_t pad[2];
};
static_assert(sizeof(FlatRow) == 32, "FlatRow layout");

// ---- full-vocabulary rows in the flat step -------------------------------------------------------------
// The same idea carried through the full-vocabulary pipeline (stg_rowdist.cuh has it as ONE CTA per
// row): every pass over the V elements of a row is a flat kernel of small CTAs over pieces of the
// row, every strictly serial part (the walks of the exact sequential sums, the top-p cut) a
// one-CTA-per-row kernel that touches per-sub-tile summaries or candidates only.  Between them the
// row lives in device memory (the 126 MB L2 holds the exp values of some 200 rows of 151,936):
//
//   prep     history / bias overrides of the row -> a sorted (token, adjusted logit) list
//   stream   HBM read: mask, overrides, 1/T -> x (stored), running max key
//   exp      e = exp(x - max) (stored over x), sub-tile sums, exp-value histogram; then, in the same
//            CTA, the guessed binade of every sub-tile of the piece (fp64 prefix of the sub-tile sums:
//            the pieces before it publish their totals, a bounded look-back collects them) and the
//            composite increment of every sub-tile under its guess
//   walk     exact softmax sum; min-p threshold
//   plan     (beside the walk, on a stream of its own) top-p plan from the histogram and the fp64 sum
//            of the sub-tile sums: nucleus bound, bin starts, flagged bins
//   scatter  (behind the plan) exp values above the bound into bin order
//   nosum    rows without top-p: fp64 partial sums of their probabilities
//   ties     candidates whose addition would be an exact rounding tie flag their bin
//   cut      flagged-bin sorts and the emulated sorted-order sum -> top-p threshold; normalise
//   sums     the same over the final probabilities (sub-tile sums, look-back, guesses, composites)
//   draw     the walk that finds the token the uniform lands on
//
// A row the flat step cannot finish (its nucleus bound proved too tight, or a look-back ran out) is
// flagged and redone by the self-contained row kernel, on the side stream beside the last two kernels.
constexpr int kFullMaxPieces = 16;  // 262144 / kFlatPiece
constexpr int kFullMaxParts = 32;   // per-piece partial sums of the phase kernels (8192-element pieces)

struct FullRow {
    unsigned long long maxkey;          // (max, lowest index) key of the adjusted, scaled logits
    unsigned long long rawkey;          // descriptor mode: arg-max key of the masked raw logits
    RowDist dist;
    float sum;                          // exact sequential softmax sum
    int32_t n_ov;                       // entries of the override list
    int32_t ov_piece[kFullMaxPieces + 1];  // first override entry of every piece
    int32_t c_lo, bound;                // top-p plan: lowest candidate bin, candidates the histogram counted
    int32_t surv;                       // survivors of the filters before top-p (counted by scatter)
    int32_t redo;                       // 1: redo the row with the self-contained row kernel
    uint32_t flags;                     // STG_ROW_* bits gathered on the way
    int32_t pad;
    double part[kFullMaxParts];         // rows without top-p: per-piece fp64 sums of the probabilities
    // look-back between the CTAs of a per-piece phase kernel ([0]: exp values, [1]: final probabilities):
    // every piece publishes the sum of its sub-tile sums and reads those of the pieces before it
    double ptotal[2][kFullMaxParts];
    uint32_t pflag[2][kFullMaxParts];   // 1: ptotal is there (cleared by k_full_prep)
    int32_t n_cross[2];                 // crossing slots handed out (Emul2Work::xs)
    int32_t pad2[2];
};

struct Emul2Work;
// device workspace of the full-vocabulary rows of a flat step, indexed by RowPlan::flat_full
struct FullWs {
    FullRow *rows;
    float *e;                  // [n, e_stride]: x, then exp values
    int64_t e_stride;
    int32_t *ov_id;            // [n, kMaxOverride] sorted token ids
    float *ov_adj;             // [n, kMaxOverride] their adjusted (unscaled) logits
    Emul2Work *ew;             // [n] sub-tile sums, guesses, composites, crossing slots
    unsigned long long *hist;  // [n, kHistBins] count << 40 | mass
    uint32_t *bstart;          // [n, kHistBins]
    unsigned char *bin_exp;    // [n, kHistBins]
    uint32_t *flag_bits;       // [n, kHistBins / 32]
    uint32_t *cursor;          // [n, kHistBins]
    uint32_t *keys;            // [n, key_stride] candidate probabilities in bin order
    int64_t key_stride;
};

cudaError_t launch_flat_prep(const SampleArgs &a, FlatRow *fr, cudaStream_t stream);
cudaError_t launch_flat_stream(const SampleArgs &a, FlatRow *fr, const FullWs &ws, cudaStream_t stream);
// the same pass over rows of the top-k path and plain arg-max rows only (stg_flat_chunks.cu)
cudaError_t launch_flat_stream_chunks(const SampleArgs &a, FlatRow *fr, cudaStream_t stream);
// a step of plain arg-max rows only, in one launch (stg_flat_greedy.cu); needs every row's key and ticket at zero
cudaError_t launch_greedy_step(const SampleArgs &a, FlatRow *fr, cudaStream_t stream);
// flat != null: also prepares the chunked rows of the flat step (then launch_flat_prep is not needed)
cudaError_t launch_full_prep(const SampleArgs &a, const FullWs &ws, FlatRow *flat, cudaStream_t stream);
struct KernelTimer;
// speculative verification in the flat form (stg_flat_full.cu): seq_ctl holds 16 bytes per sequence, fallback one
// int per sequence (1: k_spec_finish must redo it)
struct SpecArgs;
cudaError_t launch_spec_flat(const SpecArgs &a, const FullWs &ws, void *seq_ctl, int32_t *fallback, cudaStream_t stream);
// the second stream of the full rows' phases (the plan and the scatter pass run beside the walk)
struct FullSide {
    cudaStream_t stream;
    cudaEvent_t after_exp, after_scatter;
    bool any_without_top_p;  // some full row has top-p off: its Normalize sum needs a pass of its own
    bool any_with_top_p;     // some full row has top-p on: plan, scatter and tie kernels have work
};
cudaError_t launch_full_rest(const SampleArgs &a, const FullWs &ws, const WorkItem *full_items, int n_full, int *launches,
                             KernelTimer *kt, cudaStream_t stream, int part, const FullSide &side);
// the small-CTA finishes (512 threads, two CTAs per SM; 256 threads, four per SM; a.finish_cap entries per buffer)
cudaError_t launch_flat_finish_half(const SampleArgs &a, FlatRow *fr, int grid, cudaStream_t stream);
cudaError_t launch_flat_finish_quarter(const SampleArgs &a, FlatRow *fr, int grid, cudaStream_t stream);
// grid: CTAs that share the rows of a.items between them (at most a.n_items)
cudaError_t launch_flat_finish(const SampleArgs &a, FlatRow *fr, int grid, size_t smem, cudaStream_t stream);

}  // namespace stg
