/*
 * CPU oracle for the Stingray token-sampling hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA library is
 * compared against; it is never linked into, loaded by or called from the
 * product library.  Only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg may load it.
 *
 * It restates, operation for operation and in scalar fp32, the reference's
 * managed sampler.  Every function cites the reference lines it follows
 * (paths are relative to the reference project's root).  The reference's C#
 * cannot be compiled where this was written (no .NET toolchain), so parity is
 * pinned by the reference's own inline known-answer tests
 * (tests/OpenTail.Stingray.Tests.ForwardPass.Fast/SamplerTests.cs,
 * SpeculativeSamplingTests.cs, tests/OpenTail.Stingray.Tests.Cuda/
 * CudaGpuArgmaxParityTests.cs), restated in tests/test_oracle_kat.py.
 *
 * Arithmetic that lives in third-party code the reference calls:
 *   - MathF.Exp / MathF.Pow / Math.Exp (.NET runtime 10)   -> libm expf/powf/exp
 *   - TensorPrimitives.IndexOfMax / Max / Multiply (System.Numerics.Tensors
 *     10.0.5) -> first-index-of-maximum, maximum, element-wise fp32 multiply
 *   - TensorPrimitives.Sum (same package): a vectorised sum whose association
 *     order depends on the host's vector width.  PARITY UNPINNED for that one
 *     call: `sum_mode` selects the model (0 = fp64 accumulate then round,
 *     1 = sequential fp32, 2 = 8-lane strided fp32, 3 = 16-lane strided fp32).
 *   - MemoryExtensions.Sort with a comparison (unstable): the order of equal
 *     probabilities inside ApplyTopP is PARITY UNPINNED; this file orders ties
 *     by ascending token id and reports when the nucleus cut falls inside a tie.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -fPIC -shared (see Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* Per-request knobs: SamplingParams, src/OpenTail.Stingray.Engine/Sampler.cs:648-686,795.
 * Same field order as the product's C-ABI row-parameter struct. */
typedef struct {
    float temperature;        /* :650 default 1 */
    float top_p;              /* :652 default 1 */
    float min_p;              /* :653 default 0 */
    float repetition_penalty; /* :654 default 1 */
    float presence_penalty;   /* :679 */
    float frequency_penalty;  /* :684 */
    int32_t top_k;            /* :651 default 0 */
    int32_t repeat_last_n;    /* :674 default 64 */
} OrcParams;

/* What the oracle reports beside the token, so tests can classify a mismatch. */
typedef struct {
    int32_t path;          /* 0 greedy, 1 greedy+penalties, 2 top-k fast path, 3 full-vocab path,
                              4 fast path fell back to greedy (no finite logit) */
    int32_t n_cand;        /* fast path: k; full path: number of non-zero probs before the draw */
    int32_t kept;          /* survivors after min-p / top-p */
    int32_t tie_at_cutoff; /* full path: top-p cut fell inside a group of equal probabilities */
    float margin;          /* distance from the draw to the nearest CDF boundary, in
                              probability units of the normalised kept distribution */
    float prob;            /* normalised probability of the returned token */
    float kept_sum;        /* fast path keptSum / full path final sequential CDF end value */
    int32_t fallback;      /* draw ran off the end of the CDF (rounding fallback taken) */
    float cut_margin;      /* full path with top-p: distance of the sorted running sum from top_p at
                              the cut, on the nearer side (0 when top-p did not run) */
} OrcTrace;

static const float NEG_INF = -INFINITY;

/* ---- TensorPrimitives stand-ins ------------------------------------------------------- */

/* Final-logit soft cap, applied in place to the logits before they are sampled
 * (CudaForwardPass.cs:2434): x[i] = tanh(x[i] / cap) * cap, the scalar statement of the GPU kernel
 * llm_softcap_inplace (CudaTextKernels.cs:374-383).  The reference's CPU route
 * (SimdKernels.SoftcapInPlace, src/OpenTail.Stingray.Cpu/SimdKernels.cs:7133) evaluates the same
 * function with a vectorised exp approximation; neither is pinned to the last bit by a reference
 * test, so comparisons against this function carry a tolerance. */
ORC_API void orc_softcap_inplace(float *x, int64_t n, float cap)
{
    for (int64_t i = 0; i < n; i++) x[i] = tanhf(x[i] / cap) * cap;
}

/* Sampler.Greedy, Sampler.cs:442-446 = TensorPrimitives.IndexOfMax: the highest value, the
 * lowest index on ties; pinned by CudaTextKernels.cs:396-402 and CudaGpuArgmaxParityTests.cs
 * :31-38 (strict '>' left-to-right scan).  Empty span -> 0. */
ORC_API int32_t orc_greedy(const float *logits, int32_t n)
{
    if (n <= 0) return 0;
    int32_t idx = 0;
    float best = logits[0];
    for (int32_t i = 1; i < n; i++)
        if (logits[i] > best) { best = logits[i]; idx = i; }
    return idx;
}

static float tp_max(const float *x, int32_t n)
{
    float m = x[0];
    int nan = isnan(m);
    for (int32_t i = 1; i < n; i++) {
        if (isnan(x[i])) nan = 1;
        if (x[i] > m) m = x[i];
    }
    return nan ? NAN : m; /* TensorPrimitives.Max propagates NaN */
}

static float tp_sum(const float *x, int32_t n, int mode)
{
    if (mode == 1) {
        float s = 0.f;
        for (int32_t i = 0; i < n; i++) s += x[i];
        return s;
    }
    if (mode == 2 || mode == 3) {
        int lanes = mode == 2 ? 8 : 16;
        float acc[16];
        for (int l = 0; l < lanes; l++) acc[l] = 0.f;
        int32_t i = 0;
        for (; i + lanes <= n; i += lanes)
            for (int l = 0; l < lanes; l++) acc[l] += x[i + l];
        for (int width = lanes / 2; width >= 1; width /= 2)
            for (int l = 0; l < width; l++) acc[l] += acc[l + width];
        float s = acc[0];
        for (; i < n; i++) s += x[i];
        return s;
    }
    double s = 0.0;
    for (int32_t i = 0; i < n; i++) s += (double)x[i];
    return (float)s;
}

/* ---- history penalties ------------------------------------------------------------------ */

/* RepeatWindowStart, Sampler.cs:364-365 */
static int32_t repeat_window_start(int32_t count, int32_t repeat_last_n)
{
    return (repeat_last_n <= 0 || repeat_last_n >= count) ? 0 : count - repeat_last_n;
}

static int cmp_i32(const void *a, const void *b)
{
    int32_t x = *(const int32_t *)a, y = *(const int32_t *)b;
    return (x > y) - (x < y);
}

/* SamplingParams.HasHistoryPenalty, Sampler.cs:686 */
static int has_history_penalty(const OrcParams *p)
{
    return p->repetition_penalty != 1.0f || p->presence_penalty != 0.f || p->frequency_penalty != 0.f;
}

/* ApplyHistoryPenalties, Sampler.cs:367-419: repetition once per occurrence inside the trailing
 * window, in history order; presence/frequency once per distinct id over the whole history. */
ORC_API void orc_apply_history_penalties(float *logits, int32_t n, const OrcParams *p,
                                         const int32_t *hist, int32_t hcount)
{
    if (hcount <= 0 || hist == NULL) return;
    if (p->repetition_penalty != 1.0f) {
        int32_t start = repeat_window_start(hcount, p->repeat_last_n);
        for (int32_t i = start; i < hcount; i++) {
            int32_t id = hist[i];
            if ((uint32_t)id < (uint32_t)n)
                logits[id] = logits[id] > 0.f ? logits[id] / p->repetition_penalty
                                              : logits[id] * p->repetition_penalty;
        }
    }
    if (p->presence_penalty == 0.f && p->frequency_penalty == 0.f) return;
    int32_t *ids = (int32_t *)malloc(sizeof(int32_t) * (size_t)hcount);
    int32_t kept = 0;
    for (int32_t i = 0; i < hcount; i++)
        if ((uint32_t)hist[i] < (uint32_t)n) ids[kept++] = hist[i];
    qsort(ids, (size_t)kept, sizeof(int32_t), cmp_i32);
    for (int32_t i = 0; i < kept;) {
        int32_t id = ids[i], end = i + 1;
        while (end < kept && ids[end] == id) end++;
        float fcount = (float)(end - i);
        float prod = p->frequency_penalty * fcount;
        float add = p->presence_penalty + prod;
        logits[id] = logits[id] - add;
        i = end;
    }
    free(ids);
}

/* GreedyWithHistoryPenalties, Sampler.cs:421-437 */
static int32_t greedy_with_history(const float *logits, int32_t n, const OrcParams *p,
                                   const int32_t *hist, int32_t hcount)
{
    float *adj = (float *)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
    memcpy(adj, logits, sizeof(float) * (size_t)n);
    orc_apply_history_penalties(adj, n, p, hist, hcount);
    int32_t r = orc_greedy(adj, n);
    free(adj);
    return r;
}

static int32_t greedy_dispatch(const float *logits, int32_t n, const OrcParams *p,
                               const int32_t *hist, int32_t hcount, int32_t *path)
{
    if (has_history_penalty(p) && hcount > 0) {
        if (path) *path = 1;
        return greedy_with_history(logits, n, p, hist, hcount);
    }
    if (path) *path = 0;
    return orc_greedy(logits, n);
}

/* ---- slow-path stages ------------------------------------------------------------------- */

/* Softmax, Sampler.cs:448-472 */
static void softmax_inplace(float *x, int32_t n)
{
    if (n <= 0) return;
    float max = tp_max(x, n);
    if ((isinf(max) && max < 0) || isnan(max)) {
        float uniform = 1.0f / (float)n;
        for (int32_t i = 0; i < n; i++) x[i] = uniform;
        return;
    }
    float sum = 0.f;
    for (int32_t i = 0; i < n; i++) {
        x[i] = expf(x[i] - max);
        sum += x[i];
    }
    if (sum > 0.f && sum != 1.0f) {
        float inv = 1.0f / sum;
        for (int32_t i = 0; i < n; i++) x[i] = x[i] * inv;
    }
}

/* FindKthLargest, Sampler.cs:624-645 */
static float find_kth_largest(const float *data, int32_t n, int32_t k)
{
    float *top = (float *)malloc(sizeof(float) * (size_t)k);
    for (int32_t i = 0; i < k; i++) top[i] = NEG_INF;
    for (int32_t i = 0; i < n; i++) {
        float v = data[i];
        if (v > top[k - 1]) {
            top[k - 1] = v;
            for (int32_t j = k - 1; j > 0 && top[j] > top[j - 1]; j--) {
                float t = top[j]; top[j] = top[j - 1]; top[j - 1] = t;
            }
        }
    }
    float r = top[k - 1];
    free(top);
    return r;
}

/* ApplyTopK, Sampler.cs:477-488 */
static void apply_top_k(float *probs, int32_t n, int32_t k)
{
    float kth = find_kth_largest(probs, n, k);
    for (int32_t i = 0; i < n; i++)
        if (probs[i] < kth) probs[i] = 0.f;
}

/* ApplyMinP, Sampler.cs:493-503 */
static void apply_min_p(float *probs, int32_t n, float min_p)
{
    float thr = min_p * tp_max(probs, n);
    for (int32_t i = 0; i < n; i++)
        if (probs[i] < thr) probs[i] = 0.f;
}

typedef struct { int32_t idx; float prob; } IdxProb;

static int cmp_prob_desc(const void *a, const void *b)
{
    const IdxProb *x = (const IdxProb *)a, *y = (const IdxProb *)b;
    if (x->prob > y->prob) return -1;
    if (x->prob < y->prob) return 1;
    return (x->idx > y->idx) - (x->idx < y->idx); /* unpinned in the reference; ascending id here */
}

/* ApplyTopP, Sampler.cs:516-551 */
static void apply_top_p(float *probs, int32_t n, float top_p, int32_t *tie_at_cutoff, float *cut_margin)
{
    if (cut_margin) *cut_margin = INFINITY;
    int32_t m = 0;
    for (int32_t i = 0; i < n; i++)
        if (probs[i] > 0.f) m++;
    if (m == 0) return;
    IdxProb *ix = (IdxProb *)malloc(sizeof(IdxProb) * (size_t)m);
    int32_t j = 0;
    for (int32_t i = 0; i < n; i++)
        if (probs[i] > 0.f) { ix[j].idx = i; ix[j].prob = probs[i]; j++; }
    qsort(ix, (size_t)m, sizeof(IdxProb), cmp_prob_desc);
    float cum = 0.f;
    int32_t cutoff = m;
    for (int32_t i = 0; i < m; i++) {
        float before = cum;
        cum += ix[i].prob;
        if (cum >= top_p) {
            cutoff = i + 1;
            /* how close the running sum came to top_p on either side of the cut: a cut this close
             * can move by one token when exp differs in its last bit */
            if (cut_margin) *cut_margin = fminf(cum - top_p, top_p - before);
            break;
        }
    }
    if (cut_margin && cutoff == m && cum < top_p) *cut_margin = top_p - cum;
    if (tie_at_cutoff)
        *tie_at_cutoff = (cutoff < m && ix[cutoff].prob == ix[cutoff - 1].prob) ? 1 : 0;
    for (int32_t i = cutoff; i < m; i++) probs[ix[i].idx] = 0.f;
    free(ix);
}

/* Normalize, Sampler.cs:553-562 */
static void normalize(float *probs, int32_t n, int sum_mode)
{
    float sum = tp_sum(probs, n, sum_mode);
    if (sum > 0.f && sum != 1.0f) {
        float inv = 1.0f / sum;
        for (int32_t i = 0; i < n; i++) probs[i] = probs[i] * inv;
    }
}

/* SampleFromDistribution, Sampler.cs:564-576.  `u` is the value of rng.NextDouble(). */
static int32_t sample_from_distribution(const float *probs, int32_t n, double u, OrcTrace *tr)
{
    float r = (float)u;
    float cum = 0.f;
    for (int32_t i = 0; i < n; i++) {
        float before = cum;
        cum += probs[i];
        if (r <= cum) {
            if (tr) {
                float lo = r - before, hi = cum - r;
                tr->margin = lo < hi ? lo : hi;
                tr->prob = probs[i];
                tr->fallback = 0;
            }
            return i;
        }
    }
    if (tr) { tr->margin = r - cum; tr->prob = n > 0 ? probs[n - 1] : 0.f; tr->fallback = 1; tr->kept_sum = cum; }
    return n - 1;
}

ORC_API int32_t orc_sample_from_probs(const float *probs, int32_t n, double u, OrcTrace *tr)
{
    /* SampleFromProbs, Sampler.cs:195-199 */
    return sample_from_distribution(probs, n, u, tr);
}

/* The slow pipeline shared by Sample (Sampler.cs:41-92) and BuildFilteredDistribution
 * (Sampler.cs:134-162): bias -> penalties -> 1/T -> softmax -> [top-k, normalise] -> min-p ->
 * top-p -> normalise.  `probs` holds the logits on entry and the distribution on exit. */
static void slow_pipeline(float *probs, int32_t n, const OrcParams *p, const int32_t *hist,
                          int32_t hcount, const int32_t *bias_ids, const float *bias_vals,
                          int32_t nbias, int sum_mode, int32_t *tie_at_cutoff, float *cut_margin)
{
    if (cut_margin) *cut_margin = INFINITY;
    for (int32_t b = 0; b < nbias; b++)
        if ((uint32_t)bias_ids[b] < (uint32_t)n) probs[bias_ids[b]] += bias_vals[b];
    orc_apply_history_penalties(probs, n, p, hist, hcount);
    if (p->temperature != 1.0f) {
        float inv_t = 1.0f / p->temperature;
        for (int32_t i = 0; i < n; i++) probs[i] = probs[i] * inv_t;
    }
    softmax_inplace(probs, n);
    if (p->top_k > 0 && p->top_k < n) {
        apply_top_k(probs, n, p->top_k);
        normalize(probs, n, sum_mode);
    }
    if (p->min_p > 0.f) apply_min_p(probs, n, p->min_p);
    if (tie_at_cutoff) *tie_at_cutoff = 0;
    if (p->top_p < 1.0f && p->top_p > 0.f) apply_top_p(probs, n, p->top_p, tie_at_cutoff, cut_margin);
    normalize(probs, n, sum_mode);
}

/* BuildFilteredDistribution, Sampler.cs:118-163 */
ORC_API void orc_build_filtered_distribution(const float *logits, int32_t n, const OrcParams *p,
                                             const int32_t *hist, int32_t hcount,
                                             const int32_t *bias_ids, const float *bias_vals,
                                             int32_t nbias, int sum_mode, float *probs,
                                             int32_t *tie_at_cutoff)
{
    if (p->temperature <= 0.f) {
        memset(probs, 0, sizeof(float) * (size_t)n);
        probs[greedy_dispatch(logits, n, p, hist, hcount, NULL)] = 1.f;
        if (tie_at_cutoff) *tie_at_cutoff = 0;
        return;
    }
    memcpy(probs, logits, sizeof(float) * (size_t)n);
    slow_pipeline(probs, n, p, hist, hcount, bias_ids, bias_vals, nbias, sum_mode, tie_at_cutoff, NULL);
}

/* The same, also reporting how close the top-p running sum came to top_p at the cut
 * (infinity when top-p is off): what a test needs to tell a last-bit exp difference from an error. */
ORC_API void orc_build_filtered_distribution_ex(const float *logits, int32_t n, const OrcParams *p,
                                                const int32_t *hist, int32_t hcount,
                                                const int32_t *bias_ids, const float *bias_vals,
                                                int32_t nbias, int sum_mode, float *probs,
                                                int32_t *tie_at_cutoff, float *cut_margin)
{
    if (cut_margin) *cut_margin = INFINITY;
    if (p->temperature <= 0.f) {
        orc_build_filtered_distribution(logits, n, p, hist, hcount, bias_ids, bias_vals, nbias, sum_mode, probs,
                                        tie_at_cutoff);
        return;
    }
    memcpy(probs, logits, sizeof(float) * (size_t)n);
    slow_pipeline(probs, n, p, hist, hcount, bias_ids, bias_vals, nbias, sum_mode, tie_at_cutoff, cut_margin);
}

/* SampleWithDistribution, Sampler.cs:172-187 */
ORC_API int32_t orc_sample_with_distribution(const float *logits, int32_t n, const OrcParams *p,
                                             const int32_t *hist, int32_t hcount, int sum_mode,
                                             double u, float *probs, OrcTrace *tr)
{
    if (p->temperature <= 0.f) {
        int32_t a = greedy_dispatch(logits, n, p, hist, hcount, NULL);
        memset(probs, 0, sizeof(float) * (size_t)n);
        probs[a] = 1.f;
        return a;
    }
    orc_build_filtered_distribution(logits, n, p, hist, hcount, NULL, NULL, 0, sum_mode, probs, NULL);
    return sample_from_distribution(probs, n, u, tr);
}

/* ---- fast path ------------------------------------------------------------------------- */

/* SampleTopK, Sampler.cs:216-357.  Optional outputs (may be NULL): cand_ids/cand_vals/cand_probs
 * receive the first k candidates after the penalty re-sort (ids, penalised logits, softmax
 * probabilities over the k), which is what "the top-k set" means for parity. */
static int32_t sample_top_k(const float *logits, int32_t vocab, const OrcParams *p,
                            const int32_t *hist, int32_t hcount, int has_penalty, double u,
                            OrcTrace *tr, int32_t *cand_ids, float *cand_vals, float *cand_probs)
{
    int32_t k = p->top_k;
    int32_t prev = has_penalty ? hcount : 0;
    int64_t want = (int64_t)k + (int64_t)prev;
    int32_t sel = want < vocab ? (int32_t)want : vocab;

    int32_t *idx = (int32_t *)malloc(sizeof(int32_t) * (size_t)sel);
    float *vals = (float *)malloc(sizeof(float) * (size_t)sel);
    float *probs = (float *)malloc(sizeof(float) * (size_t)k);
    for (int32_t i = 0; i < sel; i++) { vals[i] = NEG_INF; idx[i] = -1; }

    for (int32_t i = 0; i < vocab; i++) {             /* :242-249 */
        float v = logits[i];
        if (v <= vals[sel - 1]) continue;
        int32_t j = sel - 1;
        while (j > 0 && vals[j - 1] < v) { vals[j] = vals[j - 1]; idx[j] = idx[j - 1]; j--; }
        vals[j] = v; idx[j] = i;
    }

    int32_t result;
    if (idx[0] < 0 || (isinf(vals[0]) && vals[0] < 0)) {  /* :254-255 */
        if (tr) tr->path = 4;
        result = orc_greedy(logits, vocab);
        goto done;
    }

    if (has_penalty) {                                /* :261-295 */
        int32_t wstart = repeat_window_start(hcount, p->repeat_last_n);
        for (int32_t t = 0; t < sel; t++) {
            if (idx[t] < 0) continue;
            int32_t occ_w = 0, occ_all = 0;
            for (int32_t h = 0; h < hcount; h++) {
                if (hist[h] != idx[t]) continue;
                occ_all++;
                if (h >= wstart) occ_w++;
            }
            if (occ_all == 0) continue;
            if (p->repetition_penalty != 1.0f && occ_w > 0) {
                float pen = powf(p->repetition_penalty, (float)occ_w);
                vals[t] = vals[t] > 0.f ? vals[t] / pen : vals[t] * pen;
            }
            float prod = p->frequency_penalty * (float)occ_all;
            float add = p->presence_penalty + prod;
            vals[t] = vals[t] - add;
        }
        for (int32_t a = 1; a < sel; a++) {
            float v = vals[a]; int32_t id = idx[a]; int32_t b = a - 1;
            while (b >= 0 && vals[b] < v) { vals[b + 1] = vals[b]; idx[b + 1] = idx[b]; b--; }
            vals[b + 1] = v; idx[b + 1] = id;
        }
    }

    {
        float inv_t = p->temperature == 1.0f ? 1.0f : 1.0f / p->temperature;   /* :298 */
        float max = vals[0] * inv_t;
        float sum = 0.f;
        for (int32_t t = 0; t < k; t++) {
            float scaled = vals[t] * inv_t;
            float e = (isinf(vals[t]) && vals[t] < 0) ? 0.f : expf(scaled - max);
            probs[t] = e;
            sum += e;
        }
        float inv_sum = sum > 0.f ? 1.0f / sum : 0.f;
        for (int32_t t = 0; t < k; t++) probs[t] = probs[t] * inv_sum;

        int32_t count = k;
        if (p->min_p > 0.f) {                          /* :319-324 */
            float thr = p->min_p * probs[0];
            for (int32_t t = 0; t < count; t++)
                if (probs[t] < thr) { count = t; break; }
        }
        if (p->top_p < 1.0f && p->top_p > 0.f) {       /* :327-335 */
            float cum = 0.f;
            for (int32_t t = 0; t < count; t++) {
                cum += probs[t];
                if (cum >= p->top_p) { count = t + 1; break; }
            }
        }
        float kept_sum = 0.f;                          /* :340-349 */
        for (int32_t t = 0; t < count; t++) kept_sum += probs[t];
        float r = (float)u * kept_sum;
        float c = 0.f;
        result = idx[0];
        int found = 0;
        for (int32_t t = 0; t < count; t++) {
            float before = c;
            c += probs[t];
            if (r <= c && idx[t] >= 0) {
                result = idx[t];
                found = 1;
                if (tr) {
                    float lo = r - before, hi = c - r;
                    float m = lo < hi ? lo : hi;
                    tr->margin = kept_sum > 0.f ? m / kept_sum : 0.f;
                    tr->prob = kept_sum > 0.f ? probs[t] / kept_sum : 0.f;
                }
                break;
            }
        }
        if (tr) {
            tr->path = 2;
            tr->n_cand = k;
            tr->kept = count;
            tr->kept_sum = kept_sum;
            tr->fallback = !found;
            if (!found) { tr->margin = 0.f; tr->prob = kept_sum > 0.f ? probs[0] / kept_sum : 0.f; }
        }
        for (int32_t t = 0; t < k; t++) {
            if (cand_ids) cand_ids[t] = idx[t];
            if (cand_vals) cand_vals[t] = vals[t];
            if (cand_probs) cand_probs[t] = probs[t];
        }
    }
done:
    free(idx); free(vals); free(probs);
    return result;
}

/* Sampler.Sample, Sampler.cs:17-102.  `u` is the one rng.NextDouble() the call consumes when
 * temperature > 0 (none is consumed when greedy).  `probs_out` (may be NULL, length n) receives
 * the final distribution on the full-vocabulary path. */
ORC_API int32_t orc_sample(const float *logits, int32_t n, const OrcParams *p, const int32_t *hist,
                           int32_t hcount, const int32_t *bias_ids, const float *bias_vals,
                           int32_t nbias, int sum_mode, double u, OrcTrace *tr, int32_t *cand_ids,
                           float *cand_vals, float *cand_probs, float *probs_out)
{
    OrcTrace local;
    if (!tr) tr = &local;
    memset(tr, 0, sizeof(*tr));
    if (hist == NULL) hcount = 0;
    if (p->temperature <= 0.f)
        return greedy_dispatch(logits, n, p, hist, hcount, &tr->path);

    int has_bias = nbias > 0;
    int has_penalty = hcount > 0 && (p->repetition_penalty != 1.0f || p->presence_penalty != 0.f ||
                                     p->frequency_penalty != 0.f);
    if (p->top_k > 0 && p->top_k < n && !has_bias)
        return sample_top_k(logits, n, p, hist, hcount, has_penalty, u, tr, cand_ids, cand_vals,
                            cand_probs);

    float *probs = (float *)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
    memcpy(probs, logits, sizeof(float) * (size_t)n);
    float cut_margin = INFINITY;
    slow_pipeline(probs, n, p, hist, hcount, bias_ids, bias_vals, nbias, sum_mode,
                  &tr->tie_at_cutoff, &cut_margin);
    tr->cut_margin = isinf(cut_margin) ? 0.f : cut_margin;
    tr->path = 3;
    int32_t nz = 0;
    for (int32_t i = 0; i < n; i++)
        if (probs[i] > 0.f) nz++;
    tr->n_cand = nz;
    tr->kept = nz;
    int32_t tok = sample_from_distribution(probs, n, u, tr);
    if (!tr->fallback) {
        float s = 0.f;
        for (int32_t i = 0; i < n; i++) s += probs[i];
        tr->kept_sum = s;
    }
    if (probs_out) memcpy(probs_out, probs, sizeof(float) * (size_t)n);
    free(probs);
    return tok;
}

/* ---- speculative decoding ---------------------------------------------------------------- */

/* ResampleResidual, Sampler.cs:587-618.  u[0] is the first NextDouble() the call draws, u[1] the
 * second (only consumed on the rounding fallback after a non-empty residual, or never);
 * *n_used reports how many were consumed. */
ORC_API int32_t orc_resample_residual(const float *p, const float *q, int32_t n, const double *u,
                                      int32_t *n_used, OrcTrace *tr)
{
    float sum = 0.f;
    for (int32_t i = 0; i < n; i++) {
        float r = p[i] - q[i];
        if (r > 0.f) sum += r;
    }
    if (sum <= 0.f || isnan(sum)) {
        if (n_used) *n_used = 1;
        return sample_from_distribution(p, n, u[0], tr);
    }
    float target = (float)u[0] * sum;
    float cum = 0.f;
    int32_t last_pos = -1;
    for (int32_t i = 0; i < n; i++) {
        float r = p[i] - q[i];
        if (r > 0.f) {
            float before = cum;
            last_pos = i;
            cum += r;
            if (target <= cum) {
                if (n_used) *n_used = 1;
                if (tr) {
                    float lo = target - before, hi = cum - target;
                    tr->margin = (lo < hi ? lo : hi) / sum;
                    tr->prob = r / sum;
                    tr->fallback = 0;
                    tr->kept_sum = sum;
                }
                return i;
            }
        }
    }
    if (last_pos >= 0) {
        if (n_used) *n_used = 1;
        if (tr) { tr->margin = 0.f; tr->fallback = 1; tr->kept_sum = sum; }
        return last_pos;
    }
    if (n_used) *n_used = 2;
    return sample_from_distribution(p, n, u[1], tr);
}

/* The accept/reject loop of SpeculativeDecoder.StepSampled, SpeculativeDecoder.cs:529-559, for
 * one sequence.  target rows: `n_draft + 1` rows of `n` logits (row i-1 predicts the slot draft
 * token i sits in; the last row is the bonus position); draft rows: `n_draft` rows, row i-1 being
 * the logits draft token i was drawn from.  Both distributions are built with the same params
 * (BuildFilteredDistribution).  `u_accept[i]` is the NextDouble() of test i; `u_final[0..1]` are
 * the draws of the correction/bonus.  mode 0 = distribution-preserving rule (:538-543),
 * mode 1 = looser accept `px >= p_min || token == Greedy(row)` (:544-547) with a draw from p on
 * rejection (:552).  Returns the accepted count; *correction receives the residual/bonus token;
 * margins[i] (may be NULL) = |u - a| of test i; *tr describes the final draw. */
ORC_API int32_t orc_spec_step_sampled(const float *target_rows, const float *draft_rows, int32_t n,
                                      int32_t n_draft, const int32_t *draft_tokens,
                                      const OrcParams *p, int sum_mode, const double *u_accept,
                                      const double *u_final, int32_t mode, float p_min,
                                      int32_t *correction, float *accept_prob, OrcTrace *tr)
{
    float *pd = (float *)malloc(sizeof(float) * (size_t)n);
    float *qd = (float *)malloc(sizeof(float) * (size_t)n);
    int32_t accepted = 0;
    int32_t corr = -1;
    for (int32_t i = 0; i < n_draft; i++) {
        const float *trow = target_rows + (size_t)i * (size_t)n;
        orc_build_filtered_distribution(trow, n, p, NULL, 0, NULL, NULL, 0, sum_mode, pd, NULL);
        int32_t tok = draft_tokens[i];
        float px = pd[tok];
        int accept;
        if (mode == 0) {
            const float *drow = draft_rows + (size_t)i * (size_t)n;
            orc_build_filtered_distribution(drow, n, p, NULL, 0, NULL, NULL, 0, sum_mode, qd, NULL);
            float qx = qd[tok];
            float a = qx > 0.f ? fminf(1.f, px / qx) : (px > 0.f ? 1.f : 0.f);
            if (accept_prob) accept_prob[i] = a;
            accept = u_accept[i] < (double)a;
        } else {
            if (accept_prob) accept_prob[i] = px;
            accept = px >= p_min || tok == orc_greedy(trow, n);
        }
        if (accept) { accepted++; continue; }
        if (mode == 0) {
            int32_t used = 0;
            corr = orc_resample_residual(pd, qd, n, u_final, &used, tr);
        } else {
            corr = sample_from_distribution(pd, n, u_final[0], tr);
        }
        break;
    }
    if (corr < 0) {
        const float *brow = target_rows + (size_t)n_draft * (size_t)n;
        corr = orc_sample_with_distribution(brow, n, p, NULL, 0, sum_mode, u_final[0], pd, tr);
    }
    *correction = corr;
    free(pd); free(qd);
    return accepted;
}

/* Greedy accept of SpeculativeDecoder.Step, SpeculativeDecoder.cs:400-405 (DSparkDecoder.cs
 * :224-237 has the same shape): count the leading draft tokens that equal the target argmax.
 * `rows` = n_draft rows of n logits, row i predicting draft token i. */
ORC_API int32_t orc_spec_greedy_accept(const float *rows, int32_t n, int32_t n_draft,
                                       const int32_t *draft_tokens)
{
    int32_t accepted = 0;
    for (int32_t i = 0; i < n_draft; i++) {
        if (orc_greedy(rows + (size_t)i * (size_t)n, n) == draft_tokens[i]) accepted++;
        else break;
    }
    return accepted;
}

/* SoftmaxProbAt, MtpDecoder.cs:584-596: fp64 accumulation in index order. */
ORC_API float orc_softmax_prob_at(const float *logits, int32_t n, int32_t idx)
{
    float max = logits[0];
    for (int32_t i = 1; i < n; i++)
        if (logits[i] > max) max = logits[i];
    double sum = 0.0;
    for (int32_t i = 0; i < n; i++) sum += exp((double)(logits[i] - max));
    if (sum <= 0 || isnan(sum)) return 0.f;
    return (float)(exp((double)(logits[idx] - max)) / sum);
}

/* AcceptDraft, MtpDecoder.cs:562-577 (p_min <= 0 is treated as 1, MtpDecoder.cs:225). */
ORC_API int32_t orc_mtp_accept(const float *logits, int32_t n, int32_t draft, float p_min,
                               float *draft_prob)
{
    if (p_min <= 0.f) p_min = 1.f;
    int32_t target = orc_greedy(logits, n);
    if (draft == target) { if (draft_prob) *draft_prob = 0.f; return 1; }
    if (p_min >= 1.0f) { if (draft_prob) *draft_prob = 0.f; return 0; }
    float pr = orc_softmax_prob_at(logits, n, draft);
    if (draft_prob) *draft_prob = pr;
    return pr >= p_min;
}

/* ---- masks ------------------------------------------------------------------------------- */

/* The ITokenConstraint.Filter contract (Core/Grammar/ITokenConstraint.cs:31-43) in bitmask form:
 * bit i of word i>>5 (LSB first) set <=> token i is left untouched; clear <=> -infinity.
 * TokenChoiceTrie.MaskLogits (Engine/ChoiceConstraint.cs:83-104) has the same effect. */
ORC_API void orc_apply_mask(float *logits, int32_t n, const uint32_t *mask)
{
    for (int32_t i = 0; i < n; i++)
        if (!((mask[i >> 5] >> (i & 31)) & 1u)) logits[i] = NEG_INF;
}

/* AndTokenConstraint.Filter, Core/Grammar/AndTokenConstraint.cs:44-86: intersection of the
 * constraining inners; an inner in a dead state (all bits clear) is skipped; an empty
 * intersection falls back to "unmasked" (all bits set).  Returns 1 when the result masks. */
ORC_API int32_t orc_and_masks(const uint32_t *const *masks, int32_t n_masks, int32_t n,
                              uint32_t *out)
{
    int32_t words = (n + 31) / 32;
    uint32_t tail = (n & 31) ? ((1u << (n & 31)) - 1u) : 0xFFFFFFFFu;
    for (int32_t w = 0; w < words; w++) out[w] = 0xFFFFFFFFu;
    int any = 0;
    for (int32_t m = 0; m < n_masks; m++) {
        uint32_t nonzero = 0;
        for (int32_t w = 0; w < words; w++) nonzero |= masks[m][w] & (w == words - 1 ? tail : 0xFFFFFFFFu);
        if (!nonzero) continue; /* dead inner: skipped */
        any = 1;
        for (int32_t w = 0; w < words; w++) out[w] &= masks[m][w];
    }
    uint32_t legal = 0;
    for (int32_t w = 0; w < words; w++) legal |= out[w] & (w == words - 1 ? tail : 0xFFFFFFFFu);
    if (!any || !legal) {
        for (int32_t w = 0; w < words; w++) out[w] = 0xFFFFFFFFu;
        return 0;
    }
    return 1;
}

/* bf16 -> fp32 is an exact widening (the reference has fp32 logits only; a bf16 row is widened
 * and then follows the fp32 rules). */
ORC_API void orc_widen_bf16(const uint16_t *src, int32_t n, float *dst)
{
    for (int32_t i = 0; i < n; i++) {
        uint32_t b = (uint32_t)src[i] << 16;
        memcpy(&dst[i], &b, 4);
    }
}

/* ---- batched drivers (what the reference's serial per-row loop does,
 * ContinuousBatchingEngine.cs:609-644): used by the parity tests and by the CPU baseline. ---- */

ORC_API void orc_sample_rows(const void *logits, int32_t dtype_bf16, int32_t rows, int32_t n,
                             int64_t row_stride, const OrcParams *params, const int32_t *hist_ids,
                             const int32_t *hist_offsets, const uint32_t *mask,
                             int64_t mask_stride_words, const double *uniforms, int sum_mode,
                             int32_t *tokens, OrcTrace *traces)
{
    float *row = (float *)malloc(sizeof(float) * (size_t)n);
    for (int32_t r = 0; r < rows; r++) {
        if (dtype_bf16)
            orc_widen_bf16((const uint16_t *)logits + (size_t)r * (size_t)row_stride, n, row);
        else
            memcpy(row, (const float *)logits + (size_t)r * (size_t)row_stride,
                   sizeof(float) * (size_t)n);
        if (mask) orc_apply_mask(row, n, mask + (size_t)r * (size_t)mask_stride_words);
        const int32_t *h = NULL;
        int32_t hc = 0;
        if (hist_ids && hist_offsets) {
            h = hist_ids + hist_offsets[r];
            hc = hist_offsets[r + 1] - hist_offsets[r];
        }
        tokens[r] = orc_sample(row, n, &params[r], h, hc, NULL, NULL, 0, sum_mode,
                               uniforms ? uniforms[r] : 0.5, traces ? &traces[r] : NULL, NULL,
                               NULL, NULL, NULL);
    }
    free(row);
}

ORC_API int32_t orc_abi_version(void) { return 1; }
