/*
 * stingray_sampler.h - C ABI of the B200 (sm_100a) token-sampling library.
 *
 * The library replaces, for batched [rows, vocab] logits that already live in device memory, the
 * managed per-row loop of the reference host:
 *     Filter -> Sampler.Greedy | Sampler.Sample -> (speculative accept / residual resampling)
 * Each entry point below names the reference interface it stands in for (paths are relative to
 * the reference project's root).
 *
 * Binding conventions follow the reference's own native bindings
 * (src/OpenTail.Stingray.Cuda/CuBlasInterop.cs:37-41, NvrtcInterop.cs:371-380): every call returns
 * an int status with 0 = success, handles and device pointers are pointer-sized integers created
 * through an out parameter, structs are sequential-layout PODs, strings are UTF-8 copied into a
 * caller buffer.  No C++ or framework types cross this boundary.
 *
 * Threading: a handle is not re-entrant (the reference drives the backend from one batcher
 * thread, src/OpenTail.Stingray.Engine/ContinuousBatchingEngine.cs:495-500); distinct handles are
 * independent.  Work is enqueued on the caller's stream; a call blocks only when it has to hand
 * results back in host memory (STG_MEM_HOST_OUTPUTS) or is documented as blocking.
 *
 * Streams: the workspace belongs to the handle, so the sampling calls of one handle run one after
 * the other on the device.  On a single stream that is the stream's own order; a call on a different
 * stream than the previous one is put behind everything enqueued on the previous stream so far (an
 * event, no host wait), which must therefore still exist.  Inputs and outputs follow the usual
 * rule: they must be ready on, and are ready after, the stream of the call that uses them.
 *
 * Repeated steps: a decode loop calls stg_sample_batch with the same buffers and the same per-row
 * parameters step after step, only the contents of the buffers change.  The second time the library
 * sees such a call on a stream that can be captured (any stream but the legacy default stream, which
 * CUDA cannot capture) it records the step's launches - a dozen kernels on three streams - as a CUDA
 * graph, and from then on submits the step as one graph launch.  Nothing changes for the caller;
 * StgStats.graph_replays counts those steps, and STG_NO_GRAPH=1 in the environment at stg_create turns
 * the mechanism off.  Steps with host-memory inputs are never captured.
 */
#ifndef STINGRAY_SAMPLER_H
#define STINGRAY_SAMPLER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define STG_API __declspec(dllexport)
#else
#define STG_API __attribute__((visibility("default")))
#endif

#define STG_ABI_VERSION 2

/* ---- status codes --------------------------------------------------------------------------- */
enum {
    STG_OK = 0,
    STG_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, size beyond the handle's limits */
    STG_ERR_CUDA = 2,             /* a CUDA runtime call failed; stg_last_error has the text */
    STG_ERR_CAPACITY = 3,         /* request exceeds the capacities given at stg_create */
    STG_ERR_UNSUPPORTED = 4,      /* combination of options this build does not implement */
    STG_ERR_TIMEOUT = 5,          /* a bounded device-side wait gave up */
    STG_ERR_NCCL = 6,             /* NCCL could not be loaded or a collective failed */
    STG_ERR_NO_DEVICE = 7         /* no usable CUDA device: there is no CPU fallback */
};

/* ---- element types of a logits buffer --------------------------------------------------------- */
enum {
    STG_DTYPE_F32 = 0,
    STG_DTYPE_BF16 = 1 /* widened exactly to fp32 on load; the reference has fp32 logits only */
};

/* ---- where a caller array lives (bit set = host memory) ------------------------------------- */
enum {
    STG_MEM_HOST_LOGITS = 1u << 0,
    STG_MEM_HOST_HISTORY = 1u << 1,  /* history_ids */
    STG_MEM_HOST_MASK = 1u << 2,
    STG_MEM_HOST_BIAS = 1u << 3,     /* bias_ids, bias_values */
    STG_MEM_HOST_UNIFORMS = 1u << 4,
    STG_MEM_HOST_OUTPUTS = 1u << 5,  /* every output array; makes the call blocking */
    STG_MEM_HOST_DRAFT = 1u << 6,    /* stg_spec_verify: draft_tokens */
    STG_MEM_HISTORY_RING = 1u << 7   /* StgSampleBatch: row r's PreviousTokens are the handle's device-resident
                                        history of slot r (stg_history_*); history_ids / history_offsets
                                        are ignored */
};

/* ---- per-row flags written to StgSampleBatch.row_flags -------------------------------------- */
enum {
    STG_ROW_PATH_MASK = 0x7u,        /* 0 greedy, 1 greedy with penalties, 2 top-k path,
                                        3 full-vocabulary path, 4 top-k path found no finite logit */
    STG_ROW_NEAR_BOUNDARY = 1u << 3, /* the draw lies within 1e-6 (of the kept mass) of the step of the running
                                        sum below or above the sampled token: another exp or summation
                                        order could have returned the neighbouring token */
    STG_ROW_TIE_AT_CUTOFF = 1u << 4, /* the top-p cut fell inside a group of equal probabilities */
    STG_ROW_CDF_FALLBACK = 1u << 5,  /* the draw ran past the end of the CDF (rounding fallback) */
    STG_ROW_FULLY_MASKED = 1u << 6,  /* no finite logit in the row */
    STG_ROW_WIDE_NUCLEUS = 1u << 7,  /* top-p candidates did not fit on chip; global-memory sort */
    STG_ROW_READ_TWICE = 1u << 8,    /* an optimistic bound failed its check and the row was processed a second
                                        time: the filter bound of a top-k row, or the nucleus bound of a
                                        full-vocabulary row */
    STG_ROW_NEAR_CUT = 1u << 10      /* full-vocabulary path: the sorted running sum of top-p passes top_p within
                                        1e-6, so a last-bit difference in exp could move the cut by a token */
};

/* ---- per-sequence flags written to StgSpecBatch.seq_flags (STG_ROW_CDF_FALLBACK applies too) --- */
enum {
    STG_SEQ_EMPTY_RESIDUAL = 1u << 8, /* max(p - q, 0) summed to nothing: the correction was drawn from p
                                         with the second spare uniform (Sampler.cs:598-599) */
    STG_SEQ_BAD_DRAFT = 1u << 9       /* a draft token lay outside [0, vocab): it was rejected unread (the
                                         reference throws there, SpeculativeDecoder.cs:534) */
};

/* ---- StgConfig.flags ---------------------------------------------------------------------------- */
enum {
    STG_CFG_HOST_LOGITS = 1u << 0,   /* reserve device staging for max_rows x max_vocab fp32 logits and the
                                        matching mask words at stg_create, so that calls with
                                        STG_MEM_HOST_LOGITS / STG_MEM_HOST_MASK never allocate; without
                                        it that staging grows on the first such call (which then
                                        synchronises the stream once) */
};

typedef struct StgSampler_ *StgHandle;

/* Capacities fixed at creation; all device workspace is allocated once from them, so that no
 * entry point allocates on the per-step path (the reference's own rule for this path,
 * src/OpenTail.Stingray.Core/Grammar/ITokenConstraint.cs:22-23). */
typedef struct StgConfig {
    int32_t struct_size;  /* = sizeof(StgConfig) */
    int32_t device;       /* CUDA device ordinal */
    int32_t max_rows;     /* rows per call */
    int32_t max_vocab;    /* vocabulary size per row */
    int32_t max_history;  /* history entries per row; max_top_k + max_history <= 8192 */
    int32_t max_top_k;
    int32_t max_bias;     /* logit-bias entries per row */
    int32_t max_spec_draft; /* draft length of stg_spec_verify (0 = entry point unused) */
    uint32_t flags;       /* STG_CFG_* */
    int32_t max_cached_masks; /* entries of the device-resident bitmask cache (stg_mask_cache_*), each
                                 (max_vocab + 31) / 32 words; 0 = no cache */
} StgConfig;

/* SamplingParams of the reference (src/OpenTail.Stingray.Engine/Sampler.cs:648-686), the fields
 * the sampler reads.  Defaults there: temperature 1, top_k 0 (off), top_p 1 (off), min_p 0 (off),
 * repetition_penalty 1 (off), repeat_last_n 64 (0 = whole history), penalties 0. */
typedef struct StgRowParams {
    float temperature;
    float top_p;
    float min_p;
    float repetition_penalty;
    float presence_penalty;
    float frequency_penalty;
    int32_t top_k;
    int32_t repeat_last_n;
} StgRowParams;

/* One batched sampling step.  `params`, `history_offsets` and `bias_offsets` are always HOST
 * arrays (they are what the managed host builds per step, ContinuousBatchingEngine.cs:638-640);
 * the location of every other array is given by `mem_flags` (bit clear = device memory). */
typedef struct StgSampleBatch {
    int32_t struct_size;            /* = sizeof(StgSampleBatch) */
    int32_t rows;
    int32_t vocab;
    int32_t logits_dtype;           /* STG_DTYPE_* */
    const void *logits;             /* [rows, row_stride] */
    int64_t row_stride;             /* elements between rows (>= vocab) */
    const StgRowParams *params;     /* host [rows] */
    const int32_t *history_ids;     /* CSR values: PreviousTokens of each row, oldest first */
    const int32_t *history_offsets; /* host [rows + 1], or NULL: no row has a history */
    const uint32_t *mask;           /* allowed-token bitmask [rows, mask_row_stride] or NULL:
                                       bit (i & 31) of word (i >> 5) set <=> token i untouched,
                                       clear <=> -infinity (ITokenConstraint.Filter contract,
                                       ITokenConstraint.cs:31-43) */
    int64_t mask_row_stride;        /* 32-bit words between mask rows */
    const uint8_t *row_uses_mask;   /* host [rows] or NULL (= every row when mask != NULL):
                                       0 = this row is unconstrained (IsConstraining false) */
    const int32_t *bias_ids;        /* CSR values of LogitBias (Sampler.cs:50-56) */
    const float *bias_values;
    const int32_t *bias_offsets;    /* host [rows + 1] or NULL */
    const float *uniforms;          /* [rows]: (float)rng.NextDouble() of each non-greedy row */
    int32_t *tokens;                /* out [rows] */
    float *token_probs;             /* out [rows] or NULL: normalised probability of the token */
    uint32_t *row_flags;            /* out [rows] or NULL: STG_ROW_* */
    int32_t *topk_ids;              /* out [rows, topk_stride] or NULL: candidates of the top-k
                                       path after the penalty re-sort (-1 = unused slot) */
    float *topk_logits;             /* out, same shape or NULL: their penalised logits */
    float *topk_probs;              /* out, same shape or NULL: softmax over the k candidates */
    int32_t topk_stride;            /* >= the largest top_k of any row on the top-k path when a topk_*
                                       output is given (STG_ERR_INVALID_ARGUMENT otherwise) */
    uint32_t mem_flags;             /* STG_MEM_HOST_* */
    float logit_softcap;            /* != 0: every logit is read as tanh(x / cap) * cap, the final-logit
                                       soft cap the reference applies in place before it samples
                                       (llm_softcap_inplace, src/OpenTail.Stingray.Cuda/CudaTextKernels.cs:374-383;
                                       SimdKernels.SoftcapInPlace on the CPU); 0: logits as given */
} StgSampleBatch;

/* One speculative verification step over `n_seq` sequences with `n_draft` draft tokens each
 * (SpeculativeDecoder.StepSampled, src/OpenTail.Stingray.Engine/SpeculativeDecoder.cs:529-559).
 * target_logits: [n_seq, n_draft + 1, vocab] (row i predicts the slot of draft token i, the last
 * row is the bonus position); draft_logits: [n_seq, n_draft, vocab] (row i is what draft token i
 * was drawn from); both built into distributions with the same `params`. */
typedef struct StgSpecBatch {
    int32_t struct_size;
    int32_t n_seq;
    int32_t n_draft;
    int32_t vocab;
    int32_t logits_dtype;
    int32_t mode;                   /* 0: accept with min(1, p/q), residual resampling;
                                       1: looser accept p >= p_min || draft == argmax, draw from p */
    const void *target_logits;
    const void *draft_logits;       /* may be NULL when mode == 1 */
    const int32_t *draft_tokens;    /* [n_seq, n_draft]; ids outside [0, vocab) are an error when the
                                       array is in host memory and are rejected with STG_SEQ_BAD_DRAFT
                                       when it is in device memory */
    const StgRowParams *params;     /* host [n_seq]; histories and bias do not apply here (the
                                       reference turns speculation off when they are set,
                                       src/OpenTail.Stingray.Cli/RunCommand.cs:1651-1678) */
    const double *uniforms;         /* [n_seq, n_draft + 2]: rng.NextDouble() of each accept test,
                                       then the two draws the correction/bonus may consume */
    float p_min;                    /* SpecDraftPMin for mode 1 */
    int32_t *accepted;              /* out [n_seq]: number of accepted draft tokens */
    int32_t *correction;            /* out [n_seq]: residual / bonus token */
    float *accept_probs;            /* out [n_seq, n_draft] or NULL: the ratio a (mode 0) or p(x) */
    uint32_t *seq_flags;            /* out [n_seq] or NULL: STG_ROW_CDF_FALLBACK etc. */
    uint32_t mem_flags;             /* STG_MEM_HOST_LOGITS | _DRAFT | _UNIFORMS | _OUTPUTS */
    float target_softcap;           /* soft caps of the two models' logits, as StgSampleBatch.logit_softcap */
    float draft_softcap;
} StgSpecBatch;

typedef struct StgStats {
    uint64_t calls;
    uint64_t rows_sampled;
    uint64_t rows_greedy;
    uint64_t rows_topk_path;
    uint64_t rows_full_path;
    uint64_t sequences_verified;
    uint64_t kernel_launches;
    uint64_t plan_uploads;
    /* events counted on the device where a row's flags are written (stg_get_stats waits for the work
     * enqueued so far to read them) */
    uint64_t boundary_draws;     /* rows flagged STG_ROW_NEAR_BOUNDARY */
    uint64_t tie_rows;           /* STG_ROW_TIE_AT_CUTOFF */
    uint64_t cdf_fallbacks;      /* STG_ROW_CDF_FALLBACK */
    uint64_t wide_nucleus_rows;  /* STG_ROW_WIDE_NUCLEUS */
    uint64_t reread_rows;        /* STG_ROW_READ_TWICE */
    uint64_t near_cut_rows;      /* STG_ROW_NEAR_CUT */
    uint64_t fully_masked_rows;  /* STG_ROW_FULLY_MASKED on a sampled row */
    uint64_t graph_replays;      /* sampling steps submitted as one replay of a captured CUDA graph */
} StgStats;

/* ---- lifetime ---------------------------------------------------------------------------------- */

/* Allocates the workspace on `config->device`.  There is no counterpart in the reference (its
 * sampler is managed code); the shape follows cublasCreate_v2's, CuBlasInterop.cs:37-38.
 * Returns STG_ERR_NO_DEVICE when no CUDA device can be used: nothing falls back to the CPU. */
STG_API int stg_create(const StgConfig *config, StgHandle *out_handle);
STG_API int stg_destroy(StgHandle handle);
STG_API int stg_abi_version(void);

/* Copies the NUL-terminated text of the last failure on `handle` (or of the last stg_create
 * failure when handle is NULL) into buf; returns the length needed, like
 * nvrtcGetProgramLogSize + nvrtcGetProgramLog (NvrtcInterop.cs:268-272). */
STG_API size_t stg_last_error(StgHandle handle, char *buf, size_t buf_len);
STG_API int stg_get_stats(StgHandle handle, StgStats *out);
/* Diagnostic: per work item of the last sampling step, 32 device time stamps (nanoseconds) taken at
 * the boundaries of its phases.  Only recorded when the handle was created with STG_PHASE_TICKS=1
 * in the environment; blocks.  The reference's counterpart is its env-gated Stopwatch buckets
 * (src/OpenTail.Stingray.Engine/DecodeProfileTimers.cs:17-67). */
STG_API int stg_debug_phase_ticks(StgHandle handle, uint64_t *out, int32_t max_items, int32_t *n_items);

/* Checked handles: a handle created while the environment variable STG_CHECKED=1 is set puts 256
 * guard bytes of a fixed pattern behind every device buffer it owns.  This call waits for the device
 * and reads them back: n_guarded = buffers checked (0 for an unchecked handle), first_bad = index of
 * the first buffer whose guard was overwritten, or -1.  The stand-in for a memory checker where none
 * can be run. */
STG_API int stg_debug_check_guards(StgHandle handle, int32_t *n_guarded, int32_t *first_bad);

/* Diagnostic: device time (microseconds) between the kernels of the last sampling step on the caller's
 * stream, measured with CUDA events, and their names (max_items strings of name_len bytes).  Only
 * recorded when the handle was created with STG_KERNEL_TIMES=1 in the environment; blocks. */
STG_API int stg_debug_kernel_times(StgHandle handle, float *out_us, char *names, int32_t name_len,
                                   int32_t max_items, int32_t *n_items);

/* ---- the hot path ------------------------------------------------------------------------------- */

/* Per-row greedy argmax over device logits [rows, row_stride], valid length `vocab`.
 * Replaces CudaBackend.ArgmaxRowsToDevice / ArgmaxRows (src/OpenTail.Stingray.Cuda/
 * CudaBackend.cs:4141-4190) and the kernel llm_argmax_rows (CudaTextKernels.cs:465-492): out_pairs
 * holds rows x {int32 index bits, float value}; the highest value wins, the lowest index on ties
 * (Sampler.Greedy, Sampler.cs:442-446). */
STG_API int stg_argmax_rows(StgHandle handle, const void *logits, int32_t logits_dtype,
                            int32_t rows, int32_t vocab, int64_t row_stride, void *out_pairs,
                            void *stream);

/* The same arg-max for callers that cannot allocate device memory where they need it (inside
 * another component's stream capture, behind a plug-in interface that hands over a stream but no
 * allocator, under a memory budget fixed at start-up).  It has no counterpart in the reference.
 * It takes no handle and allocates nothing: its scratch is a fixed array inside the library's
 * device image (about 1 MiB per GPU that loads the library, held until exit), so at most
 * STG_STATIC_MAX_ROWS rows per call are accepted (STG_ERR_CAPACITY beyond).  The first call on a
 * device looks up that array's device address, so make one call before any stream capture starts.
 * All calls on a device share the scratch: calls whose kernels could overlap on the GPU must be
 * ordered (same stream, or events).  Uses the current device; arrays are device pointers. */
#define STG_STATIC_MAX_ROWS 4096
STG_API int stg_argmax_rows_static(const void *logits, int32_t logits_dtype, int32_t rows,
                                   int32_t vocab, int64_t row_stride, void *out_pairs, void *stream);

/* One sampling step for every row of the batch: mask, logit bias, history penalties, temperature,
 * top-k, min-p, top-p and the inverse-CDF draw.  Replaces the serial loop
 *   ctr.Filter(row) -> Sampler.Greedy(row) | Sampler.Sample(row, spWithHistory, seq.Rng)
 * of ContinuousBatchingEngine.cs:609-644 (and InferenceEngine.cs:1245-1253,
 * InferenceSession.cs:494-510) after the logits download it makes unnecessary
 * (CudaForwardPass.cs:5209-5217).  Row r consumes uniforms[r] only when its temperature > 0. */
STG_API int stg_sample_rows(StgHandle handle, const StgSampleBatch *batch, void *stream);

/* Materialises the post-filter distribution of each row into `probs` [rows, vocab] (device, or
 * host with STG_MEM_HOST_OUTPUTS): Sampler.BuildFilteredDistribution, Sampler.cs:118-163.  Uses
 * the same batch description; `uniforms`, `tokens` and the top-k outputs are ignored. */
STG_API int stg_build_distribution(StgHandle handle, const StgSampleBatch *batch, float *probs,
                                   void *stream);

/* Sampler.SampleWithDistribution (Sampler.cs:172-187), called once per draft token by the speculative
 * decoder (src/OpenTail.Stingray.Engine/SpeculativeDecoder.cs:509-513): builds the post-filter
 * distribution of every row with the full-vocabulary pipeline whatever top_k is (the top-k fast path
 * of Sampler.Sample rounds differently and is never taken here), stores it in `probs` [rows, vocab]
 * (device memory, or NULL when only the tokens are wanted) and draws the row's token from it with
 * uniforms[r].  temperature <= 0 rows return the greedy arg-max and a one-hot row. */
STG_API int stg_sample_with_distribution(StgHandle handle, const StgSampleBatch *batch, float *probs,
                                         void *stream);

/* Sampler.SampleFromProbs (Sampler.cs:195-199, :564-576) on caller-held distributions: for each row
 * the first token whose sequential fp32 running sum reaches (float)uniforms[r], the last token when
 * rounding leaves the sum short (STG_ROW_CDF_FALLBACK).  probs: device [rows, row_stride] fp32;
 * uniforms and tokens follow mem_flags (STG_MEM_HOST_UNIFORMS, STG_MEM_HOST_OUTPUTS); row_flags may
 * be NULL. */
STG_API int stg_sample_from_probs(StgHandle handle, const float *probs, int32_t rows, int32_t vocab,
                                  int64_t row_stride, const float *uniforms, int32_t *tokens,
                                  uint32_t *row_flags, uint32_t mem_flags, void *stream);

/* Sampler.ResampleResidual (Sampler.cs:587-618) on caller-held distributions p and q (device
 * [rows, row_stride] fp32 each): a token drawn in proportion to max(p - q, 0) with uniforms[2r];
 * an empty residual falls back to a draw from p with the same uniform (STG_SEQ_EMPTY_RESIDUAL); the
 * rounding fallback is the last token with a positive residual (STG_ROW_CDF_FALLBACK), and only if
 * there is none a draw from p with uniforms[2r + 1].  uniforms is [rows, 2]. */
STG_API int stg_resample_residual(StgHandle handle, const float *p, const float *q, int32_t rows,
                                  int32_t vocab, int64_t row_stride, const float *uniforms,
                                  int32_t *tokens, uint32_t *row_flags, uint32_t mem_flags, void *stream);

/* Speculative accept / reject with residual resampling for a batch of sequences: the loop of
 * SpeculativeDecoder.StepSampled (SpeculativeDecoder.cs:529-559) with Sampler.ResampleResidual
 * (Sampler.cs:587-618) and the bonus draw.  temperature <= 0 rows use the greedy accept of
 * SpeculativeDecoder.Step (SpeculativeDecoder.cs:400-405): `correction` is then the target
 * argmax at the first mismatch (or at the bonus position). */
STG_API int stg_spec_verify(StgHandle handle, const StgSpecBatch *batch, void *stream);

/* MTP verification rule for `rows` rows: accept iff draft == argmax(row) or (p_min < 1 and
 * softmax(row)[draft] >= p_min), the softmax accumulated in double: MtpDecoder.AcceptDraft +
 * SoftmaxProbAt, src/OpenTail.Stingray.Engine/MtpDecoder.cs:562-596.  Device arrays; accept is
 * int32 [rows], argmax int32 [rows] or NULL, draft_prob float [rows] or NULL. */
STG_API int stg_mtp_accept(StgHandle handle, const void *logits, int32_t logits_dtype, int32_t rows,
                           int32_t vocab, int64_t row_stride, const int32_t *draft_tokens,
                           float p_min, int32_t *accept, int32_t *argmax, float *draft_prob,
                           void *stream);

/* Composes the allowed-token bitmasks of several constraints of each row into one: the AND of the
 * inners' words, AndTokenConstraint.Filter (src/OpenTail.Stingray.Core/Grammar/
 * AndTokenConstraint.cs:44-86).  masks: device [n_masks, rows, mask_row_stride] words (n_masks <=
 * 32), same bit convention as StgSampleBatch.mask.  An inner that allows nothing is skipped; when
 * no inner constrains, or the intersection is empty, the row comes out as all ones (= unmasked)
 * and out_uses_mask[row] (device uint8 [rows], may be NULL) is 0, else 1.  The result can be passed
 * as StgSampleBatch.mask as it is. */
STG_API int stg_and_masks(StgHandle handle, const uint32_t *masks, int32_t n_masks, int32_t rows,
                          int32_t vocab, int64_t mask_row_stride, uint32_t *out,
                          int64_t out_row_stride, uint8_t *out_uses_mask, void *stream);

/* ---- bitmask cache ---------------------------------------------------------------------------------
 * The reference's schema and tool-argument constraints rebuild a row's allowed-token set with a walk
 * over the whole vocabulary on every step (JsonSchemaGrammarMasker.Filter,
 * src/OpenTail.Stingray.Core/Grammar/JsonSchemaGrammarMasker.cs:67-95), although the set depends
 * only on the constraint and its automaton state.  The cache keeps such sets on the device as
 * bitmasks under a caller-chosen 64-bit key (for instance constraint id << 32 | state id; 0 is
 * reserved for "no constraint in this slot"), so that a state seen before costs no walk and no
 * host-to-device copy, and composes the masks of each row of a step with word operations. */
enum { STG_MASK_AND = 0, STG_MASK_OR = 1 };

/* Stores the (vocab + 31) / 32 words at `words` (host memory; bit convention of StgSampleBatch.mask)
 * under `key`, replacing an entry of that key or, when the cache is full, the entry least recently
 * put or composed.  The copy is enqueued on `stream`; compositions that should see it, or that still
 * read the entry it replaces, must be ordered with it by the caller (use one stream). */
STG_API int stg_mask_cache_put(StgHandle handle, uint64_t key, const uint32_t *words, int32_t vocab,
                               void *stream);
/* 1 when `key` is cached, else 0 (never an error code; a null handle answers 0). */
STG_API int stg_mask_cache_contains(StgHandle handle, uint64_t key);
/* Writes out[row] = the composition of the cached masks keys[row * keys_per_row + 0 .. keys_per_row)
 * (host array; key 0 = empty slot), ready to be passed as StgSampleBatch.mask.  STG_MASK_AND is
 * AndTokenConstraint.Filter (AndTokenConstraint.cs:44-86) exactly as stg_and_masks states it;
 * STG_MASK_OR allows a token when any inner that allows something allows it (alternatives of a
 * grammar; the engaged branch of CompositeToolArgumentConstraint.cs:43-48 is the one-key case).  A
 * row without usable inners comes out all ones with out_uses_mask[row] = 0.  keys_per_row <= 32; a
 * key that is not cached is STG_ERR_INVALID_ARGUMENT, and nothing is written. */
STG_API int stg_mask_compose(StgHandle handle, const uint64_t *keys, int32_t keys_per_row, int32_t rows,
                             int32_t vocab, int32_t op, uint32_t *out, int64_t out_row_stride,
                             uint8_t *out_uses_mask, void *stream);

/* ---- device-resident token histories -------------------------------------------------------------
 * The reference keeps each sequence's PreviousTokens on the host and hands the sampler a fresh list
 * every step (ContinuousBatchingEngine.cs:650, :1280).  Here the handle owns max_rows histories of up
 * to max_history tokens in device memory; a step samples against them with STG_MEM_HISTORY_RING in
 * StgSampleBatch.mem_flags (batch row r = slot r) and appends its own output with
 * stg_history_append, so a decode loop moves no history bytes between host and device.  A full
 * history drops its oldest token on append; from then on the slot serves only rows that cannot
 * tell: no penalty set, or a repetition penalty alone whose repeat_last_n window (1 .. max_history)
 * lies inside what is kept (Sampler.cs:364-375: the repetition penalty sees the trailing window,
 * presence and frequency penalties the whole history).  Any other row is refused with
 * STG_ERR_CAPACITY.  The host keeps the
 * lengths (they shape the step's plan), so nothing here reads the device back. */
/* Empties the histories of slots [first_slot, first_slot + n_slots). */
STG_API int stg_history_reset(StgHandle handle, int32_t first_slot, int32_t n_slots, void *stream);
/* Replaces slot's history by tokens[0 .. n) (host memory, oldest first; n <= max_history). */
STG_API int stg_history_load(StgHandle handle, int32_t slot, const int32_t *tokens, int32_t n, void *stream);
/* Appends tokens[r] (device int32 [rows], typically StgSampleBatch.tokens of the step just enqueued
 * on the same stream) to slot r for every r < rows whose active[r] != 0 (host uint8 [rows], or NULL:
 * every row). */
STG_API int stg_history_append(StgHandle handle, const int32_t *tokens, int32_t rows, const uint8_t *active,
                               void *stream);
/* Tokens slot holds now, or a negative STG_ERR_* code. */
STG_API int stg_history_length(StgHandle handle, int32_t slot);

/* ---- vocabulary-sharded mode (no counterpart in the reference, which is single-device:
 *      src/OpenTail.Stingray.Cli/RunCommand.cs:100) ------------------------------------------------
 * Each rank holds the column slice [vocab_offset, vocab_offset + batch->vocab) of every row, the
 * layout a tensor-parallel lm-head leaves behind.  stg_shard_select picks, per row, the local
 * candidates of the top-k path (batch->vocab is the slice width, history ids are global token
 * ids) into the handle's exchange buffer; stg_shard_allgather exchanges them between ranks with
 * ONE ncclAllGather per step; stg_shard_finish merges the gathered candidates and finishes the sampling
 * chain.  Only rows on the top-k path or greedy rows without penalties are supported; other rows
 * return STG_ERR_UNSUPPORTED (use row sharding for those). */
STG_API int stg_comm_unique_id(void *out_id128); /* 128 bytes; call on rank 0, then broadcast */
STG_API int stg_comm_init(StgHandle handle, const void *id128, int32_t rank, int32_t n_ranks);
STG_API int stg_comm_destroy(StgHandle handle);
STG_API int stg_shard_select(StgHandle handle, const StgSampleBatch *batch, int32_t vocab_offset,
                             int32_t global_vocab, void *stream);
STG_API int stg_shard_allgather(StgHandle handle, void *stream);
/* Bytes this rank contributes to the all-gather of the step last selected (keys and counts of
 * every row in one block, sized by the step's largest selection count). */
STG_API int stg_shard_exchange_bytes(StgHandle handle, uint64_t *out_bytes);
STG_API int stg_shard_finish(StgHandle handle, const StgSampleBatch *batch, int32_t global_vocab,
                             void *stream);
/* Single-process variant of the exchange for tests: copies `n_ranks` handles' local candidate
 * buffers (all on the same device) into `handle`'s gather buffer as the all-gather would. */
STG_API int stg_shard_gather_local(StgHandle handle, const StgHandle *peers, int32_t n_ranks,
                                   void *stream);

#ifdef __cplusplus
}
#endif
#endif /* STINGRAY_SAMPLER_H */
