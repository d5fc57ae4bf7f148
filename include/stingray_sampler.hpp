// C++ convenience layer over stingray_sampler.h: an owning handle, exceptions instead of status
// codes, and the reference's SamplingParams defaults (src/OpenTail.Stingray.Engine/Sampler.cs:648-686).
// Header-only; link against libstingray_sampler.so.
#ifndef STINGRAY_SAMPLER_HPP
#define STINGRAY_SAMPLER_HPP

#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "stingray_sampler.h"

namespace stingray {

class Error : public std::runtime_error {
public:
    Error(int status, const std::string &what) : std::runtime_error(what), status_(status) {}
    int status() const noexcept { return status_; }

private:
    int status_;
};

// SamplingParams with the reference's defaults: temperature 1, filters off, RepeatLastN 64.
inline StgRowParams default_params()
{
    StgRowParams p{};
    p.temperature = 1.0f;
    p.top_p = 1.0f;
    p.min_p = 0.0f;
    p.repetition_penalty = 1.0f;
    p.presence_penalty = 0.0f;
    p.frequency_penalty = 0.0f;
    p.top_k = 0;
    p.repeat_last_n = 64;
    return p;
}

// SamplingParams.HasHistoryPenalty, Sampler.cs:686
inline bool has_history_penalty(const StgRowParams &p)
{
    return p.repetition_penalty != 1.0f || p.presence_penalty != 0.0f || p.frequency_penalty != 0.0f;
}

class BatchSampler {
public:
    explicit BatchSampler(const StgConfig &config)
    {
        StgConfig c = config;
        c.struct_size = (int32_t)sizeof(StgConfig);
        const int st = stg_create(&c, &h_);
        if (st != STG_OK) throw Error(st, "stg_create: " + last_error(nullptr));
    }
    BatchSampler(int device, int max_rows, int max_vocab, int max_history, int max_top_k, int max_bias = 0,
                 int max_spec_draft = 0)
        : BatchSampler(make_config(device, max_rows, max_vocab, max_history, max_top_k, max_bias, max_spec_draft))
    {
    }
    ~BatchSampler()
    {
        if (h_) stg_destroy(h_);
    }
    BatchSampler(const BatchSampler &) = delete;
    BatchSampler &operator=(const BatchSampler &) = delete;
    BatchSampler(BatchSampler &&o) noexcept : h_(std::exchange(o.h_, nullptr)) {}
    BatchSampler &operator=(BatchSampler &&o) noexcept
    {
        if (this != &o) {
            if (h_) stg_destroy(h_);
            h_ = std::exchange(o.h_, nullptr);
        }
        return *this;
    }

    StgHandle handle() const noexcept { return h_; }

    // Sampler.Greedy over device rows; out_pairs = rows x {int32 index bits, float value}
    void argmax_rows(const void *logits, int dtype, int rows, int vocab, int64_t row_stride, void *out_pairs,
                     void *stream = nullptr)
    {
        check(stg_argmax_rows(h_, logits, dtype, rows, vocab, row_stride, out_pairs, stream), "stg_argmax_rows");
    }
    // Sampler.Sample for every row of the batch
    void sample_rows(StgSampleBatch batch, void *stream = nullptr)
    {
        batch.struct_size = (int32_t)sizeof(StgSampleBatch);
        check(stg_sample_rows(h_, &batch, stream), "stg_sample_rows");
    }
    // Sampler.BuildFilteredDistribution for every row of the batch
    void build_distribution(StgSampleBatch batch, float *probs, void *stream = nullptr)
    {
        batch.struct_size = (int32_t)sizeof(StgSampleBatch);
        check(stg_build_distribution(h_, &batch, probs, stream), "stg_build_distribution");
    }
    // SpeculativeDecoder.StepSampled's accept loop and correction draw
    void spec_verify(StgSpecBatch batch, void *stream = nullptr)
    {
        batch.struct_size = (int32_t)sizeof(StgSpecBatch);
        check(stg_spec_verify(h_, &batch, stream), "stg_spec_verify");
    }
    // MtpDecoder.AcceptDraft
    void mtp_accept(const void *logits, int dtype, int rows, int vocab, int64_t row_stride, const int32_t *draft,
                    float p_min, int32_t *accept, int32_t *argmax = nullptr, float *prob = nullptr,
                    void *stream = nullptr)
    {
        check(stg_mtp_accept(h_, logits, dtype, rows, vocab, row_stride, draft, p_min, accept, argmax, prob, stream),
              "stg_mtp_accept");
    }
    StgStats stats() const
    {
        StgStats s{};
        const int st = stg_get_stats(h_, &s);
        if (st != STG_OK) throw Error(st, "stg_get_stats");
        return s;
    }

    static std::string last_error(StgHandle h)
    {
        const size_t n = stg_last_error(h, nullptr, 0);
        std::vector<char> buf(n + 1, '\0');
        stg_last_error(h, buf.data(), buf.size());
        return std::string(buf.data());
    }

    static StgConfig make_config(int device, int max_rows, int max_vocab, int max_history, int max_top_k,
                                 int max_bias, int max_spec_draft)
    {
        StgConfig c{};
        c.struct_size = (int32_t)sizeof(StgConfig);
        c.device = device;
        c.max_rows = max_rows;
        c.max_vocab = max_vocab;
        c.max_history = max_history;
        c.max_top_k = max_top_k;
        c.max_bias = max_bias;
        c.max_spec_draft = max_spec_draft;
        return c;
    }

private:
    void check(int st, const char *what) const
    {
        if (st != STG_OK) throw Error(st, std::string(what) + ": " + last_error(h_));
    }
    StgHandle h_ = nullptr;
};

}  // namespace stingray

#endif  // STINGRAY_SAMPLER_HPP
