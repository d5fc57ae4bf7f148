// Host-side check of the C++ wrapper (include/stingray_sampler.hpp), written the way the reference's
// own sampler tests read (tests/OpenTail.Stingray.Tests.ForwardPass.Fast/SamplerTests.cs:7-34, :70-85):
// greedy picks the highest logit, temperature 0 routes to greedy, top-k = 2 restricts the support.
// Without a CUDA device it checks that creation fails with STG_ERR_NO_DEVICE (no CPU fallback).
// Prints one line "host_check: <result>" and exits 0 on success.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "stingray_sampler.hpp"

#define REQUIRE(c)                                                        \
    do {                                                                  \
        if (!(c)) {                                                       \
            std::printf("host_check: FAILED %s (line %d)\n", #c, __LINE__); \
            return 1;                                                     \
        }                                                                 \
    } while (0)

int main()
{
    const int V = 1000, rows = 3;
    stingray::BatchSampler s = [&]() -> stingray::BatchSampler {
        try {
            return stingray::BatchSampler(0, rows, V, 16, 8);
        } catch (const stingray::Error &e) {
            if (e.status() != STG_ERR_NO_DEVICE) throw;
            std::printf("host_check: no device, creation refused (%s)\n", e.what());
            std::exit(0);
        }
    }();
    std::vector<float> logits((size_t)rows * V, 0.0f);
    logits[0 * V + 17] = 5.0f;                       // row 0: greedy -> 17
    logits[1 * V + 999] = 4.0f;                      // row 1: temperature 0 -> greedy -> 999
    logits[2 * V + 3] = 10.0f;                       // row 2: top-k 2 -> token in {3, 500}
    logits[2 * V + 500] = 9.5f;
    std::vector<StgRowParams> params(rows, stingray::default_params());
    params[0].temperature = 0.0f;
    params[1].temperature = 0.0f;
    params[1].top_k = 5;
    params[2].top_k = 2;
    std::vector<float> uniforms = {0.5f, 0.5f, 0.9f};
    std::vector<int32_t> tokens(rows, -1);
    std::vector<uint32_t> flags(rows, 0);

    StgSampleBatch b;
    std::memset(&b, 0, sizeof b);
    b.rows = rows;
    b.vocab = V;
    b.logits_dtype = STG_DTYPE_F32;
    b.logits = logits.data();
    b.row_stride = V;
    b.params = params.data();
    b.uniforms = uniforms.data();
    b.tokens = tokens.data();
    b.row_flags = flags.data();
    b.mem_flags = STG_MEM_HOST_LOGITS | STG_MEM_HOST_UNIFORMS | STG_MEM_HOST_OUTPUTS;
    s.sample_rows(b);
    REQUIRE(tokens[0] == 17);
    REQUIRE(tokens[1] == 999);
    REQUIRE(tokens[2] == 3 || tokens[2] == 500);
    REQUIRE((flags[2] & STG_ROW_PATH_MASK) == 2);

    // a vocabulary beyond the capacity given at creation is an error code, not a crash
    b.vocab = V + 1;
    try {
        s.sample_rows(b);
        REQUIRE(!"expected an error");
    } catch (const stingray::Error &e) {
        REQUIRE(e.status() == STG_ERR_CAPACITY || e.status() == STG_ERR_INVALID_ARGUMENT);
    }
    REQUIRE(s.stats().rows_sampled == 3);
    std::printf("host_check: ok tokens %d %d %d\n", tokens[0], tokens[1], tokens[2]);
    return 0;
}
