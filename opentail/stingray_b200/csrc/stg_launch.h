// Launchers implemented in the .cu files, called by the C-ABI layer.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <utility>

#include "stg_types.h"

namespace stg {

// Raises a kernel's dynamic shared-memory limit to `bytes` unless an earlier launch on this device
// already did: the attribute call costs microseconds that a per-step launch path should not pay.
inline cudaError_t ensure_dynamic_smem(const void *fn, size_t bytes)
{
    static std::mutex mu;
    static std::map<std::pair<const void *, int>, size_t> done;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(mu);
    size_t &cur = done[{fn, dev}];
    if (bytes <= cur) return cudaSuccess;
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) cur = bytes;
    return e;
}

// Diagnostic: CUDA events recorded between the kernels of a step (STG_KERNEL_TIMES=1), read back by
// stg_debug_kernel_times.  mark(name) stamps the end of the kernel(s) launched since the last mark.
struct KernelTimer {
    static constexpr int kMax = 32;
    cudaEvent_t ev[kMax + 1] = {};
    const char *name[kMax] = {};
    int n = 0;
    bool on = false;
    void begin(cudaStream_t s) { n = 0; if (on) cudaEventRecord(ev[0], s); }
    void mark(const char *what, cudaStream_t s)
    {
        if (!on || n >= kMax) return;
        name[n] = what;
        cudaEventRecord(ev[++n], s);
    }
};

// shared memory a row-type work item needs: sort keys + exp-value histogram
constexpr size_t kRowArenaBytes = 211968;  // layout in stg_rowdist.cuh (checked there)

cudaError_t launch_sample_chunks(const SampleArgs &a, int grid, size_t smem, cudaStream_t stream);
cudaError_t launch_sample_rows(const SampleArgs &a, int grid, cudaStream_t stream);
cudaError_t launch_shard_finish(const SampleArgs &a, const void *gather, size_t block_bytes, size_t smem,
                                cudaStream_t stream);

// speculative verification, second phase (stg_spec.cu)
struct SpecArgs {
    const void *target;
    const void *draft;
    const int32_t *draft_tokens;
    const double *uniforms;
    const RowDist *tdist;
    const RowDist *ddist;
    int32_t *accepted;
    int32_t *correction;
    float *accept_probs;
    uint32_t *seq_flags;
    float p_min;
    float target_cap, draft_cap;  // soft caps of the two models' logits, 0: none
    const int32_t *only;          // k_spec_finish: when set, only the sequences whose entry is non-zero are done
    int32_t n_seq, n_draft, vocab, dtype, mode, vec;
};
cudaError_t launch_spec_finish(const SpecArgs &a, cudaStream_t stream);
cudaError_t launch_probs_draw(const float *probs, int rows, int vocab, int64_t row_stride, const float *uniforms,
                              int32_t *tokens, uint32_t *flags, cudaStream_t stream);
cudaError_t launch_residual_draw(const float *p, const float *q, int rows, int vocab, int64_t row_stride,
                                 const float *uniforms2, int32_t *tokens, uint32_t *flags, cudaStream_t stream);
cudaError_t launch_mtp_accept(const void *logits, int dtype, int rows, int vocab, int64_t row_stride, int vec,
                              const int32_t *draft, float p_min, int32_t *accept, int32_t *argmax, float *prob,
                              cudaStream_t stream);

}  // namespace stg
