// The row kernel (full-vocabulary pipeline, one row per CTA) for bf16 logits.
#include "stg_kernels_impl.cuh"

namespace stg {

cudaError_t launch_rows_bf16(const SampleArgs &a, int grid, cudaStream_t stream)
{
    void (*fn)(const SampleArgs) = k_sample_rows<true>;
    cudaError_t e = ensure_dynamic_smem((const void *)fn, kRowArenaBytes);
    if (e != cudaSuccess) return e;
    fn<<<grid, kThreads, kRowArenaBytes, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace stg
