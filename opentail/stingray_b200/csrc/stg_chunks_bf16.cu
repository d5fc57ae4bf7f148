// The chunk kernel (streaming arg-max / top-N selection) for bf16 logits.
#include "stg_kernels_impl.cuh"

namespace stg {

cudaError_t launch_chunks_bf16(const SampleArgs &a, int grid, size_t smem, cudaStream_t stream)
{
    void (*fn)(const SampleArgs) = a.vec == 4 ? k_sample_chunks<4, true> : k_sample_chunks<1, true>;
    cudaError_t e = ensure_dynamic_smem((const void *)fn, smem);
    if (e != cudaSuccess) return e;
    fn<<<grid, kThreads, smem, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace stg
