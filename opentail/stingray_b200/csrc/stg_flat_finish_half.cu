// k_flat_finish_half: the finish of the flat step's chunked rows with 512-thread CTAs, two per SM.
//
// What remains of a top-k row after k_flat_stream is a few hundred to a few thousand candidates; the
// phases of finish_topk over them are short and separated by block barriers, so a 1024-thread CTA
// that holds a whole SM (64 registers per thread) leaves most of it idle.  This translation unit
// builds the same code (stg_flat_finish.cuh, stg_select.cuh) for 512 threads: two rows per SM at a
// time, each a little slower, the batch nearly twice as fast.  Its candidate buffers (a.finish_cap
// entries, what two CTAs per SM leave room for) are shorter than the longest candidate list; such a
// list is reduced as it is read in.
#define STG_KTHREADS 512
#include <cuda_runtime.h>
#include <stdint.h>

#include "stg_flat.cuh"
#include "stg_flat_finish.cuh"
#include "stg_launch.h"

namespace stg {

static_assert(kThreads == 512, "this translation unit is the half-size build");

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 2) k_flat_finish_half(const __grid_constant__ SampleArgs a, FlatRow *fr)
{
    extern __shared__ __align__(16) unsigned char arena[];
    __shared__ SelCtl ctl;
    __shared__ FlatShared fs;
    for (int i = blockIdx.x; i < a.n_items; i += gridDim.x) {
        flat_finish_row<BF16>(a, fr, a.items[i].row, i, a.finish_cap, arena, ctl, fs);
        __syncthreads();
    }
}

cudaError_t launch_flat_finish_half(const SampleArgs &a, FlatRow *fr, int grid, cudaStream_t stream)
{
    const size_t smem = (size_t)a.finish_cap * 16;
    void (*fn)(const SampleArgs, FlatRow *) = a.dtype == 1 ? k_flat_finish_half<true> : k_flat_finish_half<false>;
    cudaError_t e = ensure_dynamic_smem((const void *)fn, smem);
    if (e != cudaSuccess) return e;
    fn<<<grid, kThreads, smem, stream>>>(a, fr);
    return cudaGetLastError();
}

}  // namespace stg
