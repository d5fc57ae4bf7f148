// TEST INFRASTRUCTURE ONLY (never linked into the product library).
//
// Host-side launcher around the reference's own per-row arg-max kernel, `llm_argmax_rows`.  The kernel
// text is NOT in this repository: oracle/build_ref_argmax.py extracts it verbatim from the
// reference's source tree (src/OpenTail.Stingray.Cuda/CudaTextKernels.cs, the raw string that the
// reference compiles with NVRTC at run time) into oracle/_ref/llm_argmax_rows.inc, which this file
// includes.  The launch shape is the reference's: one 256-thread block per row
// (src/OpenTail.Stingray.Cuda/CudaBackend.cs:4156, ArgmaxThreads = 256).
#include <cuda_runtime.h>

#include "_ref/llm_argmax_rows.inc"

extern "C" __attribute__((visibility("default"))) int ref_argmax_rows(const float *logits, int rows, int n,
                                                                      int row_stride, void *out_pairs, void *stream)
{
    if (rows <= 0) return 0;
    llm_argmax_rows<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(logits, n, row_stride, out_pairs);
    return (int)cudaGetLastError();
}
