// stg_argmax_rows_static: the per-row arg-max for callers that cannot allocate device memory.
//
// Some hosts may not call cudaMalloc at the point where they need the arg-max: code running
// between cudaStreamBeginCapture and cudaStreamEndCapture of another component, a plug-in that is
// handed a stream but no allocator, or a process whose memory budget was fixed at start-up.  The
// regular entry point (stg_argmax_rows) needs a handle, and creating a handle allocates its
// workspace.  This variant needs no handle: the few bytes of scratch the kernel uses (one partial
// result per chunk of a row, one arrival counter per row) live in file-scope __device__ arrays
// that every GPU loading this library holds until the process exits (about 1 MiB).
//
// Consequences the caller must know:
//  * sizes are bounded: at most kStaticMaxRows rows per call; larger calls are rejected;
//  * the first call on a device resolves the arrays' device addresses (cudaGetSymbolAddress) and
//    should therefore be made once before any stream capture begins;
//  * every call on a device shares the same scratch, so two calls whose kernels overlap on the GPU
//    (different streams, no ordering between them) race; order them on one stream or with events.
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../../include/stingray_sampler.h"
#include "stg_select.cuh"
#include "stg_types.h"

namespace stg {

constexpr int kStaticMaxRows = STG_STATIC_MAX_ROWS;
constexpr int kStaticMaxChunks = 32;

// Scratch of the allocation-free arg-max.  In host code these names are host-side stand-ins, not
// device addresses: the launcher below asks the runtime for the real addresses once per device.
static __device__ __align__(256) unsigned long long g_static_partial[kStaticMaxRows * kStaticMaxChunks];
static __device__ __align__(256) unsigned int g_static_ticket[kStaticMaxRows];

template <int VEC, bool BF16>
__global__ void __launch_bounds__(kThreads) k_argmax_static(const void *logits, int vocab, int64_t row_stride,
                                                            int chunk_len, int n_chunks, u64 *partial,
                                                            unsigned int *ticket, void *out_pairs)
{
    __shared__ u64 red[32];
    __shared__ int last;
    const int row = blockIdx.y, chunk = blockIdx.x;
    const int esz = BF16 ? 2 : 4;
    const LogitRow rowp{(const char *)logits + (int64_t)row * row_stride * esz, 0.f};
    const int begin = chunk * chunk_len, end = min(vocab, begin + chunk_len);
    constexpr int U = 4;
    float best = -CUDART_INF_F;
    int best_i = -1;
    for (int base = begin; base < end; base += kThreads * 4 * U) {
        float v[U][4];
        int idx[U][4];
#pragma unroll
        for (int u = 0; u < U; u++) load_items<VEC, BF16, true>(rowp, nullptr, base, u, end, v[u], idx[u]);
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (v[u][e] > best) { best = v[u][e]; best_i = idx[u][e]; }
    }
    u64 k = best_i >= 0 ? make_key(best, best_i) : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        u64 t = __shfl_xor_sync(0xFFFFFFFFu, k, o);
        k = t > k ? t : k;
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = k;
    __syncthreads();
    if (threadIdx.x < 32) {
        k = red[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            u64 t = __shfl_xor_sync(0xFFFFFFFFu, k, o);
            k = t > k ? t : k;
        }
    }
    if (threadIdx.x == 0) {
        partial[(int64_t)row * kStaticMaxChunks + chunk] = k;
        __threadfence();
        unsigned old = atomicAdd(&ticket[row], 1u);
        last = (old == (unsigned)(n_chunks - 1));
        if (last) {
            ticket[row] = 0u;  // the array must read zero again when the next call starts
            __threadfence();
            u64 b = 0ull;
            for (int c = 0; c < n_chunks; c++) {
                u64 t = __ldcg(partial + (int64_t)row * kStaticMaxChunks + c);
                b = t > b ? t : b;
            }
            int tok = 0;
            float val;
            if (b != 0ull) { tok = key_idx(b); val = key_val(b); }
            else val = BF16 ? load_one<true>(rowp, 0) : load_one<false>(rowp, 0);
            ((int32_t *)out_pairs)[2 * row] = tok;
            ((float *)out_pairs)[2 * row + 1] = val;
        }
    }
}

struct StaticDev {
    bool ready = false;
    u64 *partial = nullptr;
    unsigned int *ticket = nullptr;
    int sm_count = 0;
};
static StaticDev g_static_dev[64];
static std::mutex g_static_mu;

}  // namespace stg

using namespace stg;

extern "C" int stg_argmax_rows_static(const void *logits, int32_t dtype, int32_t rows, int32_t vocab,
                                      int64_t row_stride, void *out_pairs, void *stream_)
{
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!logits || !out_pairs || rows < 0 || vocab <= 0 || row_stride < vocab) return STG_ERR_INVALID_ARGUMENT;
    if (dtype != STG_DTYPE_F32 && dtype != STG_DTYPE_BF16) return STG_ERR_INVALID_ARGUMENT;
    if (rows > kStaticMaxRows) return STG_ERR_CAPACITY;  // beyond the fixed scratch: use stg_argmax_rows
    if (rows == 0) return STG_OK;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return STG_ERR_NO_DEVICE;
    StaticDev sd;
    {
        std::lock_guard<std::mutex> lock(g_static_mu);
        if (!g_static_dev[dev].ready) {
            // set-up, once per device, with that device current: the symbols' device addresses
            void *p = nullptr, *t = nullptr;
            if (cudaGetSymbolAddress(&p, g_static_partial) != cudaSuccess) return STG_ERR_CUDA;
            if (cudaGetSymbolAddress(&t, g_static_ticket) != cudaSuccess) return STG_ERR_CUDA;
            int sms = 0;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return STG_ERR_CUDA;
            g_static_dev[dev].partial = (u64 *)p;
            g_static_dev[dev].ticket = (unsigned int *)t;
            g_static_dev[dev].sm_count = sms;
            g_static_dev[dev].ready = true;
        }
        sd = g_static_dev[dev];
    }
    // The counters are shared by every call and keep what the last call left; a call that was cut
    // short could leave them non-zero, so they are cleared on the stream before each launch.
    if (cudaMemsetAsync(sd.ticket, 0, sizeof(unsigned int) * (size_t)rows, stream) != cudaSuccess) return STG_ERR_CUDA;
    int want = (4 * sd.sm_count + rows - 1) / rows;  // about four chunk CTAs per SM
    int max_s = (vocab + 16383) / 16384;
    int S = want < max_s ? want : max_s;
    if (S > kStaticMaxChunks) S = kStaticMaxChunks;
    if (S < 1) S = 1;
    int chunk_len = ((vocab + S - 1) / S + kSubTile - 1) / kSubTile * kSubTile;
    int n_chunks = (vocab + chunk_len - 1) / chunk_len;
    const size_t esz = dtype == STG_DTYPE_BF16 ? 2 : 4, need = dtype == STG_DTYPE_BF16 ? 8 : 16;
    const bool aligned = ((uintptr_t)logits % need) == 0 && ((size_t)row_stride * esz) % need == 0;
    dim3 grid((unsigned)n_chunks, (unsigned)rows);
    if (dtype == STG_DTYPE_BF16) {
        if (aligned) k_argmax_static<4, true><<<grid, kThreads, 0, stream>>>(logits, vocab, row_stride, chunk_len, n_chunks, sd.partial, sd.ticket, out_pairs);
        else k_argmax_static<1, true><<<grid, kThreads, 0, stream>>>(logits, vocab, row_stride, chunk_len, n_chunks, sd.partial, sd.ticket, out_pairs);
    } else {
        if (aligned) k_argmax_static<4, false><<<grid, kThreads, 0, stream>>>(logits, vocab, row_stride, chunk_len, n_chunks, sd.partial, sd.ticket, out_pairs);
        else k_argmax_static<1, false><<<grid, kThreads, 0, stream>>>(logits, vocab, row_stride, chunk_len, n_chunks, sd.partial, sd.ticket, out_pairs);
    }
    return cudaGetLastError() == cudaSuccess ? STG_OK : STG_ERR_CUDA;
}
