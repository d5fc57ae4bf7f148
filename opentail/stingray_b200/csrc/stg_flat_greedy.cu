// A step whose rows are all plain arg-max rows (Sampler.Greedy, Sampler.cs:83-99: temperature <= 0,
// no history penalties) as ONE launch: the HBM pass of the flat step with its prep and its finish
// folded in.  Each CTA reduces its piece of a row to a (value, lowest index) key and raises the row's
// key with it; the CTA that arrives last at the row's ticket writes the row's outputs and leaves the
// key and the ticket at zero, which is the state every step leaves and this kernel starts from (the
// per-row finish of the other forms resets a key it consumed, stg_flat_finish.cuh).  A translation
// unit of its own: the streaming kernel of the general form (stg_flat.cu) is not touched by it.
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "stg_flat.cuh"
#include "stg_launch.h"
#include "stg_select.cuh"
#include "stg_types.h"

namespace stg {

template <bool BF16>
__device__ __forceinline__ void greedy_load4(const LogitRow rowp, const uint32_t *mrow, int i, int end, float v[4])
{
    if (i + 3 < end) {
        load_vec4<BF16, true>(rowp, i, v);
    } else {
#pragma unroll
        for (int e = 0; e < 4; e++) v[e] = (i + e < end) ? load_one<BF16>(rowp, i + e) : -CUDART_INF_F;
    }
    if (mrow != nullptr && i < end) {
        const uint32_t bits = __ldg(mrow + (i >> 5)) >> (i & 31);
#pragma unroll
        for (int e = 0; e < 4; e++)
            if (!((bits >> e) & 1u)) v[e] = -CUDART_INF_F;
    }
}

// grid (pieces of kFlatPiece elements, rows of a.items); 256 threads; in step s thread t reads elements
// 4096 s + 1024 u + 4 t .. + 3 (u = 0..3) of the piece as four independent 16-byte loads.
// Measured on the 256 x 151,936 batch, microseconds per step: this form 29.5 (launch bounds 256 x 5; the
// same source under 256 x 6 or 256 x 8 gives 34.0 and 31.4, all at 31-40 registers - the difference is
// the instruction schedule); the next four loads prefetched into a second register set (60 registers,
// four CTAs per SM) 31.6; a grid resident all at once with equal runs of 4096-element units per CTA
// 31.5; deeper prefetch at fewer CTAs per SM (3 x 3 units, 2 x 4 units in registers) 39.7 and 39.9.
template <bool BF16, bool CAP>
__global__ void __launch_bounds__(kFlatThreads, 5) k_greedy_step(const __grid_constant__ SampleArgs a, FlatRow *fr)
{
    __shared__ unsigned long long red[kFlatThreads / 32];
    const int row = __ldg(&a.items[blockIdx.y].row), tid = threadIdx.x, lane = tid & 31;
    const RowPlan *rpp = a.plans + row;
    const int begin = blockIdx.x * kFlatPiece;
    const int end = min(a.vocab, begin + kFlatPiece);
    const int esz = BF16 ? 2 : 4;
    const LogitRow rowp{(const char *)a.logits + (int64_t)row * a.row_stride * esz, CAP ? a.softcap : 0.f};
    const uint32_t *mrow = (__ldg(&rpp->use_mask) && a.mask) ? a.mask + (int64_t)row * a.mask_stride : nullptr;
    const int i0 = begin + tid * 4;

    // No register double-buffering: a thread has the four 16-byte loads of one step in flight and the
    // other warps of the SM (40 registers: six CTAs) cover their latency.
    float best = -CUDART_INF_F;
    int best_i = -1;
#pragma unroll 1
    for (int s = 0; s < kFlatPiece / 4096; s++) {
        float cur[4][4];
#pragma unroll
        for (int u = 0; u < 4; u++) greedy_load4<BF16>(rowp, mrow, i0 + (s * 4 + u) * 1024, end, cur[u]);
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int e = 0; e < 4; e++)
                if (cur[u][e] > best) { best = cur[u][e]; best_i = i0 + (s * 4 + u) * 1024 + e; }
    }
    // a thread visits ascending indices, so it holds its lowest index of the value; the key order
    // (value, then lower index) settles ties between threads, pieces and CTAs
    unsigned long long k = best_i >= 0 ? make_key(best, best_i) : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long t = __shfl_xor_sync(0xFFFFFFFFu, k, o);
        k = t > k ? t : k;
    }
    if (lane == 0) red[tid >> 5] = k;
    __syncthreads();
    if (tid != 0) return;
    for (int w = 1; w < kFlatThreads / 32; w++) k = red[w] > k ? red[w] : k;
    FlatRow *f = fr + row;
    if (k != 0ull) atomicMax(&f->key, k);
    __threadfence();
    if (atomicAdd(&f->ticket, 1) != (int)gridDim.x - 1) return;
    // last piece of the row to arrive: every other piece's key is in (its fence came before its ticket)
    __threadfence();
    const unsigned long long key = atomicExch(&f->key, 0ull);
    atomicExch(&f->ticket, 0);
    int tok = 0;
    float val;
    uint32_t fl = kPathGreedy;
    if (key != 0ull) {
        tok = key_idx(key);
        val = key_val(key);
    } else {
        val = load_one<BF16>(rowp, 0);  // Greedy of a row without a finite value: token 0
        fl |= (1u << 6);
    }
    if (a.pairs_out) {
        ((int32_t *)a.pairs_out)[2 * row] = tok;
        ((float *)a.pairs_out)[2 * row + 1] = val;
    }
    if (a.tokens) a.tokens[row] = tok;
    if (a.token_probs) a.token_probs[row] = 1.0f;
    if (a.row_flags) a.row_flags[row] = fl;
    count_row_flags(a.counters, fl);
}

cudaError_t launch_greedy_step(const SampleArgs &a, FlatRow *fr, cudaStream_t stream)
{
    const dim3 grid((unsigned)((a.vocab + kFlatPiece - 1) / kFlatPiece), (unsigned)a.n_items);
    const bool cap = a.softcap != 0.f;
    if (a.dtype == 1) { if (cap) k_greedy_step<true, true><<<grid, kFlatThreads, 0, stream>>>(a, fr); else k_greedy_step<true, false><<<grid, kFlatThreads, 0, stream>>>(a, fr); }
    else { if (cap) k_greedy_step<false, true><<<grid, kFlatThreads, 0, stream>>>(a, fr); else k_greedy_step<false, false><<<grid, kFlatThreads, 0, stream>>>(a, fr); }
    return cudaGetLastError();
}

}  // namespace stg
