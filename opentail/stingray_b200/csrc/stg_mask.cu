// stg_and_masks: composition of the allowed-token bitmasks of several constraints, per row.
//
// AndTokenConstraint.Filter (src/OpenTail.Stingray.Core/Grammar/AndTokenConstraint.cs:44-86)
// masks a token when any constraining inner masks it: in bitmask form the result is the AND of the
// inners' words.  An inner in a dead state (it allows nothing) is skipped (:62-70); when no inner
// constrains, or the intersection is empty, the logits are returned unmasked (:80-85) - here a row
// of all-ones words, which stg_sample_rows treats as "nothing masked".
//
// One CTA per row.  The row's K masks are read twice (which inners are alive, then the AND); the
// second read comes from L2.  Pure word traffic: (K + 1) * words * 4 bytes per row.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/stingray_sampler.h"
#include "stg_handle.h"
#include "stg_types.h"

namespace stg {

constexpr int kMaxAndMasks = 32;

__global__ void __launch_bounds__(kThreads) k_and_masks(const uint32_t *masks, int n_masks, int rows, int vocab,
                                                        int64_t row_stride, uint32_t *out, int64_t out_stride,
                                                        uint8_t *uses)
{
    __shared__ unsigned alive_bits;  // bit m: inner m allows at least one token of this row
    __shared__ unsigned legal;       // OR of the intersection's words
    const int row = blockIdx.x, tid = threadIdx.x;
    const int words = (vocab + 31) >> 5;
    const uint32_t tail = (vocab & 31) ? ((1u << (vocab & 31)) - 1u) : 0xFFFFFFFFu;
    if (tid == 0) { alive_bits = 0u; legal = 0u; }
    __syncthreads();
    unsigned mine = 0u;
    for (int m = 0; m < n_masks; m++) {
        const uint32_t *src = masks + ((int64_t)m * rows + row) * row_stride;
        uint32_t acc = 0u;
        for (int w = tid; w < words; w += kThreads) acc |= __ldg(src + w) & (w == words - 1 ? tail : 0xFFFFFFFFu);
        if (__any_sync(0xFFFFFFFFu, acc != 0u)) mine |= 1u << m;
    }
    if ((tid & 31) == 0 && mine) atomicOr(&alive_bits, mine);
    __syncthreads();
    const unsigned alive = alive_bits;
    uint32_t any_legal = 0u;
    uint32_t *dst = out + (int64_t)row * out_stride;
    for (int w = tid; w < words; w += kThreads) {
        uint32_t v = 0xFFFFFFFFu;
        for (int m = 0; m < n_masks; m++)
            if ((alive >> m) & 1u) v &= __ldg(masks + ((int64_t)m * rows + row) * row_stride + w);
        dst[w] = v;
        any_legal |= v & (w == words - 1 ? tail : 0xFFFFFFFFu);
    }
    if (__any_sync(0xFFFFFFFFu, any_legal != 0u) && (tid & 31) == 0) atomicOr(&legal, 1u);
    __syncthreads();
    const bool masking = alive != 0u && legal != 0u;
    if (!masking)
        for (int w = tid; w < words; w += kThreads) dst[w] = 0xFFFFFFFFu;
    if (tid == 0 && uses) uses[row] = masking ? 1 : 0;
}

}  // namespace stg

extern "C" int stg_and_masks(StgHandle h, const uint32_t *masks, int32_t n_masks, int32_t rows, int32_t vocab,
                             int64_t mask_row_stride, uint32_t *out, int64_t out_row_stride, uint8_t *out_uses_mask,
                             void *stream)
{
    using namespace stg;
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (!masks || !out || n_masks < 0 || rows < 0 || vocab <= 0) return fail(h, STG_ERR_INVALID_ARGUMENT, "stg_and_masks: null array or negative size");
    if (n_masks > kMaxAndMasks) return fail(h, STG_ERR_CAPACITY, "stg_and_masks: at most 32 masks per row");
    const int64_t words = ((int64_t)vocab + 31) / 32;
    if (mask_row_stride < words || out_row_stride < words) return fail(h, STG_ERR_INVALID_ARGUMENT, "stg_and_masks: row stride shorter than the vocabulary");
    if (rows == 0) return STG_OK;
    CK(cudaSetDevice(h->cfg.device));
    k_and_masks<<<rows, kThreads, 0, (cudaStream_t)stream>>>(masks, n_masks, rows, vocab, mask_row_stride, out,
                                                             out_row_stride, out_uses_mask);
    CK(cudaGetLastError());
    h->stats.kernel_launches++;
    return STG_OK;
}
