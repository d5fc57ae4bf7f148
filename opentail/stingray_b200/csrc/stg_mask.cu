// Allowed-token bitmasks: stg_and_masks (composition of ready masks) and the device-resident cache
// of per-state masks with its composition, stg_mask_cache_put / _contains / stg_mask_compose.
//
// AndTokenConstraint.Filter (src/OpenTail.Stingray.Core/Grammar/AndTokenConstraint.cs:44-86)
// masks a token when any constraining inner masks it: in bitmask form the result is the AND of the
// inners' words.  An inner in a dead state (it allows nothing) is skipped (:62-70); when no inner
// constrains, or the intersection is empty, the logits are returned unmasked (:80-85) - here a row
// of all-ones words, which stg_sample_rows treats as "nothing masked".
//
// One CTA per row.  The row's K masks are read twice (which inners are alive, then the composition);
// the second read comes from L2.  Pure word traffic: (K + 1) * words * 4 bytes per row.
//
// The cache exists because the reference pays a walk over the whole vocabulary per constrained row
// and step to rebuild a set that depends on the automaton state only
// (JsonSchemaGrammarMasker.Filter, src/OpenTail.Stingray.Core/Grammar/JsonSchemaGrammarMasker.cs:67-95):
// the host walks once per new state, stores the words under (constraint, state), and every later
// step names the state by its key.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/stingray_sampler.h"
#include "stg_handle.h"
#include "stg_types.h"

#include <string.h>

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

// The same composition over cached masks: slot[row * K + m] is the cache entry of the row's m-th
// inner, or -1.  op 0: AND of the inners that allow something; op 1: their OR.
__global__ void __launch_bounds__(kThreads) k_mask_compose(const uint32_t *cache, int64_t cache_stride, const int32_t *slot,
                                                           int K, int vocab, int op, uint32_t *out, int64_t out_stride,
                                                           uint8_t *uses)
{
    __shared__ unsigned alive_bits;
    __shared__ unsigned legal;
    __shared__ int32_t sl[kMaxAndMasks];
    const int row = blockIdx.x, tid = threadIdx.x;
    const int words = (vocab + 31) >> 5;
    const uint32_t tail = (vocab & 31) ? ((1u << (vocab & 31)) - 1u) : 0xFFFFFFFFu;
    if (tid == 0) { alive_bits = 0u; legal = 0u; }
    if (tid < K) sl[tid] = slot[(int64_t)row * K + tid];
    __syncthreads();
    unsigned mine = 0u;
    for (int m = 0; m < K; m++) {
        if (sl[m] < 0) continue;
        const uint32_t *src = cache + (int64_t)sl[m] * cache_stride;
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
        uint32_t v = op == 0 ? 0xFFFFFFFFu : 0u;
        for (int m = 0; m < K; m++)
            if ((alive >> m) & 1u) {
                const uint32_t x = __ldg(cache + (int64_t)sl[m] * cache_stride + w);
                v = op == 0 ? (v & x) : (v | x);
            }
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

// entry of `key`, or -1
static int mc_find(StgHandle h, uint64_t key)
{
    auto it = h->mc_index.find(key);
    return it == h->mc_index.end() ? -1 : it->second;
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

extern "C" int stg_mask_cache_put(StgHandle h, uint64_t key, const uint32_t *words, int32_t vocab, void *stream)
{
    using namespace stg;
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (h->mc_key.empty()) return fail(h, STG_ERR_CAPACITY, "stg_mask_cache_put: the handle was created with max_cached_masks 0");
    if (key == 0 || !words || vocab <= 0) return fail(h, STG_ERR_INVALID_ARGUMENT, "stg_mask_cache_put: key 0, null words or bad vocab");
    if (vocab > h->cfg.max_vocab) return fail(h, STG_ERR_CAPACITY, "stg_mask_cache_put: vocab larger than max_vocab");
    CK(cudaSetDevice(h->cfg.device));
    int e = mc_find(h, key);
    if (e < 0) {
        // a free entry (tick 0), else the one used longest ago
        e = 0;
        for (size_t i = 1; i < h->mc_key.size() && h->mc_used[e] != 0; i++)
            if (h->mc_used[i] < h->mc_used[e]) e = (int)i;
        if (h->mc_key[e] != 0) h->mc_index.erase(h->mc_key[e]);
        h->mc_index[key] = e;
    }
    const size_t words_n = ((size_t)vocab + 31) / 32;
    CK(cudaMemcpyAsync((uint32_t *)h->mc_words.p + (int64_t)e * h->mc_stride, words, words_n * 4, cudaMemcpyHostToDevice,
                       (cudaStream_t)stream));
    h->mc_key[e] = key;
    h->mc_used[e] = ++h->mc_tick;
    return STG_OK;
}

extern "C" int stg_mask_cache_contains(StgHandle h, uint64_t key)
{
    return (h && key != 0 && stg::mc_find(h, key) >= 0) ? 1 : 0;
}

extern "C" int stg_mask_compose(StgHandle h, const uint64_t *keys, int32_t keys_per_row, int32_t rows, int32_t vocab, int32_t op,
                                uint32_t *out, int64_t out_row_stride, uint8_t *out_uses_mask, void *stream)
{
    using namespace stg;
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (h->mc_key.empty()) return fail(h, STG_ERR_CAPACITY, "stg_mask_compose: the handle was created with max_cached_masks 0");
    if (!keys || !out || keys_per_row <= 0 || rows < 0 || vocab <= 0 || (op != STG_MASK_AND && op != STG_MASK_OR))
        return fail(h, STG_ERR_INVALID_ARGUMENT, "stg_mask_compose: null array, bad size or unknown operation");
    if (keys_per_row > kMaxAndMasks) return fail(h, STG_ERR_CAPACITY, "stg_mask_compose: at most 32 keys per row");
    if (rows > h->cfg.max_rows || vocab > h->cfg.max_vocab) return fail(h, STG_ERR_CAPACITY, "stg_mask_compose: rows or vocab beyond the handle's limits");
    if (out_row_stride < ((int64_t)vocab + 31) / 32) return fail(h, STG_ERR_INVALID_ARGUMENT, "stg_mask_compose: row stride shorter than the vocabulary");
    if (rows == 0) return STG_OK;
    std::vector<int32_t> &sl = h->mc_slot_scratch;
    sl.resize((size_t)rows * keys_per_row);
    for (size_t i = 0; i < sl.size(); i++) {
        if (keys[i] == 0) { sl[i] = -1; continue; }
        sl[i] = mc_find(h, keys[i]);
        if (sl[i] < 0) return fail(h, STG_ERR_INVALID_ARGUMENT, "stg_mask_compose: key " + std::to_string(keys[i]) + " is not cached");
    }
    ++h->mc_tick;
    for (size_t i = 0; i < sl.size(); i++)
        if (sl[i] >= 0) h->mc_used[sl[i]] = h->mc_tick;
    CK(cudaSetDevice(h->cfg.device));
    // pageable source: the runtime stages it before the call returns, so the scratch may be reused at once
    CK(cudaMemcpyAsync(h->mc_slots.p, sl.data(), sl.size() * 4, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    k_mask_compose<<<rows, kThreads, 0, (cudaStream_t)stream>>>((const uint32_t *)h->mc_words.p, h->mc_stride, (const int32_t *)h->mc_slots.p,
                                                               keys_per_row, vocab, op, out, out_row_stride, out_uses_mask);
    CK(cudaGetLastError());
    h->stats.kernel_launches++;
    return STG_OK;
}
