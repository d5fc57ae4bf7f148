// Device-resident token histories: stg_history_reset / _load / _append / _length.
//
// The reference's engine appends every sampled token to the sequence's host-side list
// (ContinuousBatchingEngine.cs:650, :1280) and passes the list to Sampler.Sample as PreviousTokens
// (Sampler.cs:19, :364-401).  Here slot r of the handle owns max_history int32 entries in device
// memory, oldest first, with its length kept twice: on the device for the append kernel, on the host
// for the step's plan.  Both follow the same rule (append; a full slot drops its oldest entry), so
// they agree without ever being copied.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/stingray_sampler.h"
#include "stg_handle.h"
#include "stg_types.h"

namespace stg {

constexpr int kAppendRows = 1024;  // rows one launch of the append kernel covers (one bit each)
struct ActiveBits {
    uint32_t w[kAppendRows / 32];
};

// One warp per row.  A full slot is shifted down by one entry, 32 entries per step, every step
// reading its entries before it overwrites the ones the previous step read.
__global__ void __launch_bounds__(256) k_history_append(int32_t *ids, int32_t *len, const int32_t *tokens, int first,
                                                        int rows, int cap, const __grid_constant__ ActiveBits active)
{
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= rows || !((active.w[r >> 5] >> (r & 31)) & 1u)) return;
    int32_t *row = ids + (int64_t)(first + r) * cap;
    const int n = len[first + r];
    const int32_t tok = tokens[first + r];
    if (n < cap) {
        if (lane == 0) {
            row[n] = tok;
            len[first + r] = n + 1;
        }
        return;
    }
    for (int base = 0; base < cap - 1; base += 32) {
        const int j = base + lane;
        const int32_t v = (j + 1 < cap) ? row[j + 1] : 0;
        __syncwarp();
        if (j + 1 < cap) row[j] = v;
        __syncwarp();
    }
    if (lane == 0) row[cap - 1] = tok;
}

__global__ void k_history_set_len(int32_t *len, int first, int n, int value)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) len[first + i] = value;
}

}  // namespace stg

using namespace stg;

extern "C" {

int stg_history_reset(StgHandle h, int32_t first_slot, int32_t n_slots, void *stream)
{
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (first_slot < 0 || n_slots < 0 || (int64_t)first_slot + n_slots > h->cfg.max_rows)
        return fail(h, STG_ERR_INVALID_ARGUMENT, "stg_history_reset: slots outside [0, max_rows)");
    if (n_slots == 0) return STG_OK;
    CK(cudaSetDevice(h->cfg.device));
    k_history_set_len<<<(n_slots + 255) / 256, 256, 0, (cudaStream_t)stream>>>((int32_t *)h->ring_len_dev.p, first_slot, n_slots, 0);
    CK(cudaGetLastError());
    for (int i = 0; i < n_slots; i++) {
        h->ring_len[first_slot + i] = 0;
        h->ring_dropped[first_slot + i] = 0;
    }
    h->stats.kernel_launches++;
    return STG_OK;
}

int stg_history_load(StgHandle h, int32_t slot, const int32_t *tokens, int32_t n, void *stream)
{
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (slot < 0 || slot >= h->cfg.max_rows || n < 0 || (n > 0 && !tokens))
        return fail(h, STG_ERR_INVALID_ARGUMENT, "stg_history_load: bad slot or token array");
    if (n > h->cfg.max_history) return fail(h, STG_ERR_CAPACITY, "stg_history_load: more tokens than max_history");
    CK(cudaSetDevice(h->cfg.device));
    const int cap = std::max(h->cfg.max_history, 1);
    if (n > 0)
        CK(cudaMemcpyAsync((int32_t *)h->ring_ids.p + (int64_t)slot * cap, tokens, (size_t)n * 4, cudaMemcpyHostToDevice,
                           (cudaStream_t)stream));
    k_history_set_len<<<1, 32, 0, (cudaStream_t)stream>>>((int32_t *)h->ring_len_dev.p, slot, 1, n);
    CK(cudaGetLastError());
    h->ring_len[slot] = n;
    h->ring_dropped[slot] = 0;
    h->stats.kernel_launches++;
    return STG_OK;
}

int stg_history_append(StgHandle h, const int32_t *tokens, int32_t rows, const uint8_t *active, void *stream)
{
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (!tokens || rows < 0 || rows > h->cfg.max_rows) return fail(h, STG_ERR_INVALID_ARGUMENT, "stg_history_append: bad token array or row count");
    if (h->cfg.max_history <= 0) return fail(h, STG_ERR_CAPACITY, "stg_history_append: the handle was created with max_history 0");
    CK(cudaSetDevice(h->cfg.device));
    const int cap = h->cfg.max_history;
    for (int first = 0; first < rows; first += kAppendRows) {
        const int n = std::min(kAppendRows, rows - first);
        ActiveBits bits;
        memset(&bits, 0, sizeof(bits));
        bool any = false;
        for (int r = 0; r < n; r++)
            if (!active || active[first + r]) {
                bits.w[r >> 5] |= 1u << (r & 31);
                any = true;
            }
        if (!any) continue;
        k_history_append<<<(n + 7) / 8, 256, 0, (cudaStream_t)stream>>>((int32_t *)h->ring_ids.p, (int32_t *)h->ring_len_dev.p, tokens,
                                                                       first, n, cap, bits);
        CK(cudaGetLastError());
        h->stats.kernel_launches++;
        for (int r = 0; r < n; r++) {
            if (active && !active[first + r]) continue;
            if (h->ring_len[first + r] < cap) h->ring_len[first + r]++;
            else h->ring_dropped[first + r] = 1;
        }
    }
    return STG_OK;
}

int stg_history_length(StgHandle h, int32_t slot)
{
    if (!h) return -STG_ERR_INVALID_ARGUMENT;
    if (slot < 0 || slot >= h->cfg.max_rows) return -fail(h, STG_ERR_INVALID_ARGUMENT, "stg_history_length: slot outside [0, max_rows)");
    return h->ring_len[slot];
}

}  // extern "C"
