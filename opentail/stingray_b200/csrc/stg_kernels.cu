// Launch dispatch of the sampling kernels and the vocabulary-sharded finish.
#include "stg_kernels_impl.cuh"

namespace stg {

cudaError_t launch_chunks_f32(const SampleArgs &a, int grid, size_t smem, cudaStream_t stream);
cudaError_t launch_chunks_bf16(const SampleArgs &a, int grid, size_t smem, cudaStream_t stream);
cudaError_t launch_rows_f32(const SampleArgs &a, int grid, cudaStream_t stream);
cudaError_t launch_rows_bf16(const SampleArgs &a, int grid, cudaStream_t stream);

// Vocabulary-sharded mode, after the exchange: one CTA per row merges the ranks' candidate lists
// and finishes the row.  The gathered buffer holds one block of block_bytes per rank:
// [rows, stride] keys followed by [rows] counts.
__global__ void __launch_bounds__(kThreads, 1) k_shard_finish(const __grid_constant__ SampleArgs a,
                                                              const unsigned char *gather, size_t block_bytes)
{
    extern __shared__ __align__(16) unsigned char arena[];
    __shared__ SelCtl ctl;
    __shared__ ItemShared ish;
    const int row = blockIdx.x;
    const RowPlan rp = a.plans[row];
    if (rp.path == kPathGreedy) {
        if (threadIdx.x == 0) {
            u64 best = 0ull;
            for (int r = 0; r < a.n_ranks; r++) {
                const u64 *keys = (const u64 *)(gather + (size_t)r * block_bytes);
                const int32_t *cnt = (const int32_t *)(keys + (size_t)a.rows * a.xchg_stride);
                if (cnt[row] > 0) {
                    u64 t = keys[(int64_t)row * a.xchg_stride];
                    best = t > best ? t : best;
                }
            }
            a.tokens[row] = best ? key_idx(best) : 0;
            if (a.token_probs) a.token_probs[row] = 1.f;
            if (a.row_flags) a.row_flags[row] = kPathGreedy | (best ? 0u : (1u << 6));
        }
        return;
    }
    Sel s;
    s.c = &ctl;
    s.buf[0] = (u64 *)arena;
    s.buf[1] = s.buf[0] + a.cap;
    s.cap = a.cap;
    s.n = rp.sel;
    s.idx_off = 0;
    sel_reset(s);
    for (int r = 0; r < a.n_ranks; r++) {
        const u64 *keys = (const u64 *)(gather + (size_t)r * block_bytes);
        const int32_t *cnt = (const int32_t *)(keys + (size_t)a.rows * a.xchg_stride);
        sel_append_keys(s, keys + (int64_t)row * a.xchg_stride, cnt[row]);
    }
    const int32_t *hist = a.hist_ids ? a.hist_ids + rp.hist_off : nullptr;
    const float *ptab = (a.pow_tab && rp.pow_off >= 0) ? a.pow_tab + rp.pow_off : nullptr;
    float u = a.uniforms ? __ldg(a.uniforms + row) : 0.5f;
    int64_t o = (int64_t)row * a.topk_stride;
    finish_topk(s, rp, hist, ptab, u, &ish.fout, a.topk_ids ? a.topk_ids + o : nullptr,
                a.topk_logits ? a.topk_logits + o : nullptr, a.topk_probs ? a.topk_probs + o : nullptr);
    if (threadIdx.x == 0) {
        a.tokens[row] = ish.fout.token;
        if (a.token_probs) a.token_probs[row] = ish.fout.prob;
        if (a.row_flags) a.row_flags[row] = ish.fout.flags;
        count_row_flags(a.counters, ish.fout.flags);
    }
}

cudaError_t launch_shard_finish(const SampleArgs &a, const void *gather, size_t block_bytes, size_t smem,
                                cudaStream_t stream)
{
    cudaError_t e = ensure_dynamic_smem((const void *)k_shard_finish, smem);
    if (e != cudaSuccess) return e;
    k_shard_finish<<<a.rows, kThreads, smem, stream>>>(a, (const unsigned char *)gather, block_bytes);
    return cudaGetLastError();
}

cudaError_t launch_sample_chunks(const SampleArgs &a, int grid, size_t smem, cudaStream_t stream)
{
    return a.dtype == 1 ? launch_chunks_bf16(a, grid, smem, stream) : launch_chunks_f32(a, grid, smem, stream);
}

cudaError_t launch_sample_rows(const SampleArgs &a, int grid, cudaStream_t stream)
{
    return a.dtype == 1 ? launch_rows_bf16(a, grid, stream) : launch_rows_f32(a, grid, stream);
}

}  // namespace stg
