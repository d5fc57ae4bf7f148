// C ABI, second part: speculative verification, the MTP accept rule, and the vocabulary-sharded
// mode with its NCCL exchange.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "stg_handle.h"
#include "stg_flat.cuh"
#include "stg_emul2.cuh"
#include "stg_launch.h"

using namespace stg;
using stg::round_up;

namespace {

bool rows_aligned2(const void *p, int64_t row_stride, int dtype)
{
    const size_t esz = dtype == STG_DTYPE_BF16 ? 2 : 4;
    const size_t need = dtype == STG_DTYPE_BF16 ? 8 : 16;
    return ((uintptr_t)p % need) == 0 && ((size_t)row_stride * esz) % need == 0;
}

// ---- NCCL through dlopen: the library has no link-time dependency on it ------------------------
struct NcclId { char internal[128]; };
typedef int (*fn_get_unique_id)(NcclId *);
typedef int (*fn_comm_init_rank)(void **, int, NcclId, int);
typedef int (*fn_comm_destroy)(void *);
typedef int (*fn_all_gather)(const void *, void *, size_t, int, void *, cudaStream_t);
typedef const char *(*fn_error_string)(int);

struct NcclApi {
    void *lib = nullptr;
    fn_get_unique_id get_unique_id = nullptr;
    fn_comm_init_rank comm_init_rank = nullptr;
    fn_comm_destroy comm_destroy = nullptr;
    fn_all_gather all_gather = nullptr;
    fn_error_string error_string = nullptr;
};
NcclApi g_nccl;

bool load_nccl(std::string &why)
{
    if (g_nccl.lib) return true;
    const char *env = getenv("STG_NCCL_LIB");
    const char *names[] = {env, "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        if (!n || !*n) continue;
        g_nccl.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.lib) break;
    }
    if (!g_nccl.lib) { why = std::string("cannot load libnccl: ") + dlerror(); return false; }
    g_nccl.get_unique_id = (fn_get_unique_id)dlsym(g_nccl.lib, "ncclGetUniqueId");
    g_nccl.comm_init_rank = (fn_comm_init_rank)dlsym(g_nccl.lib, "ncclCommInitRank");
    g_nccl.comm_destroy = (fn_comm_destroy)dlsym(g_nccl.lib, "ncclCommDestroy");
    g_nccl.all_gather = (fn_all_gather)dlsym(g_nccl.lib, "ncclAllGather");
    g_nccl.error_string = (fn_error_string)dlsym(g_nccl.lib, "ncclGetErrorString");
    if (!g_nccl.get_unique_id || !g_nccl.comm_init_rank || !g_nccl.comm_destroy || !g_nccl.all_gather) {
        why = "libnccl lacks a required symbol";
        return false;
    }
    return true;
}

int nccl_fail(StgHandle h, int code, const char *what)
{
    std::string msg = std::string(what) + ": ";
    msg += g_nccl.error_string ? g_nccl.error_string(code) : "NCCL error";
    return fail(h, STG_ERR_NCCL, msg);
}

int ensure_exchange(StgHandle h, int n_ranks)
{
    // capacity of one rank's block: [max_rows, max_top_k + max_history] keys and [max_rows] counts
    const size_t R = (size_t)h->cfg.max_rows;
    const size_t sel = std::max<size_t>(1, (size_t)h->cfg.max_top_k + h->cfg.max_history);
    const size_t local = round_up(R * sel * 8 + R * 4, 16) + 16, gather = local * (size_t)n_ranks;
    int rc = STG_OK;
    if (h->xchg_local.bytes < local) {
        dev_free(h->xchg_local);
        rc = dev_alloc(h, h->xchg_local, local);
    }
    if (!rc && h->xchg_gather.bytes < gather) {
        // only the receive side grows with the number of ranks; this rank's own candidates stay
        dev_free(h->xchg_gather);
        rc = dev_alloc(h, h->xchg_gather, gather);
    }
    if (rc) return rc;
    h->shard_sel = (int)sel;
    h->shard_rows = (int)R;
    return STG_OK;
}

}  // namespace

extern "C" {

int stg_spec_verify(StgHandle h, const StgSpecBatch *b, void *stream_)
{
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (!b || b->struct_size != (int32_t)sizeof(StgSpecBatch)) return fail(h, STG_ERR_INVALID_ARGUMENT, "bad StgSpecBatch");
    const int S = b->n_seq, L = b->n_draft, V = b->vocab;
    if (S < 0 || L < 0 || V <= 0) return fail(h, STG_ERR_INVALID_ARGUMENT, "n_seq, n_draft >= 0 and vocab > 0 are required");
    if (S == 0) return STG_OK;
    if (L > h->cfg.max_spec_draft) return fail(h, STG_ERR_CAPACITY, "n_draft exceeds max_spec_draft");
    if ((int64_t)S * (L + 1) > h->cfg.max_rows) return fail(h, STG_ERR_CAPACITY, "n_seq * (n_draft + 1) exceeds max_rows");
    if (V > h->cfg.max_vocab) return fail(h, STG_ERR_CAPACITY, "vocab exceeds max_vocab");
    if (!b->target_logits || !b->params || !b->uniforms || !b->accepted || !b->correction || (L > 0 && !b->draft_tokens))
        return fail(h, STG_ERR_INVALID_ARGUMENT, "a required array is null");
    if (b->mode != 0 && b->mode != 1) return fail(h, STG_ERR_INVALID_ARGUMENT, "mode must be 0 or 1");
    bool any_sampled = false;
    for (int s = 0; s < S; s++) any_sampled |= b->params[s].temperature > 0.f;
    if (b->mode == 0 && L > 0 && any_sampled && !b->draft_logits)
        return fail(h, STG_ERR_INVALID_ARGUMENT, "draft_logits are required for the p/q accept rule");
    if (b->mem_flags & STG_MEM_HOST_LOGITS) return fail(h, STG_ERR_UNSUPPORTED, "stg_spec_verify takes device logits");
    if (b->mem_flags & STG_MEM_HOST_DRAFT)
        for (int64_t i = 0; i < (int64_t)S * L; i++)
            if ((uint32_t)b->draft_tokens[i] >= (uint32_t)V)
                return fail(h, STG_ERR_INVALID_ARGUMENT, "a draft token lies outside [0, vocab)");
    CK(cudaSetDevice(h->cfg.device));

    RowDist *tdist = (RowDist *)h->dists.p;
    RowDist *ddist = tdist + (size_t)S * (L + 1);
    // phase one: a distribution descriptor per target row, then per draft row
    for (int which = 0; which < 2; which++) {
        const int per = which == 0 ? L + 1 : L;
        const void *logits = which == 0 ? b->target_logits : b->draft_logits;
        if (per == 0 || logits == nullptr || (which == 1 && b->mode == 1)) continue;
        std::vector<StgRowParams> params((size_t)S * per);
        for (int s = 0; s < S; s++)
            for (int i = 0; i < per; i++) params[(size_t)s * per + i] = b->params[s];
        StgSampleBatch sb;
        memset(&sb, 0, sizeof(sb));
        sb.struct_size = sizeof(sb);
        sb.rows = S * per; sb.vocab = V; sb.logits_dtype = b->logits_dtype; sb.logits = logits; sb.row_stride = V;
        sb.params = params.data();
        sb.logit_softcap = which == 0 ? b->target_softcap : b->draft_softcap;
        BatchExtra x;
        x.mode = 2;
        x.dists_out = which == 0 ? tdist : ddist;
        int rc = run_batch(h, &sb, x, stream);
        if (rc) return rc;
    }
    const void *p;
    int rc = stage_in(h, b->draft_tokens, (size_t)S * L * 4, b->mem_flags & STG_MEM_HOST_DRAFT, h->sp_draft, stream, &p);
    if (rc) return rc;
    SpecArgs a;
    memset(&a, 0, sizeof(a));
    a.draft_tokens = (const int32_t *)p;
    rc = stage_in(h, b->uniforms, (size_t)S * (L + 2) * 8, b->mem_flags & STG_MEM_HOST_UNIFORMS, h->sp_uniforms, stream, &p);
    if (rc) return rc;
    a.uniforms = (const double *)p;
    const bool host_out = b->mem_flags & STG_MEM_HOST_OUTPUTS;
    a.target = b->target_logits; a.draft = b->mode == 0 ? b->draft_logits : nullptr;
    a.tdist = tdist; a.ddist = b->mode == 0 ? ddist : nullptr;
    a.accepted = host_out ? (int32_t *)h->sp_accepted.p : b->accepted;
    a.correction = host_out ? (int32_t *)h->sp_correction.p : b->correction;
    a.accept_probs = b->accept_probs ? (host_out ? (float *)h->sp_aprobs.p : b->accept_probs) : nullptr;
    a.seq_flags = b->seq_flags ? (host_out ? (uint32_t *)h->sp_flags.p : b->seq_flags) : nullptr;
    a.p_min = b->p_min;
    a.target_cap = b->target_softcap; a.draft_cap = b->draft_softcap;
    a.n_seq = S; a.n_draft = L; a.vocab = V; a.dtype = b->logits_dtype; a.mode = b->mode;
    a.vec = rows_aligned2(b->target_logits, V, b->logits_dtype) &&
            (!b->draft_logits || rows_aligned2(b->draft_logits, V, b->logits_dtype)) ? 4 : 1;
    // The flat form (stg_flat_full.cu) takes every sequence it can - up to 32 draft tokens, the handle's
    // full-row workspace, rows the sub-tile machinery covers - and flags the few that need one of the
    // draw's fall-backs; k_spec_finish then does exactly those (all of them when the flat form is off).
    cudaError_t e = cudaSuccess;
    static const bool no_flat_spec = getenv("STG_NO_FLAT_SPEC") != nullptr;
    const bool rows_ok = rows_aligned2(b->target_logits, V, b->logits_dtype) &&
                         (!b->draft_logits || rows_aligned2(b->draft_logits, V, b->logits_dtype));
    if (!no_flat_spec && !getenv("STG_NO_FLAT") && S <= h->full_cap && h->fw_rows.p && L <= 32 && rows_ok && V >= 4096 &&
        V <= kSub * kMaxSubTiles && h->sp_rowstats.p) {
        FullWs ws;
        memset(&ws, 0, sizeof(ws));
        ws.rows = (FullRow *)h->fw_rows.p; ws.e = (float *)h->fw_e.p; ws.e_stride = h->escratch_stride;
        ws.ew = (Emul2Work *)h->fw_ew.p;
        int32_t *fallback = (int32_t *)((char *)h->sp_rowstats.p + (size_t)S * 16);
        e = launch_spec_flat(a, ws, h->sp_rowstats.p, fallback, stream);
        if (e != cudaSuccess) return cuda_fail(h, e, "flat verification launch");
        h->stats.kernel_launches += 3;
        a.only = fallback;
    }
    e = launch_spec_finish(a, stream);
    if (e != cudaSuccess) return cuda_fail(h, e, "k_spec_finish launch");
    h->stats.kernel_launches++;
    h->stats.sequences_verified += S;
    if (host_out) {
        CK(cudaMemcpyAsync(b->accepted, a.accepted, (size_t)S * 4, cudaMemcpyDeviceToHost, stream));
        CK(cudaMemcpyAsync(b->correction, a.correction, (size_t)S * 4, cudaMemcpyDeviceToHost, stream));
        if (b->accept_probs) CK(cudaMemcpyAsync(b->accept_probs, a.accept_probs, (size_t)S * L * 4, cudaMemcpyDeviceToHost, stream));
        if (b->seq_flags) CK(cudaMemcpyAsync(b->seq_flags, a.seq_flags, (size_t)S * 4, cudaMemcpyDeviceToHost, stream));
        CK(cudaStreamSynchronize(stream));
    }
    return STG_OK;
}

int stg_mtp_accept(StgHandle h, const void *logits, int32_t dtype, int32_t rows, int32_t vocab, int64_t row_stride,
                   const int32_t *draft, float p_min, int32_t *accept, int32_t *argmax, float *prob, void *stream)
{
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (!logits || !draft || !accept || rows < 0 || vocab <= 0 || row_stride < vocab)
        return fail(h, STG_ERR_INVALID_ARGUMENT, "bad arguments to stg_mtp_accept");
    if (dtype != STG_DTYPE_F32 && dtype != STG_DTYPE_BF16) return fail(h, STG_ERR_INVALID_ARGUMENT, "unknown logits_dtype");
    if (rows == 0) return STG_OK;
    CK(cudaSetDevice(h->cfg.device));
    cudaError_t e = launch_mtp_accept(logits, dtype, rows, vocab, row_stride, rows_aligned2(logits, row_stride, dtype) ? 4 : 1,
                                      draft, p_min, accept, argmax, prob, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(h, e, "k_mtp_accept launch");
    h->stats.kernel_launches++;
    return STG_OK;
}

}  // extern "C"

namespace {

// shared by the two draws on caller-held distributions: stages uniforms, launches, returns tokens
int draw_rows(StgHandle h, const float *p, const float *q, int32_t rows, int32_t vocab, int64_t row_stride,
              const float *uniforms, int per_row, int32_t *tokens, uint32_t *row_flags, uint32_t mem_flags, void *stream_)
{
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (!p || (per_row == 2 && !q) || !uniforms || !tokens || rows < 0 || vocab <= 0 || row_stride < vocab)
        return fail(h, STG_ERR_INVALID_ARGUMENT, "bad arguments to a draw on caller-held distributions");
    if (rows > h->cfg.max_rows) return fail(h, STG_ERR_CAPACITY, "rows exceed max_rows");
    if (rows == 0) return STG_OK;
    CK(cudaSetDevice(h->cfg.device));
    const void *u;
    int rc = stage_in(h, uniforms, (size_t)rows * per_row * 4, mem_flags & STG_MEM_HOST_UNIFORMS, h->st_uniforms, stream, &u);
    if (rc) return rc;
    const bool host_out = mem_flags & STG_MEM_HOST_OUTPUTS;
    int32_t *d_tok = host_out ? (int32_t *)h->o_tokens.p : tokens;
    uint32_t *d_fl = row_flags ? (host_out ? (uint32_t *)h->o_flags.p : row_flags) : nullptr;
    cudaError_t e = per_row == 2 ? launch_residual_draw(p, q, rows, vocab, row_stride, (const float *)u, d_tok, d_fl, stream)
                                 : launch_probs_draw(p, rows, vocab, row_stride, (const float *)u, d_tok, d_fl, stream);
    if (e != cudaSuccess) return cuda_fail(h, e, "draw kernel launch");
    h->stats.kernel_launches++;
    if (host_out) {
        CK(cudaMemcpyAsync(tokens, d_tok, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream));
        if (row_flags) CK(cudaMemcpyAsync(row_flags, d_fl, (size_t)rows * 4, cudaMemcpyDeviceToHost, stream));
        CK(cudaStreamSynchronize(stream));
    }
    return STG_OK;
}

}  // namespace

extern "C" int stg_sample_from_probs(StgHandle h, const float *probs, int32_t rows, int32_t vocab, int64_t row_stride,
                                     const float *uniforms, int32_t *tokens, uint32_t *row_flags, uint32_t mem_flags,
                                     void *stream)
{
    return draw_rows(h, probs, nullptr, rows, vocab, row_stride, uniforms, 1, tokens, row_flags, mem_flags, stream);
}

extern "C" int stg_resample_residual(StgHandle h, const float *p, const float *q, int32_t rows, int32_t vocab,
                                     int64_t row_stride, const float *uniforms, int32_t *tokens, uint32_t *row_flags,
                                     uint32_t mem_flags, void *stream)
{
    return draw_rows(h, p, q, rows, vocab, row_stride, uniforms, 2, tokens, row_flags, mem_flags, stream);
}

extern "C" {

// ---- vocabulary-sharded mode ---------------------------------------------------------------------

int stg_comm_unique_id(void *out_id128)
{
    std::string why;
    if (!out_id128) return STG_ERR_INVALID_ARGUMENT;
    if (!load_nccl(why)) return fail(nullptr, STG_ERR_NCCL, why);
    NcclId id;
    int rc = g_nccl.get_unique_id(&id);
    if (rc != 0) return nccl_fail(nullptr, rc, "ncclGetUniqueId");
    memcpy(out_id128, &id, sizeof(id));
    return STG_OK;
}

int stg_comm_init(StgHandle h, const void *id128, int32_t rank, int32_t n_ranks)
{
    if (!h || !id128 || n_ranks < 1 || rank < 0 || rank >= n_ranks) return fail(h, STG_ERR_INVALID_ARGUMENT, "bad communicator arguments");
    std::string why;
    if (!load_nccl(why)) return fail(h, STG_ERR_NCCL, why);
    CK(cudaSetDevice(h->cfg.device));
    NcclId id;
    memcpy(&id, id128, sizeof(id));
    void *comm = nullptr;
    int rc = g_nccl.comm_init_rank(&comm, n_ranks, id, rank);
    if (rc != 0) return nccl_fail(h, rc, "ncclCommInitRank");
    h->nccl_comm = comm;
    h->rank = rank;
    h->n_ranks = n_ranks;
    return ensure_exchange(h, n_ranks);
}

int stg_comm_destroy(StgHandle h)
{
    if (h && h->nccl_comm && g_nccl.comm_destroy) {
        g_nccl.comm_destroy(h->nccl_comm);
        h->nccl_comm = nullptr;
    }
    return STG_OK;
}

int stg_shard_select(StgHandle h, const StgSampleBatch *b, int32_t vocab_offset, int32_t global_vocab, void *stream)
{
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    int rc = ensure_exchange(h, h->n_ranks);
    if (rc) return rc;
    BatchExtra x;
    x.shard_mode = 1;
    x.vocab_offset = vocab_offset;
    x.global_vocab = global_vocab;
    return run_batch(h, b, x, stream);
}

int stg_shard_allgather(StgHandle h, void *stream)
{
    if (!h) return STG_ERR_INVALID_ARGUMENT;
    if (!h->nccl_comm) return fail(h, STG_ERR_NCCL, "stg_comm_init has not been called");
    if (h->shard_block_bytes == 0) return fail(h, STG_ERR_INVALID_ARGUMENT, "stg_shard_select has not been called");
    // ONE collective per step: every rank's keys and counts travel in the same block, and the block
    // is as large as this step's selection counts need, not as the handle's capacities allow
    int rc = g_nccl.all_gather(h->xchg_local.p, h->xchg_gather.p, h->shard_block_bytes, 1 /* ncclUint8 */, h->nccl_comm,
                               (cudaStream_t)stream);
    if (rc != 0) return nccl_fail(h, rc, "ncclAllGather(candidates)");
    h->stats.kernel_launches++;
    return STG_OK;
}

int stg_shard_exchange_bytes(StgHandle h, uint64_t *out_bytes)
{
    if (!h || !out_bytes) return STG_ERR_INVALID_ARGUMENT;
    *out_bytes = (uint64_t)h->shard_block_bytes;
    return STG_OK;
}

int stg_shard_gather_local(StgHandle h, const StgHandle *peers, int32_t n_ranks, void *stream_)
{
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!h || !peers || n_ranks < 1) return STG_ERR_INVALID_ARGUMENT;
    h->n_ranks = n_ranks;
    int rc = ensure_exchange(h, n_ranks);
    if (rc) return rc;
    if (!peers[0]) return fail(h, STG_ERR_INVALID_ARGUMENT, "peer handle is null");
    h->shard_rows_used = peers[0]->shard_rows_used;
    h->shard_stride_used = peers[0]->shard_stride_used;
    h->shard_block_bytes = peers[0]->shard_block_bytes;
    const size_t lb = h->shard_block_bytes;
    for (int r = 0; r < n_ranks; r++) {
        StgHandle p = peers[r];
        if (!p || p->shard_block_bytes != lb || p->shard_rows_used != h->shard_rows_used || !p->xchg_local.p)
            return fail(h, STG_ERR_INVALID_ARGUMENT, "peer handles must have selected the same batch shape");
        CK(cudaMemcpyAsync((char *)h->xchg_gather.p + lb * r, p->xchg_local.p, lb, cudaMemcpyDeviceToDevice, stream));
    }
    return STG_OK;
}

int stg_shard_finish(StgHandle h, const StgSampleBatch *b, int32_t global_vocab, void *stream_)
{
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!h || !b) return STG_ERR_INVALID_ARGUMENT;
    if (!h->xchg_gather.p) return fail(h, STG_ERR_INVALID_ARGUMENT, "nothing has been gathered");
    // Re-plan with the same inputs as stg_shard_select (row paths, selection counts, pow table);
    // only the arrays the finish reads are staged.
    BatchExtra x;
    x.shard_mode = 2;
    x.global_vocab = global_vocab;
    return run_batch(h, b, x, stream);
}

}  // extern "C"
