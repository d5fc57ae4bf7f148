// The finish of one chunked row of the flat step by one CTA (shared by the full-size kernel in
// stg_flat.cu and the half-size one in stg_flat_finish_half.cu, which is built with 512 threads).
#pragma once
#include <math_constants.h>

#include "stg_flat.cuh"
#include "stg_select.cuh"

namespace stg {

struct FlatShared {
    FinishOut fout;
    int ok;
};

// One row of the flat step by one CTA: any top_k, any penalties, and the second chance of a row whose
// candidate list failed its check.  `cap`: entries per candidate buffer in `arena`, at least
// N + 4096 + 512; a list longer than that is reduced as it is read in (sel_append_keys).
template <bool BF16>
__device__ void flat_finish_row(const SampleArgs &a, FlatRow *fr, int row, int item, int cap, unsigned char *arena, SelCtl &ctl,
                                FlatShared &fs)
{
    const RowPlan rp = a.plans[row];
    const int esz = BF16 ? 2 : 4;
    const LogitRow rowp{(const char *)a.logits + (int64_t)row * a.row_stride * esz, a.softcap};
    if (rp.path == kPathGreedy) {
        if (a.shard_mode == 1) {
            // vocabulary-sharded mode: this rank's best (value, global token) goes to the exchange buffer
            // (the streaming kernel numbers tokens by column; the global id is column + vocab_offset, and
            // a key's low half holds ~token, so the offset is subtracted)
            if (threadIdx.x == 0) {
                const unsigned long long key = fr[row].key;
                fr[row].key = 0ull;  // consumed: keys are zero between steps (stg_flat_greedy.cu starts from that)
                a.xchg_local[(int64_t)row * a.xchg_stride] = key ? key - (unsigned long long)a.vocab_offset : 0ull;
                a.xchg_count[row] = key ? 1 : 0;
            }
            return;
        }
        if (threadIdx.x == 0) {
            const unsigned long long key = fr[row].key;
            fr[row].key = 0ull;  // consumed: keys are zero between steps (stg_flat_greedy.cu starts from that)
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
        return;
    }
    const uint32_t *mrow = (rp.use_mask && a.mask) ? a.mask + (int64_t)row * a.mask_stride : nullptr;
    unsigned long long *tk = a.phase_ticks ? a.phase_ticks + (int64_t)(a.item_base + item) * 32 : nullptr;
    tick(tk, 0);
    Sel s;
    s.c = &ctl;
    s.buf[0] = (u64 *)arena;
    s.buf[1] = s.buf[0] + cap;
    s.cap = cap;
    s.n = rp.sel;
    s.idx_off = a.vocab_offset;
    sel_reset(s);
    if (threadIdx.x == 0) {
        const FlatRow f = fr[row];
        fs.ok = (f.cnt >= rp.sel && f.cnt <= f.cap && f.tau > -CUDART_INF_F) ? f.cnt : -1;
    }
    __syncthreads();
    const int cnt = fs.ok;
    if (cnt >= 0) {
        // the list holds exactly the logits above the bound, N or more of them: a superset of the N best
        // (when no penalty can promote a logit the finish works on the whole list, see finish_topk_select)
        sel_append_keys(s, a.cand + rp.cand_off, cnt, !(rp.top_k <= kFastFinishK && penalties_only_demote(rp)));
    } else {
        // the bound was off (or dropped candidates): the row is read again by this CTA, with a generous
        // bound first (about 8 N survivors, capacity permitting) and the exact selection behind it
        const int over = (int)max(5ll, min(16ll, (long long)s.cap / max(s.n, 1)));
        const FlatRow f = fr[row];
        bool preset = false;
        float bound = 0.f;
        if (f.tau > -CUDART_INF_F && f.cnt > f.cap && f.cap > rp.sel && f.cap <= s.cap) {
            // too many passed the first bound: the list kept f.cap of them, some subset.  The N-th best of a
            // subset is no higher than the N-th best of the row, so everything at or above it is a superset of
            // the row's best N - and a far smaller one than before
            sel_append_keys(s, a.cand + rp.cand_off, f.cap, false);
            sel_raise(s);
            const uint32_t o = ord32(ctl.tau);
            bound = unord32(o > 0u ? o - 1u : 0u);  // the next value below: the strict test then keeps ties with the bound
            preset = true;
            __syncthreads();
            sel_reset(s);
        }
        sel_stream_generous<4, BF16>(s, rowp, mrow, 0, a.vocab, over, preset, bound);
    }
    if (a.shard_mode == 1) {
        // vocabulary-sharded mode: hand this rank's best `sel` survivors to the exchange buffer
        __syncthreads();
        if (ctl.cnt > rp.sel) sel_compact(s);
        const int m = ctl.cnt;
        const u64 *src = s.buf[ctl.cur];
        u64 *dst = a.xchg_local + (int64_t)row * a.xchg_stride;
        // keys from the streaming kernel's list carry column numbers, keys of a second pass global ids
        const u64 shift = cnt >= 0 ? (u64)a.vocab_offset : 0ull;
        for (int e = threadIdx.x; e < m; e += kThreads) dst[e] = src[e] - shift;
        if (threadIdx.x == 0) a.xchg_count[row] = m;
        return;
    }
    tick(tk, 1);
    if (tk && threadIdx.x == 0) { tk[8] = (unsigned long long)(long long)cnt; tk[9] = (unsigned long long)fr[row].cnt; tk[10] = (unsigned long long)fr[row].cap; }
    const int32_t *hist = a.hist_ids ? a.hist_ids + rp.hist_off : nullptr;
    const float *ptab = (a.pow_tab && rp.pow_off >= 0) ? a.pow_tab + rp.pow_off : nullptr;
    const float u = a.uniforms ? __ldg(a.uniforms + row) : 0.5f;
    const int64_t o = (int64_t)row * a.topk_stride;
    finish_topk(s, rp, hist, ptab, u, &fs.fout, a.topk_ids ? a.topk_ids + o : nullptr,
                a.topk_logits ? a.topk_logits + o : nullptr, a.topk_probs ? a.topk_probs + o : nullptr, tk);
    tick(tk, 3);
    if (threadIdx.x == 0) {
        a.tokens[row] = fs.fout.token;
        if (a.token_probs) a.token_probs[row] = fs.fout.prob;
        const uint32_t fl = fs.fout.flags | (cnt < 0 ? kFlagFlatRedo : 0u);
        if (a.row_flags) a.row_flags[row] = fl;
        count_row_flags(a.counters, fl);
    }
}


}  // namespace stg
