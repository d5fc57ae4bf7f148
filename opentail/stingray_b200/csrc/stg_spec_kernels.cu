// Second phase of speculative verification and the MTP accept rule.
//
// Phase one (k_sample in descriptor mode) leaves a RowDist per target and draft row, from which
// p[i] and q[i] are evaluated pointwise out of the logits.  k_spec_finish then runs, per sequence,
// the accept chain of SpeculativeDecoder.StepSampled
// (src/OpenTail.Stingray.Engine/SpeculativeDecoder.cs:532-559) and the one draw it ends with:
// ResampleResidual (Sampler.cs:587-618), a draw from p, or the bonus draw.  The sequential fp32
// sums of those draws are reproduced exactly by emul_scan.
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "stg_launch.h"
#include "stg_rowdist.cuh"
#include "stg_spec_prov.cuh"

namespace stg {

struct SpecShared {
    EmulCtl em;
    Emul2Ctl em2;
    int accepted;
    int bad_draft;
    int red_i[32];
};

template <bool BF16>
__global__ void __launch_bounds__(kThreads, 1) k_spec_finish(const __grid_constant__ SpecArgs a)
{
    __shared__ SpecShared sh;
    extern __shared__ __align__(16) unsigned char spec_dyn[];
    Emul2Work *wk2 = (Emul2Work *)spec_dyn;
    const int tid = threadIdx.x;
    const int s = blockIdx.x;
    if (a.only != nullptr && a.only[s] == 0) return;  // the flat form has finished this sequence
    const int L = a.n_draft, V = a.vocab;
    const int esz = BF16 ? 2 : 4;
    const RowDist *td = a.tdist + (int64_t)s * (L + 1);
    const RowDist *dd = a.ddist ? a.ddist + (int64_t)s * L : nullptr;
    const char *trows = (const char *)a.target + (int64_t)s * (L + 1) * V * esz;
    const char *drows = a.draft ? (const char *)a.draft + (int64_t)s * L * V * esz : nullptr;
    const double *u = a.uniforms + (int64_t)s * (L + 2);
    const bool greedy = (td[0].flags & kDistOneHot) != 0;

    if (tid == 0) {
        int acc = 0;
        bool bad_draft = false;
        for (int i = 0; i < L; i++) {
            const int tok = a.draft_tokens[(int64_t)s * L + i];
            bool ok;
            float shown;
            if ((unsigned)tok >= (unsigned)V) {
                // a draft token outside the vocabulary (the reference's pDist[tokens[i]] throws,
                // SpeculativeDecoder.cs:534): never read, rejected, and reported in the flags
                ok = false;
                shown = 0.f;
                bad_draft = true;
            } else if (greedy) {
                // SpeculativeDecoder.Step, SpeculativeDecoder.cs:400-405
                ok = (tok == td[i].tie_idx_max);
                shown = ok ? 1.f : 0.f;
            } else {
                const float px = eval_point<BF16>(LogitRow{trows + (int64_t)i * V * esz, a.target_cap}, tok, td[i]);
                if (a.mode == 0) {
                    const float qx = eval_point<BF16>(LogitRow{drows + (int64_t)i * V * esz, a.draft_cap}, tok, dd[i]);
                    const float r = qx > 0.f ? fminf(1.f, __fdiv_rn(px, qx)) : (px > 0.f ? 1.f : 0.f);
                    ok = u[i] < (double)r;
                    shown = r;
                } else {
                    ok = px >= a.p_min || tok == td[i].argmax;
                    shown = px;
                }
            }
            if (a.accept_probs) a.accept_probs[(int64_t)s * L + i] = shown;
            if (!ok) break;
            acc++;
        }
        // positions after the first rejection are not tested
        if (a.accept_probs)
            for (int i = acc + 1; i < L; i++) a.accept_probs[(int64_t)s * L + i] = 0.f;
        sh.accepted = acc;
        sh.bad_draft = bad_draft ? 1 : 0;
    }
    __syncthreads();
    const int acc = sh.accepted;
    uint32_t fl = sh.bad_draft ? (1u << 9) : 0u;
    int corr;
    if (greedy) {
        corr = td[acc].tie_idx_max;
    } else {
        const bool al = a.vec == 4;
        const LogitRow prow{trows + (int64_t)acc * V * esz, a.target_cap};
        ProvRow<BF16> pp{SrcLogits<BF16>{prow, nullptr, al, td[acc].inv_t, td[acc].inv_t != 1.0f}, td[acc]};
        const float u0 = __double2float_rn(u[L]);
        const float u1 = __double2float_rn(u[L + 1]);
        float cum;
        if (acc == L || a.mode == 1) {
            // bonus draw from the last target row (:555-559), or a draw from p after a looser-rule
            // rejection (:552): SampleFromDistribution, Sampler.cs:564-576
            corr = emul_any<ProvRow<BF16>, false>(&sh.em, &sh.em2, wk2, pp, V, u0, true, &cum);
            if (corr < 0) { corr = V - 1; fl |= (1u << 5); }
        } else {
            const LogitRow qrow{drows + (int64_t)acc * V * esz, a.draft_cap};
            ProvRow<BF16> qq{SrcLogits<BF16>{qrow, nullptr, al, dd[acc].inv_t, dd[acc].inv_t != 1.0f}, dd[acc]};
            ProvResidual<BF16> rr{pp, qq};
            float sum;
            emul_any<ProvResidual<BF16>, true>(&sh.em, &sh.em2, wk2, rr, V, 0.f, false, &sum);
            if (sum <= 0.f || isnan(sum)) {
                corr = emul_any<ProvRow<BF16>, false>(&sh.em, &sh.em2, wk2, pp, V, u0, true, &cum);
                if (corr < 0) { corr = V - 1; fl |= (1u << 5); }
                fl |= (1u << 8);  // empty residual
            } else {
                const float target = __fmul_rn(u0, sum);
                corr = emul_any<ProvResidual<BF16>, true>(&sh.em, &sh.em2, wk2, rr, V, target, true, &cum);
                if (corr < 0) {
                    // rounding fallback: the last token with a positive residual
                    int lastp = -1;
                    for (int base = tid * 8; base < V; base += kThreads * 8) {
                        float x[8];
                        rr.load(base, V, x);
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            if (base + j < V && x[j] > 0.f) lastp = base + j;
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) lastp = max(lastp, __shfl_xor_sync(0xFFFFFFFFu, lastp, o));
                    __syncthreads();
                    if ((tid & 31) == 0) sh.red_i[tid >> 5] = lastp;
                    __syncthreads();
                    lastp = -1;
                    for (int w = 0; w < 32; w++) lastp = max(lastp, sh.red_i[w]);
                    fl |= (1u << 5);
                    if (lastp >= 0) {
                        corr = lastp;
                    } else {
                        corr = emul_any<ProvRow<BF16>, false>(&sh.em, &sh.em2, wk2, pp, V, u1, true, &cum);
                        if (corr < 0) corr = V - 1;
                    }
                }
            }
        }
    }
    if (tid == 0) {
        a.accepted[s] = acc;
        a.correction[s] = corr;
        if (a.seq_flags) a.seq_flags[s] = fl;
    }
}

cudaError_t launch_spec_finish(const SpecArgs &a, cudaStream_t stream)
{
    if (a.dtype == 1) k_spec_finish<true><<<a.n_seq, kThreads, sizeof(Emul2Work), stream>>>(a);
    else k_spec_finish<false><<<a.n_seq, kThreads, sizeof(Emul2Work), stream>>>(a);
    return cudaGetLastError();
}

// ---- draws on caller-held distributions -------------------------------------------------------------
struct ProvPlain {  // a probability row as it is
    const float *p;
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
#pragma unroll
        for (int j = 0; j < 8; j++) x[j] = (base + j < n) ? __ldg(p + base + j) : 0.f;
    }
    __device__ __forceinline__ void reload(int base, int n, float x[8]) const { load(base, n, x); }
};
struct ProvPlainResidual {  // positive part of p - q
    const float *p, *q;
    __device__ __forceinline__ void load(int base, int n, float x[8]) const
    {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float r = (base + j < n) ? __fsub_rn(__ldg(p + base + j), __ldg(q + base + j)) : 0.f;
            x[j] = r > 0.f ? r : 0.f;
        }
    }
    __device__ __forceinline__ void reload(int base, int n, float x[8]) const { load(base, n, x); }
};

// SampleFromDistribution (Sampler.cs:564-576), one CTA per row
__device__ __forceinline__ int draw_from_probs(SpecShared &sh, Emul2Work *wk2, const float *row, int n, float u, uint32_t &fl)
{
    if (!(u > 0.f)) return 0;  // r <= cum holds at the first token whatever its probability
    ProvPlain pp{row};
    float cum;
    int tok = emul_any<ProvPlain, false>(&sh.em, &sh.em2, wk2, pp, n, u, true, &cum);
    if (tok < 0) { tok = n - 1; fl |= (1u << 5); }
    return tok;
}

__global__ void __launch_bounds__(kThreads, 1) k_probs_draw(const float *probs, int vocab, int64_t row_stride,
                                                            const float *uniforms, int32_t *tokens, uint32_t *flags)
{
    __shared__ SpecShared sh;
    extern __shared__ __align__(16) unsigned char spec_dyn[];
    const int row = blockIdx.x;
    uint32_t fl = 0u;
    const int tok = draw_from_probs(sh, (Emul2Work *)spec_dyn, probs + (int64_t)row * row_stride, vocab, __ldg(uniforms + row), fl);
    if (threadIdx.x == 0) {
        tokens[row] = tok;
        if (flags) flags[row] = fl;
    }
}

// ResampleResidual (Sampler.cs:587-618), one CTA per row
__global__ void __launch_bounds__(kThreads, 1) k_residual_draw(const float *p, const float *q, int vocab, int64_t row_stride,
                                                               const float *uniforms2, int32_t *tokens, uint32_t *flags)
{
    __shared__ SpecShared sh;
    extern __shared__ __align__(16) unsigned char spec_dyn[];
    Emul2Work *wk2 = (Emul2Work *)spec_dyn;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float *pr = p + (int64_t)row * row_stride, *qr = q + (int64_t)row * row_stride;
    const float u0 = __ldg(uniforms2 + 2 * row), u1 = __ldg(uniforms2 + 2 * row + 1);
    ProvPlainResidual rr{pr, qr};
    uint32_t fl = 0u;
    int tok;
    float sum, cum;
    emul_any<ProvPlainResidual, true>(&sh.em, &sh.em2, wk2, rr, vocab, 0.f, false, &sum);
    if (sum <= 0.f || isnan(sum)) {
        fl |= (1u << 8);  // empty residual: a draw from p
        tok = draw_from_probs(sh, wk2, pr, vocab, u0, fl);
    } else {
        const float target = __fmul_rn(u0, sum);
        tok = emul_any<ProvPlainResidual, true>(&sh.em, &sh.em2, wk2, rr, vocab, target, true, &cum);
        if (tok < 0) {
            // rounding fallback: the last token with a positive residual
            int lastp = -1;
            for (int base = tid * 8; base < vocab; base += kThreads * 8) {
                float x[8];
                rr.load(base, vocab, x);
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (base + j < vocab && x[j] > 0.f) lastp = base + j;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) lastp = max(lastp, __shfl_xor_sync(0xFFFFFFFFu, lastp, o));
            __syncthreads();
            if ((tid & 31) == 0) sh.red_i[tid >> 5] = lastp;
            __syncthreads();
            lastp = -1;
            for (int w = 0; w < 32; w++) lastp = max(lastp, sh.red_i[w]);
            fl |= (1u << 5);
            tok = lastp >= 0 ? lastp : draw_from_probs(sh, wk2, pr, vocab, u1, fl);
        }
    }
    if (tid == 0) {
        tokens[row] = tok;
        if (flags) flags[row] = fl;
    }
}

cudaError_t launch_probs_draw(const float *probs, int rows, int vocab, int64_t row_stride, const float *uniforms,
                              int32_t *tokens, uint32_t *flags, cudaStream_t stream)
{
    k_probs_draw<<<rows, kThreads, sizeof(Emul2Work), stream>>>(probs, vocab, row_stride, uniforms, tokens, flags);
    return cudaGetLastError();
}

cudaError_t launch_residual_draw(const float *p, const float *q, int rows, int vocab, int64_t row_stride,
                                 const float *uniforms2, int32_t *tokens, uint32_t *flags, cudaStream_t stream)
{
    k_residual_draw<<<rows, kThreads, sizeof(Emul2Work), stream>>>(p, q, vocab, row_stride, uniforms2, tokens, flags);
    return cudaGetLastError();
}

// MtpDecoder.AcceptDraft + SoftmaxProbAt, src/OpenTail.Stingray.Engine/MtpDecoder.cs:562-596
template <bool BF16>
__global__ void __launch_bounds__(kThreads) k_mtp_accept(const void *logits, int vocab, int64_t row_stride, int vec,
                                                         const int32_t *draft, float p_min, int32_t *accept,
                                                         int32_t *argmax, float *prob)
{
    __shared__ u64 red_k[32];
    __shared__ double red_d[32];
    const int row = blockIdx.x, tid = threadIdx.x;
    const int esz = BF16 ? 2 : 4;
    const LogitRow rowp{(const char *)logits + (int64_t)row * row_stride * esz, 0.f};
    SrcLogits<BF16> raw{rowp, nullptr, vec == 4, 1.f, false};
    const u64 mk = pass_max(raw, vocab, red_k);
    const int am = mk ? key_idx(mk) : 0;
    const int d = draft[row];
    if (p_min <= 0.f) p_min = 1.f;  // MtpDecoder.cs:225
    int ok = 0;
    float pr = 0.f;
    if (d == am) {
        ok = 1;
    } else if (p_min < 1.0f) {
        // the maximum as SoftmaxProbAt's scan finds it (seeded with logits[0])
        const float mx = mk ? key_val(mk) : load_one<BF16>(rowp, 0);
        double part = 0.0;
        for (int base = tid * 8; base < vocab; base += kThreads * 8) {
            float x[8];
            raw.get8(base, vocab, x);
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (base + j < vocab) part += exp((double)__fsub_rn(x[j], mx));
        }
        const double sum = block_sum_double(part, red_d);
        if (!(sum <= 0.0) && !isnan(sum) && (unsigned)d < (unsigned)vocab)
            pr = (float)(exp((double)__fsub_rn(load_one<BF16>(rowp, d), mx)) / sum);
        ok = pr >= p_min;
    }
    if (tid == 0) {
        accept[row] = ok;
        if (argmax) argmax[row] = am;
        if (prob) prob[row] = pr;
    }
}

cudaError_t launch_mtp_accept(const void *logits, int dtype, int rows, int vocab, int64_t row_stride, int vec,
                              const int32_t *draft, float p_min, int32_t *accept, int32_t *argmax, float *prob,
                              cudaStream_t stream)
{
    if (dtype == 1) k_mtp_accept<true><<<rows, kThreads, 0, stream>>>(logits, vocab, row_stride, vec, draft, p_min, accept, argmax, prob);
    else k_mtp_accept<false><<<rows, kThreads, 0, stream>>>(logits, vocab, row_stride, vec, draft, p_min, accept, argmax, prob);
    return cudaGetLastError();
}

}  // namespace stg
