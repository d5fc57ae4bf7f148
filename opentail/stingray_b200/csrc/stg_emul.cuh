// Block-parallel, bit-exact emulation of a SEQUENTIAL fp32 running sum.
//
// The reference accumulates probabilities one by one in fp32, in index order
// (Softmax, src/OpenTail.Stingray.Engine/Sampler.cs:460-465; SampleFromDistribution, :567-573;
// ApplyTopP's cumulative cut, :536-546; ResampleResidual, :594-614).  Which token a uniform lands
// on depends on every rounding of that running sum, so a tree reduction or an fp64 sum does not
// reproduce it.  This file does, in parallel:
//
//   while the running sum s stays inside one binade [2^E, 2^(E+1)) it is an integer multiple of
//   u = 2^(E-23), and fl(s + x) = s + rn_u(x): x rounded to a multiple of u, ties to the multiple
//   that makes the new sum even.  So inside a binade the sequential sum is an INTEGER sum, whose
//   only order dependence is the parity rule for exact ties; an element is therefore the pair
//   (d0, d1) = increment if the sum before it is even / odd, pairs compose associatively, and a
//   block-wide scan gives every intermediate sum.  The first element whose addition leaves the
//   binade is added with a real fp32 add, after which the scan restarts in the new binade.
#pragma once
#include <cuda_runtime.h>
#include <limits.h>
#include <stdint.h>

#include "stg_types.h"

namespace stg {

struct EmulCtl {
    float s;      // running sum so far (bit-exact)
    int start;    // first element not yet added
    int event;    // first element of the tile that leaves the binade or reaches the target
    int hit;      // element at which the target was reached, -1 if none yet
    int wa0[32], wa1[32];
};

static __device__ __forceinline__ int sat_add(int a, int b)
{
    int s = a + b;
    return s > (1 << 28) ? (1 << 28) : s;
}

// (a0, a1) then (b0, b1): offset for an even / odd starting sum
static __device__ __forceinline__ void comp(int a0, int a1, int b0, int b1, int &r0, int &r1)
{
    r0 = sat_add(a0, (a0 & 1) ? b1 : b0);
    r1 = sat_add(a1, ((1 + a1) & 1) ? b1 : b0);
}

// increments of x >= 0 in units of 2^(eb-150), eb the biased exponent of the running sum (>= 1)
static __device__ __forceinline__ void unit_incr(float x, int eb, int &d0, int &d1)
{
    uint32_t xb = __float_as_uint(x);
    if (!(x > 0.f)) { d0 = d1 = 0; return; }  // zero, negative or NaN terms add nothing here
    int xe = (int)(xb >> 23) & 255;
    uint32_t m = xb & 0x7FFFFFu;
    if (xe) m |= 0x800000u; else xe = 1;
    int shift = eb - xe;
    if (shift < 0 || xe == 255) { d0 = d1 = 1 << 24; return; }  // x alone leaves the binade
    if (shift == 0) { d0 = d1 = (int)m; return; }
    if (shift > 24) { d0 = d1 = 0; return; }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half) { d0 = d1 = (int)q + 1; }
    else if (rem < half) { d0 = d1 = (int)q; }
    else { d0 = (int)(q + (q & 1u)); d1 = (int)(q + 1u - (q & 1u)); }
}

// Runs s = fl(s + x_i) for i = 0..n-1 with s starting at 0 and returns the first i at which
// s >= target (the reference's `r <= cum` / `cum >= topP` tests), or -1.  *sum_out receives s at
// the hit, or the final sum.  POS_ONLY: only elements > 0 are added and tested (ResampleResidual).
// Prov::load(int base, int n, float x[kEmulItems]) yields elements base..base+7 (0 beyond n).
template <class Prov, bool POS_ONLY>
static __device__ int emul_scan(EmulCtl *c, const Prov &pv, int n, float target, bool has_target,
                         float *sum_out)
{
    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    __syncthreads();
    if (tid == 0) { c->s = 0.f; c->start = 0; c->hit = -1; c->event = INT_MAX; }
    __syncthreads();
    for (int tile0 = 0; tile0 < n; tile0 += kEmulTile) {
        float x[kEmulItems];
        const int g0 = tile0 + tid * kEmulItems;
        pv.load(g0, n, x);
        for (;;) {
            const float s = c->s;
            const int start = c->start;
            const uint32_t sb = __float_as_uint(s);
            const int ef = (int)(sb >> 23) & 255;
            const int eb = ef ? ef : 1;
            const int sint = (int)((sb & 0x7FFFFFu) | (ef ? 0x800000u : 0u));
            const bool frozen = (ef == 255);  // inf / NaN: nothing changes any more
            long long tint = LLONG_MAX;
            if (has_target) {
                double td = ceil(ldexp((double)target, 150 - eb));
                tint = td >= 1073741824.0 ? (1ll << 30) : (td <= -1073741824.0 ? -(1ll << 30) : (long long)td);
            }
            int d0[kEmulItems], d1[kEmulItems];
            int a0 = 0, a1 = 0;
#pragma unroll
            for (int j = 0; j < kEmulItems; j++) {
                int g = g0 + j;
                bool active = g >= start && g < n && !frozen;
                if (active) unit_incr(x[j], eb, d0[j], d1[j]); else { d0[j] = 0; d1[j] = 0; }
                a0 += (a0 & 1) ? d1[j] : d0[j];
                a1 += ((1 + a1) & 1) ? d1[j] : d0[j];
            }
            a0 = min(a0, 1 << 28);
            a1 = min(a1, 1 << 28);
            // inclusive scan over the warp, then over the warps
            int i0 = a0, i1 = a1;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int p0 = __shfl_up_sync(0xFFFFFFFFu, i0, o);
                int p1 = __shfl_up_sync(0xFFFFFFFFu, i1, o);
                if (lane >= o) { int r0, r1; comp(p0, p1, i0, i1, r0, r1); i0 = r0; i1 = r1; }
            }
            int e0 = __shfl_up_sync(0xFFFFFFFFu, i0, 1);
            int e1 = __shfl_up_sync(0xFFFFFFFFu, i1, 1);
            if (lane == 0) { e0 = 0; e1 = 0; }
            if (lane == 31) { c->wa0[warp] = i0; c->wa1[warp] = i1; }
            __syncthreads();
            if (warp == 0) {
                int w0 = c->wa0[lane], w1 = c->wa1[lane];
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    int p0 = __shfl_up_sync(0xFFFFFFFFu, w0, o);
                    int p1 = __shfl_up_sync(0xFFFFFFFFu, w1, o);
                    if (lane >= o) { int r0, r1; comp(p0, p1, w0, w1, r0, r1); w0 = r0; w1 = r1; }
                }
                c->wa0[lane] = w0; c->wa1[lane] = w1;
            }
            __syncthreads();
            int b0 = 0, b1 = 0;
            if (warp > 0) { b0 = c->wa0[warp - 1]; b1 = c->wa1[warp - 1]; }
            int x0, x1;
            comp(b0, b1, e0, e1, x0, x1);
            int S = sat_add(sint, (sint & 1) ? x1 : x0);
            int ev = INT_MAX, sbef = 0, dsel = 0;
            float xsel = 0.f;
#pragma unroll
            for (int j = 0; j < kEmulItems; j++) {
                int g = g0 + j;
                bool active = g >= start && g < n && !frozen && (!POS_ONLY || x[j] > 0.f);
                if (active) {
                    int d = (S & 1) ? d1[j] : d0[j];
                    int sn = sat_add(S, d);
                    bool fire = sn >= (1 << 24) || (long long)sn >= tint;
                    if (fire && ev == INT_MAX) { ev = g; sbef = S; dsel = d; xsel = x[j]; }
                    S = sn;
                }
            }
            if (ev != INT_MAX) atomicMin(&c->event, ev);
            __syncthreads();
            const int first = c->event;
            __syncthreads();  // everyone has read the event before its owner clears it
            if (first == INT_MAX) {
                if (tid == kThreads - 1 && !frozen) c->s = ldexpf((float)S, eb - 150);
                __syncthreads();
                break;  // tile done, no event
            }
            if (ev == first) {
                float snew;
                bool hit;
                if (sbef + dsel < (1 << 24)) {
                    snew = ldexpf((float)(sbef + dsel), eb - 150);
                    hit = true;  // stayed in the binade, so the event is the target
                } else {
                    snew = __fadd_rn(ldexpf((float)sbef, eb - 150), xsel);
                    hit = has_target && snew >= target;
                }
                c->s = snew;
                c->start = first + 1;
                if (hit) c->hit = first;
                c->event = INT_MAX;
            }
            __syncthreads();
            if (c->hit >= 0) {
                if (sum_out) *sum_out = c->s;
                int h = c->hit;
                __syncthreads();
                return h;
            }
        }
    }
    if (sum_out) *sum_out = c->s;
    __syncthreads();
    return -1;
}

// ---- deterministic block sums ----------------------------------------------------------------
static __device__ __forceinline__ double block_sum_double(double v, double *scratch /* 32 */)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        v = scratch[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if (threadIdx.x == 0) scratch[0] = v;
    }
    __syncthreads();
    v = scratch[0];
    __syncthreads();
    return v;
}

static __device__ __forceinline__ int block_sum_int(int v, int *scratch /* 32 */)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        v = scratch[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        if (threadIdx.x == 0) scratch[0] = v;
    }
    __syncthreads();
    v = scratch[0];
    __syncthreads();
    return v;
}

}  // namespace stg
