// Segment-parallel form of the sequential-fp32-sum emulation (see stg_emul.cuh for the arithmetic).
//
// The sequence is cut into sub-tiles of 256 elements.  All warps first reduce their sub-tiles to a
// plain sum; a block scan (fp64) of those gives, for every sub-tile, a good guess of the binade the
// running sum is in when the sequential loop reaches it.  All warps then reduce each sub-tile to
// its composite increment (for an even / odd start) under that guess.  One warp finally walks the
// sub-tiles in order with the EXACT running sum: a sub-tile whose composite keeps the sum inside
// the binade it was computed for (and below the target) is consumed whole - 32 of them per warp
// scan - and only a sub-tile in which the sum leaves its binade, meets the target, or was guessed
// wrongly is replayed with real fp32 additions, one element after the other.  The result is
// bit-identical to the one-by-one loop; the guesses only decide how much is replayed.
//
// Per element the hot phases cost a handful of instructions: with u = 2^(E-23) the unit of the
// running sum, the increment of x is rint(x / u) (round-half-even, one multiply by a power of two
// and one convert), and exact ties - where the parity of the running sum decides - are detected
// by their fraction of exactly one half and handled on a slow path.
#pragma once
#include <type_traits>

#include "stg_emul.cuh"

namespace stg {

// ---- staged reads ----------------------------------------------------------------------------------
// A provider whose elements sit in global memory as 16-byte quads (kQuadsLoad / kQuadsReload per
// thread and sub-tile) can have them copied to shared memory a few sub-tiles ahead with cp.async,
// so that the latency of L2 is not paid with registers.  Every thread copies and reads only its
// own slots: no block-wide synchronisation is involved.
constexpr int kStageBytes = 131072;  // shared memory the staged loops use at most (4 stages of 32 bytes per thread)
__device__ __forceinline__ void cp_async_wait_dyn(int pending)
{
    if (pending >= 3) asm volatile("cp.async.wait_group 3;" ::: "memory");
    else if (pending == 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
    else if (pending == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
}
// stages of Q quads per thread that fit `bytes` of shared memory (at most 4; below 2 staging is off)
__device__ __forceinline__ int stage_depth(int bytes, int quads)
{
    const int d = bytes / (quads * 16 * kThreads);
    return d > 4 ? 4 : d;
}
template <class P, class = void>
struct StageQ { static constexpr int load = 0, reload = 0; };
template <class P>
struct StageQ<P, std::void_t<decltype(P::kQuadsLoad)>> {
    static constexpr int load = P::kQuadsLoad, reload = P::kQuadsReload;
};
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem)
{
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// quad q of stage s of this thread: consecutive threads are 16 bytes apart (conflict-free LDS.128)
template <int NQ>
__device__ __forceinline__ float4 *stage_slot(unsigned char *stage, int s, int q)
{
    return (float4 *)(stage + ((size_t)(s * NQ + q) * kThreads + threadIdx.x) * 16);
}

constexpr int kSub = 256;           // elements per sub-tile (8 consecutive per lane)
constexpr int kMaxSubTiles = 1024;  // => sequences of up to 262144 elements

constexpr int kMaxCross = 12;       // sub-tiles per scan with a prepared binade crossing

// per-lane composites of a sub-tile in which the running sum is expected to pass from binade g to
// g + 1: with them the walk crosses without touching the sub-tile's elements (except one lane's 8)
struct CrossSlot {
    int lo[32][2];                  // lane composite (even / odd start) under binade g
    int hi[32][2];                  // ... under binade g + 1
};

struct Emul2Work {                  // lives in dynamic shared memory (20 KB)
    float sums[kMaxSubTiles];       // sum of each sub-tile (a guess only needs float accuracy)
    int comp[kMaxSubTiles][2];      // composite increment under the guessed binade: even / odd start
    unsigned char guess[kMaxSubTiles];  // guessed biased exponent of the running sum at the sub-tile
    unsigned char xslot[kMaxSubTiles];  // 1 + index of the sub-tile's CrossSlot, 0: none
    CrossSlot xs[kMaxCross];
};
static_assert(sizeof(Emul2Work) >= 16384, "other phases borrow 16 KB of this area");

struct Emul2Ctl {
    double wsum[32];
    int n_cross;                    // CrossSlots handed out
    float s;
    int hit;
    int abort_at;                   // sub-tile that needed a replay the caller had forbidden, or -1
    float hit_before;               // running sum just before the element that met the target (with `s` just
                                    // after it: how close the target lies to a step of the running sum)
};

// increment of x (>= 0) in units of 1/scale, for an even (d0) and an odd (d1) running sum
__device__ __forceinline__ void unit_incr_fast(float x, float scale, int &d0, int &d1, bool &tie)
{
    const float xs = x * scale;            // exact: scale is a power of two
    int d = __float2int_rn(xs);            // round half to even, saturating
    d = d > (1 << 24) ? (1 << 24) : d;
    const float tr = truncf(xs);
    tie = (xs - tr) == 0.5f;               // exact below 2^24; 0 above
    d0 = d;
    d1 = tie ? 2 * (int)tr + 1 - d : d;
}

// composite of a lane's 8 consecutive elements under binade eb (saturating)
__device__ __forceinline__ void lane_composite(const float x[8], int eb, int &a0, int &a1)
{
    a0 = 0; a1 = 0;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        int d0, d1;
        unit_incr(x[j], eb, d0, d1);
        a0 += (a0 & 1) ? d1 : d0;
        a1 += ((1 + a1) & 1) ? d1 : d0;
    }
    a0 = min(a0, 1 << 25);
    a1 = min(a1, 1 << 25);
}

__device__ __forceinline__ int exp_of_double(double v)
{
    if (!(v > 0.0)) return 1;
    int e = ilogb(v) + 127;
    return e < 1 ? 1 : (e > 254 ? 254 : e);
}

__device__ __forceinline__ long long target_units(float target, bool has_target, int eb)
{
    if (!has_target) return LLONG_MAX;
    if (eb >= 24) {
        const float ts = target * __int_as_float((277 - eb) << 23);  // target * 2^(150-eb)
        return ts >= 33554432.f ? (1ll << 25) : (long long)__float2int_ru(ts);
    }
    double td = ceil(ldexp((double)target, 150 - eb));
    return td >= 1073741824.0 ? (1ll << 30) : (td <= -1073741824.0 ? -(1ll << 30) : (long long)td);
}

// composite of one sub-tile (8 consecutive elements per lane) under binade `eb`; all lanes get it.
// FORCE: a tie inside the sub-tile makes the composite "unknown" (saturated), which forces a replay.
template <bool FORCE>
__device__ __forceinline__ void subtile_composite(const float x[8], int eb, int &r0, int &r1)
{
    if (eb >= 24) {
        // common case first: no element is an exact tie, so the increment does not depend on the
        // parity of the running sum and the composite is a plain integer sum
        const float scale = __int_as_float((277 - eb) << 23);
        int a = 0;
        bool any_tie = false;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float xs = x[j] * scale;
            a += min(__float2int_rn(xs), 1 << 24);
            any_tie |= (xs - truncf(xs)) == 0.5f;
        }
        a = min(a, 1 << 24);
        if (__ballot_sync(0xFFFFFFFFu, any_tie) == 0u) {
            r0 = r1 = __reduce_add_sync(0xFFFFFFFFu, a);
            return;
        }
    }
    if (FORCE) { r0 = r1 = 1 << 28; return; }
    int a0 = 0, a1 = 0;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        int d0, d1;
        unit_incr(x[j], eb, d0, d1);
        a0 += (a0 & 1) ? d1 : d0;
        a1 += ((1 + a1) & 1) ? d1 : d0;
    }
    a0 = min(a0, 1 << 24);
    a1 = min(a1, 1 << 24);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int p0 = __shfl_down_sync(0xFFFFFFFFu, a0, o);
        int p1 = __shfl_down_sync(0xFFFFFFFFu, a1, o);
        int n0, n1;
        comp(a0, a1, p0, p1, n0, n1);
        a0 = n0; a1 = n1;  // only lane 0's chain is meaningful
    }
    r0 = __shfl_sync(0xFFFFFFFFu, a0, 0);
    r1 = __shfl_sync(0xFFFFFFFFu, a1, 0);
}

// Replays one sub-tile exactly (one warp, 8 consecutive elements per lane).  Lanes are consumed in
// order: a warp scan of the lanes' composites under the current binade finds the first lane in which
// the sum leaves the binade or meets the target; the lanes before it are taken whole, that lane
// adds its 8 elements with real fp32 additions, and the scan restarts behind it in the new binade.
// `s` is the exact running sum before the sub-tile; returns the hit index or -1.
template <bool POS_ONLY>
__device__ __forceinline__ int replay_subtile(const float x[8], int base, int n, float target, bool has_target,
                                              float &s, float &before)
{
    const int lane = threadIdx.x & 31;
    const int g0 = base + lane * 8;
    int start_lane = 0;
    for (;;) {
        const uint32_t sb = __float_as_uint(s);
        const int ef = (int)(sb >> 23) & 255;
        const int eb = ef ? ef : 1;
        const int sint = (int)((sb & 0x7FFFFFu) | (ef ? 0x800000u : 0u));
        if (ef == 255) return -1;
        const long long tint = target_units(target, has_target, eb);
        int a0 = 0, a1 = 0;
        if (lane >= start_lane) {
            if (eb >= 24) {
                const float scale = __int_as_float((277 - eb) << 23);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    int d0, d1;
                    bool tie;
                    const float v = (g0 + j < n && (!POS_ONLY || x[j] > 0.f)) ? x[j] : 0.f;
                    unit_incr_fast(v, scale, d0, d1, tie);
                    a0 += (a0 & 1) ? d1 : d0;
                    a1 += ((1 + a1) & 1) ? d1 : d0;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    int d0, d1;
                    const float v = (g0 + j < n && (!POS_ONLY || x[j] > 0.f)) ? x[j] : 0.f;
                    unit_incr(v, eb, d0, d1);
                    a0 += (a0 & 1) ? d1 : d0;
                    a1 += ((1 + a1) & 1) ? d1 : d0;
                }
            }
            a0 = min(a0, 1 << 25);
            a1 = min(a1, 1 << 25);
        }
        int i0 = a0, i1 = a1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int p0 = __shfl_up_sync(0xFFFFFFFFu, i0, o);
            int p1 = __shfl_up_sync(0xFFFFFFFFu, i1, o);
            if (lane >= o) { int r0, r1; comp(p0, p1, i0, i1, r0, r1); i0 = r0; i1 = r1; }
        }
        const int S = sat_add(sint, (sint & 1) ? i1 : i0);  // sum after lanes 0 .. lane
        // a target that is already met fires at the first element still to come
        const bool fire = lane >= start_lane && (S >= (1 << 24) || (long long)S >= tint);
        const unsigned fm = __ballot_sync(0xFFFFFFFFu, fire);
        if (fm == 0u) {
            const int send = __shfl_sync(0xFFFFFFFFu, S, 31);
            s = ldexpf((float)send, eb - 150);
            return -1;
        }
        const int L = __ffs(fm) - 1;
        int sprev = __shfl_sync(0xFFFFFFFFu, S, L > 0 ? L - 1 : 0);
        if (L == 0) sprev = sint;
        float acc = ldexpf((float)sprev, eb - 150);
        float prev = acc;
        int hit = -1;
        if (lane == L) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                if (g0 + j < n && (!POS_ONLY || x[j] > 0.f) && hit < 0) {
                    prev = acc;
                    acc = __fadd_rn(acc, x[j]);
                    if (has_target && acc >= target) hit = g0 + j;
                }
            }
        }
        s = __shfl_sync(0xFFFFFFFFu, acc, L);
        hit = __shfl_sync(0xFFFFFFFFu, hit, L);
        if (hit >= 0) { before = __shfl_sync(0xFFFFFFFFu, prev, L); return hit; }
        start_lane = L + 1;
        if (start_lane >= 32) return -1;
    }
}

// Phase B on its own: exclusive fp64 prefix of the sub-tile sums in wk->sums[0..nsub) -> guessed
// binade of the running sum at every sub-tile (wk->guess) and a crossing slot (wk->xslot) for the
// sub-tiles in which the sum should pass into the next binade.  All kThreads threads call it.
__device__ __forceinline__ void emul2_guess(Emul2Ctl *c, Emul2Work *wk, int nsub)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    {
        double v = tid < nsub ? (double)wk->sums[tid] : 0.0;
        double inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            double t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) c->wsum[warp] = inc;
        __syncthreads();
        if (warp == 0) {
            double w = c->wsum[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                double t = __shfl_up_sync(0xFFFFFFFFu, w, o);
                if (lane >= o) w += t;
            }
            c->wsum[lane] = w;
        }
        __syncthreads();
        double excl = inc - v + (warp ? c->wsum[warp - 1] : 0.0);
        if (tid < nsub) { wk->guess[tid] = (unsigned char)exp_of_double(excl); wk->xslot[tid] = 0; }
        if (tid == 0) c->n_cross = 0;
    }
    __syncthreads();
    // sub-tiles in which the sum should pass into the next binade get a CrossSlot
    if (tid + 1 < nsub && (int)wk->guess[tid + 1] == (int)wk->guess[tid] + 1 && wk->sums[tid] > 0.f) {
        const int slot = atomicAdd(&c->n_cross, 1);
        if (slot < kMaxCross) wk->xslot[tid] = (unsigned char)(slot + 1);
    }
}

// Phase D on its own: ONE WARP walks the sub-tiles of a sequence whose per-sub-tile sums, guessed
// binades, composites and crossing slots are in `wk` (shared memory), with the exact running sum.
// Leaves the final sum in c->s and the hit (or -1, or -2 with c->abort_at for a forbidden replay) in
// c->hit.  Called by all 32 lanes of one warp; the caller synchronises the block afterwards.
template <class Prov, bool POS_ONLY, bool FORCE>
__device__ __forceinline__ void emul2_walk(Emul2Ctl *c, Emul2Work *wk, const Prov &pv, int n, int nsub, float target,
                                           bool has_target, const unsigned char *replay_ok, unsigned long long *tk)
{
    const int lane = threadIdx.x & 31;
    float s = 0.f, before = 0.f;
    int hit = -1;
    int t = 0;
    int abort_at = -1;
    int n_iter = 0, n_replay = 0, n_fast = 0;
    while (t < nsub && hit < 0) {
        n_iter++;
        const uint32_t sb = __float_as_uint(s);
        const int ef = (int)(sb >> 23) & 255;
        const int eb = ef ? ef : 1;
        const int sint = (int)((sb & 0x7FFFFFu) | (ef ? 0x800000u : 0u));
        if (ef == 255) break;  // inf / NaN: nothing changes any more
        const long long tint = target_units(target, has_target, eb);
        // lane l proposes sub-tile t + l
        const int tt = t + lane;
        int a0 = 0, a1 = 0;
        bool valid = false;
        if (tt < nsub) {
            a0 = wk->comp[tt][0];
            a1 = wk->comp[tt][1];
            valid = (wk->guess[tt] == eb) || (a0 == 0 && a1 == 0 && wk->sums[tt] == 0.f);
        }
        int i0 = a0, i1 = a1;
        if (__any_sync(0xFFFFFFFFu, a0 != a1)) {
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int p0 = __shfl_up_sync(0xFFFFFFFFu, i0, o);
                int p1 = __shfl_up_sync(0xFFFFFFFFu, i1, o);
                if (lane >= o) { int r0, r1; comp(p0, p1, i0, i1, r0, r1); i0 = r0; i1 = r1; }
            }
        } else {
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                int p0 = __shfl_up_sync(0xFFFFFFFFu, i0, o);
                if (lane >= o) i0 = sat_add(i0, p0);
            }
            i1 = i0;
        }
        const int S = sat_add(sint, (sint & 1) ? i1 : i0);  // sum after sub-tiles t .. t+lane
        const bool bad = tt >= nsub || !valid || S >= (1 << 24) || (long long)S >= tint;
        const unsigned badmask = __ballot_sync(0xFFFFFFFFu, bad);
        const int ok = badmask ? __ffs(badmask) - 1 : 32;  // sub-tiles consumed whole
        if (ok > 0) {
            const int send = __shfl_sync(0xFFFFFFFFu, S, ok - 1);
            s = ldexpf((float)send, eb - 150);
            t += ok;
        }
        if (ok < 32 && t < nsub) {
            if (wk->guess[t] != eb && !(wk->sums[t] == 0.f)) {
                // the binade was guessed wrongly for this sub-tile (it follows a crossing closely):
                // its composite under the actual binade needs no order, so recompute it and retry
                float x[8];
                pv.reload(t * kSub + lane * 8, n, x);
                if (POS_ONLY) {
#pragma unroll
                    for (int j = 0; j < 8; j++) x[j] = x[j] > 0.f ? x[j] : 0.f;
                }
                int a0, a1;
                subtile_composite<FORCE>(x, eb, a0, a1);
                if (lane == 0) { wk->comp[t][0] = a0; wk->comp[t][1] = a1; wk->guess[t] = (unsigned char)eb; wk->xslot[t] = 0; }
                __syncwarp();
                continue;
            }
            if (FORCE && replay_ok != nullptr && !replay_ok[t]) { abort_at = t; break; }
            float x[8];
            pv.reload(t * kSub + lane * 8, n, x);
            // prepared crossing: the lanes before the one in which the sum leaves the binade are
            // taken by their composites, that lane adds its 8 elements for real, the lanes behind
            // it are taken by their composites under the next binade
            bool crossed = false;
            const int xsl = wk->xslot[t];
            if (xsl && eb < 253) {
                const CrossSlot &cs = wk->xs[xsl - 1];
                int i0 = cs.lo[lane][0], i1 = cs.lo[lane][1];
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    int p0 = __shfl_up_sync(0xFFFFFFFFu, i0, o);
                    int p1 = __shfl_up_sync(0xFFFFFFFFu, i1, o);
                    if (lane >= o) { int r0, r1; comp(p0, p1, i0, i1, r0, r1); i0 = r0; i1 = r1; }
                }
                const uint32_t sb1 = __float_as_uint(s);  // s has moved on since the top of the round
                const int sint1 = (int)((sb1 & 0x7FFFFFu) | (((sb1 >> 23) & 255u) ? 0x800000u : 0u));
                const int S1 = sat_add(sint1, (sint1 & 1) ? i1 : i0);  // sum after lanes 0 .. lane
                const unsigned over = __ballot_sync(0xFFFFFFFFu, S1 >= (1 << 24));
                const unsigned tgt = __ballot_sync(0xFFFFFFFFu, (long long)S1 >= tint);
                const int L = over ? __ffs(over) - 1 : 32;
                if (L < 32 && (tgt & ((1u << L) - 1u)) == 0u) {
                    int sprev = __shfl_sync(0xFFFFFFFFu, S1, L > 0 ? L - 1 : 0);
                    if (L == 0) sprev = sint1;
                    float acc = ldexpf((float)sprev, eb - 150);
                    int hit_l = -1;
                    if (lane == L) {
                        const int g0 = t * kSub + lane * 8;
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            if (g0 + j < n && (!POS_ONLY || x[j] > 0.f) && hit_l < 0) {
                                acc = __fadd_rn(acc, x[j]);
                                if (has_target && acc >= target) hit_l = g0 + j;
                            }
                        }
                    }
                    acc = __shfl_sync(0xFFFFFFFFu, acc, L);
                    hit_l = __shfl_sync(0xFFFFFFFFu, hit_l, L);
                    const uint32_t ab = __float_as_uint(acc);
                    const int ef2 = (int)(ab >> 23) & 255;
                    if (hit_l >= 0) {
                        s = acc; hit = hit_l; crossed = true;
                    } else if (ef2 == eb + 1) {
                        const int sint2 = (int)((ab & 0x7FFFFFu) | 0x800000u);
                        const long long tint2 = target_units(target, has_target, ef2);
                        int j0 = lane > L ? cs.hi[lane][0] : 0, j1 = lane > L ? cs.hi[lane][1] : 0;
#pragma unroll
                        for (int o = 1; o < 32; o <<= 1) {
                            int p0 = __shfl_up_sync(0xFFFFFFFFu, j0, o);
                            int p1 = __shfl_up_sync(0xFFFFFFFFu, j1, o);
                            if (lane >= o) { int r0, r1; comp(p0, p1, j0, j1, r0, r1); j0 = r0; j1 = r1; }
                        }
                        const int S2 = sat_add(sint2, (sint2 & 1) ? j1 : j0);
                        const bool fire2 = S2 >= (1 << 24) || (long long)S2 >= tint2;
                        if (__ballot_sync(0xFFFFFFFFu, fire2) == 0u) {
                            const int send = __shfl_sync(0xFFFFFFFFu, S2, 31);
                            s = ldexpf((float)send, ef2 - 150);
                            crossed = true;
                            n_fast++;
                        }
                    }
                }
            }
            if (!crossed) hit = replay_subtile<POS_ONLY>(x, t * kSub, n, target, has_target, s, before);
            t += 1;
            n_replay++;
        }
    }
    if (lane == 0) { c->s = s; c->hit = abort_at >= 0 ? -2 : hit; c->abort_at = abort_at; c->hit_before = before; }
    tick(tk, 3);
    if (tk && lane == 0) { tk[4] = (unsigned long long)n_iter; tk[5] = (unsigned long long)n_replay; tk[6] = (unsigned long long)n_fast; }
}

// Same contract as emul_scan (stg_emul.cuh), for n <= kSub * kMaxSubTiles.  `Prov::load` may have
// side effects and is called exactly once per element; `Prov::reload` must be pure.
// FORCE: the elements are only partially ordered (ordered between groups, arbitrary inside a
// group): any sub-tile that needs its internal order - a replay, or a parity tie - is checked
// against replay_ok[sub-tile]; when that says 0 the scan stops and returns -2 with the sub-tile in
// c->abort_at, so that the caller can order that part and run again.
template <class Prov, bool POS_ONLY, bool FORCE, int UN = 2>
__device__ __noinline__ int emul_scan2(Emul2Ctl *c, Emul2Work *wk, const Prov &pv_in, int n, float target,
                                       bool has_target, float *sum_out, const unsigned char *replay_ok,
                                       unsigned long long *tk, unsigned char *stage = nullptr,
                                       int stage_bytes = kStageBytes)
{
    // out of line, with its own copy of the provider: the loops below then get a register
    // allocation of their own instead of sharing one with the caller's other phases
    const Prov pv = pv_in;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nsub = (n + kSub - 1) / kSub;
    __syncthreads();
    // phase A: sum of every sub-tile
    constexpr int W = kThreads / 32;
    constexpr int QL = StageQ<Prov>::load, QR = StageQ<Prov>::reload;
    bool staged = false;
    if constexpr (QL > 0)
        staged = stage != nullptr && pv.stage_ok() && stage_depth(stage_bytes, QL) >= 2 && stage_depth(stage_bytes, QR) >= 2;
    if constexpr (QL > 0) {
        if (staged) {
            const int D = stage_depth(stage_bytes, QL);
            int tq = warp;
            for (int sidx = 0; sidx < D; sidx++, tq += W) {
                const int b = tq * kSub + lane * 8;
                if (tq < nsub && b + 8 <= n) {
                    const char *g = pv.stage_src(b, false);
#pragma unroll
                    for (int q = 0; q < QL; q++) cp_async16(stage_slot<QL>(stage, sidx, q), g + q * 16);
                }
                cp_async_commit();
            }
            int sidx = 0;
            for (int t = warp; t < nsub; t += W) {
                cp_async_wait_dyn(D - 1);
                const int b = t * kSub + lane * 8;
                float x[8];
                if (b + 8 <= n) {
                    float4 qd[QL];
#pragma unroll
                    for (int q = 0; q < QL; q++) qd[q] = *stage_slot<QL>(stage, sidx, q);
                    pv.load_from(b, n, qd, x);
                } else {
                    pv.load(b, n, x);
                }
                float acc = 0.f;
#pragma unroll
                for (int j = 0; j < 8; j++) acc += (x[j] > 0.f) ? x[j] : 0.f;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
                if (lane == 0) wk->sums[t] = acc;
                const int bq = tq * kSub + lane * 8;
                if (tq < nsub && bq + 8 <= n) {
                    const char *g = pv.stage_src(bq, false);
#pragma unroll
                    for (int q = 0; q < QL; q++) cp_async16(stage_slot<QL>(stage, sidx, q), g + q * 16);
                }
                cp_async_commit();
                tq += W;
                sidx = sidx + 1 == D ? 0 : sidx + 1;
            }
            cp_async_wait<0>();
        }
    }
    for (int t = warp; t < nsub && !staged; t += UN * W) {
        float x[UN][8];
#pragma unroll
        for (int h = 0; h < UN; h++)
            if (t + h * W < nsub) pv.load((t + h * W) * kSub + lane * 8, n, x[h]);
#pragma unroll
        for (int h = 0; h < UN; h++) {
            if (t + h * W < nsub) {
                float acc = 0.f;
#pragma unroll
                for (int j = 0; j < 8; j++) acc += (x[h][j] > 0.f) ? x[h][j] : 0.f;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
                if (lane == 0) wk->sums[t + h * W] = acc;
            }
        }
    }
    __syncthreads();
    tick(tk, 0);
    emul2_guess(c, wk, nsub);
    __syncthreads();
    tick(tk, 1);
    // phase C: composite of every sub-tile under its guessed binade
    if constexpr (QR > 0) {
        if (staged) {
            const int D = stage_depth(stage_bytes, QR);
            int tq = warp;
            for (int sidx = 0; sidx < D; sidx++, tq += W) {
                const int b = tq * kSub + lane * 8;
                if (tq < nsub && b + 8 <= n && !(wk->sums[tq] == 0.f)) {
                    const char *g = pv.stage_src(b, true);
#pragma unroll
                    for (int q = 0; q < QR; q++) cp_async16(stage_slot<QR>(stage, sidx, q), g + q * 16);
                }
                cp_async_commit();
            }
            int sidx = 0;
            for (int t = warp; t < nsub; t += W) {
                cp_async_wait_dyn(D - 1);
                const int b = t * kSub + lane * 8;
                int a0 = 0, a1 = 0;
                if (!(wk->sums[t] == 0.f)) {
                    float x[8];
                    if (b + 8 <= n) {
                        float4 qd[QR];
#pragma unroll
                        for (int q = 0; q < QR; q++) qd[q] = *stage_slot<QR>(stage, sidx, q);
                        pv.reload_from(b, n, qd, x);
                    } else {
                        pv.reload(b, n, x);
                    }
                    if (POS_ONLY) {
#pragma unroll
                        for (int j = 0; j < 8; j++) x[j] = x[j] > 0.f ? x[j] : 0.f;
                    }
                    subtile_composite<FORCE>(x, wk->guess[t], a0, a1);
                    const int xsl = wk->xslot[t];
                    if (xsl) {
                        CrossSlot &cs = wk->xs[xsl - 1];
                        int l0, l1, h0, h1;
                        lane_composite(x, wk->guess[t], l0, l1);
                        lane_composite(x, wk->guess[t] + 1, h0, h1);
                        cs.lo[lane][0] = l0; cs.lo[lane][1] = l1;
                        cs.hi[lane][0] = h0; cs.hi[lane][1] = h1;
                    }
                }
                if (lane == 0) { wk->comp[t][0] = a0; wk->comp[t][1] = a1; }
                const int bq = tq * kSub + lane * 8;
                if (tq < nsub && bq + 8 <= n && !(wk->sums[tq] == 0.f)) {
                    const char *g = pv.stage_src(bq, true);
#pragma unroll
                    for (int q = 0; q < QR; q++) cp_async16(stage_slot<QR>(stage, sidx, q), g + q * 16);
                }
                cp_async_commit();
                tq += W;
                sidx = sidx + 1 == D ? 0 : sidx + 1;
            }
            cp_async_wait<0>();
        }
    }
    for (int t = warp; t < nsub && !staged; t += UN * W) {
        float x[UN][8];
        bool z[UN];
#pragma unroll
        for (int h = 0; h < UN; h++) {
            const int tt = t + h * W;
            z[h] = tt >= nsub || wk->sums[tt] == 0.f;  // nothing to add: composite 0
            if (!z[h]) pv.reload(tt * kSub + lane * 8, n, x[h]);
        }
#pragma unroll
        for (int h = 0; h < UN; h++) {
            const int tt = t + h * W;
            if (tt < nsub) {
                int a0 = 0, a1 = 0;
                if (!z[h]) {
                    if (POS_ONLY) {
#pragma unroll
                        for (int j = 0; j < 8; j++) x[h][j] = x[h][j] > 0.f ? x[h][j] : 0.f;
                    }
                    subtile_composite<FORCE>(x[h], wk->guess[tt], a0, a1);
                    const int xsl = wk->xslot[tt];
                    if (xsl) {
                        CrossSlot &cs = wk->xs[xsl - 1];
                        int l0, l1, h0, h1;
                        lane_composite(x[h], wk->guess[tt], l0, l1);
                        lane_composite(x[h], wk->guess[tt] + 1, h0, h1);
                        cs.lo[lane][0] = l0; cs.lo[lane][1] = l1;
                        cs.hi[lane][0] = h0; cs.hi[lane][1] = h1;
                    }
                }
                if (lane == 0) { wk->comp[tt][0] = a0; wk->comp[tt][1] = a1; }
            }
        }
    }
    __syncthreads();
    tick(tk, 2);
    // phase D: one warp walks the sub-tiles with the exact sum
    if (warp == 0) emul2_walk<Prov, POS_ONLY, FORCE>(c, wk, pv, n, nsub, target, has_target, replay_ok, tk);
    __syncthreads();
    if (sum_out) *sum_out = c->s;
    const int h = c->hit;
    __syncthreads();
    return h;
}

// picks the segment-parallel form whenever the sequence fits it
template <class Prov, bool POS_ONLY>
__device__ int emul_any(EmulCtl *c1, Emul2Ctl *c2, Emul2Work *wk, const Prov &pv, int n, float target,
                        bool has_target, float *sum_out, unsigned long long *tk = nullptr,
                        unsigned char *stage = nullptr, int stage_bytes = kStageBytes)
{
    if (n <= kSub * kMaxSubTiles && wk != nullptr)
        return emul_scan2<Prov, POS_ONLY, false>(c2, wk, pv, n, target, has_target, sum_out, nullptr, tk, stage,
                                                 stage_bytes);
    return emul_scan<Prov, POS_ONLY>(c1, pv, n, target, has_target, sum_out);
}

}  // namespace stg
