// round_kernel.cuh -- one prover round on the device.
//
// The reference's round is ROUND-KERNEL-CODE (src/sumcheck.lisp:190-258): for every pair (lo, hi)
// of every table the line values lo, hi, hi + s, .. (s = hi - lo), the statement at X = 0, 2, ..,
// the value weighted by LOW[l] and, once per block of |LOW| pairs, by HIGH[h]; then
// FOLD-FLAT-TABLE (:84-104) rewrites every table as lo + r (hi - lo).  Here the fold by the
// previous challenge happens on the way into the next round: a thread reads entries 4i .. 4i+3
// of the previous table, folds them to the pair (2i, 2i+1) of the current one in registers,
// writes that pair once and sums the round on it.
//
// Work split: the pairs are cut into chunks of max(2^logL, blockDim) consecutive pairs, chunk c
// going to block c mod gridDim.  Inside a chunk thread t takes pairs t, t + blockDim, ..
// (coalesced 128-bit loads).  While a thread stays under one high weight it sums
// low[l] F in registers; when the high index changes it multiplies that sum by high[h] once
// and adds it to its total.  Totals are reduced by warp shuffles, then through shared memory,
// to one partial per block; the last block to finish adds the partials, applies the final
// factor and writes canonical words (no block ever waits for another).
#pragma once
#include "device.h"

namespace sc {

using namespace scf;

template <int D> __device__ __forceinline__ Ext<D> load_ext(const u32 *p) {
    Ext<D> e;
#pragma unroll
    for (int q = 0; q < D; q += 4) {
        uint4 w = __ldcs(reinterpret_cast<const uint4 *>(p + q));
        e.v[q] = w.x; e.v[q + 1] = w.y; e.v[q + 2] = w.z; e.v[q + 3] = w.w;
    }
    return e;
}
template <int D> __device__ __forceinline__ void store_ext(u32 *p, const Ext<D> &e) {
#pragma unroll
    for (int q = 0; q < D; q += 4) *reinterpret_cast<uint4 *>(p + q) = make_uint4(e.v[q], e.v[q + 1], e.v[q + 2], e.v[q + 3]);
}
template <int D> __device__ __forceinline__ Ext<D> lift(u32 x) { Ext<D> e = ezero<D>(); e.v[0] = x; return e; }

template <int D, int NT> __device__ __forceinline__ Ext<D> pick(const Ext<D> (&val)[NT], int idx) {
    Ext<D> o = val[0];
#pragma unroll
    for (int t = 1; t < NT; t++)
        if (idx == t) o = val[t];
    return o;
}

// The statement at one point: sum of coefficient * product of the tables' values (in Montgomery form).
template <int D, int NT> __device__ __forceinline__ Ext<D> eval_statement(const DevStatement &st, const Ext<D> (&val)[NT]) {
    Ext<D> acc = ezero<D>();
    for (int t = 0; t < st.nterms; t++) {
        const DevTerm &tm = st.terms[t];
        Ext<D> prod;
        if (tm.nf == 0) {
#pragma unroll
            for (int c = 0; c < D; c++) prod.v[c] = tm.coeff[c];
            acc = eadd<D>(acc, prod);
            continue;
        }
        prod = pick<D, NT>(val, tm.f[0]);
        for (int k = 1; k < tm.nf; k++) prod = emul<D>(prod, pick<D, NT>(val, tm.f[k]));
        if (tm.ckind == CK_BASE) prod = escale<D>(prod, tm.coeff[0]);
        else if (tm.ckind == CK_EXT) {
            Ext<D> c;
#pragma unroll
            for (int q = 0; q < D; q++) c.v[q] = tm.coeff[q];
            prod = emul<D>(prod, c);
        }
        acc = eadd<D>(acc, prod);
    }
    return acc;
}

// The pair (lo, hi) of table t for pair index i, in Montgomery form.
template <int D, bool FOLD>
__device__ __forceinline__ void load_pair(const RoundArgs &a, int t, u64 i, const ExtM<D> &rm, Ext<D> &lo, Ext<D> &hi) {
    const u32 *src = a.src[t];
    if (!FOLD) {
        if (a.src_base[t]) {
            uint2 w = __ldcs(reinterpret_cast<const uint2 *>(src) + i);
            lo = lift<D>(a.raw ? to_mont(w.x) : w.x);
            hi = lift<D>(a.raw ? to_mont(w.y) : w.y);
        } else {
            lo = load_ext<D>(src + 2 * i * D);
            hi = load_ext<D>(src + (2 * i + 1) * D);
            if (a.raw) { lo = eto_mont<D>(lo); hi = eto_mont<D>(hi); }
        }
        return;
    }
    // fold entries 4i .. 4i+3 by r: e0 + r (e1 - e0), e2 + r (e3 - e2)  (FOLD-FLAT-TABLE, src/sumcheck.lisp:84-104)
    if (a.src_base[t]) {
        uint4 w = __ldcs(reinterpret_cast<const uint4 *>(src) + i);
        const u32 s0 = fsub(w.y, w.x), s1 = fsub(w.w, w.z);
        // the slope is a base element: D base products (:96-98); r carries the factor that puts the product in Montgomery form
#pragma unroll
        for (int c = 0; c < D; c++) { lo.v[c] = mmul(rm.v[c], s0); hi.v[c] = mmul(rm.v[c], s1); }
        lo.v[0] = fadd(lo.v[0], a.raw ? to_mont(w.x) : w.x);
        hi.v[0] = fadd(hi.v[0], a.raw ? to_mont(w.z) : w.z);
    } else {
        Ext<D> e0 = load_ext<D>(src + (4 * i) * D), e1 = load_ext<D>(src + (4 * i + 1) * D);
        Ext<D> e2 = load_ext<D>(src + (4 * i + 2) * D), e3 = load_ext<D>(src + (4 * i + 3) * D);
        Ext<D> p0 = emul<D>(esub<D>(e1, e0), rm), p1 = emul<D>(esub<D>(e3, e2), rm);
        if (a.raw) { e0 = eto_mont<D>(e0); e2 = eto_mont<D>(e2); }
        lo = eadd<D>(e0, p0);
        hi = eadd<D>(e2, p1);
    }
    u32 *dst = a.dst[t];
    store_ext<D>(dst + (2 * i) * D, lo);
    store_ext<D>(dst + (2 * i + 1) * D, hi);
}

template <int D, int PTS, int NT, bool FOLD>
__global__ void __launch_bounds__(ROUND_THREADS) round_kernel(const __grid_constant__ RoundArgs a) {
    extern __shared__ __align__(16) u32 smem[];
    __shared__ u32 red[ROUND_THREADS / 32][PTS * D];
    __shared__ bool is_last;
    const int tid = threadIdx.x;
    const u32 L = 1u << a.logL;

    if (a.use_low) {   // the low multipliers of this round: (v, 3v) per entry
        const uint4 *g = reinterpret_cast<const uint4 *>(a.low);
        uint4 *s = reinterpret_cast<uint4 *>(smem);
        for (u32 k = tid; k < L * (2 * D / 4); k += ROUND_THREADS) s[k] = g[k];
        __syncthreads();
    }
    ExtM<D> rm;
    if (FOLD) {
        Ext<D> r;
#pragma unroll
        for (int c = 0; c < D; c++) r.v[c] = a.r[c];
        rm = eprep<D>(r);
    }

    Ext<D> total[PTS], inner[PTS];
#pragma unroll
    for (int x = 0; x < PTS; x++) { total[x] = ezero<D>(); inner[x] = ezero<D>(); }
    u64 cur_h = ~0ull;

    auto flush = [&]() {   // total += high[h] * inner  (src/sumcheck.lisp:256-257)
        if (a.use_high) {
            Ext<D> hw = *reinterpret_cast<const Ext<D> *>(a.high + cur_h * D);
            ExtM<D> hm = eprep<D>(hw);
#pragma unroll
            for (int x = 0; x < PTS; x++) total[x] = eadd<D>(total[x], emul<D>(inner[x], hm));
        } else {
#pragma unroll
            for (int x = 0; x < PTS; x++) total[x] = eadd<D>(total[x], inner[x]);
        }
#pragma unroll
        for (int x = 0; x < PTS; x++) inner[x] = ezero<D>();
    };

    const u64 chunk = L > (u32)ROUND_THREADS ? L : ROUND_THREADS;
    for (u64 base = (u64)blockIdx.x * chunk; base < a.npairs; base += (u64)gridDim.x * chunk) {
        for (u64 q = tid; q < chunk; q += ROUND_THREADS) {
            const u64 i = base + q;
            if (i >= a.npairs) break;
            const u64 h = i >> a.logL;
            if (h != cur_h) {
                if (cur_h != ~0ull) flush();
                cur_h = h;
            }
            Ext<D> val[NT], slope[NT];
#pragma unroll
            for (int t = 0; t < NT; t++) {
                Ext<D> hi;
                load_pair<D, FOLD>(a, t, i, rm, val[t], hi);
                slope[t] = esub<D>(hi, val[t]);
            }
            // tables beyond the statement's are only folded
            if (FOLD) {
                for (int t = NT; t < a.ntables; t++) { Ext<D> lo, hi; load_pair<D, true>(a, t, i, rm, lo, hi); }
            }
            ExtM<D> lw;
            if (a.use_low) {
                const u32 *w = smem + (size_t)(i & (L - 1)) * 2 * D;
#pragma unroll
                for (int c = 0; c < D; c += 4) {
                    uint4 v = *reinterpret_cast<const uint4 *>(w + c), t3 = *reinterpret_cast<const uint4 *>(w + D + c);
                    lw.v[c] = v.x; lw.v[c + 1] = v.y; lw.v[c + 2] = v.z; lw.v[c + 3] = v.w;
                    lw.t[c] = t3.x; lw.t[c + 1] = t3.y; lw.t[c + 2] = t3.z; lw.t[c + 3] = t3.w;
                }
            }
#pragma unroll
            for (int x = 0; x < PTS; x++) {
                if (x == 1) {   // X = 2: lo + 2 s
#pragma unroll
                    for (int t = 0; t < NT; t++) val[t] = eadd<D>(eadd<D>(val[t], slope[t]), slope[t]);
                } else if (x > 1) {
#pragma unroll
                    for (int t = 0; t < NT; t++) val[t] = eadd<D>(val[t], slope[t]);
                }
                Ext<D> f = eval_statement<D, NT>(a.st, val);
                if (a.use_low) f = emul<D>(f, lw);
                inner[x] = eadd<D>(inner[x], f);
            }
        }
    }
    if (cur_h != ~0ull) flush();

    // block reduction of the totals
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int x = 0; x < PTS; x++)
#pragma unroll
        for (int c = 0; c < D; c++) {
            u32 v = total[x].v[c];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v = fadd(v, __shfl_down_sync(0xffffffffu, v, off));
            if (lane == 0) red[warp][x * D + c] = v;
        }
    __syncthreads();
    if (tid < PTS * D) {
        u32 v = red[0][tid];
#pragma unroll
        for (int w = 1; w < ROUND_THREADS / 32; w++) v = fadd(v, red[w][tid]);
        a.partials[(size_t)blockIdx.x * (PTS * D) + tid] = v;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) is_last = atomicAdd(a.counter, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();

    // the last block: add the partials, apply the final factor, leave Montgomery form
    {
        constexpr int W = PTS * D;                 // <= 32 words
        constexpr int ROWS = ROUND_THREADS / 32;
        const int k = tid & 31, row = tid >> 5;
        u32 v = 0;
        if (k < W)
            for (unsigned g = row; g < gridDim.x; g += ROWS) v = fadd(v, __ldcg(a.partials + (size_t)g * W + k));
        __syncthreads();
        if (k < W) red[row][k] = v;
        __syncthreads();
        if (tid < PTS) {
            Ext<D> s;
#pragma unroll
            for (int c = 0; c < D; c++) {
                u32 acc = red[0][tid * D + c];
#pragma unroll
                for (int w = 1; w < ROWS; w++) acc = fadd(acc, red[w][tid * D + c]);
                s.v[c] = acc;
            }
            if (a.use_post) {
                Ext<D> pf;
#pragma unroll
                for (int c = 0; c < D; c++) pf.v[c] = a.post[c];
                s = emul<D>(s, pf);
            }
            s = efrom_mont<D>(s);
#pragma unroll
            for (int c = 0; c < D; c++) {
                a.out_dev[tid * D + c] = s.v[c];
                if (a.out_host) a.out_host[tid * D + c] = s.v[c];
            }
        }
        if (tid == 0) *a.counter = 0;
        __threadfence_system();
    }
}

template <int D, int PTS, int NT>
static cudaError_t launch_round_dpn(bool fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    if (fold) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(round_kernel<D, PTS, NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        round_kernel<D, PTS, NT, true><<<grid, ROUND_THREADS, smem, stream>>>(args);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(round_kernel<D, PTS, NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        round_kernel<D, PTS, NT, false><<<grid, ROUND_THREADS, smem, stream>>>(args);
    }
    return cudaGetLastError();
}

template <int D, int PTS>
static cudaError_t launch_round_dp(int nt, bool fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    switch (nt) {
    case 1: return launch_round_dpn<D, PTS, 1>(fold, args, grid, smem, stream);
    case 2: return launch_round_dpn<D, PTS, 2>(fold, args, grid, smem, stream);
    case 3: return launch_round_dpn<D, PTS, 3>(fold, args, grid, smem, stream);
    case 4: return launch_round_dpn<D, PTS, 4>(fold, args, grid, smem, stream);
    default: return cudaErrorInvalidValue;
    }
}

template <int D>
static cudaError_t launch_round_d(int points, int nt, bool fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    switch (points) {
    case 1: return launch_round_dp<D, 1>(nt, fold, args, grid, smem, stream);
    case 2: return launch_round_dp<D, 2>(nt, fold, args, grid, smem, stream);
    case 3: return launch_round_dp<D, 3>(nt, fold, args, grid, smem, stream);
    case 4: return launch_round_dp<D, 4>(nt, fold, args, grid, smem, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace sc
