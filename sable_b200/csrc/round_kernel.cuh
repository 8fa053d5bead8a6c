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

#ifndef SC_MINBLOCKS
#define SC_MINBLOCKS 2
#endif
#ifndef SC_MINBLOCKS_D8
#define SC_MINBLOCKS_D8 2
#endif
#ifndef SC_MINBLOCKS_R0
#define SC_MINBLOCKS_R0 2
#endif

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

// The end of a round, run by every thread of the one block that holds the round's W sums (canonical words, in
// shared memory).  Several GPUs: the sums go to every rank's mailbox and come back added up.  Then the sums are
// written for the host and for whatever follows on the device, and the launch number after them.
static __device__ __forceinline__ void publish_round(const RoundArgs &a, u32 *sums, int W) {
    const int tid = threadIdx.x;
    __shared__ int missing;
    u32 posted = a.seq;
    if (a.xseq) {
        const bool dead = a.dead && *reinterpret_cast<const volatile u32 *>(a.dead) != 0;
        // hand the sums to every rank (this one included), the exchange number after them
        const size_t box = ((size_t)(a.xseq & 1) * a.world + a.rank) * MAIL_WORDS;
        if (tid < W)
            for (int r = 0; r < a.world; r++) a.mail[r][box + tid] = sums[tid];
        __threadfence_system();
        __syncthreads();
        if (tid < a.world) *reinterpret_cast<volatile u32 *>(a.mail[tid] + box + MAIL_FLAG) = a.xseq;
        // wait for every rank's number in this rank's own mailbox: bounded
        if (tid == 0) missing = dead ? 1 : 0;
        __syncthreads();
        if (tid < a.world && !dead) {
            const volatile u32 *flag = a.mail[a.rank] + ((size_t)(a.xseq & 1) * a.world + tid) * MAIL_WORDS + MAIL_FLAG;
            unsigned poll = 0;
            while (*flag != a.xseq && ++poll < a.mail_polls) __nanosleep(64);
            if (*flag != a.xseq) atomicAdd(&missing, 1);
        }
        __syncthreads();
        if (missing) posted |= EXCHANGE_FAILED;
        else if (tid < W) {
            u32 v = 0;
            for (int r = 0; r < a.world; r++)
                v = fadd(v, *reinterpret_cast<const volatile u32 *>(a.mail[a.rank] + ((size_t)(a.xseq & 1) * a.world + r) * MAIL_WORDS + tid));
            sums[tid] = v;
        }
        __syncthreads();
    }
    if (tid < W) {
        a.out_dev[tid] = sums[tid];
        if (a.out_host) a.out_host[tid] = sums[tid];
    }
    if (tid == 0 && a.chained) a.out_dev[MAX_PARTIAL_WORDS] = posted;
    __syncthreads();
    if (tid == 0 && a.out_host) {   // the host polls this word: the sums above are visible before it (the fence is cumulative)
        __threadfence_system();
        *reinterpret_cast<volatile u32 *>(a.out_host + MAX_PARTIAL_WORDS) = posted;
    }
}

// The statement at one point: sum of coefficient * product of the tables' values.  Values are
// canonical words; a product of two of them leaves REDC's factor 1/R behind, which the
// coefficients and the final factor of the round make up for (see DevStatement).  With BASEAWARE
// (a round on the caller's tables) a value that is a base element multiplies by D base products,
// or one when both factors are base elements (the reference's base variant, src/sumcheck.lisp:237-246).
// *ALL_BASE comes back true when the value is a base element.
template <int D, int NT, bool BASEAWARE>
__device__ __forceinline__ Ext<D> eval_statement(const DevStatement &st, const Ext<D> (&val)[NT], unsigned base_mask, bool *all_base) {
    Ext<D> acc = ezero<D>();
    bool abase = true;
    for (int t = 0; t < st.nterms; t++) {
        const DevTerm &tm = st.terms[t];
        Ext<D> prod;
        bool pbase = false;
        if (tm.nf == 0) {
#pragma unroll
            for (int c = 0; c < D; c++) prod.v[c] = tm.coeff[c];
            acc = eadd<D>(acc, prod);
            abase = abase && tm.ckind != CK_EXT;
            continue;
        }
        prod = pick<D, NT>(val, tm.f[0]);
        if (BASEAWARE) pbase = (base_mask >> tm.f[0]) & 1;
        for (int k = 1; k < tm.nf; k++) {
            const Ext<D> v = pick<D, NT>(val, tm.f[k]);
            if (BASEAWARE) {
                const bool vbase = (base_mask >> tm.f[k]) & 1;
                if (pbase && vbase) prod.v[0] = mmul(prod.v[0], v.v[0]);
                else if (vbase) prod = escale<D>(prod, v.v[0]);
                else if (pbase) { prod = escale<D>(v, prod.v[0]); pbase = false; }
                else prod = emul<D>(prod, v);
            } else {
                prod = emul<D>(prod, v);
            }
        }
        if (tm.ckind == CK_BASE) {
            if (BASEAWARE && pbase) prod.v[0] = mmul(prod.v[0], tm.coeff[0]);
            else prod = escale<D>(prod, tm.coeff[0]);
        } else if (tm.ckind == CK_EXT) {
            Ext<D> c;
#pragma unroll
            for (int q = 0; q < D; q++) c.v[q] = tm.coeff[q];
            if (BASEAWARE && pbase) { prod = escale<D>(c, prod.v[0]); pbase = false; }
            else prod = emul<D>(prod, c);
        }
        abase = abase && pbase;
        acc = eadd<D>(acc, prod);
    }
    if (BASEAWARE) *all_base = abase;
    return acc;
}

// The sums a listed statement (device.h) keeps in the kernels that sum base-field values (the base-table round kernel,
// the small-value pass): one for its terms with base-field coefficients, if it has any, and one for its term with an
// extension-field coefficient, if it has one (at most one: MAX_GROUPS).
template <class S> __host__ __device__ constexpr int listed_ext_terms() { int n = 0; for (int t = 0; t < S::NTERMS; t++) n += S::ck(t) == CK_EXT; return n; }
template <class S> __host__ __device__ constexpr int listed_groups() { return (listed_ext_terms<S>() < S::NTERMS ? 1 : 0) + listed_ext_terms<S>(); }
template <class S> __host__ __device__ constexpr int listed_group(int t) { return S::ck(t) == CK_EXT && listed_ext_terms<S>() < S::NTERMS ? 1 : 0; }

// A statement of the list (device.h): the same evaluation as eval_statement with every loop bound, table index
// and coefficient kind a compile-time constant, so it unrolls into straight-line code.
template <int D, class S, bool BASEAWARE>
__device__ __forceinline__ Ext<D> eval_listed(const DevStatement &st, const Ext<D> (&val)[S::NT], unsigned base_mask, bool *all_base) {
    Ext<D> acc = ezero<D>();
    bool abase = true;
#pragma unroll
    for (int t = 0; t < S::NTERMS; t++) {
        Ext<D> prod = val[S::f(t, 0)];
        bool pbase = BASEAWARE && ((base_mask >> S::f(t, 0)) & 1);
#pragma unroll
        for (int k = 1; k < S::nf(t); k++) {
            const Ext<D> &v = val[S::f(t, k)];
            if (BASEAWARE) {
                const bool vbase = (base_mask >> S::f(t, k)) & 1;
                if (pbase && vbase) prod.v[0] = mmul(prod.v[0], v.v[0]);
                else if (vbase) prod = escale<D>(prod, v.v[0]);
                else if (pbase) { prod = escale<D>(v, prod.v[0]); pbase = false; }
                else prod = emul<D>(prod, v);
            } else {
                prod = emul<D>(prod, v);
            }
        }
        if (S::ck(t) == CK_BASE) {
            if (BASEAWARE && pbase) prod.v[0] = mmul(prod.v[0], st.terms[t].coeff[0]);
            else prod = escale<D>(prod, st.terms[t].coeff[0]);
        } else {
            Ext<D> c;
#pragma unroll
            for (int q = 0; q < D; q++) c.v[q] = st.terms[t].coeff[q];
            if (BASEAWARE && pbase) { prod = escale<D>(c, prod.v[0]); pbase = false; }
            else prod = emul<D>(prod, c);
        }
        abase = abase && pbase;
        acc = eadd<D>(acc, prod);
    }
    if (BASEAWARE) *all_base = abase;
    return acc;
}

// A pure product of the NT tables (the coefficient rides in the round's final factor).
template <int D, int NT, bool BASEAWARE>
__device__ __forceinline__ Ext<D> eval_product(const Ext<D> (&val)[NT], unsigned base_mask, bool *all_base) {
    Ext<D> prod = val[0];
    bool pbase = BASEAWARE && (base_mask & 1);
#pragma unroll
    for (int t = 1; t < NT; t++) {
        if (BASEAWARE) {
            const bool vbase = (base_mask >> t) & 1;
            if (pbase && vbase) prod.v[0] = mmul(prod.v[0], val[t].v[0]);
            else if (vbase) prod = escale<D>(prod, val[t].v[0]);
            else if (pbase) { prod = escale<D>(val[t], prod.v[0]); pbase = false; }
            else prod = emul<D>(prod, val[t]);
        } else {
            prod = emul<D>(prod, val[t]);
        }
    }
    if (BASEAWARE) *all_base = pbase;
    return prod;
}

// The layer statement of LogUp-GKR, a d + b c + lam c d for the tables (a, b, c, d) at positions
// (0, 1, 2, 3) (reference LAYER-STATEMENT, src/gkr.lisp:30-41), as (a + lam c) d + b c: three
// products, one of them by the constant.
template <int D, bool BASEAWARE>
__device__ __forceinline__ Ext<D> eval_gkr(const Ext<D> (&val)[4], const ExtM<D> &lam, unsigned base_mask) {
    const bool ab = BASEAWARE && (base_mask & 1), bb = BASEAWARE && (base_mask & 2), cb = BASEAWARE && (base_mask & 4),
               db = BASEAWARE && (base_mask & 8);
    Ext<D> u;
    if (cb) {
#pragma unroll
        for (int k = 0; k < D; k++) u.v[k] = mmul(lam.v[k], val[2].v[0]);
    } else {
        u = emul<D>(val[2], lam);
    }
    if (ab) u.v[0] = fadd(u.v[0], val[0].v[0]); else u = eadd<D>(u, val[0]);
    if (bb && !cb && !db) return emul_plus_scaled<D>(u, eprep<D>(val[3]), val[2], val[1].v[0]);   // u d + b c, one reduction per coordinate
    if (!bb && !cb && !db) return emul2<D>(u, eprep<D>(val[3]), val[1], eprep<D>(val[2]));   // u d + b c, one reduction per coordinate
    Ext<D> f = db ? escale<D>(u, val[3].v[0]) : emul<D>(u, val[3]);
    Ext<D> g;
    if (bb && cb) g = lift<D>(mmul(val[1].v[0], val[2].v[0]));
    else if (bb) g = escale<D>(val[2], val[1].v[0]);
    else if (cb) g = escale<D>(val[1], val[2].v[0]);
    else g = emul<D>(val[1], val[2]);
    return eadd<D>(f, g);
}

template <int D, int PTS, int NT, int FOLD, int SHAPE>
__global__ void __launch_bounds__(ROUND_THREADS, NT > 4 ? 1 : (D == 8 ? SC_MINBLOCKS_D8 : (FOLD ? SC_MINBLOCKS : SC_MINBLOCKS_R0))) round_kernel(const __grid_constant__ RoundArgs a) {
    extern __shared__ __align__(16) u32 smem[];
    __shared__ u32 red[ROUND_THREADS / 32][PTS * D];
    __shared__ bool is_last;
    const int tid = threadIdx.x;
    const u32 L = 1u << a.logL;
    constexpr int NE = FOLD == 1 ? 4 : 2;   // entries read per table and pair (FOLD = 2: two blocks of four base entries)

    if (a.use_low) {   // the low multipliers of this round: (v, 3v) per entry
        const uint4 *g = reinterpret_cast<const uint4 *>(a.low);
        uint4 *s = reinterpret_cast<uint4 *>(smem);
        for (u32 k = tid; k < L * (2 * D / 4); k += ROUND_THREADS) s[k] = g[k];
        __syncthreads();
    }
    ExtM<D> rm;
    if (FOLD == 1) {
        Ext<D> r;
#pragma unroll
        for (int c = 0; c < D; c++) r.v[c] = a.r_dev ? a.r_dev[c] : a.r[c];
        rm = eprep<D>(r);
    }
    u32 bind[4][D];   // FOLD = 2: the weights of the four entries of a block
    if (FOLD == 2) {
#pragma unroll
        for (int b = 0; b < 4; b++)
#pragma unroll
            for (int c = 0; c < D; c++) bind[b][c] = a.bind[b][c];
    }
    // a block of four base entries bound to two challenges at once: sum_b bind[b] e[b]  (BIND-PREFIX, src/sumcheck.lisp:496-510)
    auto bound = [&](const Ext<D> &e4) {
        Ext<D> o;
#pragma unroll
        for (int c = 0; c < D; c++) {
            u64 acc = 0;
#pragma unroll
            for (int b = 0; b < 4; b++) acc += (u64)bind[b][c] * e4.v[b];
            o.v[c] = redc4(acc);
        }
        return o;
    };
    // a block of eight base entries bound to three challenges at once: the eight products do not fit one 64-bit sum, two sums of four do
    auto bound3 = [&](const u32 (&e8)[8]) {
        Ext<D> o;
#pragma unroll
        for (int c = 0; c < D; c++) {
            u64 lo4 = 0, hi4 = 0;
#pragma unroll
            for (int b = 0; b < 4; b++) { lo4 += (u64)a.bind3[b][c] * e8[b]; hi4 += (u64)a.bind3[4 + b][c] * e8[4 + b]; }
            o.v[c] = fadd(redc4(lo4), redc4(hi4));
        }
        return o;
    };
    // the two blocks of eight base entries of pair i of table t, bound: entries 16 i .. 16 i + 15
    auto bound3_pair = [&](const u32 *src, u64 i, Ext<D> &lo, Ext<D> &hi) {
        const uint4 *p = reinterpret_cast<const uint4 *>(src) + 4 * i;
        const uint4 w0 = __ldcs(p), w1 = __ldcs(p + 1), w2 = __ldcs(p + 2), w3 = __ldcs(p + 3);
        const u32 b0[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w}, b1[8] = {w2.x, w2.y, w2.z, w2.w, w3.x, w3.y, w3.z, w3.w};
        lo = bound3(b0);
        hi = bound3(b1);
    };
    unsigned base_mask = 0;
#pragma unroll
    for (int t = 0; t < NT; t++) base_mask |= (a.src_base[t] ? 1u : 0u) << t;
    ExtM<D> lam;
    if (SHAPE == SHAPE_GKR) {
        Ext<D> c;
#pragma unroll
        for (int k = 0; k < D; k++) c.v[k] = a.st.terms[0].coeff[k];
        lam = eprep<D>(c);
    }

    Ext<D> total[PTS], inner[PTS];
#pragma unroll
    for (int x = 0; x < PTS; x++) { total[x] = ezero<D>(); inner[x] = ezero<D>(); }
    u64 cur_h = ~0ull;
    // Round 0 with low weights (LAZY): the products with the low weight are summed over a run of pairs before they are
    // reduced (64-bit sums, one p off the high word of both sides before each addition keeps them below 2 p 2^32)
    constexpr bool LAZY = FOLD == 0 && D == 4 && NT <= 4 && PTS <= 2;   // where the wider sums fit the registers
    u64 inner64[LAZY ? PTS : 1][D];
#pragma unroll
    for (int x = 0; x < (LAZY ? PTS : 1); x++)
#pragma unroll
        for (int c = 0; c < D; c++) inner64[x][c] = 0;

    auto flush = [&]() {   // total += high[h] * inner  (src/sumcheck.lisp:256-257)
        if (LAZY && a.use_low) {
#pragma unroll
            for (int x = 0; x < PTS; x++)
#pragma unroll
                for (int c = 0; c < D; c++) { inner[x].v[c] = redc4(inner64[LAZY ? x : 0][c]); inner64[LAZY ? x : 0][c] = 0; }
        }
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
            // F_p^4: every load of the pair first, so that they are all in flight together; F_p^8: table by
            // table (the entries of four tables at once would not fit the register file)
            constexpr bool HOIST = D == 4 && NT <= 4;
            auto load_table = [&](int t, Ext<D> (&et)[NE]) {
                if (FOLD == 3) {
                    // read where it is bound, below
                } else if (FOLD == 2) {
                    const uint4 w0 = __ldcs(reinterpret_cast<const uint4 *>(a.src[t]) + 2 * i), w1 = __ldcs(reinterpret_cast<const uint4 *>(a.src[t]) + 2 * i + 1);
                    et[0].v[0] = w0.x; et[0].v[1] = w0.y; et[0].v[2] = w0.z; et[0].v[3] = w0.w;
                    et[1].v[0] = w1.x; et[1].v[1] = w1.y; et[1].v[2] = w1.z; et[1].v[3] = w1.w;
                } else if ((base_mask >> t) & 1) {
                    if (FOLD == 1) {
                        const uint4 w = __ldcs(reinterpret_cast<const uint4 *>(a.src[t]) + i);
                        et[0].v[0] = w.x; et[1 % NE].v[0] = w.y; et[2 % NE].v[0] = w.z; et[3 % NE].v[0] = w.w;
                    } else {
                        const uint2 w = __ldcs(reinterpret_cast<const uint2 *>(a.src[t]) + i);
                        et[0].v[0] = w.x; et[1].v[0] = w.y;
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < NE; k++) et[k] = load_ext<D>(a.src[t] + (NE * i + k) * D);
                }
            };
            Ext<D> e[HOIST ? NT : 1][NE];
            if (HOIST) {
#pragma unroll
                for (int t = 0; t < NT; t++) load_table(t, e[HOIST ? t : 0]);
            }
            Ext<D> val[NT], slope[NT];
#pragma unroll
            for (int t = 0; t < NT; t++) {
                const bool tb = (base_mask >> t) & 1;
                if (!HOIST) load_table(t, e[0]);
                Ext<D> (&et)[NE] = e[HOIST ? t : 0];
                if (FOLD == 3) {
                    Ext<D> lo, hi;
                    bound3_pair(a.src[t], i, lo, hi);
                    store_ext<D>(a.dst[t] + (2 * i) * D, lo);
                    store_ext<D>(a.dst[t] + (2 * i + 1) * D, hi);
                    val[t] = lo;
                    slope[t] = esub<D>(hi, lo);
                    if (PTS == 2) slope[t] = eadd<D>(slope[t], hi);
                } else if (FOLD == 2) {
                    const Ext<D> lo = bound(et[0]), hi = bound(et[1]);
                    store_ext<D>(a.dst[t] + (2 * i) * D, lo);
                    store_ext<D>(a.dst[t] + (2 * i + 1) * D, hi);
                    val[t] = lo;
                    slope[t] = esub<D>(hi, lo);
                    if (PTS == 2) slope[t] = eadd<D>(slope[t], hi);
                } else if (!FOLD) {
                    if (tb) {
                        val[t] = lift<D>(et[0].v[0]);
                        const u32 sl = fsub(et[1].v[0], et[0].v[0]);
                        slope[t] = lift<D>(PTS == 2 ? fadd(sl, et[1].v[0]) : sl);
                    } else {
                        val[t] = et[0];
                        slope[t] = esub<D>(et[1], et[0]);
                        if (PTS == 2) slope[t] = eadd<D>(slope[t], et[1]);
                    }
                } else {
                    // fold entries 4i .. 4i+3 by r: e0 + r (e1 - e0), e2 + r (e3 - e2)  (FOLD-FLAT-TABLE, src/sumcheck.lisp:84-104)
                    Ext<D> lo, hi;
                    if (tb) {   // the slope is a base element: D base products (:96-98)
                        const u32 s0 = fsub(et[1].v[0], et[0].v[0]), s1 = fsub(et[3 % NE].v[0], et[2 % NE].v[0]);
#pragma unroll
                        for (int c = 0; c < D; c++) { lo.v[c] = mmul(rm.v[c], s0); hi.v[c] = mmul(rm.v[c], s1); }
                        lo.v[0] = fadd(lo.v[0], et[0].v[0]);
                        hi.v[0] = fadd(hi.v[0], et[2 % NE].v[0]);
                    } else {
                        lo = eadd<D>(et[0], emul<D>(esub<D>(et[1], et[0]), rm));
                        hi = eadd<D>(et[2 % NE], emul<D>(esub<D>(et[3 % NE], et[2 % NE]), rm));
                    }
                    store_ext<D>(a.dst[t] + (2 * i) * D, lo);
                    store_ext<D>(a.dst[t] + (2 * i + 1) * D, hi);
                    val[t] = lo;
                    slope[t] = esub<D>(hi, lo);
                    if (PTS == 2) slope[t] = eadd<D>(slope[t], hi);
                }
            }
            // tables beyond the statement's are only folded
            if (FOLD == 3) {
                for (int t = NT; t < a.ntables; t++) {
                    Ext<D> lo, hi;
                    bound3_pair(a.src[t], i, lo, hi);
                    store_ext<D>(a.dst[t] + (2 * i) * D, lo);
                    store_ext<D>(a.dst[t] + (2 * i + 1) * D, hi);
                }
            } else if (FOLD == 2) {
                for (int t = NT; t < a.ntables; t++) {
                    const uint4 w0 = __ldcs(reinterpret_cast<const uint4 *>(a.src[t]) + 2 * i), w1 = __ldcs(reinterpret_cast<const uint4 *>(a.src[t]) + 2 * i + 1);
                    Ext<D> b0, b1;
                    b0.v[0] = w0.x; b0.v[1] = w0.y; b0.v[2] = w0.z; b0.v[3] = w0.w;
                    b1.v[0] = w1.x; b1.v[1] = w1.y; b1.v[2] = w1.z; b1.v[3] = w1.w;
                    store_ext<D>(a.dst[t] + (2 * i) * D, bound(b0));
                    store_ext<D>(a.dst[t] + (2 * i + 1) * D, bound(b1));
                }
            } else if (FOLD == 1) {
                for (int t = NT; t < a.ntables; t++) {
                    Ext<D> lo, hi;
                    if (a.src_base[t]) {
                        const uint4 w = __ldcs(reinterpret_cast<const uint4 *>(a.src[t]) + i);
                        const u32 s0 = fsub(w.y, w.x), s1 = fsub(w.w, w.z);
#pragma unroll
                        for (int c = 0; c < D; c++) { lo.v[c] = mmul(rm.v[c], s0); hi.v[c] = mmul(rm.v[c], s1); }
                        lo.v[0] = fadd(lo.v[0], w.x);
                        hi.v[0] = fadd(hi.v[0], w.z);
                    } else {
                        const u32 *src = a.src[t] + 4 * i * D;
                        Ext<D> e0 = load_ext<D>(src), e1 = load_ext<D>(src + D), e2 = load_ext<D>(src + 2 * D), e3 = load_ext<D>(src + 3 * D);
                        lo = eadd<D>(e0, emul<D>(esub<D>(e1, e0), rm));
                        hi = eadd<D>(e2, emul<D>(esub<D>(e3, e2), rm));
                    }
                    store_ext<D>(a.dst[t] + (2 * i) * D, lo);
                    store_ext<D>(a.dst[t] + (2 * i + 1) * D, hi);
                }
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
                if (x == 1) {   // X = 2: lo + 2 s; with two points the array holds 2 hi - lo already
#pragma unroll
                    for (int t = 0; t < NT; t++) val[t] = PTS == 2 ? slope[t] : eadd<D>(eadd<D>(val[t], slope[t]), slope[t]);
                } else if (x > 1) {
#pragma unroll
                    for (int t = 0; t < NT; t++) val[t] = eadd<D>(val[t], slope[t]);
                }
                bool fbase = false;
                Ext<D> f;
                if (SHAPE == SHAPE_PRODUCT) f = eval_product<D, NT, FOLD == 0>(val, base_mask, &fbase);
                else if (SHAPE == SHAPE_GKR) f = eval_gkr<D, FOLD == 0>(reinterpret_cast<const Ext<D>(&)[4]>(val), lam, base_mask);
                else if (SHAPE >= SHAPE_LISTED) {
                    typedef Listed<(SHAPE >= SHAPE_LISTED ? SHAPE - SHAPE_LISTED : 0)> S;
                    f = eval_listed<D, S, FOLD == 0>(a.st, reinterpret_cast<const Ext<D>(&)[S::NT]>(val), FOLD ? 0u : base_mask, &fbase);
                }
                else f = eval_statement<D, NT, FOLD == 0>(a.st, val, FOLD ? 0u : base_mask, &fbase);
                if (LAZY && a.use_low) {
                    if (fbase) {   // a base value times the weight: D base products (EXT-SCALE, src/sumcheck.lisp:246), unreduced
                        const u32 fb = f.v[0];
#pragma unroll
                        for (int c = 0; c < D; c++) inner64[LAZY ? x : 0][c] = presub(inner64[LAZY ? x : 0][c]) + (u64)lw.v[c] * fb;
                    } else {
                        const ExtRaw<D> raw = emul_raw<D>(f, lw);
#pragma unroll
                        for (int c = 0; c < D; c++) inner64[LAZY ? x : 0][c] = presub(inner64[LAZY ? x : 0][c]) + presub(raw.v[c]);
                    }
                    continue;
                }
                if (a.use_low) {
                    if (!FOLD && fbase) {   // a base value times the weight: D base products (EXT-SCALE, src/sumcheck.lisp:246)
                        const u32 fb = f.v[0];
#pragma unroll
                        for (int c = 0; c < D; c++) f.v[c] = mmul(lw.v[c], fb);
                    } else {
                        f = emul<D>(f, lw);
                    }
                }
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
    constexpr int W = PTS * D;                 // <= 64 words
    constexpr int ROWS = ROUND_THREADS / 32;
    constexpr int KW = W > 32 ? 64 : 32;       // threads across a row of partial sums
    if (gridDim.x > 1) {
        if (tid < W) {
            u32 v = red[0][tid];
#pragma unroll
            for (int w = 1; w < ROWS; w++) v = fadd(v, red[w][tid]);
            a.partials[(size_t)blockIdx.x * W + tid] = v;
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) is_last = atomicAdd(a.counter, 1u) == gridDim.x - 1;
        __syncthreads();
        if (!is_last) return;
        __threadfence();
        // the last block: add the partials (a single block has its rows in shared memory already)
        const int k = tid % KW, row = tid / KW;
        constexpr int NROW = ROUND_THREADS / KW;
        u32 v = 0;
        if (k < W)
            for (unsigned g = row; g < gridDim.x; g += NROW) v = fadd(v, __ldcg(a.partials + (size_t)g * W + k));
        __syncthreads();
        if (k < W) red[row][k] = v;
        if (k < W && NROW < ROWS) for (int w = NROW + row; w < ROWS; w += NROW) red[w][k] = 0;
        __syncthreads();
        if (tid == 0) *a.counter = 0;
    }
    // apply the final factor and publish
    {
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
#pragma unroll
            for (int c = 0; c < D; c++) red[0][tid * D + c] = s.v[c];
        }
        __syncthreads();
        publish_round(a, &red[0][0], W);
    }
}

template <int D, int PTS, int NT, int SHAPE>
static cudaError_t launch_round_dpns(int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    if (fold == 1) {
        if (smem > 40 * 1024) cudaFuncSetAttribute(round_kernel<D, PTS, NT, 1, SHAPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        round_kernel<D, PTS, NT, 1, SHAPE><<<grid, ROUND_THREADS, smem, stream>>>(args);
    } else if (fold == 0) {
        if (smem > 40 * 1024) cudaFuncSetAttribute(round_kernel<D, PTS, NT, 0, SHAPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        round_kernel<D, PTS, NT, 0, SHAPE><<<grid, ROUND_THREADS, smem, stream>>>(args);
    } else if (fold == 2) {
        // base tables bound to two challenges on the way in (after the small-value rounds: at most three tables, degree three)
        if constexpr (NT <= 3 && PTS <= 3 && SHAPE != SHAPE_GKR) {
            if (smem > 40 * 1024) cudaFuncSetAttribute(round_kernel<D, PTS, NT, 2, SHAPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            round_kernel<D, PTS, NT, 2, SHAPE><<<grid, ROUND_THREADS, smem, stream>>>(args);
        } else {
            return cudaErrorInvalidValue;
        }
    } else if (fold == 3) {
        // base tables bound to three challenges on the way in (after three small-value rounds: degree at most two)
        if constexpr (NT <= 3 && PTS <= 2 && SHAPE != SHAPE_GKR) {
            if (smem > 40 * 1024) cudaFuncSetAttribute(round_kernel<D, PTS, NT, 3, SHAPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            round_kernel<D, PTS, NT, 3, SHAPE><<<grid, ROUND_THREADS, smem, stream>>>(args);
        } else {
            return cudaErrorInvalidValue;
        }
    } else {
        return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}
template <int D, int PTS>
static cudaError_t launch_round_dp(int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    switch (nt) {
    case 1: return launch_round_dpns<D, PTS, 1, SHAPE_GENERIC>(fold, args, grid, smem, stream);
    case 2: return launch_round_dpns<D, PTS, 2, SHAPE_GENERIC>(fold, args, grid, smem, stream);
    case 3: return launch_round_dpns<D, PTS, 3, SHAPE_GENERIC>(fold, args, grid, smem, stream);
    case 4: return launch_round_dpns<D, PTS, 4, SHAPE_GENERIC>(fold, args, grid, smem, stream);
    default: return cudaErrorInvalidValue;
    }
}

// The kernels with the statement built in: a product of nt tables at nt points, the GKR layer.
template <int D>
static cudaError_t launch_round_shape(int shape, int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    if (shape == SHAPE_GKR && points == 2 && nt == 4) return launch_round_dpns<D, 2, 4, SHAPE_GKR>(fold, args, grid, smem, stream);
    if (shape == SHAPE_LISTED + 0) return launch_round_dpns<D, Listed<0>::PTS, Listed<0>::NT, SHAPE_LISTED + 0>(fold, args, grid, smem, stream);
    if (shape == SHAPE_LISTED + 1) return launch_round_dpns<D, Listed<1>::PTS, Listed<1>::NT, SHAPE_LISTED + 1>(fold, args, grid, smem, stream);
    if (shape == SHAPE_LISTED + 2) return launch_round_dpns<D, Listed<2>::PTS, Listed<2>::NT, SHAPE_LISTED + 2>(fold, args, grid, smem, stream);
    if (shape == SHAPE_PRODUCT && points == nt) {
        switch (nt) {
        case 1: return launch_round_dpns<D, 1, 1, SHAPE_PRODUCT>(fold, args, grid, smem, stream);
        case 2: return launch_round_dpns<D, 2, 2, SHAPE_PRODUCT>(fold, args, grid, smem, stream);
        case 3: return launch_round_dpns<D, 3, 3, SHAPE_PRODUCT>(fold, args, grid, smem, stream);
        case 4: return launch_round_dpns<D, 4, 4, SHAPE_PRODUCT>(fold, args, grid, smem, stream);
        }
    }
    return cudaErrorInvalidValue;
}

// Statements over five to eight tables: the term-table kernel for six or eight tables (a statement
// over five or seven gets one more position, a copy of position 0 that no term names).
template <int D, int PTS>
static cudaError_t launch_round_wide_p(int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    if (nt == 6) return launch_round_dpns<D, PTS, 6, SHAPE_GENERIC>(fold, args, grid, smem, stream);
    if (nt == 8) return launch_round_dpns<D, PTS, 8, SHAPE_GENERIC>(fold, args, grid, smem, stream);
    return cudaErrorInvalidValue;
}
template <int D>
static cudaError_t launch_round_wide(int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    switch (points) {
    case 1: return launch_round_wide_p<D, 1>(nt, fold, args, grid, smem, stream);
    case 2: return launch_round_wide_p<D, 2>(nt, fold, args, grid, smem, stream);
    case 3: return launch_round_wide_p<D, 3>(nt, fold, args, grid, smem, stream);
    case 4: return launch_round_wide_p<D, 4>(nt, fold, args, grid, smem, stream);
    default: return cudaErrorInvalidValue;
    }
}

// Degrees five to eight: the term-table kernel with more points.
template <int D>
static cudaError_t launch_round_high(int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    switch (points) {
    case 5: return launch_round_dp<D, 5>(nt, fold, args, grid, smem, stream);
    case 6: return launch_round_dp<D, 6>(nt, fold, args, grid, smem, stream);
    case 7: return launch_round_dp<D, 7>(nt, fold, args, grid, smem, stream);
    case 8: return launch_round_dp<D, 8>(nt, fold, args, grid, smem, stream);
    default: return cudaErrorInvalidValue;
    }
}

template <int D>
static cudaError_t launch_round_d(int shape, int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    if (shape != SHAPE_GENERIC) return launch_round_shape<D>(shape, points, nt, fold, args, grid, smem, stream);
    switch (points) {
    case 1: return launch_round_dp<D, 1>(nt, fold, args, grid, smem, stream);
    case 2: return launch_round_dp<D, 2>(nt, fold, args, grid, smem, stream);
    case 3: return launch_round_dp<D, 3>(nt, fold, args, grid, smem, stream);
    case 4: return launch_round_dp<D, 4>(nt, fold, args, grid, smem, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace sc
