// round_base.cu -- round 0 when every table of the statement is in the base field.
//
// The reference's base variant (ROUND-KERNEL-CODE with BASE, src/sumcheck.lisp:194-195,237-246):
// line values and the statement are base-field integers and a term costs one base-times-extension
// product by its weight.  Here that product is four (or eight) 32x32 -> 64-bit multiply-adds into
// 64-bit sums that are reduced once per run of pairs under one high weight: four products below
// p^2 fit a 64-bit word (REDUCED-SUM, src/field.lisp:213-218), and after every second pair the
// sums' high words lose one p, which makes room for two more; the high weight multiplies once per run.
// Terms with an extension-field coefficient keep a sum of their own and meet their coefficient
// in the last block, so the pairs never see an extension-by-extension product.
#include "round_kernel.cuh"

namespace sc {

template <int NT> __device__ __forceinline__ u32 pick_base(const u32 (&val)[NT], int idx) {
    u32 o = val[0];
#pragma unroll
    for (int t = 1; t < NT; t++)
        if (idx == t) o = val[t];
    return o;
}

// SHAPE: SHAPE_GENERIC (term descriptors from the arguments, kept in registers), SHAPE_PRODUCT, or a listed statement
template <int D, int PTS, int NT, int NG, int SHAPE>
__global__ void __launch_bounds__(ROUND_THREADS, round_base_blocks_per_sm(D, SHAPE, PTS, NG)) round_base_kernel(const __grid_constant__ RoundArgs a) {
    extern __shared__ __align__(16) u32 smem[];
    constexpr int W = NG * PTS * D;
    __shared__ u32 red[ROUND_THREADS / 32][W];
    __shared__ u32 out[PTS * D];
    __shared__ bool is_last;
    const int tid = threadIdx.x;
    const u32 L = 1u << a.logL;

    if (a.use_low) {
        const uint4 *g = reinterpret_cast<const uint4 *>(a.low);
        uint4 *s = reinterpret_cast<uint4 *>(smem);
        for (u32 k = tid; k < L * (2 * D / 4); k += ROUND_THREADS) s[k] = g[k];
        __syncthreads();
    }

    // term descriptors in registers: factors | kind | group | table positions, and the base coefficient
    const int nterms = a.st.nterms;
    u32 desc[BASE_MAX_TERMS], coef[BASE_MAX_TERMS];
#pragma unroll
    for (int t = 0; t < BASE_MAX_TERMS; t++) {
        desc[t] = 0; coef[t] = 0;
        if (t < nterms) {
            const DevTerm &tm = a.st.terms[t];
            u32 ds = (u32)tm.nf | ((u32)tm.ckind << 4) | ((u32)tm.group << 6);
            for (int k = 0; k < BASE_MAX_FACTORS && k < tm.nf; k++) ds |= (u32)tm.f[k] << (8 + 4 * k);
            desc[t] = ds;
            coef[t] = tm.coeff[0];
        }
    }
    u32 total[NG][PTS][D];
    u64 acc[NG][PTS][D];
#pragma unroll
    for (int g = 0; g < NG; g++)
#pragma unroll
        for (int x = 0; x < PTS; x++)
#pragma unroll
            for (int c = 0; c < D; c++) { total[g][x][c] = 0; acc[g][x][c] = 0; }
    int pending = 0;            // products added to each 64-bit sum since its high word last lost a p (see presub)
    bool dirty = false;         // the 64-bit sums hold something
    u64 cur_h = ~0ull;
    u32 inner[NG][PTS][D];      // reduced sums of the current run
    bool have_inner = false;

    auto reduce = [&]() {       // acc -> inner (mod p)
#pragma unroll
        for (int g = 0; g < NG; g++)
#pragma unroll
            for (int x = 0; x < PTS; x++)
#pragma unroll
                for (int c = 0; c < D; c++) {
                    const u32 v = redc4(acc[g][x][c]);
                    inner[g][x][c] = have_inner ? fadd(inner[g][x][c], v) : v;
                    acc[g][x][c] = 0;
                }
        have_inner = true;
        pending = 0;
        dirty = false;
    };
    auto settle = [&]() {       // two more products fit after this (four fit from zero)
#pragma unroll
        for (int g = 0; g < NG; g++)
#pragma unroll
            for (int x = 0; x < PTS; x++)
#pragma unroll
                for (int c = 0; c < D; c++) acc[g][x][c] = presub(acc[g][x][c]);
        pending = 0;
    };
    auto flush = [&]() {        // total += high[h] * inner  (src/sumcheck.lisp:256-257)
        if (dirty) reduce();
        if (!have_inner) return;
        if (a.use_high) {
            Ext<D> hw = *reinterpret_cast<const Ext<D> *>(a.high + cur_h * D);
            const ExtM<D> hm = eprep<D>(hw);
#pragma unroll
            for (int g = 0; g < NG; g++)
#pragma unroll
                for (int x = 0; x < PTS; x++) {
                    Ext<D> in;
#pragma unroll
                    for (int c = 0; c < D; c++) in.v[c] = inner[g][x][c];
                    const Ext<D> pr = emul<D>(in, hm);
#pragma unroll
                    for (int c = 0; c < D; c++) total[g][x][c] = fadd(total[g][x][c], pr.v[c]);
                }
        } else {
#pragma unroll
            for (int g = 0; g < NG; g++)
#pragma unroll
                for (int x = 0; x < PTS; x++)
#pragma unroll
                    for (int c = 0; c < D; c++) total[g][x][c] = fadd(total[g][x][c], inner[g][x][c]);
        }
        have_inner = false;
    };

    // two neighbouring pairs per thread and iteration: one 128-bit load per table keeps twice the bytes in flight
    const u64 chunk = L > (u32)(2 * ROUND_THREADS) ? L : 2 * ROUND_THREADS;
    for (u64 base = (u64)blockIdx.x * chunk; base < a.npairs; base += (u64)gridDim.x * chunk) {
        for (u64 q = 2 * (u64)tid; q < chunk; q += 2 * ROUND_THREADS) {
            const u64 i0 = base + q;
            if (i0 >= a.npairs) break;
            const bool two = i0 + 1 < a.npairs;
            u32 lo2[2][NT], hi2[2][NT];
#pragma unroll
            for (int t = 0; t < NT; t++) {
                if (two) {
                    const uint4 w = __ldcs(reinterpret_cast<const uint4 *>(a.src[t] + 2 * i0));
                    lo2[0][t] = w.x; hi2[0][t] = w.y; lo2[1][t] = w.z; hi2[1][t] = w.w;
                } else {
                    const uint2 w = __ldcs(reinterpret_cast<const uint2 *>(a.src[t]) + i0);
                    lo2[0][t] = w.x; hi2[0][t] = w.y; lo2[1][t] = 0; hi2[1][t] = 0;
                }
            }
#pragma unroll
            for (int pp = 0; pp < 2; pp++) {
            if (pp == 1 && !two) break;
            const u64 i = i0 + pp;
            const u64 h = i >> a.logL;
            if (h != cur_h) {
                if (cur_h != ~0ull) flush();
                cur_h = h;
            }
            u32 val[NT], slope[NT];
#pragma unroll
            for (int t = 0; t < NT; t++) {
                val[t] = lo2[pp][t];
                slope[t] = fsub(hi2[pp][t], lo2[pp][t]);
            }
            u32 lw[D];
            if (a.use_low) {
                const u32 *w = smem + (size_t)(i & (L - 1)) * 2 * D;
#pragma unroll
                for (int c = 0; c < D; c += 4) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(w + c);
                    lw[c] = v.x; lw[c + 1] = v.y; lw[c + 2] = v.z; lw[c + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int c = 0; c < D; c++) lw[c] = c == 0 ? R1 : 0u;
            }
#pragma unroll
            for (int x = 0; x < PTS; x++) {
                if (x == 1) {
#pragma unroll
                    for (int t = 0; t < NT; t++) val[t] = fadd(fadd(val[t], slope[t]), slope[t]);
                } else if (x > 1) {
#pragma unroll
                    for (int t = 0; t < NT; t++) val[t] = fadd(val[t], slope[t]);
                }
                u32 m[NG];
#pragma unroll
                for (int g = 0; g < NG; g++) m[g] = 0;
                if (SHAPE == SHAPE_PRODUCT) {
                    u32 pr = val[0];
#pragma unroll
                    for (int t = 1; t < NT; t++) pr = mmul(pr, val[t]);
                    m[0] = pr;
                } else if (SHAPE >= SHAPE_LISTED) {
                    typedef Listed<(SHAPE >= SHAPE_LISTED ? SHAPE - SHAPE_LISTED : 0)> S;
#pragma unroll
                    for (int t = 0; t < S::NTERMS; t++) {
                        u32 pr = val[S::f(t, 0) < NT ? S::f(t, 0) : 0];
#pragma unroll
                        for (int k = 1; k < S::nf(t); k++) pr = mmul(pr, val[S::f(t, k) < NT ? S::f(t, k) : 0]);
                        if (S::ck(t) == CK_BASE) pr = mmul(pr, coef[t < BASE_MAX_TERMS ? t : 0]);
                        const int g = listed_group<S>(t) < NG ? listed_group<S>(t) : 0;
                        m[g] = fadd(m[g], pr);
                    }
                } else {
                    // the terms, from the descriptors held in registers (see BASE_MAX_TERMS)
#pragma unroll
                    for (int t = 0; t < BASE_MAX_TERMS; t++) {
                        if (t < nterms) {
                            const u32 ds = desc[t];
                            const int nf = ds & 15, ckind = (ds >> 4) & 3, group = (ds >> 6) & 3;
                            u32 pr;
                            if (nf == 0) pr = coef[t];
                            else {
                                pr = pick_base<NT>(val, (ds >> 8) & 15);
#pragma unroll
                                for (int k = 1; k < BASE_MAX_FACTORS; k++)
                                    if (k < nf) pr = mmul(pr, pick_base<NT>(val, (ds >> (8 + 4 * k)) & 15));
                                if (ckind == CK_BASE) pr = mmul(pr, coef[t]);
                            }
                            if (NG == 1 || group == 0) m[0] = fadd(m[0], pr);
                            else m[NG - 1] = fadd(m[NG - 1], pr);
                        }
                    }
                }
#pragma unroll
                for (int g = 0; g < NG; g++)
#pragma unroll
                    for (int c = 0; c < D; c++) acc[g][x][c] += (u64)lw[c] * m[g];
            }
            dirty = true;
            if (++pending == 2) settle();
            }
        }
    }
    if (cur_h != ~0ull) flush();

    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int g = 0; g < NG; g++)
#pragma unroll
        for (int x = 0; x < PTS; x++)
#pragma unroll
            for (int c = 0; c < D; c++) {
                u32 v = total[g][x][c];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v = fadd(v, __shfl_down_sync(0xffffffffu, v, off));
                if (lane == 0) red[warp][(g * PTS + x) * D + c] = v;
            }
    __syncthreads();
    if (tid < W) {
        u32 v = red[0][tid];
#pragma unroll
        for (int w = 1; w < ROUND_THREADS / 32; w++) v = fadd(v, red[w][tid]);
        a.partials[(size_t)blockIdx.x * W + tid] = v;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) is_last = atomicAdd(a.counter, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    {
        // the last block: add the partials; each group's sum times its coefficient; the final factor
        constexpr int ROWS = ROUND_THREADS / 64;     // W <= 64 words
        const int k = tid & 63, row = tid >> 6;
        u32 v = 0;
        if (k < W)
            for (unsigned g = row; g < gridDim.x; g += ROWS) v = fadd(v, __ldcg(a.partials + (size_t)g * W + k));
        __syncthreads();
        if (k < W) red[row][k] = v;
        __syncthreads();
        if (tid < PTS) {
            Ext<D> s = ezero<D>();
#pragma unroll
            for (int g = 0; g < NG; g++) {
                Ext<D> sg, cg;
#pragma unroll
                for (int c = 0; c < D; c++) {
                    u32 accw = red[0][(g * PTS + tid) * D + c];
#pragma unroll
                    for (int w = 1; w < ROWS; w++) accw = fadd(accw, red[w][(g * PTS + tid) * D + c]);
                    sg.v[c] = accw;
                    cg.v[c] = a.gcoef[g][c];
                }
                s = eadd<D>(s, emul<D>(sg, cg));
            }
            if (a.use_post) {
                Ext<D> pf;
#pragma unroll
                for (int c = 0; c < D; c++) pf.v[c] = a.post[c];
                s = emul<D>(s, pf);
            }
#pragma unroll
            for (int c = 0; c < D; c++) out[tid * D + c] = s.v[c];
        }
        __syncthreads();
        if (tid == 0) *a.counter = 0;
        publish_round(a, out, PTS * D);
    }
}

template <int D, int PTS, int NT, int NG, int SHAPE>
static cudaError_t launch_base_one(const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    if (smem > 40 * 1024) cudaFuncSetAttribute(round_base_kernel<D, PTS, NT, NG, SHAPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    round_base_kernel<D, PTS, NT, NG, SHAPE><<<grid, ROUND_THREADS, smem, stream>>>(args);
    return cudaGetLastError();
}
template <int D, int PTS, int NT>
static cudaError_t launch_base_dpn(int ng, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    if (ng == 1) return launch_base_one<D, PTS, NT, 1, SHAPE_GENERIC>(args, grid, smem, stream);
    return launch_base_one<D, PTS, NT, 2, SHAPE_GENERIC>(args, grid, smem, stream);
}
template <int D, int PTS>
static cudaError_t launch_base_dp(int nt, int ng, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    switch (nt) {
    case 1: return launch_base_dpn<D, PTS, 1>(ng, args, grid, smem, stream);
    case 2: return launch_base_dpn<D, PTS, 2>(ng, args, grid, smem, stream);
    case 3: return launch_base_dpn<D, PTS, 3>(ng, args, grid, smem, stream);
    case 4: return launch_base_dpn<D, PTS, 4>(ng, args, grid, smem, stream);
    default: return cudaErrorInvalidValue;
    }
}
template <int D, int K>
static cudaError_t launch_base_listed(const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    typedef Listed<K> S;
    return launch_base_one<D, S::PTS, S::NT, listed_groups<S>(), SHAPE_LISTED + K>(args, grid, smem, stream);
}
template <int D>
static cudaError_t launch_base_d(int shape, int points, int nt, int ng, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    if (shape == SHAPE_PRODUCT && points == nt && ng == 1) {
        switch (nt) {
        case 1: return launch_base_one<D, 1, 1, 1, SHAPE_PRODUCT>(args, grid, smem, stream);
        case 2: return launch_base_one<D, 2, 2, 1, SHAPE_PRODUCT>(args, grid, smem, stream);
        case 3: return launch_base_one<D, 3, 3, 1, SHAPE_PRODUCT>(args, grid, smem, stream);
        case 4: return launch_base_one<D, 4, 4, 1, SHAPE_PRODUCT>(args, grid, smem, stream);
        }
    }
    // the listed statements with at most one extension-field coefficient (the kernel keeps two sums at most)
    if (shape == SHAPE_LISTED + 0) return launch_base_listed<D, 0>(args, grid, smem, stream);
    if (shape == SHAPE_LISTED + 1) return launch_base_listed<D, 1>(args, grid, smem, stream);
    switch (points) {
    case 1: return launch_base_dp<D, 1>(nt, ng, args, grid, smem, stream);
    case 2: return launch_base_dp<D, 2>(nt, ng, args, grid, smem, stream);
    case 3: return launch_base_dp<D, 3>(nt, ng, args, grid, smem, stream);
    case 4: return launch_base_dp<D, 4>(nt, ng, args, grid, smem, stream);
    default: return cudaErrorInvalidValue;
    }
}

// the groups a listed statement runs this kernel with, or 0 when it cannot (more than one extension-field coefficient)
int listed_base_groups(int shape) {
    if (shape == SHAPE_LISTED + 0) return listed_groups<Listed<0>>();
    if (shape == SHAPE_LISTED + 1) return listed_groups<Listed<1>>();
    return 0;
}
int listed_base_group_of(int shape, int term) {
    if (shape == SHAPE_LISTED + 0) return listed_group<Listed<0>>(term);
    if (shape == SHAPE_LISTED + 1) return listed_group<Listed<1>>(term);
    return 0;
}

cudaError_t launch_round_base(int D, int shape, int points, int nt_used, int ngroups, const RoundArgs &args, int grid, size_t smem,
                              cudaStream_t stream) {
    if (ngroups < 1 || ngroups > MAX_GROUPS) return cudaErrorInvalidValue;
    if (D == 4) return launch_base_d<4>(shape, points, nt_used, ngroups, args, grid, smem, stream);
    if (D == 8) return launch_base_d<8>(shape, points, nt_used, ngroups, args, grid, smem, stream);
    return cudaErrorInvalidValue;
}

}  // namespace sc
