// round_sv.cu -- rounds 0 and 1 of a statement over base-field tables from one pass (see SvArgs): the reference's
// small-value rounds (SMALL-VALUE-CODE and GRID-CODE, src/sumcheck.lisp:344-427) with L0 = 2.
//
// Work split: a thread keeps one low index l of the split eq weights and walks the high indices h
// of its block's share, reading block y = h L + l of every table (one 128-bit load per table;
// neighbouring threads read neighbouring blocks).  Per block it adds w_high[h] F(z) into G^2 D
// 64-bit sums that are reduced once, at the end (the reference reduces once per four products, REDUCED-SUM,
// src/field.lisp:213-218; here a sum's high word loses one p before every second block, which keeps it within
// 64 bits: presub, field.cuh); the low weight multiplies once at the very end.  Blocks' rows are added by the last block to finish (no waiting).
// The grid of G^2 points is cut along its second variable (blockIdx.y) so that a thread's sums fit its
// registers: two rows per block at D = 4 (rows z1 < 2 are the entries' own rows), one row at D = 8 or with two groups.
// The statement at a grid point is a product of the tables (SHAPE_PRODUCT), a listed statement resolved at
// compile time, or the term table with its descriptors in registers, as in the base-table round kernel; as there,
// a term with an extension-field coefficient is summed without it in a group of its own (NG = 2), and the last
// block multiplies each group's accumulators by the group's coefficient before it adds them up: so a statement
// with constants takes these rounds too (the reference folds those from round 0: its kernel works on base values
// only, src/sumcheck.lisp:535-539), and the proof bytes are the same.
#include "round_kernel.cuh"

namespace sc {

template <int NT> __device__ __forceinline__ u32 sv_pick(const u32 (&val)[NT], int idx) {
    u32 o = val[0];
#pragma unroll
    for (int t = 1; t < NT; t++)
        if (idx == t) o = val[t];
    return o;
}

// One sum per grid point (every coefficient in the base field, or a product whose coefficient rides in the final factor).
template <int D, int G, int NT, int SHAPE>
__global__ void __launch_bounds__(ROUND_THREADS, G > 2 ? 2 : 1) sv_kernel(const __grid_constant__ SvArgs a) {
    constexpr int ROWS1 = D == 4 ? 2 : 1;         // rows of the grid (values of z1) a block handles, at most
    constexpr int Z = G * ROWS1, W = Z * D;       // this block's share of the accumulators
    constexpr int WALL = G * G * D;               // all of them
    const int z1lo = blockIdx.y * ROWS1;          // its first row
    const int nrows = (G - z1lo) < ROWS1 ? (G - z1lo) : ROWS1;
    extern __shared__ __align__(16) u32 tot[];   // [W][ROUND_THREADS]
    __shared__ bool is_last;
    const int tid = threadIdx.x;
    const u32 L = 1u << a.logL;
    const u32 lchunks = L / ROUND_THREADS;
    const u32 lc = blockIdx.x % lchunks, hg = blockIdx.x / lchunks, nhg = gridDim.x / lchunks;
    const u64 NH = a.nblocks >> a.logL;
    const u64 h0 = NH * hg / nhg, h1 = NH * (hg + 1) / nhg;
    const u32 l = lc * ROUND_THREADS + tid;

    // the term table's descriptors in registers: factors | positions, and the base coefficient
    const int nterms = a.st.nterms;
    u32 desc[BASE_MAX_TERMS], coef[BASE_MAX_TERMS];
#pragma unroll
    for (int t = 0; t < BASE_MAX_TERMS; t++) {
        desc[t] = 0; coef[t] = 0;
        if (SHAPE != SHAPE_PRODUCT && t < nterms) {
            const DevTerm &tm = a.st.terms[t];
            u32 ds = (u32)tm.nf | ((u32)tm.ckind << 4);
            for (int k = 0; k < BASE_MAX_FACTORS && k < tm.nf; k++) ds |= (u32)tm.f[k] << (8 + 4 * k);
            desc[t] = ds;
            coef[t] = tm.coeff[0];
        }
    }
    // the statement on the tables' values at one grid point (base field; the factor R^-e the products leave behind
    // is the final factor's business, as in every round kernel)
    auto statement = [&](const u32 (&val)[NT]) -> u32 {
        if (SHAPE == SHAPE_PRODUCT) {
            u32 f = val[0];
#pragma unroll
            for (int t = 1; t < NT; t++) f = mmul(f, val[t]);
            return f;
        } else if (SHAPE >= SHAPE_LISTED) {
            typedef Listed<(SHAPE >= SHAPE_LISTED ? SHAPE - SHAPE_LISTED : 0)> S;
            u32 f = 0;
#pragma unroll
            for (int t = 0; t < S::NTERMS; t++) {
                u32 pr = val[S::f(t, 0) < NT ? S::f(t, 0) : 0];
#pragma unroll
                for (int k = 1; k < S::nf(t); k++) pr = mmul(pr, val[S::f(t, k) < NT ? S::f(t, k) : 0]);
                pr = mmul(pr, coef[t < BASE_MAX_TERMS ? t : 0]);   // a listed statement's coefficients here are base elements
                f = fadd(f, pr);
            }
            return f;
        } else {
            u32 f = 0;
#pragma unroll
            for (int t = 0; t < BASE_MAX_TERMS; t++) {
                if (t < nterms) {
                    const u32 ds = desc[t];
                    const int nf = ds & 15, ckind = (ds >> 4) & 3;
                    u32 pr;
                    if (nf == 0) pr = coef[t];
                    else {
                        pr = sv_pick<NT>(val, (ds >> 8) & 15);
#pragma unroll
                        for (int k = 1; k < BASE_MAX_FACTORS; k++)
                            if (k < nf) pr = mmul(pr, sv_pick<NT>(val, (ds >> (8 + 4 * k)) & 15));
                        if (ckind == CK_BASE) pr = mmul(pr, coef[t]);
                    }
                    f = fadd(f, pr);
                }
            }
            return f;
        }
    };

    u64 acc[Z][D];
#pragma unroll
    for (int z = 0; z < Z; z++)
#pragma unroll
        for (int c = 0; c < D; c++) acc[z][c] = 0;
    // The 64-bit sums run on without a reduction: before every second block each sum's high word loses one p when it can
    // (presub, field.cuh), which keeps a sum below p 2^32 there and below 2 p 2^32 after two more products: what redc4 takes.
    bool second = false;

    // the next block's entries are asked for before this block's arithmetic starts
    uint4 next[NT];
    if (h0 < h1) {
#pragma unroll
        for (int t = 0; t < NT; t++) next[t] = __ldcs(reinterpret_cast<const uint4 *>(a.src[t]) + (h0 * L + l));
    }
    for (u64 h = h0; h < h1; h++) {
        uint4 cur[NT];
#pragma unroll
        for (int t = 0; t < NT; t++) cur[t] = next[t];
        if (h + 1 < h1) {
#pragma unroll
            for (int t = 0; t < NT; t++) next[t] = __ldcs(reinterpret_cast<const uint4 *>(a.src[t]) + ((h + 1) * L + l));
        }
        u32 g[NT][Z];
#pragma unroll
        for (int t = 0; t < NT; t++) {
            const uint4 e = cur[t];
            // entries (b0, b1) = e.x (0,0), e.y (1,0), e.z (0,1), e.w (1,1); extend variable 0, then variable 1, by additions
            u32 row[2][G];
            row[0][0] = e.x; row[0][1] = e.y; row[1][0] = e.z; row[1][1] = e.w;
#pragma unroll
            for (int b1 = 0; b1 < 2; b1++) {
                const u32 s = fsub(row[b1][1], row[b1][0]);
#pragma unroll
                for (int z0 = 2; z0 < G; z0++) row[b1][z0] = fadd(row[b1][z0 - 1], s);
            }
#pragma unroll
            for (int z0 = 0; z0 < G; z0++) {
                if (ROWS1 == 2) {
                    if (z1lo == 0) {           // rows 0 and 1: the entries' own rows
                        g[t][z0] = row[0][z0];
                        g[t][(z0 + G) % Z] = row[1][z0];
                    } else {                   // rows 2 and 3: row 1 plus one and two slopes
                        const u32 s = fsub(row[1][z0], row[0][z0]);
                        g[t][z0] = fadd(row[1][z0], s);
                        g[t][(z0 + G) % Z] = fadd(g[t][z0], s);
                    }
                } else {                       // one row: z1 = z1lo, row 0 plus z1lo slopes
                    u32 v = z1lo == 0 ? row[0][z0] : row[1][z0];
                    const u32 s = fsub(row[1][z0], row[0][z0]);
                    for (int k = 1; k < z1lo; k++) v = fadd(v, s);
                    g[t][z0] = v;
                }
            }
        }
        u32 hw[D];
        if (a.use_high) {
            const uint4 *hp = reinterpret_cast<const uint4 *>(a.high + h * D);
#pragma unroll
            for (int c = 0; c < D; c += 4) { const uint4 v = __ldg(hp + c / 4); hw[c] = v.x; hw[c + 1] = v.y; hw[c + 2] = v.z; hw[c + 3] = v.w; }
        } else {
#pragma unroll
            for (int c = 0; c < D; c++) hw[c] = c == 0 ? R1 : 0u;
        }
#pragma unroll
        for (int z = 0; z < Z; z++) {
            u32 val[NT];
#pragma unroll
            for (int t = 0; t < NT; t++) val[t] = g[t][z];
            const u32 f = statement(val);
#pragma unroll
            for (int c = 0; c < D; c++) acc[z][c] = (second ? presub(acc[z][c]) : acc[z][c]) + (u64)hw[c] * f;
        }
        second = !second;
    }
#pragma unroll
    for (int z = 0; z < Z; z++)
#pragma unroll
        for (int c = 0; c < D; c++) tot[(z * D + c) * ROUND_THREADS + tid] = redc4(acc[z][c]);

    // the low weight, once per thread
    if (a.use_low) {
        const u32 *w = a.low + (size_t)l * 2 * D;
        ExtM<D> lw;
#pragma unroll
        for (int c = 0; c < D; c++) { lw.v[c] = __ldg(w + c); lw.t[c] = __ldg(w + D + c); }
        for (int z = 0; z < Z; z++) {
            Ext<D> v;
#pragma unroll
            for (int c = 0; c < D; c++) v.v[c] = tot[(z * D + c) * ROUND_THREADS + tid];
            v = emul<D>(v, lw);
#pragma unroll
            for (int c = 0; c < D; c++) tot[(z * D + c) * ROUND_THREADS + tid] = v.v[c];
        }
    }
    __syncthreads();
    // the block's share of its row of partial sums: word k summed over the threads
    for (int k = tid >> 5; k < nrows * G * D; k += ROUND_THREADS / 32) {
        u32 v = 0;
        for (int j = tid & 31; j < ROUND_THREADS; j += 32) v = fadd(v, tot[k * ROUND_THREADS + j]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v = fadd(v, __shfl_down_sync(0xffffffffu, v, off));
        if ((tid & 31) == 0) a.partials[(size_t)blockIdx.x * WALL + z1lo * G * D + k] = v;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) is_last = atomicAdd(a.counter, 1u) == gridDim.x * gridDim.y - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    __shared__ u32 row[SV_MAX_WORDS];
    if (tid < WALL) {
        u32 v = 0;
        for (unsigned b = 0; b < gridDim.x; b++) v = fadd(v, __ldcg(a.partials + (size_t)b * WALL + tid));
        row[tid] = v;
    }
    __syncthreads();
    if (tid < G * G) {
        Ext<D> s;
#pragma unroll
        for (int c = 0; c < D; c++) s.v[c] = row[tid * D + c];
        if (a.use_post) {
            Ext<D> pf;
#pragma unroll
            for (int c = 0; c < D; c++) pf.v[c] = a.post[c];
            s = emul<D>(s, pf);
        }
#pragma unroll
        for (int c = 0; c < D; c++) {
            if (a.out_dev) a.out_dev[tid * D + c] = s.v[c];
            if (a.out_host) a.out_host[tid * D + c] = s.v[c];
        }
    }
    __syncthreads();
    if (tid == 0) {
        *a.counter = 0;
        if (a.out_host) {
            __threadfence_system();
            *reinterpret_cast<volatile u32 *>(a.out_host + SV_FLAG) = a.seq;
        }
    }
}

// Two sums per grid point: the same pass with the accumulators doubled, one row of the grid per block.  Kept apart from the
// kernel above, which the benchmark configs C2 and C5 run: the two were measured as one template, and that one was 8 % slower
// on them (12.2 against 13.2 ms for the pass of C5) although its code for one sum is the same.
template <int D, int NG> __host__ __device__ constexpr int sv_rows() { return D == 4 && NG == 1 ? 2 : 1; }

template <int D, int G, int NT, int SHAPE, int NG>
__global__ void __launch_bounds__(ROUND_THREADS, G > 2 ? (D == 4 && G == 3 ? 3 : 2) : 1) sv_groups_kernel(const __grid_constant__ SvArgs a) {
    constexpr int ROWS1 = sv_rows<D, NG>();       // rows of the grid (values of z1) a block handles, at most
    constexpr int Z = G * ROWS1, W = NG * Z * D;  // this block's share of the accumulators
    constexpr int WONE = G * G * D;               // one group's accumulators
    constexpr int WALL = NG * WONE;               // all of them
    const int z1lo = blockIdx.y * ROWS1;          // its first row
    const int nrows = (G - z1lo) < ROWS1 ? (G - z1lo) : ROWS1;
    extern __shared__ __align__(16) u32 tot[];   // [W][ROUND_THREADS]
    __shared__ bool is_last;
    const int tid = threadIdx.x;
    const u32 L = 1u << a.logL;
    const u32 lchunks = L / ROUND_THREADS;
    const u32 lc = blockIdx.x % lchunks, hg = blockIdx.x / lchunks, nhg = gridDim.x / lchunks;
    const u64 NH = a.nblocks >> a.logL;
    const u64 h0 = NH * hg / nhg, h1 = NH * (hg + 1) / nhg;
    const u32 l = lc * ROUND_THREADS + tid;

    // the term table's descriptors in registers: factors | positions, and the base coefficient
    const int nterms = a.st.nterms;
    u32 desc[BASE_MAX_TERMS], coef[BASE_MAX_TERMS];
#pragma unroll
    for (int t = 0; t < BASE_MAX_TERMS; t++) {
        desc[t] = 0; coef[t] = 0;
        if (SHAPE != SHAPE_PRODUCT && t < nterms) {
            const DevTerm &tm = a.st.terms[t];
            u32 ds = (u32)tm.nf | ((u32)tm.ckind << 4) | ((u32)(tm.group & 1) << 6);
            for (int k = 0; k < BASE_MAX_FACTORS && k < tm.nf; k++) ds |= (u32)tm.f[k] << (8 + 4 * k);
            desc[t] = ds;
            coef[t] = tm.coeff[0];
        }
    }
    // the statement on the tables' values at one grid point (base field; the factor R^-e the products leave behind
    // is the final factor's business, as in every round kernel)
    auto statement = [&](const u32 (&val)[NT], u32 (&f)[NG]) {
#pragma unroll
        for (int g = 0; g < NG; g++) f[g] = 0;
        if (SHAPE == SHAPE_PRODUCT) {
            u32 pr = val[0];
#pragma unroll
            for (int t = 1; t < NT; t++) pr = mmul(pr, val[t]);
            f[0] = pr;
        } else if (SHAPE >= SHAPE_LISTED) {
            typedef Listed<(SHAPE >= SHAPE_LISTED ? SHAPE - SHAPE_LISTED : 0)> S;
#pragma unroll
            for (int t = 0; t < S::NTERMS; t++) {
                u32 pr = val[S::f(t, 0) < NT ? S::f(t, 0) : 0];
#pragma unroll
                for (int k = 1; k < S::nf(t); k++) pr = mmul(pr, val[S::f(t, k) < NT ? S::f(t, k) : 0]);
                if (S::ck(t) == CK_BASE) pr = mmul(pr, coef[t < BASE_MAX_TERMS ? t : 0]);   // the others wait for the group's coefficient
                const int g = listed_group<S>(t) < NG ? listed_group<S>(t) : 0;
                f[g] = fadd(f[g], pr);
            }
        } else {
#pragma unroll
            for (int t = 0; t < BASE_MAX_TERMS; t++) {
                if (t < nterms) {
                    const u32 ds = desc[t];
                    const int nf = ds & 15, ckind = (ds >> 4) & 3, group = (ds >> 6) & 1;
                    u32 pr;
                    if (nf == 0) pr = coef[t];
                    else {
                        pr = sv_pick<NT>(val, (ds >> 8) & 15);
#pragma unroll
                        for (int k = 1; k < BASE_MAX_FACTORS; k++)
                            if (k < nf) pr = mmul(pr, sv_pick<NT>(val, (ds >> (8 + 4 * k)) & 15));
                        if (ckind == CK_BASE) pr = mmul(pr, coef[t]);
                    }
                    if (NG > 1 && group) f[NG - 1] = fadd(f[NG - 1], pr);
                    else f[0] = fadd(f[0], pr);
                }
            }
        }
    };

    u64 acc[NG][Z][D];
#pragma unroll
    for (int g = 0; g < NG; g++)
#pragma unroll
        for (int z = 0; z < Z; z++)
#pragma unroll
            for (int c = 0; c < D; c++) acc[g][z][c] = 0;
    bool second = false;   // the sums run on without a reduction, as in sv_kernel

    // the next block's entries are asked for before this block's arithmetic starts
    uint4 next[NT];
    if (h0 < h1) {
#pragma unroll
        for (int t = 0; t < NT; t++) next[t] = __ldcs(reinterpret_cast<const uint4 *>(a.src[t]) + (h0 * L + l));
    }
    for (u64 h = h0; h < h1; h++) {
        uint4 cur[NT];
#pragma unroll
        for (int t = 0; t < NT; t++) cur[t] = next[t];
        if (h + 1 < h1) {
#pragma unroll
            for (int t = 0; t < NT; t++) next[t] = __ldcs(reinterpret_cast<const uint4 *>(a.src[t]) + ((h + 1) * L + l));
        }
        u32 g[NT][Z];
#pragma unroll
        for (int t = 0; t < NT; t++) {
            const uint4 e = cur[t];
            // entries (b0, b1) = e.x (0,0), e.y (1,0), e.z (0,1), e.w (1,1); extend variable 0, then variable 1, by additions
            u32 row[2][G];
            row[0][0] = e.x; row[0][1] = e.y; row[1][0] = e.z; row[1][1] = e.w;
#pragma unroll
            for (int b1 = 0; b1 < 2; b1++) {
                const u32 s = fsub(row[b1][1], row[b1][0]);
#pragma unroll
                for (int z0 = 2; z0 < G; z0++) row[b1][z0] = fadd(row[b1][z0 - 1], s);
            }
#pragma unroll
            for (int z0 = 0; z0 < G; z0++) {
                if (ROWS1 == 2) {
                    if (z1lo == 0) {           // rows 0 and 1: the entries' own rows
                        g[t][z0] = row[0][z0];
                        g[t][(z0 + G) % Z] = row[1][z0];
                    } else {                   // rows 2 and 3: row 1 plus one and two slopes
                        const u32 s = fsub(row[1][z0], row[0][z0]);
                        g[t][z0] = fadd(row[1][z0], s);
                        g[t][(z0 + G) % Z] = fadd(g[t][z0], s);
                    }
                } else {                       // one row: z1 = z1lo, row 0 plus z1lo slopes
                    u32 v = z1lo == 0 ? row[0][z0] : row[1][z0];
                    const u32 s = fsub(row[1][z0], row[0][z0]);
                    for (int k = 1; k < z1lo; k++) v = fadd(v, s);
                    g[t][z0] = v;
                }
            }
        }
        u32 hw[D];
        if (a.use_high) {
            const uint4 *hp = reinterpret_cast<const uint4 *>(a.high + h * D);
#pragma unroll
            for (int c = 0; c < D; c += 4) { const uint4 v = __ldg(hp + c / 4); hw[c] = v.x; hw[c + 1] = v.y; hw[c + 2] = v.z; hw[c + 3] = v.w; }
        } else {
#pragma unroll
            for (int c = 0; c < D; c++) hw[c] = c == 0 ? R1 : 0u;
        }
#pragma unroll
        for (int z = 0; z < Z; z++) {
            u32 val[NT];
#pragma unroll
            for (int t = 0; t < NT; t++) val[t] = g[t][z];
            u32 f[NG];
            statement(val, f);
#pragma unroll
            for (int g = 0; g < NG; g++)
#pragma unroll
                for (int c = 0; c < D; c++) acc[g][z][c] = (second ? presub(acc[g][z][c]) : acc[g][z][c]) + (u64)hw[c] * f[g];
        }
        second = !second;
    }
#pragma unroll
    for (int g = 0; g < NG; g++)
#pragma unroll
        for (int z = 0; z < Z; z++)
#pragma unroll
            for (int c = 0; c < D; c++) tot[((g * Z + z) * D + c) * ROUND_THREADS + tid] = redc4(acc[g][z][c]);

    // the low weight, once per thread
    if (a.use_low) {
        const u32 *w = a.low + (size_t)l * 2 * D;
        ExtM<D> lw;
#pragma unroll
        for (int c = 0; c < D; c++) { lw.v[c] = __ldg(w + c); lw.t[c] = __ldg(w + D + c); }
        for (int z = 0; z < NG * Z; z++) {
            Ext<D> v;
#pragma unroll
            for (int c = 0; c < D; c++) v.v[c] = tot[(z * D + c) * ROUND_THREADS + tid];
            v = emul<D>(v, lw);
#pragma unroll
            for (int c = 0; c < D; c++) tot[(z * D + c) * ROUND_THREADS + tid] = v.v[c];
        }
    }
    __syncthreads();
    // the block's share of its row of partial sums: word k summed over the threads
    for (int gk = tid >> 5; gk < NG * nrows * G * D; gk += ROUND_THREADS / 32) {
        const int g = gk / (nrows * G * D), k = gk % (nrows * G * D);
        u32 v = 0;
        for (int j = tid & 31; j < ROUND_THREADS; j += 32) v = fadd(v, tot[(g * Z * D + k) * ROUND_THREADS + j]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v = fadd(v, __shfl_down_sync(0xffffffffu, v, off));
        if ((tid & 31) == 0) a.partials[(size_t)blockIdx.x * WALL + g * WONE + z1lo * G * D + k] = v;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) is_last = atomicAdd(a.counter, 1u) == gridDim.x * gridDim.y - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    __shared__ u32 row[MAX_GROUPS * SV_MAX_WORDS];
    static_assert(WALL <= ROUND_THREADS && WALL <= MAX_GROUPS * SV_MAX_WORDS, "one thread per accumulator word");
    if (tid < WALL) {
        u32 v = 0;
        for (unsigned b = 0; b < gridDim.x; b++) v = fadd(v, __ldcg(a.partials + (size_t)b * WALL + tid));
        row[tid] = v;
    }
    __syncthreads();
    if (tid < G * G) {
        Ext<D> s;
#pragma unroll
        for (int c = 0; c < D; c++) s.v[c] = row[tid * D + c];
        if (NG > 1 || a.use_gcoef) {   // each group's accumulators times the group's coefficient
            s = ezero<D>();
#pragma unroll
            for (int g = 0; g < NG; g++) {
                Ext<D> v, gc;
#pragma unroll
                for (int c = 0; c < D; c++) { v.v[c] = row[g * WONE + tid * D + c]; gc.v[c] = a.gcoef[g][c]; }
                s = eadd<D>(s, emul<D>(v, gc));
            }
        }
        if (a.use_post) {
            Ext<D> pf;
#pragma unroll
            for (int c = 0; c < D; c++) pf.v[c] = a.post[c];
            s = emul<D>(s, pf);
        }
#pragma unroll
        for (int c = 0; c < D; c++) {
            if (a.out_dev) a.out_dev[tid * D + c] = s.v[c];
            if (a.out_host) a.out_host[tid * D + c] = s.v[c];
        }
    }
    __syncthreads();
    if (tid == 0) {
        *a.counter = 0;
        if (a.out_host) {
            __threadfence_system();
            *reinterpret_cast<volatile u32 *>(a.out_host + SV_FLAG) = a.seq;
        }
    }
}

template <int D, int G, int NT, int SHAPE, int NG> static cudaError_t launch_sv_one(const SvArgs &args, int grid, cudaStream_t stream) {
    if constexpr (NG == 1) {
        constexpr int ROWS1 = D == 4 ? 2 : 1;
        const size_t smem = (size_t)G * ROWS1 * D * ROUND_THREADS * 4;
        cudaFuncSetAttribute(sv_kernel<D, G, NT, SHAPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        sv_kernel<D, G, NT, SHAPE><<<dim3(grid, (G + ROWS1 - 1) / ROWS1), ROUND_THREADS, smem, stream>>>(args);
    } else {
        constexpr int ROWS1 = sv_rows<D, NG>();
        const size_t smem = (size_t)NG * G * ROWS1 * D * ROUND_THREADS * 4;
        cudaFuncSetAttribute(sv_groups_kernel<D, G, NT, SHAPE, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        sv_groups_kernel<D, G, NT, SHAPE, NG><<<dim3(grid, (G + ROWS1 - 1) / ROWS1), ROUND_THREADS, smem, stream>>>(args);
    }
    return cudaGetLastError();
}
template <int D, int G, int NG> static cudaError_t launch_sv_generic(int nt, const SvArgs &args, int grid, cudaStream_t stream) {
    switch (nt) {
    case 1: return launch_sv_one<D, G, 1, SHAPE_GENERIC, NG>(args, grid, stream);
    case 2: return launch_sv_one<D, G, 2, SHAPE_GENERIC, NG>(args, grid, stream);
    case 3: return launch_sv_one<D, G, 3, SHAPE_GENERIC, NG>(args, grid, stream);
    }
    return cudaErrorInvalidValue;
}
template <int D, int K> static cudaError_t launch_sv_listed(const SvArgs &args, int grid, cudaStream_t stream) {
    typedef Listed<K> S;   // the groups its entry says, as in the base-table kernel
    return launch_sv_one<D, S::PTS + 1, S::NT, SHAPE_LISTED + K, listed_groups<S>()>(args, grid, stream);
}
template <int D> static cudaError_t launch_sv_d(int shape, int G, int nt, int ng, const SvArgs &args, int grid, cudaStream_t stream) {
    if (shape == SHAPE_PRODUCT && G == nt + 1 && ng == 1) {
        switch (nt) {
        case 1: return launch_sv_one<D, 2, 1, SHAPE_PRODUCT, 1>(args, grid, stream);
        case 2: return launch_sv_one<D, 3, 2, SHAPE_PRODUCT, 1>(args, grid, stream);
        case 3: return launch_sv_one<D, 4, 3, SHAPE_PRODUCT, 1>(args, grid, stream);
        }
    }
    // a listed statement: one sum when all its coefficients are base elements, else the sums its entry says
    if (shape == SHAPE_LISTED + 0 && ng == 1) return launch_sv_one<D, Listed<0>::PTS + 1, Listed<0>::NT, SHAPE_LISTED + 0, 1>(args, grid, stream);
    if (shape == SHAPE_LISTED + 1 && ng == 1) return launch_sv_one<D, Listed<1>::PTS + 1, Listed<1>::NT, SHAPE_LISTED + 1, 1>(args, grid, stream);
    if (shape == SHAPE_LISTED + 0 && ng == listed_groups<Listed<0>>()) return launch_sv_listed<D, 0>(args, grid, stream);
    if (shape == SHAPE_LISTED + 1 && ng == listed_groups<Listed<1>>()) return launch_sv_listed<D, 1>(args, grid, stream);
    if (ng == 1) {
        switch (G) {
        case 2: return launch_sv_generic<D, 2, 1>(nt, args, grid, stream);
        case 3: return launch_sv_generic<D, 3, 1>(nt, args, grid, stream);
        case 4: return launch_sv_generic<D, 4, 1>(nt, args, grid, stream);
        }
    } else {
        switch (G) {
        case 2: return launch_sv_generic<D, 2, 2>(nt, args, grid, stream);
        case 3: return launch_sv_generic<D, 3, 2>(nt, args, grid, stream);
        case 4: return launch_sv_generic<D, 4, 2>(nt, args, grid, stream);
        }
    }
    return cudaErrorInvalidValue;
}
// The thread blocks along x a pass is launched with.  The kernels cut the grid of points over blockIdx.y; one block along x per
// SM gives them one or two full waves of thread blocks, except for three rounds at D = 4, where a plane of the grid per thread
// block (G of them, two blocks per SM) fills the GPU once with 2 / G blocks along x per SM (measured: 444 blocks on 296 places
// ran a wave and a half).
int small_values_grid_x(int D, int G, int ngroups, int l0, int sms) {
    (void)ngroups;
    if (l0 == 3 && D == 4) { const int x = sms * 2 / G; return x > 0 ? x : 1; }
    return sms;
}
// G = points + 1 grid values per variable: degree at most three, at most three tables in the statement
bool small_values_supported(int D, int G, int nt) { return (D == 4 || D == 8) && nt >= 1 && nt <= 3 && G >= 2 && G <= 4; }
cudaError_t launch_small_values(int D, int shape, int G, int nt, const SvArgs &args, int grid, cudaStream_t stream) {
    if (!small_values_supported(D, G, nt) || args.ngroups < 1 || args.ngroups > MAX_GROUPS) return cudaErrorInvalidValue;
    if (shape == SHAPE_LISTED + 2 || shape == SHAPE_GKR) shape = SHAPE_GENERIC;
    return D == 4 ? launch_sv_d<4>(shape, G, nt, args.ngroups, args, grid, stream) : launch_sv_d<8>(shape, G, nt, args.ngroups, args, grid, stream);
}

}  // namespace sc
