// round_sv3.cu -- rounds 0, 1 and 2 of a statement of degree at most two over base-field tables from one pass: the
// reference's small-value rounds (SMALL-VALUE-CODE and GRID-CODE, src/sumcheck.lisp:344-427) with L0 = 3, what
// CHOOSE-SMALL-VALUE-KERNEL (:450-455) takes when the kernel's code fits its limit.
//
// The pass is that of round_sv.cu with blocks of eight entries and a grid of G^3 points: a thread keeps one low index
// l of the split eq weights (those of round 2: the variables after the first three) and walks the high indices h of
// its block's share, reading block y = h L + l of every table (two 128-bit loads per table).  The block's values on
// {0..G-1}^3 come by additions: variable 2 first (the plane z2 of this thread block: blockIdx.y), then variable 1,
// then variable 0.  A thread block keeps the accumulators of one plane at D = 4 (G^2 points) and of one row of a plane
// at D = 8 (G points), so that they fit the registers.  Per block of entries it adds w_high[h] F(z) into 64-bit sums,
// reduced once at the end; the low weight multiplies once at the very end; the last thread block to finish adds the
// rows of partial sums.  One sum per grid point: every coefficient is a base element (a product's rides in the final factor).
#include "round_kernel.cuh"

namespace sc {

template <int NT> __device__ __forceinline__ u32 sv3_pick(const u32 (&val)[NT], int idx) {
    u32 o = val[0];
#pragma unroll
    for (int t = 1; t < NT; t++)
        if (idx == t) o = val[t];
    return o;
}

template <int D, int G> __host__ __device__ constexpr int sv3_rows() { return D == 4 ? G : 1; }   // rows (values of z1) per thread block

template <int D, int G, int NT, int SHAPE>
__global__ void __launch_bounds__(ROUND_THREADS, 2) sv3_kernel(const __grid_constant__ SvArgs a) {
    constexpr int ROWS = sv3_rows<D, G>();
    constexpr int Z = G * ROWS, W = Z * D;        // this thread block's share of the accumulators
    constexpr int WALL = G * G * G * D;           // all of them
    constexpr int YPP = G / ROWS;                 // thread blocks per plane
    const int z2 = blockIdx.y / YPP, z1lo = (blockIdx.y % YPP) * ROWS;
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
                pr = mmul(pr, coef[t < BASE_MAX_TERMS ? t : 0]);   // base elements, all of them, on this path
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
                        pr = sv3_pick<NT>(val, (ds >> 8) & 15);
#pragma unroll
                        for (int k = 1; k < BASE_MAX_FACTORS; k++)
                            if (k < nf) pr = mmul(pr, sv3_pick<NT>(val, (ds >> (8 + 4 * k)) & 15));
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
    // v + k s for k = 0 .. G-1 at position k (k = 0: v, k = 1: w = v + s given, k = 2: w + s)
    auto at = [](u32 v, u32 w, int k) -> u32 {
        if (k == 0) return v;
        if (k == 1) return w;
        return fadd(w, fsub(w, v));
    };

    for (u64 h = h0; h < h1; h++) {
        u32 g[NT][Z];
#pragma unroll
        for (int t = 0; t < NT; t++) {
            const uint4 *p = reinterpret_cast<const uint4 *>(a.src[t]) + 2 * (h * L + l);
            const uint4 e0 = __ldcs(p), e1 = __ldcs(p + 1);
            // entries (b0, b1, b2): e0 = (0,0,0) (1,0,0) (0,1,0) (1,1,0), e1 the same with b2 = 1
            const u32 lo[4] = {e0.x, e0.y, e0.z, e0.w}, hi[4] = {e1.x, e1.y, e1.z, e1.w};
            u32 pl[4];   // the plane z2: variable 2 extended
#pragma unroll
            for (int b = 0; b < 4; b++) pl[b] = at(lo[b], hi[b], z2);
#pragma unroll
            for (int r = 0; r < ROWS; r++) {
                const int z1 = z1lo + r;
                const u32 r0 = at(pl[0], pl[2], z1), r1 = at(pl[1], pl[3], z1);   // variable 1 extended: (b0 = 0), (b0 = 1)
#pragma unroll
                for (int z0 = 0; z0 < G; z0++) g[t][r * G + z0] = at(r0, r1, z0);
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

    if (a.use_low) {   // the low weight, once per thread
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
    // this thread block's share of its row of partial sums: word k summed over the threads; grid point z = z0 + G z1 + G^2 z2
    for (int k = tid >> 5; k < W; k += ROUND_THREADS / 32) {
        u32 v = 0;
        for (int j = tid & 31; j < ROUND_THREADS; j += 32) v = fadd(v, tot[k * ROUND_THREADS + j]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v = fadd(v, __shfl_down_sync(0xffffffffu, v, off));
        if ((tid & 31) == 0) a.partials[(size_t)blockIdx.x * WALL + ((size_t)z2 * G * G + (size_t)z1lo * G) * D + k] = v;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) is_last = atomicAdd(a.counter, 1u) == gridDim.x * gridDim.y - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    static_assert(WALL <= ROUND_THREADS && WALL <= SV3_MAX_WORDS, "one thread per accumulator word");
    __shared__ u32 row[SV3_MAX_WORDS];
    if (tid < WALL) {
        u32 v = 0;
        for (unsigned b = 0; b < gridDim.x; b++) v = fadd(v, __ldcg(a.partials + (size_t)b * WALL + tid));
        row[tid] = v;
    }
    __syncthreads();
    if (tid < G * G * G) {
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
            *reinterpret_cast<volatile u32 *>(a.out_host + SV3_FLAG) = a.seq;
        }
    }
}

template <int D, int G, int NT, int SHAPE> static cudaError_t launch_sv3_one(const SvArgs &args, int grid, cudaStream_t stream) {
    constexpr int ROWS = sv3_rows<D, G>();
    const size_t smem = (size_t)G * ROWS * D * ROUND_THREADS * 4;
    cudaFuncSetAttribute(sv3_kernel<D, G, NT, SHAPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sv3_kernel<D, G, NT, SHAPE><<<dim3(grid, G * (G / ROWS)), ROUND_THREADS, smem, stream>>>(args);
    return cudaGetLastError();
}
template <int D, int G> static cudaError_t launch_sv3_generic(int nt, const SvArgs &args, int grid, cudaStream_t stream) {
    switch (nt) {
    case 1: return launch_sv3_one<D, G, 1, SHAPE_GENERIC>(args, grid, stream);
    case 2: return launch_sv3_one<D, G, 2, SHAPE_GENERIC>(args, grid, stream);
    case 3: return launch_sv3_one<D, G, 3, SHAPE_GENERIC>(args, grid, stream);
    }
    return cudaErrorInvalidValue;
}
template <int D> static cudaError_t launch_sv3_d(int shape, int G, int nt, const SvArgs &args, int grid, cudaStream_t stream) {
    if (shape == SHAPE_PRODUCT && G == nt + 1) {
        switch (nt) {
        case 1: return launch_sv3_one<D, 2, 1, SHAPE_PRODUCT>(args, grid, stream);
        case 2: return launch_sv3_one<D, 3, 2, SHAPE_PRODUCT>(args, grid, stream);
        }
    }
    if (shape == SHAPE_LISTED + 0) return launch_sv3_one<D, Listed<0>::PTS + 1, Listed<0>::NT, SHAPE_LISTED + 0>(args, grid, stream);
    switch (G) {
    case 2: return launch_sv3_generic<D, 2>(nt, args, grid, stream);
    case 3: return launch_sv3_generic<D, 3>(nt, args, grid, stream);
    }
    return cudaErrorInvalidValue;
}
// G = points + 1 grid values per variable: degree at most two (G^3 D sums), at most three tables in the statement
bool small_values3_supported(int D, int G, int nt) { return (D == 4 || D == 8) && nt >= 1 && nt <= 3 && G >= 2 && G <= 3; }
cudaError_t launch_small_values3(int D, int shape, int G, int nt, const SvArgs &args, int grid, cudaStream_t stream) {
    if (!small_values3_supported(D, G, nt) || args.ngroups != 1) return cudaErrorInvalidValue;
    if (shape != SHAPE_PRODUCT && shape != SHAPE_LISTED + 0) shape = SHAPE_GENERIC;
    return D == 4 ? launch_sv3_d<4>(shape, G, nt, args, grid, stream) : launch_sv3_d<8>(shape, G, nt, args, grid, stream);
}

}  // namespace sc
