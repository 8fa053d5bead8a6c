// aux_kernels.cu -- the small kernels around the rounds: eq weight tables, the stand-alone fold,
// export to canonical words, the seeded table generator, the sum over ranks, and the dispatch of
// the round kernels by extension degree.
#include "round_kernel.cuh"

namespace sc {

cudaError_t launch_round_d4(int shape, int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream);
cudaError_t launch_round_d8(int shape, int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream);

cudaError_t launch_round_d4w(int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream);
cudaError_t launch_round_d8w(int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream);

cudaError_t launch_round_d4h(int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream);
cudaError_t launch_round_d8h(int points, int nt, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream);

bool round_supported(int D, int points, int nt_used) {
    if (!(D == 4 || D == 8) || points < 1 || points > SC_MAX_POINTS || nt_used < 1 || nt_used > 8) return false;
    return points <= FAST_POINTS || nt_used <= 4;   // degree above four: at most four tables in the statement
}
cudaError_t launch_round(int D, int shape, int points, int nt_used, int fold, const RoundArgs &args, int grid, size_t smem, cudaStream_t stream) {
    if (fold == 2 && (points > 3 || nt_used > 3)) return cudaErrorInvalidValue;
    if (fold == 3 && (points > 2 || nt_used > 3)) return cudaErrorInvalidValue;
    if (points > FAST_POINTS) {
        if (fold >= 2 || nt_used > 4) return cudaErrorInvalidValue;
        return D == 4 ? launch_round_d4h(points, nt_used, fold, args, grid, smem, stream) : launch_round_d8h(points, nt_used, fold, args, grid, smem, stream);
    }
    if (nt_used > 4) {   // kernels exist for six and eight tables
        const int nt = nt_used <= 6 ? 6 : 8;
        if (fold >= 2) return cudaErrorInvalidValue;
        return D == 4 ? launch_round_d4w(points, nt, fold, args, grid, smem, stream) : launch_round_d8w(points, nt, fold, args, grid, smem, stream);
    }
    if (D == 4) return launch_round_d4(shape, points, nt_used, fold, args, grid, smem, stream);
    if (D == 8) return launch_round_d8(shape, points, nt_used, fold, args, grid, smem, stream);
    return cudaErrorInvalidValue;
}

// ------------------------------------------------------------------ eq weights
//
// eq(r[s..s+b), x) = prod_k (x_k ? r_{s+k} : 1 - r_{s+k})  (EQ-TABLE, src/field.lisp:354-363, bit k of
// x pairing with the k-th element).  The tables of all rounds are built in two launches: first
// the tables of every start s and width w <= 8 by the product itself, then every larger table
// as a product of at most four of those, one per 8-bit chunk of x.

template <int D> __global__ void eq_chunks_kernel(const u32 *r_mont, int n, u32 *chunks) {
    // one thread per (start s, width w, x < 2^w): element offset s * 512 + 2^w + x
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = idx >> 9, off = idx & 511;
    if (s >= n || off < 2) return;
    const int w = 31 - __clz(off);          // 2^w <= off < 2^(w+1)
    const int x = off - (1 << w);
    if (s + w > n) return;
    Ext<D> acc = eone_mont<D>();
    Ext<D> one = eone_mont<D>();
    for (int k = 0; k < w; k++) {
        Ext<D> rk = *reinterpret_cast<const Ext<D> *>(r_mont + (size_t)(s + k) * D);
        Ext<D> f = ((x >> k) & 1) ? rk : esub<D>(one, rk);
        acc = emul<D>(acc, f);
    }
    *reinterpret_cast<Ext<D> *>(chunks + ((size_t)s * 512 + off) * D) = acc;
}

template <int D> __global__ void weight_tables_kernel(const u32 *chunks, const WeightDesc *descs, int ndescs, const u32 *bw_mont,
                                                      u32 *weights, u64 total_entries) {
    for (u64 e = (u64)blockIdx.x * blockDim.x + threadIdx.x; e < total_entries; e += (u64)gridDim.x * blockDim.x) {
        // find the table of entry e
        u64 first = 0;
        int d = 0;
        for (; d < ndescs; d++) {
            const u64 count = descs[d].entries * (u64)(descs[d].blocks > 0 ? descs[d].blocks : 1);
            if (e < first + count) break;
            first += count;
        }
        if (d >= ndescs) return;
        const WeightDesc ds = descs[d];
        const u64 local = e - first;
        const u64 x = local % ds.entries;
        const u64 b = local / ds.entries;
        Ext<D> acc = eone_mont<D>();
        bool have = false;
        for (int done = 0; done < ds.bits; done += 8) {
            const int w = ds.bits - done < 8 ? ds.bits - done : 8;
            const u32 xc = (u32)(x >> done) & ((1u << w) - 1);
            Ext<D> f = *reinterpret_cast<const Ext<D> *>(chunks + ((size_t)(ds.start + done) * 512 + (1u << w) + xc) * D);
            acc = have ? emul<D>(acc, f) : f;
            have = true;
        }
        if (ds.blocks > 0) {
            Ext<D> w = *reinterpret_cast<const Ext<D> *>(bw_mont + b * D);
            acc = emul<D>(acc, w);
        }
        if (ds.kind == 0) {
            *reinterpret_cast<Ext<D> *>(weights + ds.out_word + local * D) = acc;
        } else {
            u32 *o = weights + ds.out_word + local * 2 * D;
#pragma unroll
            for (int c = 0; c < D; c++) { o[c] = acc.v[c]; o[D + c] = ftriple(acc.v[c]); }
        }
    }
}

cudaError_t launch_eq_chunks(int D, const u32 *r_mont, int n, u32 *chunks, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    const int total = n * 512;
    if (D == 4) eq_chunks_kernel<4><<<(total + 255) / 256, 256, 0, stream>>>(r_mont, n, chunks);
    else eq_chunks_kernel<8><<<(total + 255) / 256, 256, 0, stream>>>(r_mont, n, chunks);
    return cudaGetLastError();
}
cudaError_t launch_weight_tables(int D, const u32 *chunks, const WeightDesc *descs, int ndescs, const u32 *bw_mont, u32 *weights,
                                 u64 total_entries, cudaStream_t stream) {
    if (!total_entries) return cudaSuccess;
    u64 blocks = (total_entries + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (D == 4) weight_tables_kernel<4><<<(unsigned)blocks, 256, 0, stream>>>(chunks, descs, ndescs, bw_mont, weights, total_entries);
    else weight_tables_kernel<8><<<(unsigned)blocks, 256, 0, stream>>>(chunks, descs, ndescs, bw_mont, weights, total_entries);
    return cudaGetLastError();
}

// ------------------------------------------------------------------ stand-alone fold (FOLD-FLAT-TABLE, src/sumcheck.lisp:84-104)

template <int D> __global__ void fold_kernel(const __grid_constant__ FoldArgs a) {
    Ext<D> r;
#pragma unroll
    for (int c = 0; c < D; c++) r.v[c] = a.r_dev ? a.r_dev[c] : a.r[c];
    const ExtM<D> rm = eprep<D>(r);
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < a.nout; i += (u64)gridDim.x * blockDim.x) {
        for (int t = 0; t < a.ntables; t++) {
            Ext<D> o;
            if (a.src_base[t]) {
                const uint2 w = reinterpret_cast<const uint2 *>(a.src[t])[i];
                const u32 s = fsub(w.y, w.x);
#pragma unroll
                for (int c = 0; c < D; c++) o.v[c] = mmul(rm.v[c], s);
                o.v[0] = fadd(o.v[0], w.x);
            } else {
                Ext<D> e0 = load_ext<D>(a.src[t] + (2 * i) * D), e1 = load_ext<D>(a.src[t] + (2 * i + 1) * D);
                o = eadd<D>(e0, emul<D>(esub<D>(e1, e0), rm));
            }
            store_ext<D>(a.dst[t] + i * D, o);
        }
    }
}
cudaError_t launch_fold(int D, const FoldArgs &args, cudaStream_t stream) {
    if (!args.nout || !args.ntables) return cudaSuccess;
    u64 blocks = (args.nout + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (D == 4) fold_kernel<4><<<(unsigned)blocks, 256, 0, stream>>>(args);
    else fold_kernel<8><<<(unsigned)blocks, 256, 0, stream>>>(args);
    return cudaGetLastError();
}

// ------------------------------------------------------------------ export: entries as extension elements

template <int D> __global__ void export_kernel(const __grid_constant__ ExportArgs a) {
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < a.count; i += (u64)gridDim.x * blockDim.x) {
        for (int t = 0; t < a.ntables; t++) {
            Ext<D> e;
            if (a.src_base[t]) e = lift<D>(a.src[t][i]);
            else e = load_ext<D>(a.src[t] + i * D);
            store_ext<D>(a.out + ((u64)t * a.count + i) * D, e);
        }
    }
}
cudaError_t launch_export(int D, const ExportArgs &args, cudaStream_t stream) {
    if (!args.count || !args.ntables) return cudaSuccess;
    u64 blocks = (args.count + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (D == 4) export_kernel<4><<<(unsigned)blocks, 256, 0, stream>>>(args);
    else export_kernel<8><<<(unsigned)blocks, 256, 0, stream>>>(args);
    return cudaGetLastError();
}

// ------------------------------------------------------------------ seeded inputs

__device__ __forceinline__ u64 splitmix64(u64 x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__global__ void generate_kernel(u32 *out, u64 seed, int table_id, u64 first, u64 entries, int stride, int nonzero) {
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < entries; i += (u64)gridDim.x * blockDim.x) {
        bool all0 = true;
        for (int c = 0; c < stride; c++) {
            const u32 v = (u32)(splitmix64(seed ^ ((u64)table_id << 56) ^ ((u64)c << 48) ^ (first + i)) % P);
            out[i * stride + c] = v;
            all0 = all0 && v == 0;
        }
        if (nonzero && all0) out[i * stride] = 1;
    }
}
cudaError_t launch_generate(u32 *out, u64 seed, int table_id, u64 first, u64 entries, int stride, int nonzero, cudaStream_t stream) {
    if (!entries) return cudaSuccess;
    u64 blocks = (entries + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    generate_kernel<<<(unsigned)blocks, 256, 0, stream>>>(out, seed, table_id, first, entries, stride, nonzero);
    return cudaGetLastError();
}

__global__ void reduce_words_kernel(u32 *w, u64 count) {
    for (u64 i = (u64)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (u64)gridDim.x * blockDim.x) {
        const u32 v = w[i];
        if (v >= P) w[i] = v % P;
    }
}
cudaError_t launch_reduce_words(u32 *words, u64 count, cudaStream_t stream) {
    if (!count) return cudaSuccess;
    u64 blocks = (count + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    reduce_words_kernel<<<(unsigned)blocks, 256, 0, stream>>>(words, count);
    return cudaGetLastError();
}

// ------------------------------------------------------------------ sum of the ranks' partial sums (canonical words)

__global__ void sum_ranks_kernel(const u32 *gathered, int world, int words, u32 *out_dev, u32 *out_host, int flag_word, u32 seq) {
    const int k = threadIdx.x;
    if (k < words) {
        u32 acc = 0;
        for (int r = 0; r < world; r++) acc = fadd(acc, gathered[r * words + k]);
        out_dev[k] = acc;
        if (out_host) out_host[k] = acc;
        __threadfence_system();
    }
    __syncthreads();
    if (k == 0 && out_host) {
        __threadfence_system();
        *reinterpret_cast<volatile u32 *>(out_host + flag_word) = seq;
    }
}
cudaError_t launch_sum_ranks(const u32 *gathered, int world, int words, u32 *out_dev, u32 *out_host, int flag_word, u32 seq, cudaStream_t stream) {
    if (words > 256) return cudaErrorInvalidValue;   // one thread per word: a round's sums, or the small-value accumulators (at most SV3_MAX_WORDS)
    sum_ranks_kernel<<<1, 256, 0, stream>>>(gathered, world, words, out_dev, out_host, flag_word, seq);
    return cudaGetLastError();
}

}  // namespace sc
