// round_tail.cu -- the last rounds of a proof in one launch (see TailArgs in device.h).
//
// The arithmetic of a round is that of round_kernel with FOLD: entries 4i .. 4i+3 of every table
// are folded by the last challenge into the pair (2i, 2i+1), written, and the statement is summed
// over the pairs with the round's eq weights (one weight per pair: the tables are small, the
// weights are not split); when the launch starts at a round that has no challenge to fold by (round 0, or the round
// after a gather) its first round sums the pairs as they lie.  What differs is that the block stays resident between rounds and gets
// each challenge from the host through mapped memory, so a round costs a few microseconds
// instead of a launch and a completion.  Every wait is bounded: a block that hears nothing for
// its limit of polls, or is told to stop, records why and returns.
//
// The words that cross PCIe on the way carry their own "here" mark: every element word is below p < 2^31, so bit 31
// of each word says that the word has been written (the host clears the words before the launch).  The host polls the
// sums' words and the block polls the challenge's words themselves -- one read over PCIe instead of a flag and then
// the data, and no fence between data and flag on the device.
//
// With own_transcript the block does not wait at all: it carries the transcript's hash state on
// (transcript.cuh) and derives every challenge itself (SEND of its sums, CHALLENGE), posting sums and
// challenges for the host, which replays the same steps on its transcript and checks that they agree.
#include "round_kernel.cuh"

namespace sc {

__device__ __forceinline__ u32 ld_sys(const u32 *p) {
    u32 v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ u32 timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return (u32)t;
}
__device__ __forceinline__ void st_sys(u32 *p, u32 v) { asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

template <int D, int PTS, int NT, int SHAPE>
__global__ void __launch_bounds__(ROUND_THREADS) tail_kernel(const __grid_constant__ TailArgs a) {
    __shared__ u32 red[ROUND_THREADS / 32][PTS * D];
    __shared__ u32 chal[8];
    __shared__ u32 msg[PTS * D];
    __shared__ u32 hash[B3_STATE_WORDS];
    __shared__ TrWork tw;
    __shared__ int go;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int W = PTS * D, ROWS = ROUND_THREADS / 32;

    ExtM<D> lam;
    if (SHAPE == SHAPE_GKR) {
        Ext<D> c;
#pragma unroll
        for (int k = 0; k < D; k++) c.v[k] = a.st.terms[0].coeff[k];
        lam = eprep<D>(c);
    }
    Ext<D> r;
#pragma unroll
    for (int c = 0; c < D; c++) r.v[c] = a.r_dev ? a.r_dev[c] : a.r[c];
    ExtM<D> rm = eprep<D>(r);

    if (a.own_transcript && tid < B3_STATE_WORDS - 4) hash[tid] = a.tstate ? a.tstate[tid] : a.tstate0[tid];
    for (int k = 0; k < a.nrounds; k++) {
        const u32 t_round = timer_ns();
        const TailRound rd = a.rd[k];
        const bool plain = a.nofold && k == 0;   // nothing to fold by yet: the pairs (2i, 2i+1) as they lie, nothing written
        const int kk = k - a.nofold;             // the number of this round's fold
        const int out = kk & 1;
        Ext<D> total[PTS];
#pragma unroll
        for (int x = 0; x < PTS; x++) total[x] = ezero<D>();
        for (u64 i = tid; plain && i < rd.npairs; i += ROUND_THREADS) {
            Ext<D> hw;
            if (rd.use_high) hw = *reinterpret_cast<const Ext<D> *>(a.weights + rd.high_word + i * D);
            Ext<D> val[NT], slope[NT];
#pragma unroll
            for (int t = 0; t < NT; t++) {
                Ext<D> e0 = ezero<D>(), e1 = ezero<D>();
                if (a.src_base[t]) {
                    const uint2 w = *reinterpret_cast<const uint2 *>(a.src[t] + 2 * i);
                    e0.v[0] = w.x; e1.v[0] = w.y;
                } else {
                    e0 = load_ext<D>(a.src[t] + (2 * i) * D);
                    e1 = load_ext<D>(a.src[t] + (2 * i + 1) * D);
                }
                val[t] = e0;
                slope[t] = esub<D>(e1, e0);
            }
            Ext<D> sum[PTS];
#pragma unroll
            for (int x = 0; x < PTS; x++) {
                if (x == 1) {
#pragma unroll
                    for (int t = 0; t < NT; t++) val[t] = eadd<D>(eadd<D>(val[t], slope[t]), slope[t]);
                } else if (x > 1) {
#pragma unroll
                    for (int t = 0; t < NT; t++) val[t] = eadd<D>(val[t], slope[t]);
                }
                bool unused = false;
                if (SHAPE == SHAPE_PRODUCT) sum[x] = eval_product<D, NT, false>(val, 0u, &unused);
                else if (SHAPE == SHAPE_GKR) sum[x] = eval_gkr<D, false>(reinterpret_cast<const Ext<D>(&)[4]>(val), lam, 0u);
                else if (SHAPE >= SHAPE_LISTED) {
                    typedef Listed<(SHAPE >= SHAPE_LISTED ? SHAPE - SHAPE_LISTED : 0)> S;
                    sum[x] = eval_listed<D, S, false>(a.st, reinterpret_cast<const Ext<D>(&)[S::NT]>(val), 0u, &unused);
                }
                else sum[x] = eval_statement<D, NT, false>(a.st, val, 0u, &unused);
            }
            if (rd.use_high) {
                const ExtM<D> hm = eprep<D>(hw);
#pragma unroll
                for (int x = 0; x < PTS; x++) total[x] = eadd<D>(total[x], emul<D>(sum[x], hm));
            } else {
#pragma unroll
                for (int x = 0; x < PTS; x++) total[x] = eadd<D>(total[x], sum[x]);
            }
        }
        for (u64 i = tid; !plain && i < rd.npairs; i += ROUND_THREADS) {
            // the weight and every table's entries are asked for first: a round here is a chain of latencies
            Ext<D> hw;
            if (rd.use_high) hw = *reinterpret_cast<const Ext<D> *>(a.weights + rd.high_word + i * D);
            Ext<D> e[NT][4];
#pragma unroll
            for (int t = 0; t < NT; t++) {
                const u32 *src = kk == 0 ? a.src[t] : a.buf[out ^ 1][t];
                if (kk == 0 && a.src_base[t]) {
                    const uint4 w = *reinterpret_cast<const uint4 *>(src + 4 * i);
                    e[t][0].v[0] = w.x; e[t][1].v[0] = w.y; e[t][2].v[0] = w.z; e[t][3].v[0] = w.w;
                } else {
#pragma unroll
                    for (int q = 0; q < 4; q++) e[t][q] = load_ext<D>(src + (4 * i + q) * D);
                }
            }
            Ext<D> val[NT], slope[NT];
#pragma unroll
            for (int t = 0; t < NT; t++) {
                Ext<D> lo, hi;
                if (kk == 0 && a.src_base[t]) {   // base entries: D base products (FOLD-FLAT-TABLE, src/sumcheck.lisp:95-98)
                    const u32 s0 = fsub(e[t][1].v[0], e[t][0].v[0]), s1 = fsub(e[t][3].v[0], e[t][2].v[0]);
#pragma unroll
                    for (int c = 0; c < D; c++) { lo.v[c] = mmul(rm.v[c], s0); hi.v[c] = mmul(rm.v[c], s1); }
                    lo.v[0] = fadd(lo.v[0], e[t][0].v[0]);
                    hi.v[0] = fadd(hi.v[0], e[t][2].v[0]);
                } else {
                    lo = eadd<D>(e[t][0], emul<D>(esub<D>(e[t][1], e[t][0]), rm));
                    hi = eadd<D>(e[t][2], emul<D>(esub<D>(e[t][3], e[t][2]), rm));
                }
                u32 *dst = a.buf[out][t];
                store_ext<D>(dst + (2 * i) * D, lo);
                store_ext<D>(dst + (2 * i + 1) * D, hi);
                val[t] = lo;
                slope[t] = esub<D>(hi, lo);
            }
            for (int t = NT; t < a.ntables; t++) {   // tables outside the statement are only folded
                const u32 *src = kk == 0 ? a.src[t] : a.buf[out ^ 1][t];
                Ext<D> lo, hi;
                if (kk == 0 && a.src_base[t]) {
                    const uint4 w = *reinterpret_cast<const uint4 *>(src + 4 * i);
                    const u32 s0 = fsub(w.y, w.x), s1 = fsub(w.w, w.z);
#pragma unroll
                    for (int c = 0; c < D; c++) { lo.v[c] = mmul(rm.v[c], s0); hi.v[c] = mmul(rm.v[c], s1); }
                    lo.v[0] = fadd(lo.v[0], w.x);
                    hi.v[0] = fadd(hi.v[0], w.z);
                } else {
                    const u32 *ee = src + 4 * i * D;
                    const Ext<D> e0 = load_ext<D>(ee), e1 = load_ext<D>(ee + D), e2 = load_ext<D>(ee + 2 * D), e3 = load_ext<D>(ee + 3 * D);
                    lo = eadd<D>(e0, emul<D>(esub<D>(e1, e0), rm));
                    hi = eadd<D>(e2, emul<D>(esub<D>(e3, e2), rm));
                }
                store_ext<D>(a.buf[out][t] + (2 * i) * D, lo);
                store_ext<D>(a.buf[out][t] + (2 * i + 1) * D, hi);
            }
            Ext<D> sum[PTS];
#pragma unroll
            for (int x = 0; x < PTS; x++) {
                if (x == 1) {
#pragma unroll
                    for (int t = 0; t < NT; t++) val[t] = eadd<D>(eadd<D>(val[t], slope[t]), slope[t]);
                } else if (x > 1) {
#pragma unroll
                    for (int t = 0; t < NT; t++) val[t] = eadd<D>(val[t], slope[t]);
                }
                bool unused = false;
                if (SHAPE == SHAPE_PRODUCT) sum[x] = eval_product<D, NT, false>(val, 0u, &unused);
                else if (SHAPE == SHAPE_GKR) sum[x] = eval_gkr<D, false>(reinterpret_cast<const Ext<D>(&)[4]>(val), lam, 0u);
                else if (SHAPE >= SHAPE_LISTED) {
                    typedef Listed<(SHAPE >= SHAPE_LISTED ? SHAPE - SHAPE_LISTED : 0)> S;
                    sum[x] = eval_listed<D, S, false>(a.st, reinterpret_cast<const Ext<D>(&)[S::NT]>(val), 0u, &unused);
                }
                else sum[x] = eval_statement<D, NT, false>(a.st, val, 0u, &unused);
            }
            if (rd.use_high) {
                const ExtM<D> hm = eprep<D>(hw);
#pragma unroll
                for (int x = 0; x < PTS; x++) total[x] = eadd<D>(total[x], emul<D>(sum[x], hm));
            } else {
#pragma unroll
                for (int x = 0; x < PTS; x++) total[x] = eadd<D>(total[x], sum[x]);
            }
        }
        // the block's sums
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
        u32 *slot = a.host + (size_t)k * TAIL_SLOT_WORDS;
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
            for (int c = 0; c < D; c++) {
                if (a.own_transcript) { slot[tid * D + c] = s.v[c]; msg[tid * D + c] = s.v[c]; }
                else st_sys(slot + tid * D + c, s.v[c] | TAIL_HERE);   // each word says for itself that it is there
            }
        }
        __syncthreads();   // also: every store of the folded tables is done before the next round reads them
        if (a.own_transcript) {
            // the transcript's next steps, here: SEND of the sums, then the challenge; the host replays both and compares
            const u32 s0 = timer_ns();
            transcript_round(&tw, hash, msg, W, D, hash);
            __syncthreads();
            if (tid < D) { chal[tid] = tw.chal[tid]; slot[52 + tid] = tw.chal[tid]; }
            if (tid == 0) { slot[60] = s0 - t_round; slot[61] = timer_ns() - s0; go = 1; }   // nanoseconds: the round's arithmetic, its transcript steps
            __syncthreads();
            if (tid == 0) {
                __threadfence_system();   // cumulative: the sums and the challenge written before the barrier are visible before the words below
                st_sys(slot + 32, a.seq + (u32)k);
                st_sys(slot + 50, a.seq + (u32)k);
            }
        } else if (tid == 0) {
            // wait for the challenge, a bounded number of polls: its words in one 128-bit read per four (each read is a
            // trip over PCIe), every one of them marked by the host
            int ok = 0;
            for (unsigned poll = 0; poll < a.poll_limit; poll++) {
                u32 here = TAIL_HERE;
#pragma unroll
                for (int c = 0; c < D; c += 4) {
                    uint4 v;
                    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(slot + 40 + c) : "memory");
                    chal[c] = v.x & ~TAIL_HERE; chal[c + 1] = v.y & ~TAIL_HERE; chal[c + 2] = v.z & ~TAIL_HERE; chal[c + 3] = v.w & ~TAIL_HERE;
                    here &= v.x & v.y & v.z & v.w;
                }
                if (here) { ok = 1; break; }
                if ((poll & 63) == 63 && ld_sys(a.host + TAIL_STOP) == a.seq) { ok = -1; break; }
            }
            if (ok != 1) st_sys(a.host + TAIL_STATUS, ok == 0 ? 2u : 3u);
            go = ok == 1;
        }
        __syncthreads();
        if (!go) return;
#pragma unroll
        for (int c = 0; c < D; c++) r.v[c] = to_mont(chal[c]);
        rm = eprep<D>(r);
        __syncthreads();
    }
    // the last fold: one entry per table and block, posted to the host and left in the buffer the next round would read
    {
        const int folds = a.nrounds - a.nofold;   // folds done so far: the tables are in the caller's arrays still when there was none
        const int last = (folds - 1) & 1;
        if (tid < a.ntables * a.blocks) {
            const int t = tid / a.blocks, b = tid % a.blocks;
            Ext<D> e0 = ezero<D>(), e1 = ezero<D>();
            if (folds == 0 && a.src_base[t]) { e0.v[0] = a.src[t][2 * b]; e1.v[0] = a.src[t][2 * b + 1]; }
            else {
                const u32 *e = (folds == 0 ? a.src[t] : a.buf[last][t]) + (size_t)2 * b * D;
                e0 = load_ext<D>(e); e1 = load_ext<D>(e + D);
            }
            const Ext<D> f = eadd<D>(e0, emul<D>(esub<D>(e1, e0), rm));
            store_ext<D>(a.buf[folds == 0 ? 0 : last ^ 1][t] + (size_t)b * D, f);
#pragma unroll
            for (int c = 0; c < D; c++) st_sys(a.host + TAIL_FINALS + tid * D + c, f.v[c] | TAIL_HERE);
        }
        if (tid == 0) st_sys(a.host + TAIL_STATUS, 1u);
    }
}

template <int D, int PTS, int NT, int SHAPE> static cudaError_t launch_tail_one(const TailArgs &args, cudaStream_t stream) {
    tail_kernel<D, PTS, NT, SHAPE><<<1, ROUND_THREADS, 0, stream>>>(args);
    return cudaGetLastError();
}
template <int D, int PTS> static cudaError_t launch_tail_dp(int nt, const TailArgs &args, cudaStream_t stream) {
    switch (nt) {
    case 1: return launch_tail_one<D, PTS, 1, SHAPE_GENERIC>(args, stream);
    case 2: return launch_tail_one<D, PTS, 2, SHAPE_GENERIC>(args, stream);
    case 3: return launch_tail_one<D, PTS, 3, SHAPE_GENERIC>(args, stream);
    case 4: return launch_tail_one<D, PTS, 4, SHAPE_GENERIC>(args, stream);
    default: return cudaErrorInvalidValue;
    }
}
template <int D> static cudaError_t launch_tail_d(int shape, int points, int nt, const TailArgs &args, cudaStream_t stream) {
    if (shape == SHAPE_GKR && points == 2 && nt == 4) return launch_tail_one<D, 2, 4, SHAPE_GKR>(args, stream);
    if (shape == SHAPE_LISTED + 0) return launch_tail_one<D, Listed<0>::PTS, Listed<0>::NT, SHAPE_LISTED + 0>(args, stream);
    if (shape == SHAPE_LISTED + 1) return launch_tail_one<D, Listed<1>::PTS, Listed<1>::NT, SHAPE_LISTED + 1>(args, stream);
    if (shape == SHAPE_LISTED + 2) return launch_tail_one<D, Listed<2>::PTS, Listed<2>::NT, SHAPE_LISTED + 2>(args, stream);
    if (shape == SHAPE_PRODUCT && points == nt) {
        switch (nt) {
        case 1: return launch_tail_one<D, 1, 1, SHAPE_PRODUCT>(args, stream);
        case 2: return launch_tail_one<D, 2, 2, SHAPE_PRODUCT>(args, stream);
        case 3: return launch_tail_one<D, 3, 3, SHAPE_PRODUCT>(args, stream);
        case 4: return launch_tail_one<D, 4, 4, SHAPE_PRODUCT>(args, stream);
        }
    }
    switch (points) {
    case 1: return launch_tail_dp<D, 1>(nt, args, stream);
    case 2: return launch_tail_dp<D, 2>(nt, args, stream);
    case 3: return launch_tail_dp<D, 3>(nt, args, stream);
    case 4: return launch_tail_dp<D, 4>(nt, args, stream);
    default: return cudaErrorInvalidValue;
    }
}
// The transcript's part of a round kernel's round (see TranscriptArgs): one block behind the round kernel.
__global__ void __launch_bounds__(ROUND_THREADS) transcript_kernel(const __grid_constant__ TranscriptArgs a) {
    __shared__ u32 sums[MAX_PARTIAL_WORDS];
    __shared__ u32 state[B3_STATE_WORDS];
    __shared__ TrWork tw;
    const int tid = threadIdx.x;
    if (tid < a.W) sums[tid] = a.sums[tid];
    if (tid < B3_STATE_WORDS - 4) state[tid] = a.tinit ? a.tstate0[tid] : a.tstate[tid];
    u32 posted = a.sums[MAX_PARTIAL_WORDS];
    if (!a.tinit && a.tstate[CHAIN_DEAD] != 0) posted |= EXCHANGE_FAILED;   // a round before this one failed
    __syncthreads();
    if (posted & EXCHANGE_FAILED) {
        if (tid == 0) a.tstate[CHAIN_DEAD] = 1;
    } else {
        transcript_round(&tw, state, sums, a.W, a.D, state);
        __syncthreads();
        if (tid < B3_STATE_WORDS - 4) a.tstate[tid] = state[tid];
        if (tid < a.D) {
            const u32 c = tw.chal[tid];
            a.chal_dev[tid] = to_mont(c);
            a.chal_dev[a.D + tid] = c;
            a.out_host[CHAIN_CHAL_WORD + tid] = c;
        }
        if (tid == 0 && a.tinit) a.tstate[CHAIN_DEAD] = 0;
    }
    if (tid < a.W) a.out_host[tid] = sums[tid];
    __syncthreads();
    if (tid == 0) {   // the host polls this word: the words above are visible before it (the fence is cumulative)
        __threadfence_system();
        *reinterpret_cast<volatile u32 *>(a.out_host + MAX_PARTIAL_WORDS) = (posted & EXCHANGE_FAILED) | a.seq;
    }
}
cudaError_t launch_transcript_round(const TranscriptArgs &args, cudaStream_t stream) {
    transcript_kernel<<<1, ROUND_THREADS, 0, stream>>>(args);
    return cudaGetLastError();
}

cudaError_t launch_tail(int D, int shape, int points, int nt_used, const TailArgs &args, cudaStream_t stream) {
    if (D == 4) return launch_tail_d<4>(shape, points, nt_used, args, stream);
    if (D == 8) return launch_tail_d<8>(shape, points, nt_used, args, stream);
    return cudaErrorInvalidValue;
}

}  // namespace sc
