// gkr.cu -- the upper layers of the batched LogUp-GKR fraction trees (PROVE-UPPER,
// src/gkr.lisp:215-272) on top of the sumcheck contexts: the biggest caller of PROVE.
//
// A domain has K blocks of 2^n leaf fractions p/q per lookup.  The trees are built on the device
// (FRACTION-TREES, :149-188): p/q = p0/q0 + p1/q1 entry by entry.  The children of (b, x) in the
// layer of 2^m entries per block are (b, x) and (b, x + 2^m) of the layer below, that is, the
// lower and upper halves of each block -- which are also the four tables p0, p1, q0, q1 of the
// layer's sumcheck (LAYER-TABLES, :199-206).  So every layer is kept as two arrays, the lower
// halves and the upper halves of its blocks, each block-major: the tree kernel reads and writes
// them entry by entry, and the sumcheck contexts borrow them as their tables without a copy.
//
// The layer statement sum_l a_l (p0_l q1_l + p1_l q0_l) + a_l lambda q0_l q1_l (:30-41) is a sum
// over the lookups of statements on separate tables, and a round's sums are linear in the
// statement: lookup l runs in its own context with the built-in kernel of that four-table
// statement, and the host adds the L rows of sums before it sends them.  The tiny sumchecks over
// the block index (top tree, "-blk") run the same way with tables uploaded from the host.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/sumcheck_b200.h"
#include "device.h"
#include "field.cuh"
#include "part_workers.h"

namespace sc {
using namespace scf;

// One layer from the one below: COUNT = K 2^m output entries.  Output entry o = b 2^m + x goes to
// the lower or upper half of block b of the output layer (m >= 1), or to a plain array (m = 0).
template <int D>
__global__ void __launch_bounds__(256) fraction_layer_kernel(const u32 *__restrict__ p0, const u32 *__restrict__ p1,
                                                             const u32 *__restrict__ q0, const u32 *__restrict__ q1, u64 count,
                                                             int m, u32 *__restrict__ plo, u32 *__restrict__ phi,
                                                             u32 *__restrict__ qlo, u32 *__restrict__ qhi) {
    typedef uint4 V;
    constexpr int NV = D / 4;
    for (u64 o = (u64)blockIdx.x * blockDim.x + threadIdx.x; o < count; o += (u64)gridDim.x * blockDim.x) {
        Ext<D> a0, a1, b0, b1;
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const V w0 = __ldcs(reinterpret_cast<const V *>(p0) + o * NV + k), w1 = __ldcs(reinterpret_cast<const V *>(p1) + o * NV + k);
            const V w2 = __ldcs(reinterpret_cast<const V *>(q0) + o * NV + k), w3 = __ldcs(reinterpret_cast<const V *>(q1) + o * NV + k);
            a0.v[4 * k] = w0.x; a0.v[4 * k + 1] = w0.y; a0.v[4 * k + 2] = w0.z; a0.v[4 * k + 3] = w0.w;
            a1.v[4 * k] = w1.x; a1.v[4 * k + 1] = w1.y; a1.v[4 * k + 2] = w1.z; a1.v[4 * k + 3] = w1.w;
            b0.v[4 * k] = w2.x; b0.v[4 * k + 1] = w2.y; b0.v[4 * k + 2] = w2.z; b0.v[4 * k + 3] = w2.w;
            b1.v[4 * k] = w3.x; b1.v[4 * k + 1] = w3.y; b1.v[4 * k + 2] = w3.z; b1.v[4 * k + 3] = w3.w;
        }
        // the denominators in Montgomery form: a product with one of them is canonical again
        const ExtM<D> m0 = eprep<D>(eto_mont<D>(b0)), m1 = eprep<D>(eto_mont<D>(b1));
        const Ext<D> p = eadd<D>(emul<D>(a0, m1), emul<D>(a1, m0));
        const Ext<D> q = emul<D>(b0, m1);
        u32 *pd, *qd;
        u64 at;
        if (m == 0) { pd = plo; qd = qlo; at = o; }
        else {
            const u64 half = 1ull << (m - 1), b = o >> m, x = o & ((1ull << m) - 1);
            const bool up = x >= half;
            pd = up ? phi : plo; qd = up ? qhi : qlo;
            at = b * half + (x & (half - 1));
        }
#pragma unroll
        for (int k = 0; k < NV; k++) {
            reinterpret_cast<V *>(pd)[at * NV + k] = make_uint4(p.v[4 * k], p.v[4 * k + 1], p.v[4 * k + 2], p.v[4 * k + 3]);
            reinterpret_cast<V *>(qd)[at * NV + k] = make_uint4(q.v[4 * k], q.v[4 * k + 1], q.v[4 * k + 2], q.v[4 * k + 3]);
        }
    }
}

static cudaError_t launch_fraction_layer(int D, const u32 *p0, const u32 *p1, const u32 *q0, const u32 *q1, u64 count, int m,
                                         u32 *plo, u32 *phi, u32 *qlo, u32 *qhi, int sms, cudaStream_t stream) {
    u64 blocks = (count + 255) / 256;
    const u64 cap = (u64)sms * 8;
    const int grid = (int)(blocks < cap ? blocks : cap);
    if (D == 4) fraction_layer_kernel<4><<<grid, 256, 0, stream>>>(p0, p1, q0, q1, count, m, plo, phi, qlo, qhi);
    else fraction_layer_kernel<8><<<grid, 256, 0, stream>>>(p0, p1, q0, q1, count, m, plo, phi, qlo, qhi);
    return cudaGetLastError();
}

// ---- host arithmetic on canonical elements (a handful of products per layer)
struct HostField {
    int D;
    typedef std::vector<u32> E;
    E zero() const { return E((size_t)D, 0u); }
    E one() const { E o = zero(); o[0] = 1; return o; }
    E add(const E &a, const E &b) const { E o(D); for (int c = 0; c < D; c++) o[c] = fadd(a[c], b[c]); return o; }
    E sub(const E &a, const E &b) const { E o(D); for (int c = 0; c < D; c++) o[c] = fsub(a[c], b[c]); return o; }
    template <int DD> static void mul_d(const u32 *a, const u32 *b, u32 *o) {
        Ext<DD> x, y;
        for (int c = 0; c < DD; c++) { x.v[c] = a[c]; y.v[c] = b[c]; }
        const Ext<DD> z = emul<DD>(x, eprep<DD>(eto_mont<DD>(y)));
        for (int c = 0; c < DD; c++) o[c] = z.v[c];
    }
    E mul(const E &a, const E &b) const { E o(D); if (D == 4) mul_d<4>(a.data(), b.data(), o.data()); else mul_d<8>(a.data(), b.data(), o.data()); return o; }
    E fold(const E &lo, const E &hi, const E &r) const { return add(lo, mul(r, sub(hi, lo))); }   // FOLD-PAIR, :65-66
    // EQ-TABLE (src/field.lisp:354-363): bit 0 of the index pairs with r_0
    std::vector<E> eq_table(const std::vector<E> &r) const {
        std::vector<E> t{one()};
        for (const E &rb : r) {
            const size_t n = t.size();
            t.resize(2 * n);
            for (size_t i = 0; i < n; i++) { const E up = mul(t[i], rb); t[n + i] = up; t[i] = sub(t[i], up); }
        }
        return t;
    }
};

struct DeviceArrays {   // the trees' arrays, carved out of one block of the first context's workspace
    char *base = nullptr;
    u64 used = 0, cap = 0;
    static u64 round_up(u64 words) { return ((words ? words : 4) * 4 + 255) & ~(u64)255; }
    cudaError_t get(u32 **p, u64 words) {
        const u64 bytes = round_up(words);
        if (used + bytes > cap) return cudaErrorMemoryAllocation;
        *p = (u32 *)(base + used);
        used += bytes;
        return cudaSuccess;
    }
};

struct Halves { u32 *lo = nullptr, *hi = nullptr; };   // a layer: the lower and the upper halves of its blocks

struct Part {   // one lookup's share of a sumcheck
    std::string statement;
    std::vector<std::string> names, cnames;
    std::vector<const u32 *> host, dev;   // per table: one of them is set
    std::vector<u32> cvals;
    bool layer = false;                   // the statement is the layer statement (constants a, al): no need to parse it
};

// PROVE (src/sumcheck.lisp:512-571) of the sum of the parts' statements, part l on context l: one header,
// per round the sum of the parts' sums.  FINALS and FOLDED are per part, per table (blocks entries).
static int prove_parts(sc_ctx *const *ctxs, std::vector<Part> &parts, sc_transcript *tr, int n, const u32 *eq, const char *label,
                       int blocks, const u32 *bw, int degree, std::vector<HostField::E> *challenges,
                       std::vector<std::vector<u32>> *folded, PartWorkers *workers) {
    const int D = sc_transcript_degree(tr), L = (int)parts.size();
    const auto t_enter = std::chrono::steady_clock::now();
    int points = 1, rc;
    for (int l = 0; l < L; l++) {
        Part &pt = parts[l];
        const int nt = (int)pt.names.size(), nc = (int)pt.cnames.size();
        std::vector<const char *> tn, cn;
        for (auto &s : pt.names) tn.push_back(s.c_str());
        for (auto &s : pt.cnames) cn.push_back(s.c_str());
        int deg = 0, nterms = 0;
        std::vector<u32> coeffs((size_t)SC_MAX_TERMS * D);
        std::vector<int32_t> ptr(SC_MAX_TERMS + 1), idx((size_t)SC_MAX_TERMS * SC_MAX_FACTORS);
        if (pt.layer) {
            // the layer statement's term table written down directly (what sc_lower_statement gives for it: the terms in
            // the order of their table lists), a p0 q1 + a p1 q0 + al q0 q1, each times bw when that is table 0
            const int o = pt.names[0] == "bw" ? 1 : 0;
            const int lists[3][2] = {{o + 0, o + 3}, {o + 1, o + 2}, {o + 2, o + 3}};
            int used = 0;
            for (int t = 0; t < 3; t++) {
                memcpy(coeffs.data() + (size_t)t * D, pt.cvals.data() + (size_t)(t == 2 ? D : 0), 4 * (size_t)D);
                ptr[t] = used;
                if (o) idx[used++] = 0;
                idx[used++] = lists[t][0]; idx[used++] = lists[t][1];
            }
            ptr[3] = used; nterms = 3; deg = 2 + o;
        } else if ((rc = sc_lower_statement(pt.statement.c_str(), D, nt, tn.data(), nc, cn.data(), pt.cvals.data(), &deg, &nterms, coeffs.data(),
                                            ptr.data(), idx.data())))
            return rc;
        if (l == 0) { if (degree < 0) degree = deg; points = degree > 1 ? degree : 1; }
        if ((rc = sc_set_statement(ctxs[l], D, points, nt, nterms, coeffs.data(), ptr.data(), idx.data()))) return rc;
        for (int t = 0; t < nt; t++) {
            rc = pt.dev[t] ? sc_borrow_table(ctxs[l], t, pt.dev[t], (u64)blocks << n, D) : sc_upload_table(ctxs[l], t, pt.host[t], (u64)blocks << n, D);
            if (rc) return rc;
        }
        if ((rc = sc_begin(ctxs[l], n, eq, blocks, blocks > 1 ? bw : nullptr))) return rc;   // one block: its weight is 1
    }
    static const bool trace = getenv("SABLE_B200_TRACE") != nullptr;
    const auto t_begun = std::chrono::steady_clock::now();
    std::vector<uint8_t> header(label, label + strlen(label));   // label | "|" | n u16 | degree u16 | blocks u32 (:24-27)
    header.push_back('|');
    header.push_back((uint8_t)n); header.push_back((uint8_t)(n >> 8));
    header.push_back((uint8_t)degree); header.push_back((uint8_t)(degree >> 8));
    for (int b = 0; b < 4; b++) header.push_back((uint8_t)((u32)blocks >> (8 * b)));
    if ((rc = sc_transcript_absorb(tr, header.data(), header.size()))) return rc;
    // one part: its sums are the message, so the device may carry the transcript through the last rounds itself
    struct Attach { sc_ctx *c; ~Attach() { if (c) sc_attach_transcript(c, nullptr); } } attach{L == 1 ? ctxs[0] : nullptr};
    if (L == 1 && (rc = sc_attach_transcript(ctxs[0], tr))) return rc;
    u32 sums[SC_MAX_POINTS * 8], part[SC_MAX_POINTS * 8];
    for (int j = 0; j < n; j++) {
        if (workers) {   // every lookup's round at the same time
            if ((rc = workers->round(sums))) return rc;
            for (int l = 1; l < L; l++) for (int k = 0; k < points * D; k++) sums[k] = fadd(sums[k], workers->part(l)[k]);
        } else {
            for (int l = 0; l < L; l++) {
                if ((rc = sc_round(ctxs[l], l ? part : sums))) return rc;
                if (l) for (int k = 0; k < points * D; k++) sums[k] = fadd(sums[k], part[k]);
            }
        }
        if ((rc = sc_transcript_send(tr, sums, points, D))) return rc;
        HostField::E r((size_t)D);
        if ((rc = sc_transcript_challenge_base(tr, D, r.data()))) return rc;
        for (int l = 0; l < L; l++) if ((rc = sc_challenge(ctxs[l], r.data()))) return rc;
        challenges->push_back(r);
    }
    folded->clear();
    const auto t_rounds = std::chrono::steady_clock::now();
    for (int l = 0; l < L; l++) {
        std::vector<u32> out(parts[l].names.size() * (size_t)blocks * D);
        if ((rc = sc_finish(ctxs[l], out.data()))) return rc;
        folded->push_back(out);
    }
    if (trace) fprintf(stderr, "  proof of %d rounds: statement, tables and sc_begin %.1f us, rounds %.1f us, finish %.1f us\n", n,
                       std::chrono::duration<double, std::micro>(t_begun - t_enter).count(), std::chrono::duration<double, std::micro>(t_rounds - t_begun).count(),
                       std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t_rounds).count());
    return SC_OK;
}

}  // namespace sc

using namespace sc;

#define GK(call)                                                                      \
    do {                                                                              \
        cudaError_t e_ = (call);                                                      \
        if (e_ != cudaSuccess) { cudaGetLastError(); return e_ == cudaErrorMemoryAllocation ? SC_ENOMEM : SC_ECUDA; } \
    } while (0)

extern "C" int sc_gkr_prove_upper(sc_ctx *const *ctxs, int lookups, sc_transcript *tr, int n, int K, const uint32_t *const *leaves_p,
                                  const uint32_t *const *leaves_q, int leaves_on_device, const char *label, uint32_t *ri_out,
                                  uint32_t *rb_out, uint32_t *cp_out, uint32_t *cq_out) {
    if (!ctxs || !tr || !leaves_p || !leaves_q || lookups < 1 || n < 1 || n > 34 || K < 1) return SC_EINVAL;
    for (int l = 0; l < lookups; l++) {
        if (!ctxs[l] || !leaves_p[l] || !leaves_q[l]) return SC_EINVAL;
        int world = 1;
        sc_comm_info(ctxs[l], nullptr, &world);
        if (world > 1) return SC_EUNSUPPORTED;   // the trees live on one GPU
    }
    if (!label) label = "gkr";
    const int D = sc_transcript_degree(tr), L = lookups;
    if (D != 4 && D != 8) return SC_EINVAL;
    const HostField F{D};
    typedef HostField::E E;
    int lk = 0;
    while ((1 << lk) < K) lk++;                 // BLOCK-BITS, :23-25
    int rc, sms = 148, device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    cudaStream_t stream;
    GK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    struct StreamGuard { cudaStream_t s; ~StreamGuard() { cudaStreamDestroy(s); } } guard{stream};

    // ---- the trees (FRACTION-TREES): layer m >= 1 as halves, layer 0 (the blocks' roots) as one array
    DeviceArrays mem;
    {
        u64 bytes = 0;
        for (int m = n; m >= 1; m--) bytes += 4 * DeviceArrays::round_up(((u64)K << (m - 1)) * D);
        bytes += 2 * DeviceArrays::round_up((u64)K * D);
        bytes *= (u64)L;
        void *base = nullptr;
        if ((rc = sc_workspace(ctxs[0], bytes, &base))) return rc;
        mem.base = (char *)base; mem.cap = bytes;
        // the layers' proofs grow from one entry to K 2^(n-2): make the contexts' room for the largest once
        if (n >= 2) for (int l = 0; l < L; l++) if ((rc = sc_reserve(ctxs[l], D, n - 2, K, 4))) return rc;
    }
    // on every way out the contexts get tables of their own again: the trees' arrays are scratch of the first context
    struct Unborrow {
        sc_ctx *const *ctxs; int L, D;
        ~Unborrow() {
            const u32 one[8] = {1, 0, 0, 0, 0, 0, 0, 0};
            for (int l = 0; l < L; l++) for (int t = 0; t < 4; t++) sc_upload_table(ctxs[l], t, one, 1, D);
        }
    } unborrow{ctxs, L, D};
    std::vector<std::vector<Halves>> LP(L, std::vector<Halves>(n + 1)), LQ(L, std::vector<Halves>(n + 1));
    for (int l = 0; l < L; l++) {
        const u64 half = (u64)K << (n - 1);     // entries of one array of halves of the leaf layer
        GK(mem.get(&LP[l][n].lo, half * D)); GK(mem.get(&LP[l][n].hi, half * D));
        GK(mem.get(&LQ[l][n].lo, half * D)); GK(mem.get(&LQ[l][n].hi, half * D));
        const cudaMemcpyKind kind = leaves_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
        const size_t width = ((size_t)1 << (n - 1)) * D * 4;   // one half of one block
        for (int which = 0; which < 2; which++) {
            const u32 *src = which ? leaves_q[l] : leaves_p[l];
            Halves &h = which ? LQ[l][n] : LP[l][n];
            if (K > 16 && width <= ((size_t)1 << 28)) {   // many small blocks: one strided copy per half
                GK(cudaMemcpy2DAsync(h.lo, width, src, 2 * width, width, (size_t)K, kind, stream));
                GK(cudaMemcpy2DAsync(h.hi, width, (const char *)src + width, 2 * width, width, (size_t)K, kind, stream));
            } else {
                for (int b = 0; b < K; b++) {
                    GK(cudaMemcpyAsync((char *)h.lo + (size_t)b * width, (const char *)src + (size_t)2 * b * width, width, kind, stream));
                    GK(cudaMemcpyAsync((char *)h.hi + (size_t)b * width, (const char *)src + (size_t)(2 * b + 1) * width, width, kind, stream));
                }
            }
            GK(launch_reduce_words(h.lo, half * D, stream));   // COERCE-EXT reduces its input (src/field.lisp:115-117)
            GK(launch_reduce_words(h.hi, half * D, stream));
        }
        for (int m = n - 1; m >= 0; m--) {
            const u64 count = (u64)K << m, out_half = m ? (u64)K << (m - 1) : (u64)K;
            GK(mem.get(&LP[l][m].lo, out_half * D)); GK(mem.get(&LQ[l][m].lo, out_half * D));
            if (m) { GK(mem.get(&LP[l][m].hi, out_half * D)); GK(mem.get(&LQ[l][m].hi, out_half * D)); }
            GK(launch_fraction_layer(D, LP[l][m + 1].lo, LP[l][m + 1].hi, LQ[l][m + 1].lo, LQ[l][m + 1].hi, count, m, LP[l][m].lo, LP[l][m].hi,
                                     LQ[l][m].lo, LQ[l][m].hi, sms, stream));
        }
    }
    // the top tree over the block index, on the host: the blocks' roots padded with 0/1 (:176-188)
    const int KP = 1 << lk;
    std::vector<std::vector<std::vector<E>>> TP(L, std::vector<std::vector<E>>(lk + 1)), TQ(L, std::vector<std::vector<E>>(lk + 1));
    {
        std::vector<u32> hp((size_t)K * D), hq((size_t)K * D);
        for (int l = 0; l < L; l++) {
            GK(cudaMemcpyAsync(hp.data(), LP[l][0].lo, hp.size() * 4, cudaMemcpyDeviceToHost, stream));
            GK(cudaMemcpyAsync(hq.data(), LQ[l][0].lo, hq.size() * 4, cudaMemcpyDeviceToHost, stream));
            GK(cudaStreamSynchronize(stream));
            TP[l][lk].assign(KP, F.zero()); TQ[l][lk].assign(KP, F.one());
            for (int b = 0; b < K; b++) {
                TP[l][lk][b].assign(hp.begin() + (size_t)b * D, hp.begin() + (size_t)(b + 1) * D);
                TQ[l][lk][b].assign(hq.begin() + (size_t)b * D, hq.begin() + (size_t)(b + 1) * D);
            }
            for (int j = lk - 1; j >= 0; j--) {
                const int h = 1 << j;
                TP[l][j].resize(h); TQ[l][j].resize(h);
                for (int b = 0; b < h; b++) {
                    const E &p0 = TP[l][j + 1][b], &p1 = TP[l][j + 1][b + h], &q0 = TQ[l][j + 1][b], &q1 = TQ[l][j + 1][b + h];
                    TP[l][j][b] = F.add(F.mul(p0, q1), F.mul(p1, q0));
                    TQ[l][j][b] = F.mul(q0, q1);
                }
            }
        }
    }

    // ---- the proof: the roots, then every layer from the one above (:224-272)
    std::vector<E> cp(L), cq(L);
    for (int l = 0; l < L; l++) {
        u32 root[16];
        memcpy(root, TP[l][0][0].data(), 4 * (size_t)D); memcpy(root + D, TQ[l][0][0].data(), 4 * (size_t)D);
        if ((rc = sc_transcript_send(tr, root, 2, D))) return rc;
        cp[l] = TP[l][0][0]; cq[l] = TQ[l][0][0];
    }
    const char *tnames[4] = {"p0", "p1", "q0", "q1"};
    const std::string layer_statement = "(+ (* a p0 q1) (* a p1 q0) (* al q0 q1))";   // LAYER-STATEMENT (:30-41), one lookup's terms
    auto layer_parts = [&](std::vector<Part> &parts, bool with_bw) -> int {             // LAYER-CHALLENGES (:43-51)
        std::vector<u32> as((size_t)L * D);
        E lam((size_t)D);
        int r;
        if ((r = sc_transcript_challenge_base(tr, L * D, as.data()))) return r;
        if ((r = sc_transcript_challenge_base(tr, D, lam.data()))) return r;
        parts.assign(L, Part());
        for (int l = 0; l < L; l++) {
            Part &pt = parts[l];
            pt.statement = with_bw ? "(* bw " + layer_statement + ")" : layer_statement;
            if (with_bw) pt.names.push_back("bw");
            for (const char *nm : tnames) pt.names.push_back(nm);
            pt.cnames = {"a", "al"};
            pt.layer = true;
            const E a(as.begin() + (size_t)l * D, as.begin() + (size_t)(l + 1) * D), al = F.mul(a, lam);
            pt.cvals.insert(pt.cvals.end(), a.begin(), a.end());
            pt.cvals.insert(pt.cvals.end(), al.begin(), al.end());
            pt.host.assign(pt.names.size(), nullptr); pt.dev.assign(pt.names.size(), nullptr);
        }
        return SC_OK;
    };
    // SEND-FINALS (:208-213) and NEXT-CLAIMS (:57-63); FINALS per lookup: p0, p1, q0, q1, D words each
    auto finish_layer = [&](const std::vector<std::vector<E>> &finals, E *tt) -> int {
        int r;
        for (int l = 0; l < L; l++)
            for (int t = 0; t < 4; t++)
                if ((r = sc_transcript_send(tr, finals[l][t].data(), 1, D))) return r;
        tt->assign((size_t)D, 0u);
        if ((r = sc_transcript_challenge_base(tr, D, tt->data()))) return r;
        for (int l = 0; l < L; l++) { cp[l] = F.fold(finals[l][0], finals[l][1], *tt); cq[l] = F.fold(finals[l][2], finals[l][3], *tt); }
        return SC_OK;
    };
    auto flat = [&](const std::vector<E> &v) { std::vector<u32> o; for (const E &e : v) o.insert(o.end(), e.begin(), e.end()); return o; };

    std::vector<E> r;
    std::vector<Part> parts;
    std::vector<std::vector<u32>> folded;
    std::unique_ptr<PartWorkers> workers;    // several lookups: their rounds run side by side
    if (L > 1) workers.reset(new PartWorkers(std::vector<sc_ctx *>(ctxs, ctxs + L)));
    for (int j = 0; j < lk; j++) {              // the top tree
        if ((rc = layer_parts(parts, false))) return rc;
        const int h = 1 << j;
        std::vector<std::vector<u32>> keep;      // the tables' words, alive until the proof has read them
        for (int l = 0; l < L; l++) {
            const std::vector<E> &tp = TP[l][j + 1], &tq = TQ[l][j + 1];
            keep.push_back(flat(std::vector<E>(tp.begin(), tp.begin() + h))); keep.push_back(flat(std::vector<E>(tp.begin() + h, tp.end())));
            keep.push_back(flat(std::vector<E>(tq.begin(), tq.begin() + h))); keep.push_back(flat(std::vector<E>(tq.begin() + h, tq.end())));
        }
        for (int l = 0; l < L; l++) for (int t = 0; t < 4; t++) parts[l].host[t] = keep[(size_t)4 * l + t].data();
        const std::vector<u32> eq = flat(r);
        const std::string lab = std::string(label) + "-top";
        std::vector<E> rho;
        if ((rc = prove_parts(ctxs, parts, tr, j, j > 0 ? eq.data() : nullptr, lab.c_str(), 1, nullptr, j > 0 ? 2 : 0, &rho, &folded, workers.get()))) return rc;
        std::vector<std::vector<E>> finals(L, std::vector<E>(4));
        for (int l = 0; l < L; l++) for (int t = 0; t < 4; t++) finals[l][t].assign(folded[l].begin() + (size_t)t * D, folded[l].begin() + (size_t)(t + 1) * D);
        E tt;
        if ((rc = finish_layer(finals, &tt))) return rc;
        r = rho; r.push_back(tt);
    }
    std::vector<E> rb = r, ri;
    if (KP != K) {                               // the padded blocks' roots have denominators 1 (PADDED-MASS, :68-71)
        const std::vector<E> e = F.eq_table(rb);
        E mass = F.zero();
        for (int b = K; b < KP; b++) mass = F.add(mass, e[b]);
        for (int l = 0; l < L; l++) cq[l] = F.sub(cq[l], mass);
    }
    const bool trace = getenv("SABLE_B200_TRACE") != nullptr;   // per-layer host times on stderr
    for (int layer = 0; layer + 1 < n; layer++) {   // the in-block layers
        const auto t_layer = std::chrono::steady_clock::now();
        if ((rc = layer_parts(parts, false))) return rc;
        std::vector<E> bw;                       // BLOCK-WEIGHTS (:73-77)
        if (rb.empty()) bw.push_back(F.one());
        else { const std::vector<E> e = F.eq_table(rb); bw.assign(e.begin(), e.begin() + K); }
        for (int l = 0; l < L; l++) {
            const Halves &p = LP[l][layer + 1], &q = LQ[l][layer + 1];
            parts[l].dev[0] = p.lo; parts[l].dev[1] = p.hi; parts[l].dev[2] = q.lo; parts[l].dev[3] = q.hi;
        }
        GK(cudaStreamSynchronize(stream));       // the trees are complete before a context reads them
        const std::vector<u32> eq = flat(ri), bwf = flat(bw);
        std::vector<E> rho;
        std::vector<Part> saved = parts;
        if (trace) fprintf(stderr, "gkr layer %d: %.1f us before its proof\n", layer, std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t_layer).count());
        if ((rc = prove_parts(ctxs, parts, tr, layer, layer > 0 ? eq.data() : nullptr, label, K, bwf.data(), layer > 0 ? 2 : 0, &rho, &folded, workers.get()))) return rc;
        std::vector<std::vector<E>> finals(L, std::vector<E>(4));
        std::vector<E> rbn;
        if (lk > 0) {
            // bind the block index: the blocks' values and weights, padded with zeros (:254-265)
            std::vector<Part> blk(L);
            std::vector<std::vector<u32>> keep;
            std::vector<u32> bwp = bwf;
            bwp.resize((size_t)KP * D, 0u);
            for (int l = 0; l < L; l++) {
                blk[l] = saved[l];
                blk[l].statement = "(* bw " + layer_statement + ")";
                blk[l].names.insert(blk[l].names.begin(), "bw");
                for (int t = 0; t < 4; t++) {
                    std::vector<u32> v(folded[l].begin() + (size_t)t * K * D, folded[l].begin() + (size_t)(t + 1) * K * D);
                    v.resize((size_t)KP * D, 0u);
                    keep.push_back(v);
                }
            }
            for (int l = 0; l < L; l++) {
                blk[l].host.assign(5, nullptr); blk[l].dev.assign(5, nullptr);
                blk[l].host[0] = bwp.data();
                for (int t = 0; t < 4; t++) blk[l].host[t + 1] = keep[(size_t)4 * l + t].data();
            }
            const std::string lab = std::string(label) + "-blk";
            std::vector<std::vector<u32>> fblk;
            if ((rc = prove_parts(ctxs, blk, tr, lk, nullptr, lab.c_str(), 1, nullptr, -1, &rbn, &fblk, workers.get()))) return rc;
            for (int l = 0; l < L; l++) for (int t = 0; t < 4; t++) finals[l][t].assign(fblk[l].begin() + (size_t)(t + 1) * D, fblk[l].begin() + (size_t)(t + 2) * D);
        } else {
            for (int l = 0; l < L; l++) for (int t = 0; t < 4; t++) finals[l][t].assign(folded[l].begin() + (size_t)t * K * D, folded[l].begin() + (size_t)t * K * D + D);
        }
        E tt;
        if ((rc = finish_layer(finals, &tt))) return rc;
        ri = rho; ri.push_back(tt);
        rb = rbn;
        if (trace) fprintf(stderr, "gkr layer %d: %.1f us\n", layer, std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t_layer).count());
    }
    if (ri_out) for (size_t i = 0; i < ri.size(); i++) memcpy(ri_out + i * D, ri[i].data(), 4 * (size_t)D);
    if (rb_out) for (size_t i = 0; i < rb.size(); i++) memcpy(rb_out + i * D, rb[i].data(), 4 * (size_t)D);
    if (cp_out) for (int l = 0; l < L; l++) memcpy(cp_out + (size_t)l * D, cp[l].data(), 4 * (size_t)D);
    if (cq_out) for (int l = 0; l < L; l++) memcpy(cq_out + (size_t)l * D, cq[l].data(), 4 * (size_t)D);
    return SC_OK;
}
