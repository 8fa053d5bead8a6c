// field.cuh -- KoalaBear arithmetic for the device: F_p with p = 2^31 - 2^24 + 1 and the tower
// F_p^D = F_p[w]/(w^D - 3), D = 4 or 8, on the 32-bit integer pipes.
//
// The reference computes a product as (mod (* a b) p) on 64-bit words (src/field.lisp:70-72) and an
// extension product as a schoolbook sum with one reduction per four products (mul*, :220-234).
// Here a product is a 64-bit product followed by Montgomery's REDC (R = 2^32), which leaves the
// factor 1/R: constants (challenges, weights, coefficients) are kept as c R so that constant
// times value needs no correction, and the factors left by products of two table values are
// collected into one constant per round (see DevTerm in device.h).  Tables hold canonical
// residues in [0, p) on the device as they do at the library boundary.
//
// An extension element is D words in the reference's tower order: word i holds the coefficient of
// w^bitrev(i) (power-order, src/field.lisp:195-204).
#pragma once
#include <cstdint>

namespace scf {

typedef uint32_t u32;
typedef uint64_t u64;

constexpr u32 P = 2130706433u;       // 0x7F000001
constexpr u32 PINV = 0x81000001u;    // p^-1 mod 2^32
constexpr u32 R1 = 0x01FFFFFEu;      // 2^32 mod p   (the Montgomery form of 1)
constexpr u32 R2 = 0x17F7EFE4u;      // 2^64 mod p   (REDC(x R2) = x R: into Montgomery form)
constexpr u32 R3 = 0x18AF7F37u;      // 2^96 mod p

#ifdef __CUDACC__
#define SCF_HD __host__ __device__ __forceinline__
#else
#define SCF_HD inline
#endif

SCF_HD u32 umin32(u32 a, u32 b) { return a < b ? a : b; }
SCF_HD u32 mulhi32(u32 a, u32 b) {
#ifdef __CUDA_ARCH__
    return __umulhi(a, b);
#else
    return (u32)(((u64)a * b) >> 32);
#endif
}

// a + b and a - b for a, b in [0, p): the wrapped candidate is the larger one (fadd, fsub,
// src/field.lisp:50-60, written without the sign mask).
SCF_HD u32 fadd(u32 a, u32 b) { u32 s = a + b; return umin32(s, s - P); }
SCF_HD u32 fsub(u32 a, u32 b) { u32 d = a - b; return umin32(d, d + P); }
SCF_HD u32 fneg(u32 a) { return fsub(0u, a); }
SCF_HD u32 fdbl(u32 a) { return fadd(a, a); }
SCF_HD u32 ftriple(u32 a) { return fadd(fadd(a, a), a); }   // times-3, src/field.lisp:62-65

// Montgomery reduction of t < p 2^32: t / 2^32 mod p, in [0, p).
SCF_HD u32 redc(u64 t) {
    u32 m = (u32)t * PINV;
    u32 u = mulhi32(m, P);
    u32 r = (u32)(t >> 32) - u;
    return umin32(r, r + P);
}
// The same for t < 2 p 2^32, which holds a sum of four products of values below p
// (4 p^2 < 2 p 2^32): the high word loses one p first.
SCF_HD u32 redc4(u64 t) {
    u32 hi = (u32)(t >> 32);
    hi = umin32(hi, hi - P);
    u32 m = (u32)t * PINV;
    u32 u = mulhi32(m, P);
    u32 r = hi - u;
    return umin32(r, r + P);
}
SCF_HD u32 mmul(u32 a, u32 b) { return redc((u64)a * b); }
SCF_HD u32 to_mont(u32 x) { return mmul(x, R2); }
SCF_HD u32 from_mont(u32 x) { return redc((u64)x); }

template <int D> struct Log2;
template <> struct Log2<1> { static constexpr int v = 0; };
template <> struct Log2<2> { static constexpr int v = 1; };
template <> struct Log2<4> { static constexpr int v = 2; };
template <> struct Log2<8> { static constexpr int v = 3; };

template <int D> SCF_HD constexpr int brev(int i) {
    int r = 0;
    for (int b = 0; b < Log2<D>::v; b++) r |= ((i >> b) & 1) << (Log2<D>::v - 1 - b);
    return r;
}

template <int D> struct Ext {
    u32 v[D];
};

template <int D> SCF_HD Ext<D> ezero() { Ext<D> o;
#pragma unroll
    for (int i = 0; i < D; i++) o.v[i] = 0; return o; }
template <int D> SCF_HD Ext<D> eone_mont() { Ext<D> o = ezero<D>(); o.v[0] = R1; return o; }
template <int D> SCF_HD Ext<D> eadd(const Ext<D> &a, const Ext<D> &b) { Ext<D> o;
#pragma unroll
    for (int i = 0; i < D; i++) o.v[i] = fadd(a.v[i], b.v[i]); return o; }
template <int D> SCF_HD Ext<D> esub(const Ext<D> &a, const Ext<D> &b) { Ext<D> o;
#pragma unroll
    for (int i = 0; i < D; i++) o.v[i] = fsub(a.v[i], b.v[i]); return o; }
// a times a base element s (ext-scale, src/field.lisp:158-164)
template <int D> SCF_HD Ext<D> escale(const Ext<D> &a, u32 s) { Ext<D> o;
#pragma unroll
    for (int i = 0; i < D; i++) o.v[i] = mmul(a.v[i], s); return o; }
template <int D> SCF_HD Ext<D> eto_mont(const Ext<D> &a) { return escale<D>(a, R2); }
template <int D> SCF_HD Ext<D> efrom_mont(const Ext<D> &a) { Ext<D> o;
#pragma unroll
    for (int i = 0; i < D; i++) o.v[i] = from_mont(a.v[i]); return o; }

// A multiplier prepared once: the element with the triples of the coefficients that wrap around
// w^D = 3 (the reference triples b's wrapping coefficients first, mul* src/field.lisp:225-227).
template <int D> struct ExtM {
    u32 v[D];    // tower order
    u32 t[D];    // 3 v[i]; t[0] unused
};
template <int D> SCF_HD ExtM<D> eprep(const Ext<D> &b) { ExtM<D> m;
#pragma unroll
    for (int i = 0; i < D; i++) { m.v[i] = b.v[i]; m.t[i] = ftriple(b.v[i]); }
    return m; }

// A running sum of products below p^2 in 64 bits: four fit from zero; then the high word loses one
// p (the sum drops below p 2^32) and two more fit, and so on; the sum stays below 2 p 2^32, which is
// what redc4 takes.  So a coordinate with many products needs one reduction, not one per four.
SCF_HD u64 presub(u64 t) {
    u32 hi = (u32)(t >> 32);
    hi = umin32(hi, hi - P);
    return ((u64)hi << 32) | (u32)t;
}
// a b in F_p[w]/(w^D - 3): c_e = sum_{i+j=e} a_i b_j + 3 sum_{i+j=e+D} a_i b_j on the power-ordered
// coefficients (mul*, src/field.lisp:220-234, reduces once per four products; here once per
// coordinate).  Montgomery REDC on each sum: with both factors in Montgomery form so is the product.
template <int D> SCF_HD Ext<D> emul(const Ext<D> &a, const ExtM<D> &b) {
    Ext<D> o;
#pragma unroll
    for (int e = 0; e < D; e++) {
        u64 acc = 0;
#pragma unroll
        for (int i = 0; i < D; i++) {
            if (i >= 4 && (i & 1) == 0) acc = presub(acc);
            const int j = (e - i + D) % D;
            const u32 bj = (i > e) ? b.t[brev<D>(j)] : b.v[brev<D>(j)];
            acc += (u64)a.v[brev<D>(i)] * bj;
        }
        o.v[brev<D>(e)] = (D >= 4) ? redc4(acc) : redc(acc);
    }
    return o;
}
// a b without the reductions: per coordinate the 64-bit sum of products (below 2 p 2^32), which redc4 turns into the
// coordinate; such sums can be added up first (presub on the way) and reduced once
template <int D> struct ExtRaw { u64 v[D]; };
template <int D> SCF_HD ExtRaw<D> emul_raw(const Ext<D> &a, const ExtM<D> &b) {
    ExtRaw<D> o;
#pragma unroll
    for (int e = 0; e < D; e++) {
        u64 acc = 0;
#pragma unroll
        for (int i = 0; i < D; i++) {
            if (i >= 4 && (i & 1) == 0) acc = presub(acc);
            const int j = (e - i + D) % D;
            const u32 bj = (i > e) ? b.t[brev<D>(j)] : b.v[brev<D>(j)];
            acc += (u64)a.v[brev<D>(i)] * bj;
        }
        o.v[brev<D>(e)] = acc;
    }
    return o;
}
// a1 b1 + a2 b2 with one reduction per coordinate
template <int D> SCF_HD Ext<D> emul2(const Ext<D> &a1, const ExtM<D> &b1, const Ext<D> &a2, const ExtM<D> &b2) {
    Ext<D> o;
#pragma unroll
    for (int e = 0; e < D; e++) {
        u64 acc = 0;
#pragma unroll
        for (int k = 0; k < 2 * D; k++) {
            if (k >= 4 && (k & 1) == 0) acc = presub(acc);
            const int i = k % D;
            const int j = (e - i + D) % D;
            const Ext<D> &a = k < D ? a1 : a2;
            const ExtM<D> &b = k < D ? b1 : b2;
            const u32 bj = (i > e) ? b.t[brev<D>(j)] : b.v[brev<D>(j)];
            acc += (u64)a.v[brev<D>(i)] * bj;
        }
        o.v[brev<D>(e)] = redc4(acc);
    }
    return o;
}
template <int D> SCF_HD Ext<D> emul(const Ext<D> &a, const Ext<D> &b) { return emul<D>(a, eprep<D>(b)); }

// a b + s c for a base element s: the product s c_k joins the first four products of coordinate k
// before their reduction (the sum of four loses one p 2^32 first, so five products fit 64 bits and
// stay below 2 p 2^32), which saves a reduction and an addition per coordinate.
template <int D> SCF_HD Ext<D> emul_plus_scaled(const Ext<D> &a, const ExtM<D> &b, const Ext<D> &c, u32 s) {
    Ext<D> o;
#pragma unroll
    for (int e = 0; e < D; e++) {
        u64 acc = 0;
#pragma unroll
        for (int i = 0; i < D; i++) {
            if (i >= 4 && (i & 1) == 0) acc = presub(acc);
            const int j = (e - i + D) % D;
            const u32 bj = (i > e) ? b.t[brev<D>(j)] : b.v[brev<D>(j)];
            acc += (u64)a.v[brev<D>(i)] * bj;
        }
        acc = presub(acc) + (u64)c.v[brev<D>(e)] * s;   // after four or after two products: room for at least one more
        o.v[brev<D>(e)] = redc4(acc);
    }
    return o;
}

}  // namespace scf
