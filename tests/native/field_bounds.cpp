// field_bounds.cpp -- host-side checks of the device's 64-bit running sums (csrc/field.cuh is host/device code):
// the sums of products that the kernels carry without reducing must never wrap, for the largest operands, and must
// reduce to the exact value.  Shadow arithmetic in unsigned __int128.  Prints "ok" or the first failure.
#include <cstdio>
#include <cstdlib>

#include "../../sable_b200/csrc/field.cuh"

using namespace scf;
typedef unsigned __int128 u128;

static u64 rng_state = 88172645463325252ull;
static u32 rnd() {   // xorshift, values in [0, p)
    rng_state ^= rng_state << 13; rng_state ^= rng_state >> 7; rng_state ^= rng_state << 17;
    return (u32)(rng_state % P);
}
static u32 exact_redc(u128 t) {   // t / 2^32 mod p for any t: multiply by the inverse of 2^32
    // 2^-32 mod p: from_mont(1) = redc(1)
    const u32 rinv = redc((u64)1);
    return (u32)(((t % P) * rinv) % P);
}
static int fail(const char *what, long i) { printf("FAILED: %s at step %ld\n", what, i); return 1; }

// the small-value passes: acc = (second ? presub(acc) : acc) + w f, second toggling, redc4 at the end
static int running_sum(u32 w, u32 f, long steps) {
    u64 acc = 0;
    u128 shadow = 0, plain = 0;
    bool second = false;
    for (long i = 0; i < steps; i++) {
        if (second) { const u64 before = acc; acc = presub(acc); shadow -= (u128)(before - acc); }
        acc += (u64)w * f; shadow += (u128)w * f; plain += (u128)w * f;
        if ((u128)acc != shadow) return fail("the running sum wrapped", i);
        if (shadow >= ((u128)2 * P << 32)) return fail("the running sum left redc4's range", i);
        second = !second;
    }
    if (redc4(acc) != exact_redc(plain)) return fail("the reduced running sum is not the exact value", steps);
    return 0;
}

// round 0 with low weights: inner = presub(inner) + presub(raw), raw the unreduced coordinates of an extension product
template <int D> static int lazy_products(bool extreme, long steps) {
    u64 inner[D];
    Ext<D> want = ezero<D>();
    for (int c = 0; c < D; c++) inner[c] = 0;
    for (long i = 0; i < steps; i++) {
        Ext<D> a, b;
        for (int c = 0; c < D; c++) { a.v[c] = extreme ? P - 1 : rnd(); b.v[c] = extreme ? P - 1 : rnd(); }
        const ExtM<D> bm = eprep<D>(b);
        const ExtRaw<D> raw = emul_raw<D>(a, bm);
        const Ext<D> prod = emul<D>(a, bm);
        for (int c = 0; c < D; c++) {
            if (raw.v[c] >= ((u64)2 * P << 32)) return fail("an unreduced coordinate left redc4's range", i);
            if (redc4(raw.v[c]) != prod.v[c]) return fail("emul_raw and emul disagree", i);
            const u128 sum = (u128)presub(inner[c]) + presub(raw.v[c]);
            if (sum >= ((u128)2 * P << 32)) return fail("the sum of products left redc4's range", i);
            inner[c] = (u64)sum;
        }
        want = eadd<D>(want, prod);
    }
    for (int c = 0; c < D; c++)
        if (redc4(inner[c]) != want.v[c]) return fail("the reduced sum of products is not the sum of the reduced products", steps);
    return 0;
}

// the bind of three challenges: two sums of four products, reduced apart
static int bound_eight(bool extreme) {
    u32 w[8], e[8];
    for (int b = 0; b < 8; b++) { w[b] = extreme ? P - 1 : rnd(); e[b] = extreme ? P - 1 : rnd(); }
    u64 lo4 = 0, hi4 = 0;
    u128 plain = 0;
    for (int b = 0; b < 4; b++) { lo4 += (u64)w[b] * e[b]; hi4 += (u64)w[4 + b] * e[4 + b]; }
    for (int b = 0; b < 8; b++) plain += (u128)w[b] * e[b];
    if (fadd(redc4(lo4), redc4(hi4)) != exact_redc(plain)) return fail("eight bound entries", 0);
    return 0;
}

int main() {
    int bad = 0;
    bad |= running_sum(P - 1, P - 1, 1 << 20);          // the largest operands, a million blocks
    bad |= running_sum(P - 1, 1, 1000);
    for (int k = 0; k < 200 && !bad; k++) bad |= running_sum(rnd(), rnd(), 1 + (long)(rnd() % 5000));
    bad |= lazy_products<4>(true, 4096);
    bad |= lazy_products<4>(false, 4096);
    bad |= lazy_products<8>(true, 1024);
    bad |= lazy_products<8>(false, 1024);
    bad |= bound_eight(true);
    for (int k = 0; k < 1000 && !bad; k++) bad |= bound_eight(false);
    if (!bad) printf("ok\n");
    return bad;
}
