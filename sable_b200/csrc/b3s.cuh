// b3s.cuh -- the Fiat-Shamir transcript's hash on the device, run by one thread: sequential BLAKE3
// (B3S, src/blake3.lisp:44-155) and the challenge sampling (src/transcript.lisp:95-100, 116-135,
// 152-172).  Host/device code, so the same functions can be checked against the host transcript.
#pragma once
#include "field.cuh"

namespace sc {
using scf::u32;
using scf::u64;

#ifdef __CUDACC__
#define B3_HD __host__ __device__
#else
#define B3_HD
#endif

struct B3State {
    u32 cv[8];
    u32 pending[16];
    int fill;
    u64 blocks;
};
B3_HD inline u32 b3_ror(u32 x, int n) {
#ifdef __CUDA_ARCH__
    return __funnelshift_r(x, x, n);
#else
    return (x >> n) | (x << (32 - n));
#endif
}
#define B3_MIX(a, b, c, d, x, y)                  \
    a = a + b + (x); d = b3_ror(d ^ a, 16);       \
    c = c + d;       b = b3_ror(b ^ c, 12);       \
    a = a + b + (y); d = b3_ror(d ^ a, 8);        \
    c = c + d;       b = b3_ror(b ^ c, 7);
// COMPRESS (:44-88); OUT may alias nothing
#ifdef __CUDACC__
__host__ __device__ __noinline__
#else
inline
#endif
void b3_compress(const u32 *cv, const u32 *block, u64 counter, u32 block_len, u32 flags, u32 *out) {
    u32 v0 = cv[0], v1 = cv[1], v2 = cv[2], v3 = cv[3], v4 = cv[4], v5 = cv[5], v6 = cv[6], v7 = cv[7];
    u32 v8 = 0x6A09E667u, v9 = 0xBB67AE85u, v10 = 0x3C6EF372u, v11 = 0xA54FF53Au;
    u32 v12 = (u32)counter, v13 = (u32)(counter >> 32), v14 = block_len, v15 = flags;
    u32 m[16];
#pragma unroll
    for (int i = 0; i < 16; i++) m[i] = block[i];
#pragma unroll
    for (int round = 0; round < 7; round++) {
        B3_MIX(v0, v4, v8, v12, m[0], m[1]) B3_MIX(v1, v5, v9, v13, m[2], m[3])
        B3_MIX(v2, v6, v10, v14, m[4], m[5]) B3_MIX(v3, v7, v11, v15, m[6], m[7])
        B3_MIX(v0, v5, v10, v15, m[8], m[9]) B3_MIX(v1, v6, v11, v12, m[10], m[11])
        B3_MIX(v2, v7, v8, v13, m[12], m[13]) B3_MIX(v3, v4, v9, v14, m[14], m[15])
        if (round < 6) {   // the message permutation
            u32 t[16];
            t[0] = m[2]; t[1] = m[6]; t[2] = m[3]; t[3] = m[10]; t[4] = m[7]; t[5] = m[0]; t[6] = m[4]; t[7] = m[13];
            t[8] = m[1]; t[9] = m[11]; t[10] = m[12]; t[11] = m[5]; t[12] = m[9]; t[13] = m[14]; t[14] = m[15]; t[15] = m[8];
#pragma unroll
            for (int i = 0; i < 16; i++) m[i] = t[i];
        }
    }
    out[0] = v0 ^ v8; out[1] = v1 ^ v9; out[2] = v2 ^ v10; out[3] = v3 ^ v11;
    out[4] = v4 ^ v12; out[5] = v5 ^ v13; out[6] = v6 ^ v14; out[7] = v7 ^ v15;
    out[8] = v8 ^ cv[0]; out[9] = v9 ^ cv[1]; out[10] = v10 ^ cv[2]; out[11] = v11 ^ cv[3];
    out[12] = v12 ^ cv[4]; out[13] = v13 ^ cv[5]; out[14] = v14 ^ cv[6]; out[15] = v15 ^ cv[7];
}
// B3S-UPDATE (:118-136) of the low NBYTES (1..4) bytes of W: a full pending block is compressed only
// when more input arrives; at most two pieces per call (one up to the next word boundary, one after)
B3_HD inline void b3_put(B3State *st, u32 w, int nbytes) {
    while (nbytes > 0) {
        if (st->fill == 64) {
            u32 o[16];
            b3_compress(st->cv, st->pending, st->blocks++, 64, 0, o);
            for (int i = 0; i < 8; i++) st->cv[i] = o[i];
            for (int i = 0; i < 16; i++) st->pending[i] = 0;
            st->fill = 0;
        }
        const int at = st->fill & 3, room = 4 - at, can = nbytes < room ? nbytes : room;
        const u32 piece = can == 4 ? w : (w & ((1u << (8 * can)) - 1u));
        st->pending[st->fill >> 2] |= piece << (8 * at);
        st->fill += can;
        nbytes -= can;
        w = can == 4 ? 0u : (w >> (8 * can));
    }
}
// ABSORB (src/transcript.lisp:95-100) of a field array of WORDS values: u64 LE length in bytes, then the values as u32 LE
B3_HD inline void b3_absorb_words(B3State *st, const u32 *values, int words) {
    b3_put(st, (u32)(4 * words), 4); b3_put(st, 0u, 4);
    for (int i = 0; i < words; i++) b3_put(st, values[i], 4);
}
// SQUEEZE (:152-157) of N <= 64 bytes into OUT (as words): the output block, then "squeeze" and its first 32 bytes absorbed
B3_HD inline void b3_squeeze(B3State *st, u32 *out16, int nbytes) {
    b3_compress(st->cv, st->pending, 0, (u32)st->fill, 2u | 8u, out16);
    b3_put(st, 0x65757173u, 4);   // "sque"
    b3_put(st, 0x00657a65u, 3);   // "eze"
    const int take = nbytes < 32 ? nbytes : 32;
    for (int i = 0; i < take; i += 4) b3_put(st, out16[i >> 2], take - i < 4 ? take - i : 4);
}
// CHALLENGE-BASE (:159-172): K <= 8 base elements by rejection of 31-bit words
B3_HD inline void b3_challenge(B3State *st, int k, u32 *out) {
    int have = 0;
    while (have < k) {
        const int n = 4 * (k - have + 4);   // at most 48 bytes: one output block
        u32 o[16];
        b3_squeeze(st, o, n);
        for (int i = 0; i < n / 4 && have < k; i++) {
            const u32 w = o[i] & 0x7FFFFFFFu;
            if (w < scf::P) out[have++] = w;
        }
    }
}


}  // namespace sc
