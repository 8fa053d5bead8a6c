// transcript.cuh -- the Fiat-Shamir transcript carried on by the device: one round of it is SEND of the
// round's sums (ABSORB of a u64 length and the values as u32 LE, src/transcript.lisp:95-100, 116-135)
// followed by CHALLENGE (:152-176) over the sequential BLAKE3 of src/blake3.lisp:44-155.
//
// A block of threads runs a round together: every thread puts its bytes of the message behind the
// pending block in a small buffer (the stream is not word-aligned: SQUEEZE appends 7 + 32 bytes),
// then one thread runs the chain of compressions -- each needs the chaining value of the one before,
// so there is nothing for a second thread to do -- with the sixteen state words and the sixteen message
// words in registers, the message schedule resolved at compile time.  The four quarter-rounds of a step
// are independent instructions that one thread issues back to back, so the step already takes no longer
// than its chain of dependent operations; spreading the four columns over four lanes would add the
// shuffles of the diagonal step to that chain.
//
// Everything here is inlined into its caller and the compression has ONE call site (the loop in
// transcript_round), which keeps the two kernels that carry it (the transcript kernel behind a round kernel,
// and the resident kernel of the small rounds) small.
//
// The code is host/device: the host build runs the same statements with one "thread", so the device's
// transcript can be checked against the host transcript without a GPU.
#pragma once
#include <cstdint>

#include "field.cuh"

namespace sc {
using scf::u32;
using scf::u64;

// The hash state as it travels between launches (device memory) and from the host:
//   [0, 8) chaining value   [8, 24) pending block, little-endian words, zero padded   [24] bytes pending (0..64)
//   [25], [26] blocks compressed so far (low, high)
constexpr int B3_STATE_WORDS = 32;
constexpr int TR_BUF_WORDS = 96;     // 384 bytes: a pending block (64), a message (8 + 4 * 64), one SQUEEZE (39), rounded up to blocks

struct TrWork {          // a block's scratch for one round of the transcript (shared memory on the device)
    u32 cv[8];
    u32 buf[TR_BUF_WORDS];
    u32 out[16];         // the last compression's output
    u32 chal[8];         // the challenge, canonical words
    u32 off, total;      // byte offsets into buf: the pending block starts at off, the stream ends at total
    u32 blocks[2];
};

#ifdef __CUDA_ARCH__
#define TR_TID ((int)threadIdx.x)
#define TR_NT ((int)blockDim.x)
#define TR_SYNC() __syncthreads()
#define TR_FN __device__ __forceinline__
#define TR_INL __device__ __forceinline__
#else
#define TR_TID 0
#define TR_NT 1
#define TR_SYNC() ((void)0)
#define TR_FN inline
#define TR_INL inline
#endif

TR_INL u32 tr_ror(u32 x, int n) {
#ifdef __CUDA_ARCH__
    return __funnelshift_r(x, x, n);
#else
    return (x >> n) | (x << (32 - n));
#endif
}

#define TR_G(a, b, c, d, x, y)                     \
    a = a + b + (x); d = tr_ror(d ^ a, 16);        \
    c = c + d;       b = tr_ror(b ^ c, 12);        \
    a = a + b + (y); d = tr_ror(d ^ a, 8);         \
    c = c + d;       b = tr_ror(b ^ c, 7);
// one round: the four columns, then the four diagonals, with the sixteen message words in the order given
#define TR_ROUND(i0, i1, i2, i3, i4, i5, i6, i7, i8, i9, i10, i11, i12, i13, i14, i15)                                  \
    TR_G(v0, v4, v8, v12, m[i0], m[i1]) TR_G(v1, v5, v9, v13, m[i2], m[i3])                                             \
    TR_G(v2, v6, v10, v14, m[i4], m[i5]) TR_G(v3, v7, v11, v15, m[i6], m[i7])                                           \
    TR_G(v0, v5, v10, v15, m[i8], m[i9]) TR_G(v1, v6, v11, v12, m[i10], m[i11])                                         \
    TR_G(v2, v7, v8, v13, m[i12], m[i13]) TR_G(v3, v4, v9, v14, m[i14], m[i15])

// COMPRESS (src/blake3.lisp:44-88).  CV (8 words) and BLOCK (16 words) are read before OUT (16 words) is written,
// so OUT may be either of them.  The rows below are the message permutation (:37-40) applied 0 to 6 times.
TR_FN void tr_compress(const u32 *cv, const u32 *block, u32 counter_lo, u32 counter_hi, u32 block_len, u32 flags, u32 *out) {
    u32 m[16];
#pragma unroll
    for (int i = 0; i < 16; i++) m[i] = block[i];
    const u32 c0 = cv[0], c1 = cv[1], c2 = cv[2], c3 = cv[3], c4 = cv[4], c5 = cv[5], c6 = cv[6], c7 = cv[7];
    u32 v0 = c0, v1 = c1, v2 = c2, v3 = c3, v4 = c4, v5 = c5, v6 = c6, v7 = c7;
    u32 v8 = 0x6A09E667u, v9 = 0xBB67AE85u, v10 = 0x3C6EF372u, v11 = 0xA54FF53Au;
    u32 v12 = counter_lo, v13 = counter_hi, v14 = block_len, v15 = flags;
    TR_ROUND(0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15)
    TR_ROUND(2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8)
    TR_ROUND(3, 4, 10, 12, 13, 2, 7, 14, 6, 5, 9, 0, 11, 15, 8, 1)
    TR_ROUND(10, 7, 12, 9, 14, 3, 13, 15, 4, 0, 11, 2, 5, 8, 1, 6)
    TR_ROUND(12, 13, 9, 11, 15, 10, 14, 8, 7, 2, 5, 3, 0, 1, 6, 4)
    TR_ROUND(9, 14, 11, 5, 8, 12, 15, 1, 13, 3, 0, 10, 2, 6, 4, 7)
    TR_ROUND(11, 15, 5, 0, 1, 9, 8, 6, 14, 10, 2, 12, 3, 4, 7, 13)
    out[0] = v0 ^ v8; out[1] = v1 ^ v9; out[2] = v2 ^ v10; out[3] = v3 ^ v11;
    out[4] = v4 ^ v12; out[5] = v5 ^ v13; out[6] = v6 ^ v14; out[7] = v7 ^ v15;
    out[8] = v8 ^ c0; out[9] = v9 ^ c1; out[10] = v10 ^ c2; out[11] = v11 ^ c3;
    out[12] = v12 ^ c4; out[13] = v13 ^ c5; out[14] = v14 ^ c6; out[15] = v15 ^ c7;
}

TR_INL void tr_put_byte(TrWork *w, u32 at, u32 byte) { reinterpret_cast<unsigned char *>(w->buf)[at] = (unsigned char)byte; }

// One round of the transcript, by every thread of the block (the host build: by the caller alone).
//   STATE_IN   B3_STATE_WORDS words, the state before the round (any memory)
//   SUMS       W canonical words, the round's message (rows of D words)
//   STATE_OUT  the state after SEND and CHALLENGE (may be STATE_IN)
// The challenge, D canonical words, is left in W->chal.
TR_FN void transcript_round(TrWork *w, const u32 *state_in, const u32 *sums, int W, int D, u32 *state_out) {
    const int tid = TR_TID, nt = TR_NT;
    const u32 fill0 = state_in[24];
    for (int k = tid; k < TR_BUF_WORDS; k += nt) w->buf[k] = k < 16 ? state_in[8 + k] : 0u;
    for (int k = tid; k < 8; k += nt) w->cv[k] = state_in[k];
    TR_SYNC();
    // ABSORB: the length in bytes as u64 LE, then the values as u32 LE
    const int L = 8 + 4 * W;
    for (int k = tid; k < L; k += nt) {
        u32 byte;
        if (k < 8) byte = k < 4 ? (((u32)(4 * W)) >> (8 * k)) & 0xffu : 0u;
        else byte = (sums[(k - 8) >> 2] >> (8 * ((k - 8) & 3))) & 0xffu;
        tr_put_byte(w, fill0 + (u32)k, byte);
    }
    TR_SYNC();
    if (tid == 0) {
        w->off = 0; w->total = fill0 + (u32)L;
        w->blocks[0] = state_in[25]; w->blocks[1] = state_in[26];
        // One loop, one compression per turn.  While a full block has more input behind it, that block is chained
        // (B3S-UPDATE, src/blake3.lisp:134-142: a full block is compressed only when more input has arrived).  Else,
        // while challenge words are missing, SQUEEZE (src/transcript.lisp:152-157): the output block of the pending
        // bytes, from which CHALLENGE-BASE (:159-172) keeps the words below p, then "squeeze" and the first 32 output
        // bytes are absorbed -- which may fill a block again, and the loop chains it before it ends.
        int have = 0;
        for (;;) {
            const bool chain = w->total - w->off > 64;
            if (!chain && have >= D) break;
            if (!chain && w->total + 39u > 4u * TR_BUF_WORDS) {   // a second SQUEEZE (about once in 10^8 rounds): make room
                const u32 fill = w->total - w->off;
                for (int k = 0; k < 16; k++) w->buf[k] = w->buf[w->off / 4 + k];
                for (int k = 16; k < TR_BUF_WORDS; k++) w->buf[k] = 0;
                w->off = 0; w->total = fill;
            }
            tr_compress(w->cv, w->buf + w->off / 4, chain ? w->blocks[0] : 0u, chain ? w->blocks[1] : 0u, chain ? 64u : w->total - w->off,
                        chain ? 0u : (2u | 8u), w->out);   // the output block: CHUNK_END | ROOT, counter 0 (:113-123)
            if (chain) {
#pragma unroll
                for (int i = 0; i < 8; i++) w->cv[i] = w->out[i];
                if (++w->blocks[0] == 0) ++w->blocks[1];
                w->off += 64;
            } else {
                const int nbytes = 4 * (D - have + 4);      // at most 48: one output block
                for (int i = 0; i < nbytes / 4 && have < D; i++) {
                    const u32 v = w->out[i] & 0x7FFFFFFFu;
                    if (v < scf::P) w->chal[have++] = v;
                }
                const u32 tag[2] = {0x65757173u, 0x00657a65u};   // "sque", "eze"
                for (int k = 0; k < 7; k++) tr_put_byte(w, w->total + (u32)k, (tag[k >> 2] >> (8 * (k & 3))) & 0xffu);
                const int take = nbytes < 32 ? nbytes : 32;
                for (int k = 0; k < take; k++) tr_put_byte(w, w->total + 7u + (u32)k, (w->out[k >> 2] >> (8 * (k & 3))) & 0xffu);
                w->total += 7u + (u32)take;
            }
        }
    }
    TR_SYNC();
    const u32 off = w->off;
    for (int k = tid; k < 8; k += nt) state_out[k] = w->cv[k];
    for (int k = tid; k < 16; k += nt) state_out[8 + k] = w->buf[off / 4 + k];
    if (tid == 0) { state_out[24] = w->total - off; state_out[25] = w->blocks[0]; state_out[26] = w->blocks[1]; }
}

}  // namespace sc
