// device.h -- the structures handed to the kernels and the launchers the context calls.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/sumcheck_b200.h"
#include "field.cuh"
#include "transcript.cuh"

namespace sc {

using scf::u32;
using scf::u64;

enum CoeffKind : uint8_t { CK_ONE = 0, CK_BASE = 1, CK_EXT = 2 };

// Statements with a kernel of their own; every other statement runs the term-table kernel.
//   SHAPE_PRODUCT  c t0 t1 .. t(k-1), each table once, k points; c rides in the round's final factor
//   SHAPE_GKR      a d + b c + lam c d over the tables (a, b, c, d) = positions (0, 1, 2, 3);
//                  lam is the coefficient of term 0
//   SHAPE_LISTED + k  statement k of the list below, its term table resolved at compile time
enum Shape : int { SHAPE_GENERIC = 0, SHAPE_PRODUCT = 1, SHAPE_GKR = 2, SHAPE_LISTED = 3 };

// Statements instantiated ahead of time.  The reference compiles a kernel per statement at run time
// (ROUND-KERNEL, src/sumcheck.lisp:270-280); here a statement on this list gets kernels of its own at build time:
// the description below is all compile-time, so the term loop unrolls into straight-line code with every table
// index fixed.  A statement matches an entry when its tables can be put into the entry's positions so that the
// terms' table lists agree and no coefficient needs more than the entry's kind allows (CK_EXT takes any
// coefficient, CK_BASE one in the base field).  Every other statement runs the term-table kernel.  To add one:
// a specialisation here, a line in LISTED_SHAPES, and the instantiations in the launchers (launch_round_listed,
// launch_tail, launch_round_base).
template <int K> struct Listed;
#ifdef __CUDACC__
#define SC_CX static constexpr __host__ __device__
#else
#define SC_CX static constexpr
#endif
// c0 t0 t1 + c1 t1: a product and one of its tables again, e.g. (+ (* alpha t0 t1) (* 3 t1))
template <> struct Listed<0> {
    static constexpr int NT = 2, PTS = 2, NTERMS = 2;
    SC_CX int nf(int t) { return t == 0 ? 2 : 1; }
    SC_CX int f(int t, int k) { return t == 0 ? k : 1; }
    SC_CX int ck(int t) { return t == 0 ? CK_EXT : CK_BASE; }
};
// c0 t0 t1 t2 + c1 t2, e.g. the reference's base-table test statement (+ (* t0 t1 t2) (* 7 t1)) (tests/tests.lisp:333)
template <> struct Listed<1> {
    static constexpr int NT = 3, PTS = 3, NTERMS = 2;
    SC_CX int nf(int t) { return t == 0 ? 3 : 1; }
    SC_CX int f(int t, int k) { return t == 0 ? k : 2; }
    SC_CX int ck(int t) { return t == 0 ? CK_EXT : CK_BASE; }
};
// c0 t0 t1 + c1 t2 t3: a sum of two products over different tables
template <> struct Listed<2> {
    static constexpr int NT = 4, PTS = 2, NTERMS = 2;
    SC_CX int nf(int) { return 2; }
    SC_CX int f(int t, int k) { return 2 * t + k; }
    SC_CX int ck(int) { return CK_EXT; }
};
constexpr int LISTED_SHAPES = 3;
constexpr int LISTED_MAX_TERMS = 3, LISTED_MAX_FACTORS = 4;
// the same descriptions as data, for the host's matching
struct ListedInfo { int nt, pts, nterms, nf[LISTED_MAX_TERMS], f[LISTED_MAX_TERMS][LISTED_MAX_FACTORS], ck[LISTED_MAX_TERMS]; };
template <int K> inline ListedInfo listed_info() {
    ListedInfo o = {};
    o.nt = Listed<K>::NT; o.pts = Listed<K>::PTS; o.nterms = Listed<K>::NTERMS;
    for (int t = 0; t < o.nterms; t++) {
        o.nf[t] = Listed<K>::nf(t); o.ck[t] = Listed<K>::ck(t);
        for (int k = 0; k < o.nf[t]; k++) o.f[t][k] = Listed<K>::f(t, k);
    }
    return o;
}

// One term of the statement: coefficient times a product of tables.  Tables hold canonical words
// and constants (coefficients, weights, challenges) are in Montgomery form c R, so REDC of
// constant times value is their canonical product.  A product of m table values computed with
// m - 1 REDCs carries the factor R^-(m-1); with e = max(m - 1) over the terms, the coefficient of
// a term is stored as c R^(m-1-e) and the round's final factor carries R^e.  A term without
// factors is the constant term, stored as the canonical word c R^-e and added as it is.
struct DevTerm {
    u32 coeff[8];
    uint8_t ckind;
    uint8_t nf;
    uint8_t f[SC_MAX_FACTORS];
    uint8_t group;        // the base-table kernel: which sum the term's base value goes to (see RoundArgs::gcoef)
    uint8_t pad;
};
struct DevStatement {
    int nterms;
    DevTerm terms[SC_MAX_TERMS];
};

constexpr int ROUND_THREADS = 256;


constexpr int MAX_PARTIAL_WORDS = SC_MAX_POINTS * 8;   // points * D words per partial sum

// Everything one round kernel needs.  The kernel reads the current tables (entries 2i, 2i+1 of
// each for pair i; with FOLD entries 4i..4i+3, folded by r on the way in and written to dst),
// evaluates the statement at X = 0, 2, .., points on the line through each pair, weights the
// values by low[l] high[h] for i = h 2^logL + l, and sums over all pairs.
struct RoundArgs {
    const u32 *src[SC_MAX_TABLES];
    u32 *dst[SC_MAX_TABLES];
    uint8_t src_base[SC_MAX_TABLES];   // 1: the source holds base-field entries (one word each)
    int ntables;          // tables read (and folded); the statement may use fewer
    u32 r[8];             // the fold challenge, Montgomery form
    u64 npairs;           // pairs to sum, over all blocks
    int logL;             // pairs per high weight: 2^logL
    int use_low;          // 0: every low weight is 1 (and logL is 0 or there is no eq)
    int use_high;         // 0: every high weight is 1
    const u32 *low;       // 2^logL multipliers (ExtM layout: D words, then their D triples), Montgomery form
    const u32 *high;      // npairs >> logL elements, Montgomery form
    DevStatement st;
    u32 post[8];          // the sums are multiplied by this element at the end (Montgomery form) ...
    int use_post;         // ... when this is 1
    u32 *partials;        // gridDim.x rows of points * D words
    unsigned int *counter;// blocks that have written their partial; the last one finishes and resets it
    u32 *out_dev;         // points * D canonical words
    u32 *out_host;        // the same, in mapped host memory (may be NULL) ...
    u32 seq;              // ... followed, at word MAX_PARTIAL_WORDS, by this launch's number once the sums are visible
    // The kernel for a round whose tables are all in the base field sums base values: one sum per
    // group of terms, weighted by the eq weights, and multiplies each group's sum by its
    // coefficient at the end.  Group 0 holds the terms with base-field coefficients (their sum is a
    // base value, gcoef = 1); a term with an extension coefficient is a group of its own.
    // Several GPUs: the last block hands this rank's sums to every rank and adds up what the others hand it,
    // through mailboxes in device memory that the ranks opened to each other (peer stores over NVLink): rank r's
    // mailbox holds, for each parity of the exchange number and each sender, MAIL_WORDS words: the sums, then at
    // word MAIL_FLAG the exchange number, written last.  xseq = 0: no exchange (one GPU, or the caller exchanges).
    u32 *mail[8];         // the ranks' mailboxes, mail[rank] this rank's own
    int world, rank;
    u32 xseq;
    unsigned mail_polls;  // polls (with a short sleep each) the last block waits for the other ranks' sums
    // A chain of launches (the transcript on the device, see TranscriptArgs): the fold challenge lies at R_DEV (D words,
    // Montgomery form), left there by the transcript kernel of the round before, instead of in r; the launch number
    // is also written behind the sums at out_dev (word MAX_PARTIAL_WORDS), with EXCHANGE_FAILED when another rank's
    // sums never came; DEAD points at the chain's failure word: once it is set the last block does not wait again.
    const u32 *r_dev;
    const u32 *dead;
    int chained;          // 1: the launch is part of a chain (out_dev has room for the launch number)
    u32 bind[4][8];       // FOLD = 2: eq(rho0 rho1, b), b < 4, Montgomery form: entry y of the bound table is sum_b bind[b] T[4y + b]
    u32 bind3[8][8];      // FOLD = 3: eq(rho0 rho1 rho2, b), b < 8: entry y of the bound table is sum_b bind3[b] T[8y + b]
    int ngroups;
    u32 gcoef[2][8];      // Montgomery form
};
constexpr int CHAIN_CHAL_WORD = 72;   // a chain's slot in mapped host memory: sums at [0, 64), the posted launch number at 64, the challenge at [72, 80)
constexpr int CHAIN_SLOT_WORDS = 96;
constexpr int CHAIN_DEAD = 31;        // word of the hash state's buffer: a round of the chain failed

// The transcript's part of a round, on the device (transcript.cuh): one block, launched behind the round kernel of a
// chain.  It reads the round's sums (and the launch number behind them) where the round kernel left them, SENDs them
// and draws the CHALLENGE from the hash state in TSTATE (or, for the first launch of a chain, from TSTATE0, the host
// transcript's state), leaves the new state in TSTATE and the challenge in CHAL_DEV (D words in Montgomery form for the
// next launch's fold, then the D canonical words), and posts sums, challenge and the launch number to the chain's slot
// in mapped host memory.  So the host can enqueue every round of a proof without waiting for any of them.
// It is a kernel of its own, not the round kernel's last block, because transcript code inside the round kernels --
// called or inlined, and run by one block only -- slowed every round kernel's main loop by 2 % (measured on the
// layer statement at n = 28, alternating builds on one GPU: 12.25 ms without, 12.47 ms with).
struct TranscriptArgs {
    const u32 *sums;      // W words, then at word MAX_PARTIAL_WORDS the launch number the round kernel wrote
    int W, D;
    u32 *tstate;
    u32 *chal_dev;
    int tinit;
    u32 tstate0[B3_STATE_WORDS - 4];
    u32 *out_host;        // the chain's slot of this round
    u32 seq;
};
cudaError_t launch_transcript_round(const TranscriptArgs &args, cudaStream_t stream);
constexpr int MAIL_WORDS = 128, MAIL_FLAG = 64;
constexpr unsigned MAIL_POLL_LIMIT = 20000000u;   // polls (with a short sleep each) a rank waits for the others' sums
constexpr u32 EXCHANGE_FAILED = 0x80000000u;      // or-ed into the posted launch number when a rank's sums never came
constexpr int FAST_POINTS = 4;         // the built-in statements, the base-table, small-value and resident kernels: degree <= 4
constexpr int MAX_GROUPS = 2;
constexpr int BASE_MAX_TERMS = 4;      // the base-table kernel keeps its term descriptors in registers:
constexpr int BASE_MAX_FACTORS = 4;    // statements beyond these run the general kernel
constexpr int PARTIAL_ROW_WORDS = MAX_PARTIAL_WORDS > MAX_GROUPS * FAST_POINTS * 8 ? MAX_PARTIAL_WORDS : MAX_GROUPS * FAST_POINTS * 8;   // words per block in the partials buffer

// Launchers (defined next to their kernels).  Each returns the CUDA error of the launch.
// fold: 0 the tables as they are, 1 folded by r on the way in, 2 base tables bound to two challenges at once (args.bind)
cudaError_t launch_round(int D, int shape, int points, int nt_used, int fold, const RoundArgs &args, int grid, size_t smem,
                         cudaStream_t stream);
bool round_supported(int D, int points, int nt_used);
// The round on tables that are all in the base field (no fold): see RoundArgs::ngroups.
cudaError_t launch_round_base(int D, int shape, int points, int nt_used, int ngroups, const RoundArgs &args, int grid, size_t smem,
                              cudaStream_t stream);
// Blocks of that kernel an SM holds: three where the sums are few enough for 80 registers a thread (the built-in
// statements at D = 4 with at most 16 words of sums), else two.  The grid is sized to match.
#ifdef __CUDACC__
__host__ __device__
#endif
constexpr int round_base_blocks_per_sm(int D, int shape, int points, int ngroups) {
    return D == 4 && shape != SHAPE_GENERIC && ngroups * points * D <= 16 && points <= 3 ? 3 : 2;
}
// a listed statement in that kernel: the number of sums it keeps (0: it cannot run there) and the sum of a term
int listed_base_groups(int shape);
int listed_base_group_of(int shape, int term);

// The first two rounds of a statement over base-field tables from one pass over the tables (the
// reference's small-value rounds with L0 = 2, src/sumcheck.lisp:319-337): for every block y of four
// consecutive entries the tables' values on the grid {0..G-1}^2 of the two lowest variables are
// made by additions, the statement is evaluated on them in the base field, and the values are summed with
// the eq weights of the other variables: A[z0 + G z1] = sum_y w(y) F(T_t(z0, z1, y)).  The host reads both round
// messages off A; the tables are then bound to both challenges at once on the way into round 2.
struct SvArgs {
    const u32 *src[SC_MAX_TABLES];
    u64 nblocks;          // blocks of four entries
    int logL;             // blocks per high weight; a thread keeps one low index and walks the high ones
    int use_low, use_high;
    const u32 *low;       // multipliers (ExtM layout), Montgomery form
    const u32 *high;
    u32 post[8];          // final factor (Montgomery form), applied when use_post
    int use_post;
    u32 *partials;        // gridDim.x rows of G * G * D words
    unsigned int *counter;
    u32 *out_dev;         // G * G * D canonical words (for the all-gather of several GPUs; may be NULL)
    u32 *out_host;        // the same in mapped host memory (may be NULL), then the word below
    u32 seq;              // posted at word SV_FLAG of out_host
    DevStatement st;      // the statement, for the kernels that read the term table
    int ngroups;          // sums kept per grid point, as in the base-table round kernel (see RoundArgs::gcoef) ...
    int use_gcoef;        // ... 1: some group's coefficient is not one ...
    u32 gcoef[MAX_GROUPS][8];   // ... the groups' coefficients (Montgomery form), applied by the last block
};
constexpr int SV_MAX_WORDS = 128;  // G^2 D words: G <= 4, D <= 8
constexpr int SV_FLAG = SV_MAX_WORDS;
cudaError_t launch_small_values(int D, int shape, int G, int nt, const SvArgs &args, int grid, cudaStream_t stream);
bool small_values_supported(int D, int G, int nt);
// The same for the first three rounds (L0 = 3, degree at most two): blocks of eight entries, G^3 D words out, then the
// word SV3_FLAG; nblocks counts blocks of eight, the weights are those of round 2.  One sum per grid point only.
constexpr int SV3_MAX_WORDS = 256;  // G^3 D words: G <= 3, D <= 8
constexpr int SV3_FLAG = SV3_MAX_WORDS;
cudaError_t launch_small_values3(int D, int shape, int G, int nt, const SvArgs &args, int grid, cudaStream_t stream);
bool small_values3_supported(int D, int G, int nt);
int small_values_grid_x(int D, int G, int ngroups, int l0, int sms);   // thread blocks along x that fill the GPU once (the grid's y is the kernels' own)

// The last rounds in one launch.  Once the tables are small a round is all latency (launch,
// completion, the trip to the host and back), so a single block runs every remaining round and
// talks to the host through mapped memory: it posts a round's sums, waits -- a bounded number of
// polls -- for the challenge the host's transcript derives from them, folds, and goes on; after
// the last challenge it folds once more and posts the final entries.  The transcript stays on
// the host.  Slot k of the mapped buffer (TAIL_SLOT_WORDS words) belongs to round k of the launch:
//   [0, 32) sums   [40, 48) challenge (canonical), each word with TAIL_HERE set once it is written (cleared by the host before the launch)
//   the device's own transcript instead: [32] posted = seq + k, [50] challenge posted, [52, 60) the challenge
// word TAIL_STATUS of the buffer: 0 running, 1 finished, 2 gave up waiting, 3 told to stop;
// word TAIL_STOP: the host sets it to seq to make the kernel return at its next poll;
// the final entries (ntables * K * D words, table after table) start at word TAIL_FINALS, each word with TAIL_HERE set.
constexpr int TAIL_MAX_ROUNDS = 16;
constexpr int TAIL_SLOT_WORDS = 64;
constexpr int TAIL_STATUS = TAIL_MAX_ROUNDS * TAIL_SLOT_WORDS;
constexpr int TAIL_STOP = TAIL_STATUS + 1;
constexpr int TAIL_FINALS = TAIL_STATUS + 16;
constexpr int TAIL_FINAL_WORDS = 1024;           // room for the final entries: ntables * K * D words at most
constexpr int TAIL_WORDS = TAIL_FINALS + TAIL_FINAL_WORDS;
constexpr u32 TAIL_HERE = 0x80000000u;           // set in a word that has been written (elements are below p < 2^31)
constexpr unsigned TAIL_POLL_LIMIT = 1500000u;   // polls of mapped host memory (about a microsecond each) before giving up
struct TailRound {
    u64 npairs;
    u64 high_word;     // offset of the round's weights in the weights buffer
    int use_high;
};
struct TailArgs {
    const u32 *src[SC_MAX_TABLES];     // the tables the first round of the launch reads (4 entries per pair)
    u32 *buf[2][SC_MAX_TABLES];        // the folded tables go to buf[0], buf[1], buf[0], ..
    uint8_t src_base[SC_MAX_TABLES];
    int ntables;
    int nrounds;
    int blocks;                        // K: the tables are K blocks of entries, one after the other; one final entry per table and block
    int nofold;                        // 1: the launch's first round has no challenge to fold by: it sums the pairs of src as they lie (2 entries per pair)
    TailRound rd[TAIL_MAX_ROUNDS];
    u32 r[8];                          // the challenge of the round before the launch, Montgomery form
    const u32 *weights;
    DevStatement st;
    u32 post[8];
    int use_post;
    u32 seq;
    u32 *host;                         // the mapped buffer (device address)
    unsigned poll_limit;               // polls before the block gives up on a challenge
    // own_transcript: the block derives each challenge itself (transcript.cuh) instead of waiting for the host, which
    // replays the same messages on its transcript and checks.  The hash state it starts from is TSTATE0 (a copy of
    // the host transcript's state before this launch's first round) or, when TSTATE is set, the state the round
    // kernels before it left in device memory; then the challenge of the round before the launch is at R_DEV.
    int own_transcript;
    u32 tstate0[B3_STATE_WORDS - 4];
    u32 *tstate;
    const u32 *r_dev;
};
cudaError_t launch_tail(int D, int shape, int points, int nt_used, const TailArgs &args, cudaStream_t stream);

// Stand-alone fold of NTABLES tables: dst entry i = src[2i] + r (src[2i+1] - src[2i]).
struct FoldArgs {
    const u32 *src[SC_MAX_TABLES];
    u32 *dst[SC_MAX_TABLES];
    uint8_t src_base[SC_MAX_TABLES];
    int ntables;
    const u32 *r_dev;   // non-null: the challenge lies here, in device memory, instead of in r
    u32 r[8];     // Montgomery form
    u64 nout;     // entries written per table
};
cudaError_t launch_fold(int D, const FoldArgs &args, cudaStream_t stream);

// Entries as extension elements (base entries lifted): count entries per table.
struct ExportArgs {
    const u32 *src[SC_MAX_TABLES];
    uint8_t src_base[SC_MAX_TABLES];
    int ntables;
    u64 count;
    u32 *out;     // ntables * count * D words
};
cudaError_t launch_export(int D, const ExportArgs &args, cudaStream_t stream);

// Seeded table generator (canonical residues).
cudaError_t launch_generate(u32 *out, u64 seed, int table_id, u64 first, u64 entries, int stride, int nonzero,
                            cudaStream_t stream);
// In-place reduction of words >= p (inputs are reduced as COERCE-EXT does).
cudaError_t launch_reduce_words(u32 *words, u64 count, cudaStream_t stream);

// The eq weight tables of every round.  CHUNKS holds, for every start s < n and width w = 1..8,
// eq(r[s .. s+w)) as 2^w elements at element offset s * 512 + 2^w (Montgomery form); each
// descriptor names a table entry x -> product over 8-bit chunks of x, times an optional block
// weight, written as Ext (kind 0) or as a multiplier with triples (kind 1).
struct WeightDesc {
    u64 out_word;     // word offset of the table in the weights buffer
    u64 entries;      // entries per block
    int start;        // first eq variable
    int bits;         // variables covered: entries = 2^bits
    int kind;         // 0: Ext, 1: ExtM
    int blocks;       // > 0: the table has blocks * entries elements, element (b, x) times bw[b]
};
cudaError_t launch_eq_chunks(int D, const u32 *r_mont, int n, u32 *chunks, cudaStream_t stream);
cudaError_t launch_weight_tables(int D, const u32 *chunks, const WeightDesc *descs, int ndescs, const u32 *bw_mont,
                                 u32 *weights, u64 total_entries, cudaStream_t stream);

// out[k] = sum over ranks of gathered[rank * words + k] mod p, to device and mapped host memory.
// The launch number SEQ is posted at word FLAG_WORD of out_host once the sums are visible.
cudaError_t launch_sum_ranks(const u32 *gathered, int world, int words, u32 *out_dev, u32 *out_host, int flag_word, u32 seq,
                             cudaStream_t stream);

}  // namespace sc
