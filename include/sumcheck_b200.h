/*
 * sumcheck_b200.h -- C ABI of libsumcheck_b200.so: the sumcheck prover rounds on a B200.
 *
 * The reference (Exacta, Common Lisp) has no foreign-function interface; its operator for this
 * path is the Lisp function
 *
 *   (exacta.sumcheck:prove tr n statement tables &key eq constants label block-weights degree)
 *                                                             src/sumcheck.lisp:512-571
 *
 * The functions below are what a Lisp PROVE binds (through sb-alien) to run its rounds on the
 * device: each one names the reference code it stands in for.  Part 1 is the device layer (the
 * transcript and the statement compiler stay with the caller, as in the reference).  Part 2 is a
 * host layer in C++ behind the same ABI, for callers without a Lisp: the transcript, the
 * statement compiler and PROVE itself, with the reference's argument meaning.
 *
 * Conventions.  Every function returns 0 or a negative SC_E* code and never throws or aborts.
 * Field values cross this boundary as canonical u32 residues in [0, p), p = 2^31 - 2^24 + 1; an
 * extension element is D consecutive u32 in the reference's tower order (src/field.lisp:8-11).
 * Input values >= p are reduced, as COERCE-EXT does (src/field.lisp:115-117).  A context belongs
 * to one device and one host thread at a time; calls are synchronous unless stated.  The library
 * installs no signal handler and calls nothing back.
 */
#ifndef SUMCHECK_B200_H
#define SUMCHECK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SC_OK 0
#define SC_EINVAL (-1)      /* bad argument (the reference signals INVALID-PARAMETER, src/conditions.lisp:94-122) */
#define SC_ECUDA (-2)       /* a CUDA call failed; sc_last_error() has the text */
#define SC_ENOMEM (-3)      /* device or host memory exhausted, or over the context's memory budget */
#define SC_EUNSUPPORTED (-4)/* a shape no kernel is instantiated for (degree, table count, extension degree) */
#define SC_ESTATE (-5)      /* calls out of order (round before begin, challenge before round ...) */
#define SC_ECOMM (-6)       /* the collective layer failed or timed out */
#define SC_ESTATEMENT (-7)  /* malformed statement, or a variable that is neither a table nor a constant */

#define SC_MAX_TABLES 8        /* table slots of one context */
#define SC_MAX_WIDE_TABLES 64  /* tables of one sc_prove: a wider statement is cut into parts on child contexts */
#define SC_MAX_TERMS 16
#define SC_MAX_FACTORS 8
#define SC_MAX_POINTS 8

typedef struct sc_ctx sc_ctx;

/* ------------------------------------------------------------------ part 1: the device layer */

/* A prover context on CUDA device DEVICE (an ordinal of this process).  It owns every device
   buffer it makes: tables, folded tables, weights, partial sums.  No reference counterpart (the
   reference allocates fresh Lisp vectors per round, src/sumcheck.lisp:92). */
int sc_create(int device, sc_ctx **ctx);
int sc_destroy(sc_ctx *ctx);

/* A cap, in bytes, on the device memory the context may hold (0 = no cap).  Exceeding it makes
   the allocating call return SC_ENOMEM before any CUDA allocation is tried. */
int sc_set_memory_budget(sc_ctx *ctx, uint64_t bytes);

const char *sc_strerror(int code);
const char *sc_last_error(const sc_ctx *ctx);

/* The statement as a term table: sum over terms of coefficient * product of tables.  This is
   what EXPAND (src/forms.lisp:57-78) gives once the constants' values are multiplied into each
   monomial's coefficient; it replaces the compiled round kernel of the reference
   (ROUND-KERNEL-CODE, src/sumcheck.lisp:190-258, and STATEMENT-FUNCTION, :108-110).
     D          extension degree, 4 or 8 (TRANSCRIPT-DEGREE)
     points     max(degree, 1): the round message has POINTS rows, X = 0, 2, .., POINTS (:186-188)
     ntables    number of table slots (at most SC_MAX_TABLES); tables that occur in no term are still
                folded (:528, :562).  A statement may multiply up to eight different tables at degree
                <= 4, up to four at degree 5 to 8; otherwise SC_EUNSUPPORTED
     coeffs     nterms * D canonical words
     term_ptr   nterms + 1 offsets into term_tables (CSR); term t multiplies tables
                term_tables[term_ptr[t] .. term_ptr[t+1]), repeated indices for powers */
int sc_set_statement(sc_ctx *ctx, int D, int points, int ntables, int nterms, const uint32_t *coeffs,
                     const int32_t *term_ptr, const int32_t *term_tables);

/* Table SLOT from host memory: ENTRIES entries of STRIDE words, stride 1 (base field) or D.
   Stands in for MAKE-TABLE (src/sumcheck.lisp:61-70).  The host array is only read, and is free
   again when the call returns (from pinned memory the call waits for the copy; from pageable
   memory the data has left the array by then and the rest is ordered on the context's stream). */
int sc_upload_table(sc_ctx *ctx, int slot, const uint32_t *host, uint64_t entries, int stride);

/* Table SLOT filled on the device by the seeded generator of the benchmarks:
   word c of entry i = splitmix64(seed ^ table_id << 56 ^ c << 48 ^ (first + i)) mod p;
   with NONZERO an all-zero entry gets word 0 = 1.  No reference counterpart. */
int sc_generate_table(sc_ctx *ctx, int slot, uint64_t seed, int table_id, uint64_t first, uint64_t entries,
                      int stride, int nonzero);

/* Table SLOT is the caller's own device memory: ENTRIES entries of STRIDE words, canonical (every
   word below p; nothing reduces them), starting on a 16-byte boundary, on the context's device.
   Nothing is copied: the first rounds read the table where it lies, and it must stay unchanged
   and allocated until another table takes the slot (the folded tables are the context's own).
   The context never writes or frees it.  For callers whose tables are made on the device (the layers of a fraction tree,
   sc_gkr_prove_upper).  No reference counterpart: Lisp tables live in host memory. */
int sc_borrow_table(sc_ctx *ctx, int slot, const uint32_t *table_dev, uint64_t entries, int stride);

/* Room ahead of a run of proofs of growing size (the layers of a tree, smallest first): the folded
   tables' buffers and the weight tables for proofs of extension degree D with up to N variables
   over K blocks and NTABLES tables, so that no proof of the run frees and allocates again.
   Optional; counted in the memory budget.  No reference counterpart. */
int sc_reserve(sc_ctx *ctx, int D, int n, int K, int ntables);
/* Child INDEX (0..63) of the context at *OUT: a context of its own on the same device, made on
   first use, destroyed with its parent.  sc_prove runs the parts of a statement wider than one
   kernel on them.  No reference counterpart. */
int sc_child(sc_ctx *ctx, int index, sc_ctx **out);
/* BYTES of device memory of the context's own for the caller's scratch, at *OUT: grow-only (a
   larger request frees and allocates, the contents are lost), freed with the context, counted in
   the memory budget.  No reference counterpart. */
int sc_workspace(sc_ctx *ctx, uint64_t bytes, void **out);

/* The current (folded) contents of table SLOT as canonical extension elements, for tests.
   Writes min(entries, CAP) entries of D words; *ENTRIES gets the table's size.  SC_ESTATE while the
   folded table does not exist in memory: during the small-value rounds (rounds 1 and 2 of a product
   of base tables) and once the resident last-rounds kernel runs. */
int sc_download_table(sc_ctx *ctx, int slot, uint32_t *host, uint64_t cap, uint64_t *entries);

/* Start a proof of N rounds over the uploaded tables (each K * 2^N entries, K = 1 when
   BLOCK_WEIGHTS is NULL).  EQ: N extension elements or NULL (weights 1).  Builds the eq weight
   tables of every round on the device (WEIGHTS and SPLIT-WEIGHTS, src/sumcheck.lisp:37-49; the
   split point is chosen per round by the library, which does not change any sum). */
int sc_begin(sc_ctx *ctx, int n, const uint32_t *eq, int K, const uint32_t *block_weights);

/* Round j: the sums g_j(X) at X = 0, 2, .., POINTS over the pairs of the current tables, as
   POINTS * D canonical words, row-major (what ROUND-MESSAGE sends, src/sumcheck.lisp:313-317).
   For j > 0 the fold by the previous challenge (FOLD-FLAT-TABLE, :84-104) happens inside the
   same kernel, on the way in.  With a communicator (sc_comm_init) the sums are the whole job's. */
int sc_round(sc_ctx *ctx, uint32_t *sums);

/* The challenge of the round just computed, D canonical words (CHALLENGE, src/transcript.lisp:174).
   It is applied by the next sc_round or by sc_finish. */
int sc_challenge(sc_ctx *ctx, const uint32_t *r);

/* After the last challenge: every table folded to K entries, written as ntables * K * D canonical
   words (the third value of PROVE, src/sumcheck.lisp:567-571; its second value, the finals, is
   entry 0 of each).  With N = 0 these are the tables' own entries. */
int sc_finish(sc_ctx *ctx, uint32_t *folded);

/* Timing of the rounds of the last proof, measured with CUDA events on the context's stream. */
typedef struct sc_round_stat {
    float kernel_ms;        /* the round kernel (fold + sums) */
    uint64_t bytes;         /* algorithmic bytes: tables read once + folded tables written once */
    uint64_t pairs;         /* pairs summed in the round */
} sc_round_stat;
int sc_enable_timing(sc_ctx *ctx, int on);
int sc_round_stats(sc_ctx *ctx, sc_round_stat *stats, int cap, int *count);
/* Kernels launched by this context since it was created. */
uint64_t sc_launch_count(const sc_ctx *ctx);
/* A stopwatch of CUDA events on the context's stream: sc_timer_stop waits for the stream and
   gives the milliseconds since sc_timer_start. */
int sc_timer_start(sc_ctx *ctx);
int sc_timer_stop(sc_ctx *ctx, float *ms);
/* The caller's words of table SLOT as they lie on the device (WORDS of them), for benchmarks that
   generate a table on the device and want the same data in host memory. */
int sc_fetch_table(sc_ctx *ctx, int slot, uint32_t *host, uint64_t words);

/* Several GPUs: the hypercube is cut on its top log2(WORLD) variables, rank RANK holding entries
   [RANK * 2^N / WORLD, (RANK + 1) * 2^N / WORLD) of every table (with block weights: of every block of
   every table, block after block).  Each round's sums are combined
   with an NCCL all-gather of POINTS * D words and a sum mod p; when fewer than log2(WORLD)
   variables would remain per rank the tables are gathered and every rank finishes alike.
   NCCL_ID is the 128-byte ncclUniqueId made by rank 0 (sc_comm_unique_id) and handed to the
   others by the caller.  sc_begin's N stays the whole job's.  No reference counterpart. */
int sc_comm_unique_id(void *nccl_id128);
int sc_comm_init(sc_ctx *ctx, const void *nccl_id128, int rank, int world);
/* The context's place in its communicator (rank 0 of 1 without one). */
int sc_comm_info(const sc_ctx *ctx, int *rank, int *world);

/* One round's sums with no allocation at all, for callers that cannot allocate device memory where
   they run: code recording work into a stream capture, a service whose device memory was handed
   out completely at start-up, a plug-in that receives device pointers but no allocator.  It has
   no counterpart in the reference (which allocates freely); it computes what sc_round returns
   for round 0 of a proof without eq weights: the sums of the statement (given as for
   sc_set_statement) at X = 0, 2, .., POINTS over the pairs of the caller's device-resident
   tables (TABLES_DEV[t]: ENTRIES entries of STRIDES[t] words, canonical, below p, each table
   starting on a 16-byte boundary, as cudaMalloc and torch give them; an offset into a larger buffer
   must keep that), written as POINTS * D canonical words to the device buffer SUMS_DEV (4-byte
   aligned).  The launch is asynchronous on STREAM (a cudaStream_t, or NULL); the device that is
   current when the call is made must be the stream's and the tables' device.
   Scratch: the blocks' partial sums and a block counter live in one fixed array in the library's
   device image (256.25 KiB: 2 048 rows of 32 words and the counter, held by every GPU that loads
   the library until exit).  The limits that follow from it: ENTRIES at most 2^28 per table and
   POINTS * D at most 32; more is refused with an error code and a message naming the limit,
   and so are misaligned or null pointers -- nothing is launched then.  The first call on a device looks up
   the array's device address (cudaGetSymbolAddress), so make that first call before any stream
   capture begins.  All calls on one device share the array: the counter is cleared at the start of
   each call, the rows are overwritten, and two calls that run on the GPU at the same time race --
   order them on one stream or with events.  On the host nothing is shared between calls but the
   looked-up addresses, so calls may come from several host threads (ordering their work on the
   GPU stays the caller's job).  Nothing is allocated or freed, on the device or by any
   library, and no context is needed.  On failure the text of the error is copied to MESSAGE
   (MESSAGE_CAP bytes, may be NULL). */
int sc_round_sums_static(int D, int points, int ntables, const uint32_t *const *tables_dev, const int *strides,
                         uint64_t entries, int nterms, const uint32_t *coeffs, const int32_t *term_ptr,
                         const int32_t *term_tables, uint32_t *sums_dev, void *stream, char *message,
                         size_t message_cap);

/* ------------------------------------------------------------------ part 2: the host layer */

typedef struct sc_transcript sc_transcript;

/* MAKE-TRANSCRIPT (src/transcript.lisp:75-84), prover side: B3S over "LLM-SUMCHECK-v6-O|" | label. */
sc_transcript *sc_transcript_new(const uint8_t *label, size_t label_len, int degree);
void sc_transcript_free(sc_transcript *tr);
int sc_transcript_degree(const sc_transcript *tr);   /* TRANSCRIPT-DEGREE */
/* ABSORB (:95-100), SEND of a field array (:133-135), CHALLENGE-BASE (:166-172), B3S-DIGEST of the state */
int sc_transcript_absorb(sc_transcript *tr, const uint8_t *data, uint64_t len);
int sc_transcript_send(sc_transcript *tr, const uint32_t *values, int rows, int cols);
int sc_transcript_challenge_base(sc_transcript *tr, int k, uint32_t *out);
int sc_transcript_challenge_bits(sc_transcript *tr, int nbits, int k, uint64_t *out);
int sc_transcript_digest(const sc_transcript *tr, uint8_t *out, size_t n);
/* TRANSCRIPT-MESSAGES (:69), TRANSCRIPT-SENT-BYTES (:73) */
int sc_transcript_message_count(const sc_transcript *tr);
int sc_transcript_message(const sc_transcript *tr, int index, uint64_t dims[2], uint32_t *values);
uint64_t sc_transcript_sent_bytes(const sc_transcript *tr);
/* ENCODE-PROOF (src/proofio.lisp:44-49) of the recorded messages: returns the size; writes when CAP allows. */
uint64_t sc_transcript_encode(const sc_transcript *tr, const char magic[8], uint8_t *out, uint64_t cap);

/* The hash state of the transcript (B3S: chaining value, pending block as little-endian words,
   bytes pending, blocks compressed), for a device that carries the transcript on. */
int sc_transcript_state(const sc_transcript *tr, uint32_t cv[8], uint32_t pending[16], int *fill, uint64_t *blocks);
/* For tests: the transcript code the device runs (one round: SEND of ROWS x COLS values, then CHALLENGE of TR's
   degree), executed on the host from TR's present state without changing TR.  STATE_OUT gets 32 words: chaining
   value, pending block, bytes pending, blocks compressed (low, high); CHALLENGE gets the degree's words. */
int sc_transcript_device_round(const sc_transcript *tr, const uint32_t *values, int rows, int cols, uint32_t *state_out,
                               uint32_t *challenge);
/* The transcript on the device (an option; the default keeps it on the host, as the reference does).  Per round
   the host's part is SEND of the sums and CHALLENGE (src/transcript.lisp:116-176): a launch, a wait and a hash
   per round, which is all a small round costs.  With sc_set_device_transcript(CTX, 1) -- or
   SABLE_B200_DEVICE_TRANSCRIPT=1 in the environment when the context is made -- and the proof's transcript
   attached, the first sc_round of a proof enqueues EVERY round at once: behind each round kernel a one-block kernel
   sends the round's sums and draws the challenge (sequential BLAKE3 on the device, from a copy of the
   transcript's hash state), and the next launch folds by the challenge it finds in device memory.  The caller's
   loop stays as it is: sc_round returns each round's sums as they are posted, the caller sends them and draws
   the challenge on its own transcript, and sc_challenge checks that it is the device's (SC_ESTATE if not: the
   transcript was used for something else in between).  The proof bytes are the same.  With several GPUs every
   rank hashes the same summed words, so nothing more crosses NVLink.  The small-value first rounds of a statement
   over base tables stay with the host; the chain starts after them.
   sc_attach_transcript: TR (or NULL) is the host transcript of the proofs that follow on CTX; sc_prove attaches
   its own for the length of the call.  sc_attach_transcript_state: the same for a transcript that is not the
   library's own, such as the Lisp one: its B3S state -- chaining value, pending block as little-endian words, bytes
   pending, blocks compressed -- as it stands when the next sc_round is called; used by that call if it starts
   a chain, forgotten otherwise.  No reference counterpart: the reference's transcript is host code throughout. */
int sc_attach_transcript(sc_ctx *ctx, const sc_transcript *tr);
int sc_attach_transcript_state(sc_ctx *ctx, const uint32_t cv[8], const uint32_t pending[16], int fill, uint64_t blocks);
int sc_set_device_transcript(sc_ctx *ctx, int on);

/* EXPAND + the lowering to a term table (src/forms.lisp:57-78; STATEMENT-DEGREE,
   src/sumcheck.lisp:33-35).  STATEMENT is the form as text, e.g. "(+ (* alpha t0 t1) (* 3 t1))".
   Outputs as for sc_set_statement; *DEGREE gets the degree in the tables.  Capacities:
   SC_MAX_TERMS terms, SC_MAX_TERMS * SC_MAX_FACTORS table indices. */
int sc_lower_statement(const char *statement, int D, int ntables, const char *const *table_names, int nconstants,
                       const char *const *constant_names, const uint32_t *constant_values, int *degree, int *nterms,
                       uint32_t *coeffs, int32_t *term_ptr, int32_t *term_tables);

/* PROVE (src/sumcheck.lisp:512-571) with the reference's argument meaning.  TABLES[t] is host
   memory of K * 2^N entries of STRIDES[t] words (with a communicator: this rank's slice, 2^N / world
   entries), or NULL for a table already on the device in slot t (sc_upload_table, sc_generate_table).  DEGREE < 0 takes the statement's degree.
   Outputs (any may be NULL): CHALLENGES n * D, FINALS ntables * D, FOLDED ntables * max(K,1) * D.
   TR ends in the state, and with the recorded messages, the reference leaves it in.
   A statement with more than SC_MAX_TABLES tables or SC_MAX_TERMS terms (or, above degree four,
   more than four tables) is cut into groups of terms, each proved on a context of its own (CTX
   and its children, sc_child) with the groups' sums added per round: up to SC_MAX_WIDE_TABLES
   tables, all passed from host memory, one GPU. */
int sc_prove(sc_ctx *ctx, sc_transcript *tr, int n, const char *statement, int ntables,
             const char *const *table_names, const uint32_t *const *tables, const int *strides, const uint32_t *eq,
             int nconstants, const char *const *constant_names, const uint32_t *constant_values, const char *label,
             int K, const uint32_t *block_weights, int degree, uint32_t *challenges, uint32_t *finals,
             uint32_t *folded);

/* PROVE-UPPER (src/gkr.lisp:215-272): the upper layers of the batched LogUp-GKR fraction trees.
   A domain has K blocks of 2^N leaf fractions p/q for each of LOOKUPS lookups; LEAVES_P[l] and
   LEAVES_Q[l] are K * 2^N entries of D words, block-major (host memory, or device memory when
   LEAVES_ON_DEVICE is nonzero; they are only read).  Builds the fraction trees on the device
   (FRACTION-TREES, :149-188), sends the roots and proves every layer down to the leaves' parents
   on TR, exactly the messages and challenges of the reference.  CTXS holds one context per lookup,
   all on the current device and without a communicator: the layer statement is a sum over the
   lookups, and lookup l's share of each round's sums is computed on CTXS[l].  Tables 0..4 of the
   contexts are overwritten.  N >= 1.  Device memory: about 4 * K * 2^N * D words per lookup for
   the trees, taken from the first context's workspace (sc_workspace) and kept by it for the next
   call, besides the contexts' own buffers.
   Outputs (any may be NULL): RI (N - 1) * D words (the in-block point), RB ceil(log2 K) * D (the
   block point), CP and CQ LOOKUPS * D each (the claims on the leaf layer). */
int sc_gkr_prove_upper(sc_ctx *const *ctxs, int lookups, sc_transcript *tr, int n, int K, const uint32_t *const *leaves_p,
                       const uint32_t *const *leaves_q, int leaves_on_device, const char *label, uint32_t *ri, uint32_t *rb,
                       uint32_t *cp, uint32_t *cq);

/* PROVE-DOMAIN (src/domain.lisp:336-372): a domain of BLOCKS blocks of 2^N elements with base-field columns,
   constraints that must vanish everywhere and lookups, proved by one batched LogUp-GKR over the lookups' trees
   (sc_gkr_prove_upper) and one sumcheck over the halves of the columns (sc_prove), with the reference's messages
   and challenges.  The domain is data, as in MAKE-DOMAIN (:39-53):
     column   NAME; KIND 0 :full (every variable), 1 :row C (the variables from C on), 2 :col C (the variables
              below C); SHARED: the same in every block (never a :full column); DATA in host memory: K 2^N words
              (:full), K 2^(N-C) (:row), K 2^C (:col), without the factor K when shared
     constraints  forms over the column names, as text
     lookup   TAG, VALUES and NUM (or NULL): forms; a leaf of the lookup's tree is NUM / (Z - TAG - sum_i BETA_i VALUE_i)
   With MERGE the block index is bound inside the protocol (a second sumcheck) and a claim is one value. */
typedef struct sc_domain_column { const char *name; int kind; int c; int shared; const uint32_t *data; } sc_domain_column;
typedef struct sc_domain_lookup { const char *tag; int nvalues; const char *const *values; const char *num; } sc_domain_lookup;
typedef struct sc_domain {
    const char *name;
    int n, blocks, merge;
    int ncolumns; const sc_domain_column *columns;
    int nconstraints; const char *const *constraints;
    int nlookups; const sc_domain_lookup *lookups;
} sc_domain;
/* DOMAIN-STATEMENT (:104-125) as text (STATEMENT, CAP bytes; SC_EINVAL when it does not fit), the number of tables
   of the sumcheck (DOMAIN-TABLES, :60-78: two per column that depends on the top in-block variable), and
   DOMAIN-DEGREE (:127-156) of the main sumcheck and of the block phase.  Any output may be NULL. */
int sc_domain_statement(const sc_domain *domain, char *statement, size_t cap, int *ntables, int *degree, int *block_degree);
/* CTXS: max(1, lookups) contexts on the current device, without a communicator (the first also proves the
   sumcheck; a statement wider than one kernel runs in parts on its children).  Z (D words) and BETAS (NBETAS
   elements, at least the lookups' largest number of values) are the lookup challenges, drawn by the caller.
   LABEL: NULL for "dom".  Outputs, the column claims (DOMAIN-CLAIMS, :179-210), any may be NULL: for column c,
   POINT_LEN[c] elements at POINTS + c (N + ceil(log2 K)) D and VALUE_ROWS[c] elements at VALUES + c K D (one
   value when merged or shared, else K). */
int sc_prove_domain(sc_ctx *const *ctxs, int nctx, sc_transcript *tr, const sc_domain *domain, const uint32_t *z, const uint32_t *betas,
                    int nbetas, const char *label, int *point_len, uint32_t *points, int *value_rows, uint32_t *values);

#ifdef __cplusplus
}
#endif
#endif /* SUMCHECK_B200_H */
