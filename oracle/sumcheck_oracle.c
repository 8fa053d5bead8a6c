/*
 * sumcheck_oracle.c -- CPU restatement of the reference sumcheck prover, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA prover is compared with; it is
 * never linked into, loaded by or called from the product library.  Only the test suite, the smoke
 * check and the benchmark's CPU-baseline legs may use it.
 *
 * Parity status: PINNED.  Every function here is checked (tests/test_oracle.py) against the
 * reference's own known-answer vectors (its tests/vectors.sexp, copied as data into
 * tests/golden/vectors.json): the :ext :lagrange :eq :mle :pow :b3s :transcript :proofio :poly
 * vectors, and the four :sumcheck vectors, whose challenges, finals and proof bytes it reproduces
 * exactly.  The reference itself (Common Lisp) cannot be run where this is built.
 *
 * Each section cites the reference file and lines it follows (paths inside the reference tree).
 * The algorithm has the reference's shape: flat tables that stay in the base field until their
 * first fold, eq weights split in two halves (LOW and HIGH), one pass per round over the pairs
 * and one fold per round, statements evaluated as written.  Loops over HIGH blocks and over
 * folded entries may run on several threads (OpenMP); the sums are exact, so the thread count
 * does not change any output.
 */
#include <ctype.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define P 2130706433u /* 2^31 - 2^24 + 1, src/field.lisp:31 */
#define MAXD 8
typedef uint32_t u32;
typedef uint64_t u64;
typedef uint8_t u8;

/* ------------------------------------------------------------------ F_p, src/field.lisp:46-84 */

static inline u32 fadd(u32 a, u32 b) { u32 s = a + b; return s >= P ? s - P : s; }
static inline u32 fsub(u32 a, u32 b) { return a >= b ? a - b : a + P - b; }
static inline u32 fmul(u32 a, u32 b) { return (u32)(((u64)a * b) % P); }
static u32 fpow(u32 a, u64 e) {
    u32 r = 1, b = a % P;
    for (; e; e >>= 1) { if (e & 1) r = fmul(r, b); b = fmul(b, b); }
    return r;
}
static u32 modp_i64(long long x) { long long r = x % (long long)P; if (r < 0) r += P; return (u32)r; }

u32 orc_fpow(u32 a, u64 e) { return fpow(a, e); }

/* ------------------------------------------------------------------ F_p^D, src/field.lisp:140-164,195-234 */

static int bitrev(int i, int bits) {
    int r = 0;
    for (int b = 0; b < bits; b++) r |= ((i >> b) & 1) << (bits - 1 - b);
    return r;
}
static int log2i(int d) { int b = 0; while ((1 << b) < d) b++; return b; }

static void eadd(int D, const u32 *a, const u32 *b, u32 *o) { for (int i = 0; i < D; i++) o[i] = fadd(a[i], b[i]); }
static void esub(int D, const u32 *a, const u32 *b, u32 *o) { for (int i = 0; i < D; i++) o[i] = fsub(a[i], b[i]); }
static void escale(int D, const u32 *a, u32 s, u32 *o) { for (int i = 0; i < D; i++) o[i] = fmul(a[i], s); }
static void ezero(int D, u32 *o) { memset(o, 0, 4 * D); }
static void eone(int D, u32 *o) { ezero(D, o); o[0] = 1; }
static void ecopy(int D, const u32 *a, u32 *o) { memcpy(o, a, 4 * D); }

/* Schoolbook product in F_p[w]/(w^D - 3); coordinate i holds the coefficient of w^bitrev(i)
   (power-order, src/field.lisp:195-204; mul*, :220-234).  Up to four products below p^2 are summed
   in a 64-bit word before one reduction (reduced-sum, :213-218). */
static void emul(int D, const u32 *a, const u32 *b, u32 *o) {
    int bits = log2i(D);
    u32 ap[MAXD], bp[MAXD], b3[MAXD], c[MAXD];
    for (int e = 0; e < D; e++) { ap[e] = a[bitrev(e, bits)]; bp[e] = b[bitrev(e, bits)]; }
    for (int e = 0; e < D; e++) b3[e] = fadd(fadd(bp[e], bp[e]), bp[e]);
    for (int e = 0; e < D; e++) {
        u32 acc = 0; u64 part = 0; int cnt = 0;
        for (int i = 0; i < D; i++) {
            int j = (e - i + D) % D;
            part += (u64)ap[i] * (i > e ? b3[j] : bp[j]);
            if (++cnt == 4) { acc = fadd(acc, (u32)(part % P)); part = 0; cnt = 0; }
        }
        if (cnt) acc = fadd(acc, (u32)(part % P));
        c[e] = acc;
    }
    for (int e = 0; e < D; e++) o[e] = c[bitrev(e, bits)];
}

/* 1/a as a^(p^D - 2): the same field element as the reference's norm descent (inv*, :236-243).
   The exponent is written in base p: p^D - 2 = (p-1)(p^(D-1)+...+p) + (p-2). */
static void einv(int D, const u32 *a, u32 *o) {
    /* square-and-multiply over the digits of p^D - 2 in base 2, computed with a small bignum */
    u32 big[MAXD + 1]; memset(big, 0, sizeof big); big[0] = 1;
    int len = 1;
    for (int k = 0; k < D; k++) { /* big *= p */
        u64 carry = 0;
        for (int i = 0; i < len; i++) { u64 t = (u64)big[i] * P + carry; big[i] = (u32)t; carry = t >> 32; }
        if (carry) big[len++] = (u32)carry;
    }
    { /* big -= 2 */
        u64 borrow = 2;
        for (int i = 0; i < len && borrow; i++) { u64 t = (u64)big[i]; if (t >= borrow) { big[i] = (u32)(t - borrow); borrow = 0; } else { big[i] = (u32)(t + (1ull << 32) - borrow); borrow = 1; } }
    }
    u32 r[MAXD], base[MAXD], t[MAXD];
    eone(D, r); ecopy(D, a, base);
    for (int i = 0; i < len; i++)
        for (int b = 0; b < 32; b++) {
            if ((big[i] >> b) & 1) { emul(D, r, base, t); ecopy(D, t, r); }
            emul(D, base, base, t); ecopy(D, t, base);
        }
    ecopy(D, r, o);
}

void orc_ext_add(int D, const u32 *a, const u32 *b, u32 *o) { eadd(D, a, b, o); }
void orc_ext_sub(int D, const u32 *a, const u32 *b, u32 *o) { esub(D, a, b, o); }
void orc_ext_mul(int D, const u32 *a, const u32 *b, u32 *o) { u32 t[MAXD]; emul(D, a, b, t); ecopy(D, t, o); }
void orc_ext_inv(int D, const u32 *a, u32 *o) {
    int nz = 0; for (int i = 0; i < D; i++) nz |= a[i] != 0;
    if (nz) einv(D, a, o); else ezero(D, o);
}
/* eq(a, b) = a b + (1 - a)(1 - b), src/field.lisp:306-309 */
void orc_ext_eq1(int D, const u32 *a, const u32 *b, u32 *o) {
    u32 one[MAXD], x[MAXD], y[MAXD], z[MAXD];
    eone(D, one); emul(D, a, b, x); esub(D, one, a, y); esub(D, one, b, z); emul(D, y, z, y); eadd(D, x, y, o);
}

/* eq-table, src/field.lisp:354-363: entry e becomes e(1 - r_b) below and e r_b above. */
void orc_eq_table(int D, int k, const u32 *r, u32 *out) {
    eone(D, out);
    size_t size = 1;
    for (int b = 0; b < k; b++) {
        for (size_t i = 0; i < size; i++) {
            u32 up[MAXD];
            emul(D, out + D * i, r + D * b, up);
            esub(D, out + D * i, up, out + D * i);
            ecopy(D, up, out + D * (size + i));
        }
        size *= 2;
    }
}

/* lagrange, src/field.lisp:326-352: sum_i w_i v_i prod_{j != i} (x - j), nodes 0..d. */
void orc_lagrange(int D, int count, const u32 *values, const u32 *x, u32 *out) {
    int d = count - 1;
    u32 acc[MAXD]; ezero(D, acc);
    for (int i = 0; i <= d; i++) {
        u32 num[MAXD], t[MAXD]; ecopy(D, values + D * i, num);
        u32 w = 1;
        for (int j = 0; j <= d; j++) {
            if (j == i) continue;
            u32 xm[MAXD], jj[MAXD]; ezero(D, jj); jj[0] = (u32)j; esub(D, x, jj, xm);
            emul(D, num, xm, t); ecopy(D, t, num);
            w = fmul(w, modp_i64((long long)i - j));
        }
        escale(D, num, fpow(w, P - 2), t);
        eadd(D, acc, t, acc);
    }
    ecopy(D, acc, out);
}

/* fold-table / mle-eval, src/field.lisp:365-379 */
void orc_mle_eval(int D, int k, const u32 *values, int stride, const u32 *r, u32 *out) {
    size_t size = (size_t)1 << k;
    u32 *t = calloc(size * D, 4);
    for (size_t i = 0; i < size; i++) for (int c = 0; c < stride; c++) t[D * i + c] = values[stride * i + c] % P;
    for (int b = 0; b < k; b++) {
        size /= 2;
        for (size_t i = 0; i < size; i++) {
            u32 s[MAXD], m[MAXD];
            esub(D, t + D * (2 * i + 1), t + D * (2 * i), s); emul(D, r + D * b, s, m); eadd(D, t + D * (2 * i), m, m);
            ecopy(D, m, t + D * i);
        }
    }
    ecopy(D, t, out); free(t);
}

/* ------------------------------------------------------------------ BLAKE3 compression and B3S
   src/blake3.lisp:44-88 (compress), :99-155 (sequential mode). */

static const u32 IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au, 0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
static const int PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
static inline u32 rotr(u32 x, int n) { return (x >> n) | (x << (32 - n)); }
#define G(a, b, c, d, x, y) do { v[a] += v[b] + (x); v[d] = rotr(v[d] ^ v[a], 16); v[c] += v[d]; v[b] = rotr(v[b] ^ v[c], 12); \
                                 v[a] += v[b] + (y); v[d] = rotr(v[d] ^ v[a], 8);  v[c] += v[d]; v[b] = rotr(v[b] ^ v[c], 7); } while (0)
static void compress(const u32 cv[8], const u32 block[16], u64 counter, u32 blen, u32 flags, u32 out[16]) {
    u32 v[16], m[16], t[16];
    memcpy(v, cv, 32); memcpy(v + 8, IV, 16);
    v[12] = (u32)counter; v[13] = (u32)(counter >> 32); v[14] = blen; v[15] = flags;
    memcpy(m, block, 64);
    for (int r = 0; r < 7; r++) {
        G(0, 4, 8, 12, m[0], m[1]); G(1, 5, 9, 13, m[2], m[3]); G(2, 6, 10, 14, m[4], m[5]); G(3, 7, 11, 15, m[6], m[7]);
        G(0, 5, 10, 15, m[8], m[9]); G(1, 6, 11, 12, m[10], m[11]); G(2, 7, 8, 13, m[12], m[13]); G(3, 4, 9, 14, m[14], m[15]);
        for (int i = 0; i < 16; i++) t[i] = m[PERM[i]];
        memcpy(m, t, 64);
    }
    for (int i = 0; i < 8; i++) { out[i] = v[i] ^ v[i + 8]; out[i + 8] = v[i + 8] ^ cv[i]; }
}

typedef struct { u32 cv[8]; u8 block[64]; int used; u64 counter; } b3s;

static void b3s_init(b3s *s) { memcpy(s->cv, IV, 32); memset(s->block, 0, 64); s->used = 0; s->counter = 0; }
static void load_words(const u8 *b, u32 w[16]) { for (int i = 0; i < 16; i++) w[i] = (u32)b[4 * i] | (u32)b[4 * i + 1] << 8 | (u32)b[4 * i + 2] << 16 | (u32)b[4 * i + 3] << 24; }
static void b3s_update(b3s *s, const u8 *data, size_t len) {
    size_t i = 0;
    while (i < len) {
        if (s->used == 64) { /* a full block is compressed only when more input arrives */
            u32 w[16], o[16]; load_words(s->block, w);
            compress(s->cv, w, s->counter, 64, 0, o); memcpy(s->cv, o, 32);
            s->counter++; memset(s->block, 0, 64); s->used = 0;
        }
        size_t n = len - i; if (n > (size_t)(64 - s->used)) n = 64 - s->used;
        memcpy(s->block + s->used, data + i, n); s->used += (int)n; i += n;
    }
}
static void b3s_digest(const b3s *s, u8 *out, size_t n) {
    u32 w[16], o[16]; load_words(s->block, w);
    size_t got = 0; u64 c = 0;
    while (got < n) {
        compress(s->cv, w, c++, (u32)s->used, 2 | 8, o); /* CHUNK_END | ROOT */
        for (int i = 0; i < 64 && got < n; i++, got++) out[got] = (u8)(o[i / 4] >> (8 * (i % 4)));
    }
}

/* ------------------------------------------------------------------ transcript, src/transcript.lisp */

typedef struct { int rank; u64 dims[2]; u32 *values; size_t count; } message;
typedef struct orc_tr {
    int D; b3s st;
    message *msgs; int nmsgs, cap;
    u64 sent_bytes;
} orc_tr;

static const char DOMAIN[] = "LLM-SUMCHECK-v6-O|"; /* src/transcript.lisp:24 */

orc_tr *orc_tr_new(const u8 *label, int len, int D) {
    orc_tr *t = calloc(1, sizeof *t);
    t->D = D; b3s_init(&t->st);
    b3s_update(&t->st, (const u8 *)DOMAIN, strlen(DOMAIN));
    b3s_update(&t->st, label, (size_t)len);
    return t;
}
void orc_tr_free(orc_tr *t) { if (!t) return; for (int i = 0; i < t->nmsgs; i++) free(t->msgs[i].values); free(t->msgs); free(t); }
/* absorb: u64 LE length, then the bytes (:95-100) */
void orc_tr_absorb(orc_tr *t, const u8 *data, u64 len) {
    u8 l[8]; for (int i = 0; i < 8; i++) l[i] = (u8)(len >> (8 * i));
    b3s_update(&t->st, l, 8); b3s_update(&t->st, data, (size_t)len);
}
/* send a field array of shape (rows, cols): record it, absorb its values as u32 LE (:116-135) */
void orc_tr_send(orc_tr *t, const u32 *values, int rows, int cols) {
    if (t->nmsgs == t->cap) { t->cap = t->cap ? 2 * t->cap : 16; t->msgs = realloc(t->msgs, t->cap * sizeof(message)); }
    message *m = &t->msgs[t->nmsgs++];
    m->rank = 2; m->dims[0] = (u64)rows; m->dims[1] = (u64)cols; m->count = (size_t)rows * cols;
    m->values = malloc(4 * m->count + 4); memcpy(m->values, values, 4 * m->count);
    u8 *bytes = malloc(4 * m->count + 4);
    for (size_t i = 0; i < m->count; i++) for (int b = 0; b < 4; b++) bytes[4 * i + b] = (u8)(values[i] >> (8 * b));
    t->sent_bytes += 4 * m->count;
    orc_tr_absorb(t, bytes, 4 * m->count); free(bytes);
}
/* squeeze n bytes; then absorb "squeeze" and the first min(32, n) of them (:152-157) */
void orc_tr_squeeze(orc_tr *t, u8 *out, size_t n) {
    b3s_digest(&t->st, out, n);
    b3s_update(&t->st, (const u8 *)"squeeze", 7);
    b3s_update(&t->st, out, n < 32 ? n : 32);
}
/* k base challenges by rejection sampling of 31-bit words (:159-172) */
void orc_tr_challenge_base(orc_tr *t, int k, u32 *out) {
    int have = 0;
    u8 *buf = malloc(4 * ((size_t)k + 4));
    while (have < k) {
        size_t n = 4 * ((size_t)(k - have) + 4);
        orc_tr_squeeze(t, buf, n);
        for (size_t i = 0; i < n; i += 4) {
            u32 w = ((u32)buf[i] | (u32)buf[i + 1] << 8 | (u32)buf[i + 2] << 16 | (u32)buf[i + 3] << 24) & 0x7FFFFFFFu;
            if (w < P && have < k) out[have++] = w;
        }
    }
    free(buf);
}
void orc_tr_challenge_bits(orc_tr *t, int nbits, int k, u64 *out) { /* :186-190 */
    u8 *buf = malloc(8 * (size_t)k);
    orc_tr_squeeze(t, buf, 8 * (size_t)k);
    for (int i = 0; i < k; i++) {
        u64 w = 0; for (int b = 0; b < 8; b++) w |= (u64)buf[8 * i + b] << (8 * b);
        out[i] = nbits >= 64 ? w : w & ((1ull << nbits) - 1);
    }
    free(buf);
}
void orc_tr_digest(const orc_tr *t, u8 *out, int n) { b3s_digest(&t->st, out, (size_t)n); }
int orc_tr_nmessages(const orc_tr *t) { return t->nmsgs; }
u64 orc_tr_sent_bytes(const orc_tr *t) { return t->sent_bytes; }
int orc_tr_message(const orc_tr *t, int i, u64 dims[2], u32 *values) {
    if (i < 0 || i >= t->nmsgs) return -1;
    dims[0] = t->msgs[i].dims[0]; dims[1] = t->msgs[i].dims[1];
    if (values) memcpy(values, t->msgs[i].values, 4 * t->msgs[i].count);
    return 0;
}

/* B3S alone, for its vectors */
void orc_b3s(const u8 *const *chunks, const u64 *lens, int nchunks, u8 *out, u64 n) {
    b3s s; b3s_init(&s);
    for (int i = 0; i < nchunks; i++) b3s_update(&s, chunks[i], (size_t)lens[i]);
    b3s_digest(&s, out, (size_t)n);
}

/* proof bytes, src/proofio.lisp:1-9,30-49: magic | u32 count | per field array: 1 | rank | u64 dims | u32 values */
u64 orc_tr_encode(const orc_tr *t, const char *magic8, u8 *out, u64 cap) {
    u64 need = 12;
    for (int i = 0; i < t->nmsgs; i++) need += 2 + 8 * (u64)t->msgs[i].rank + 4 * t->msgs[i].count;
    if (!out || cap < need) return need;
    u8 *p = out; memcpy(p, magic8, 8); p += 8;
    for (int b = 0; b < 4; b++) *p++ = (u8)((u32)t->nmsgs >> (8 * b));
    for (int i = 0; i < t->nmsgs; i++) {
        const message *m = &t->msgs[i];
        *p++ = 1; *p++ = (u8)m->rank;
        for (int r = 0; r < m->rank; r++) for (int b = 0; b < 8; b++) *p++ = (u8)(m->dims[r] >> (8 * b));
        for (size_t k = 0; k < m->count; k++) for (int b = 0; b < 4; b++) *p++ = (u8)(m->values[k] >> (8 * b));
    }
    return need;
}

/* ------------------------------------------------------------------ forms, src/forms.lisp
   A form is parsed into a tree.  EXPAND (:57-78) gives the sum of monomials used for the degree
   and the variables; the values come from the tree evaluated as written (arithmetic-form,
   :113-142), over F_p or F_p^D. */

enum { N_INT, N_VAR, N_ADD, N_SUB, N_MUL, N_EXPT };
typedef struct node { int kind; long long ival; int var; int nargs; struct node **args; } node;
typedef struct { char **names; int n; } symtab;

static int sym_intern(symtab *s, const char *name) {
    for (int i = 0; i < s->n; i++) if (!strcmp(s->names[i], name)) return i;
    s->names = realloc(s->names, (s->n + 1) * sizeof(char *));
    s->names[s->n] = strdup(name);
    return s->n++;
}
static void sym_free(symtab *s) { for (int i = 0; i < s->n; i++) free(s->names[i]); free(s->names); }
static void node_free(node *x) { if (!x) return; for (int i = 0; i < x->nargs; i++) node_free(x->args[i]); free(x->args); free(x); }

static void skip_ws(const char **s) { while (**s && isspace((unsigned char)**s)) (*s)++; }
static node *parse_form(const char **s, symtab *syms, int *err) {
    skip_ws(s);
    node *x = calloc(1, sizeof *x);
    if (**s == '(') {
        (*s)++; skip_ws(s);
        char op[16]; int k = 0;
        while (**s && !isspace((unsigned char)**s) && **s != '(' && **s != ')' && k < 15) op[k++] = (char)tolower((unsigned char)*(*s)++);
        op[k] = 0;
        if (!strcmp(op, "+")) x->kind = N_ADD; else if (!strcmp(op, "-")) x->kind = N_SUB;
        else if (!strcmp(op, "*")) x->kind = N_MUL; else if (!strcmp(op, "expt")) x->kind = N_EXPT;
        else { *err = 1; return x; }
        for (;;) {
            skip_ws(s);
            if (**s == ')') { (*s)++; break; }
            if (!**s) { *err = 1; return x; }
            x->args = realloc(x->args, (x->nargs + 1) * sizeof(node *));
            x->args[x->nargs++] = parse_form(s, syms, err);
            if (*err) return x;
        }
        if (x->kind == N_EXPT && (x->nargs != 2 || x->args[1]->kind != N_INT || x->args[1]->ival < 0)) *err = 1;
        if (x->kind == N_SUB && x->nargs == 0) *err = 1;
        return x;
    }
    char tok[128]; int k = 0;
    while (**s && !isspace((unsigned char)**s) && **s != '(' && **s != ')' && k < 127) tok[k++] = (char)tolower((unsigned char)*(*s)++);
    tok[k] = 0;
    if (!k) { *err = 1; return x; }
    char *end; long long v = strtoll(tok, &end, 10);
    if (*end == 0) { x->kind = N_INT; x->ival = v; }
    else { x->kind = N_VAR; x->var = sym_intern(syms, tok); }
    return x;
}

/* polynomials: sorted, merged lists of monomials (forms.lisp:28-55) */
#define MAXDEG 24
typedef struct { int deg; int vars[MAXDEG]; u32 c; } mono;
typedef struct { mono *m; int n; } poly;
static const symtab *g_cmp_syms;
static int var_lt(int a, int b) { return strcmp(g_cmp_syms->names[a], g_cmp_syms->names[b]); }
static int mono_cmp(const void *pa, const void *pb) {
    const mono *a = pa, *b = pb;
    if (a->deg != b->deg) return a->deg - b->deg;
    for (int i = 0; i < a->deg; i++) { int c = var_lt(a->vars[i], b->vars[i]); if (c) return c; }
    return 0;
}
static void poly_collect(poly *p) {
    qsort(p->m, p->n, sizeof(mono), mono_cmp);
    int o = 0;
    for (int i = 0; i < p->n; i++) {
        if (o && mono_cmp(&p->m[o - 1], &p->m[i]) == 0) p->m[o - 1].c = fadd(p->m[o - 1].c, p->m[i].c);
        else p->m[o++] = p->m[i];
    }
    int k = 0;
    for (int i = 0; i < o; i++) if (p->m[i].c) p->m[k++] = p->m[i];
    p->n = k;
}
static poly poly_const(u32 c) { poly p; p.m = malloc(sizeof(mono)); p.n = 1; p.m[0].deg = 0; p.m[0].c = c; poly_collect(&p); return p; }
static poly poly_mul(const poly *a, const poly *b, int *err) {
    poly p; p.n = 0; p.m = malloc(sizeof(mono) * (size_t)(a->n * b->n + 1));
    for (int i = 0; i < a->n; i++) for (int j = 0; j < b->n; j++) {
        mono *m = &p.m[p.n++];
        m->deg = a->m[i].deg + b->m[j].deg;
        if (m->deg > MAXDEG) { *err = 1; p.n--; continue; }
        int x = 0, y = 0, k = 0; /* merge the sorted variable lists */
        while (x < a->m[i].deg || y < b->m[j].deg) {
            if (y >= b->m[j].deg || (x < a->m[i].deg && var_lt(a->m[i].vars[x], b->m[j].vars[y]) <= 0)) m->vars[k++] = a->m[i].vars[x++];
            else m->vars[k++] = b->m[j].vars[y++];
        }
        m->c = fmul(a->m[i].c, b->m[j].c);
    }
    poly_collect(&p);
    return p;
}
static poly expand(const node *x, int *err) {
    poly p; p.m = NULL; p.n = 0;
    switch (x->kind) {
    case N_INT: return poly_const(modp_i64(x->ival));
    case N_VAR: p.m = malloc(sizeof(mono)); p.n = 1; p.m[0].deg = 1; p.m[0].vars[0] = x->var; p.m[0].c = 1; return p;
    case N_ADD: case N_SUB: {
        for (int i = 0; i < x->nargs; i++) {
            poly q = expand(x->args[i], err);
            int negate = x->kind == N_SUB && (i > 0 || x->nargs == 1);
            p.m = realloc(p.m, sizeof(mono) * (size_t)(p.n + q.n + 1));
            for (int k = 0; k < q.n; k++) { p.m[p.n] = q.m[k]; if (negate) p.m[p.n].c = fsub(0, q.m[k].c); p.n++; }
            free(q.m);
        }
        if (!p.m) p.m = malloc(sizeof(mono));
        poly_collect(&p); return p;
    }
    case N_MUL: {
        p = poly_const(1);
        for (int i = 0; i < x->nargs; i++) { poly q = expand(x->args[i], err); poly r = poly_mul(&p, &q, err); free(p.m); free(q.m); p = r; }
        return p;
    }
    case N_EXPT: {
        p = poly_const(1);
        poly q = expand(x->args[0], err);
        for (long long i = 0; i < x->args[1]->ival; i++) { poly r = poly_mul(&p, &q, err); free(p.m); p = r; }
        free(q.m); return p;
    }
    }
    *err = 1; return p;
}

/* evaluation as written: over F_p^D (values: D words per variable) */
static void eval_ext(const node *x, int D, const u32 *const *vals, u32 *out) {
    u32 a[MAXD], b[MAXD];
    switch (x->kind) {
    case N_INT: ezero(D, out); out[0] = modp_i64(x->ival); return;
    case N_VAR: ecopy(D, vals[x->var], out); return;
    case N_ADD: ezero(D, a); for (int i = 0; i < x->nargs; i++) { eval_ext(x->args[i], D, vals, b); if (i) eadd(D, a, b, a); else ecopy(D, b, a); } ecopy(D, a, out); return;
    case N_MUL: eone(D, a); for (int i = 0; i < x->nargs; i++) { eval_ext(x->args[i], D, vals, b); if (i) { u32 t[MAXD]; emul(D, a, b, t); ecopy(D, t, a); } else ecopy(D, b, a); } ecopy(D, a, out); return;
    case N_SUB:
        eval_ext(x->args[0], D, vals, a);
        if (x->nargs == 1) { ezero(D, b); esub(D, b, a, out); return; }
        for (int i = 1; i < x->nargs; i++) { eval_ext(x->args[i], D, vals, b); esub(D, a, b, a); }
        ecopy(D, a, out); return;
    case N_EXPT: {
        eval_ext(x->args[0], D, vals, b); eone(D, a);
        for (long long i = 0; i < x->args[1]->ival; i++) { u32 t[MAXD]; emul(D, a, b, t); ecopy(D, t, a); }
        ecopy(D, a, out); return;
    }
    }
}
/* and over F_p */
static u32 eval_base(const node *x, const u32 *vals) {
    u32 a;
    switch (x->kind) {
    case N_INT: return modp_i64(x->ival);
    case N_VAR: return vals[x->var];
    case N_ADD: a = 0; for (int i = 0; i < x->nargs; i++) a = fadd(a, eval_base(x->args[i], vals)); return a;
    case N_MUL: a = 1; for (int i = 0; i < x->nargs; i++) a = fmul(a, eval_base(x->args[i], vals)); return a;
    case N_SUB:
        a = eval_base(x->args[0], vals);
        if (x->nargs == 1) return fsub(0, a);
        for (int i = 1; i < x->nargs; i++) a = fsub(a, eval_base(x->args[i], vals));
        return a;
    case N_EXPT: return fpow(eval_base(x->args[0], vals), (u64)x->args[1]->ival);
    }
    return 0;
}

/* A parsed statement with its variables resolved against tables and constants. */
typedef struct {
    node *root; symtab syms;
    int nt, nc;
    int *slot_of_var; /* symbol index -> table slot t (0..nt-1) or nt + constant index, or -1 */
    int degree;       /* in the tables, forms.lisp:101-106 with sumcheck.lisp:29-35 */
} statement;

static int stmt_parse(statement *st, const char *text, int nt, const char *const *tnames, int nc, const char *const *cnames) {
    memset(st, 0, sizeof *st);
    int err = 0; const char *s = text;
    st->root = parse_form(&s, &st->syms, &err);
    skip_ws(&s);
    if (err || *s) return -1;
    st->nt = nt; st->nc = nc;
    st->slot_of_var = malloc(sizeof(int) * (size_t)(st->syms.n + 1));
    char low[128];
    for (int v = 0; v < st->syms.n; v++) {
        st->slot_of_var[v] = -1;
        for (int t = 0; t < nt; t++) { int k = 0; for (; tnames[t][k] && k < 127; k++) low[k] = (char)tolower((unsigned char)tnames[t][k]); low[k] = 0; if (!strcmp(low, st->syms.names[v])) st->slot_of_var[v] = t; }
        for (int c = 0; c < nc; c++) { int k = 0; for (; cnames[c][k] && k < 127; k++) low[k] = (char)tolower((unsigned char)cnames[c][k]); low[k] = 0; if (!strcmp(low, st->syms.names[v])) st->slot_of_var[v] = nt + c; }
    }
    g_cmp_syms = &st->syms;
    poly p = expand(st->root, &err);
    if (err) { free(p.m); return -1; }
    /* every variable that survives the expansion must be a table or a constant */
    st->degree = 0;
    for (int i = 0; i < p.n; i++) {
        int d = 0;
        for (int k = 0; k < p.m[i].deg; k++) {
            int slot = st->slot_of_var[p.m[i].vars[k]];
            if (slot < 0) { free(p.m); return -2; }
            if (slot < nt) d++;
        }
        if (d > st->degree) st->degree = d;
    }
    free(p.m);
    /* variables that are written but cancel out must still be bound to evaluate the tree */
    for (int v = 0; v < st->syms.n; v++) if (st->slot_of_var[v] < 0) return -2;
    return 0;
}
static void stmt_free(statement *st) { node_free(st->root); sym_free(&st->syms); free(st->slot_of_var); }

/* EXPAND for its vector: terms as (variable-index list, coefficient), graded order.  VARS names
   the variables; the indices written are positions in VARS. */
int orc_expand(const char *text, int nvars, const char *const *vars, int cap, int *degs, int *idx /* cap*MAXDEG */, u32 *coeffs) {
    statement st;
    if (stmt_parse(&st, text, nvars, vars, 0, NULL)) return -1;
    int err = 0; g_cmp_syms = &st.syms;
    poly p = expand(st.root, &err);
    int n = p.n <= cap ? p.n : -1;
    for (int i = 0; i < p.n && n >= 0; i++) {
        degs[i] = p.m[i].deg; coeffs[i] = p.m[i].c;
        for (int k = 0; k < p.m[i].deg; k++) idx[MAXDEG * i + k] = st.slot_of_var[p.m[i].vars[k]];
    }
    free(p.m); stmt_free(&st);
    return n;
}
int orc_statement_degree(const char *text, int nt, const char *const *tnames, int nc, const char *const *cnames) {
    statement st; int r = stmt_parse(&st, text, nt, tnames, nc, cnames);
    int d = r ? r : st.degree; stmt_free(&st); return d;
}

/* ------------------------------------------------------------------ sumcheck, src/sumcheck.lisp */

static int n_threads(int threads) {
#ifdef _OPENMP
    return threads > 0 ? threads : omp_get_max_threads();
#else
    (void)threads; return 1;
#endif
}
int orc_max_threads(void) { return n_threads(0); }

/* header: label | "|" | n u16 | degree u16 | blocks u32 (:24-27) */
static size_t make_header(const char *label, int n, int degree, u32 blocks, u8 *out) {
    size_t l = strlen(label); memcpy(out, label, l); out[l++] = '|';
    out[l++] = (u8)n; out[l++] = (u8)(n >> 8); out[l++] = (u8)degree; out[l++] = (u8)(degree >> 8);
    for (int b = 0; b < 4; b++) out[l++] = (u8)(blocks >> (8 * b));
    return l;
}

/* weights over the variables from..to-1 (:37-41): eq-table of r[from..to), or ones */
static u32 *weights(int D, const u32 *eq, int from, int to) {
    size_t size = (size_t)1 << (to - from);
    u32 *w = malloc(4 * D * size);
    if (eq) orc_eq_table(D, to - from, eq + D * from, w);
    else for (size_t i = 0; i < size; i++) eone(D, w + D * i);
    return w;
}

typedef struct { int stride; u32 *e; size_t size; } table;

/* table-entry (:75-82): an entry as an extension element */
static inline void entry(const table *t, int D, size_t x, u32 *out) {
    if (t->stride == 1) { ezero(D, out); out[0] = t->e[x]; }
    else ecopy(D, t->e + D * x, out);
}

/* fold-flat-table (:84-104) */
static void fold_table(table *t, int D, const u32 *r, int threads) {
    size_t half = t->size / 2;
    u32 *f = malloc(4 * D * (half ? half : 1));
    int base = t->stride == 1;
#pragma omp parallel for num_threads(threads) schedule(static) if (half > 4096)
    for (size_t i = 0; i < half; i++) {
        u32 term[MAXD];
        if (base) {
            u32 lo = t->e[2 * i];
            escale(D, r, fsub(t->e[2 * i + 1], lo), term);
            term[0] = fadd(term[0], lo);
        } else {
            u32 s[MAXD];
            esub(D, t->e + D * (2 * i + 1), t->e + D * (2 * i), s);
            emul(D, r, s, term);
            eadd(D, t->e + D * (2 * i), term, term);
        }
        ecopy(D, term, f + D * i);
    }
    free(t->e); t->e = f; t->size = half; t->stride = D;
}

/* One round (:190-258 and :282-311): sums at X = 0, 2, .., points over the pairs, weight of pair
   i = h |LOW| + l being LOW[l] HIGH[h].  With BASE (all tables in the base field, no constants)
   the statement runs over F_p and each term costs one base-times-extension product. */
static void round_sums(const statement *st, int D, int points, const table *tabs, const u32 *cvals,
                       const u32 *low, size_t nlow, const u32 *high, size_t nhigh, int base, int threads, u32 *sums /* points*D */) {
    int nt = st->nt, nv = st->syms.n;
    memset(sums, 0, 4 * (size_t)points * D);
#pragma omp parallel num_threads(threads) if (nhigh * nlow > 2048)
    {
        u32 mysum[4 * 16 * MAXD]; /* points <= 16 */
        u32 *local = mysum;
        memset(local, 0, 4 * (size_t)points * D);
        u32 *lines = malloc(4 * (size_t)nt * (points + 1) * D + 64);
        u32 *inner = malloc(4 * (size_t)points * D);
        const u32 **vals = malloc(sizeof(u32 *) * (size_t)(nv + 1));
        u32 *bvals = malloc(4 * (size_t)(nv + 1));
#pragma omp for schedule(static)
        for (size_t h = 0; h < nhigh; h++) {
            memset(inner, 0, 4 * (size_t)points * D);
            for (size_t l = 0; l < nlow; l++) {
                size_t i = h * nlow + l;
                const u32 *w = low + D * l;
                u32 f[MAXD], term[MAXD];
                if (base) {
                    u32 *bl = lines; /* nt x (points+1) base line values */
                    for (int t = 0; t < nt; t++) {
                        u32 lo = tabs[t].e[2 * i], hi = tabs[t].e[2 * i + 1], s = fsub(hi, lo);
                        u32 *ln = bl + t * (points + 1);
                        ln[0] = lo; ln[1] = hi;
                        for (int x = 2; x <= points; x++) ln[x] = fadd(ln[x - 1], s);
                    }
                    for (int xi = 0; xi < points; xi++) {
                        int x = xi ? xi + 1 : 0;
                        for (int v = 0; v < nv; v++) bvals[v] = bl[st->slot_of_var[v] * (points + 1) + x];
                        escale(D, w, eval_base(st->root, bvals), term);
                        eadd(D, inner + D * xi, term, inner + D * xi);
                    }
                } else {
                    for (int t = 0; t < nt; t++) {
                        u32 *ln = lines + (size_t)t * (points + 1) * D, s[MAXD];
                        entry(&tabs[t], D, 2 * i, ln); entry(&tabs[t], D, 2 * i + 1, ln + D);
                        esub(D, ln + D, ln, s);
                        for (int x = 2; x <= points; x++) eadd(D, ln + D * (x - 1), s, ln + D * x);
                    }
                    for (int xi = 0; xi < points; xi++) {
                        int x = xi ? xi + 1 : 0;
                        for (int v = 0; v < nv; v++) {
                            int slot = st->slot_of_var[v];
                            vals[v] = slot < nt ? lines + ((size_t)slot * (points + 1) + x) * D : cvals + D * (slot - nt);
                        }
                        eval_ext(st->root, D, vals, f);
                        emul(D, w, f, term);
                        eadd(D, inner + D * xi, term, inner + D * xi);
                    }
                }
            }
            for (int xi = 0; xi < points; xi++) {
                u32 term[MAXD];
                emul(D, high + D * h, inner + D * xi, term);
                eadd(D, local + D * xi, term, local + D * xi);
            }
        }
#pragma omp critical
        for (int k = 0; k < points * D; k++) sums[k] = fadd(sums[k], local[k]);
        free(lines); free(inner); free(vals); free(bvals);
    }
}

/*
 * prove (:512-571).  Tables: K 2^n entries each (K = 1 without block weights), stride 1 (base) or
 * D.  eq: n EXTs or NULL.  K = 0 means no block weights.  degree < 0 means the statement's degree.
 * Outputs: challenges n*D, finals ntables*D, folded ntables*max(K,1)*D (any may be NULL).
 * Returns 0, or a negative error.
 */
int orc_prove(orc_tr *tr, int n, const char *statement_text,
              int nt, const char *const *tnames, const u32 *const *tdata, const int *strides,
              const u32 *eq, int nc, const char *const *cnames, const u32 *cvals,
              const char *label, int K, const u32 *bw, int degree, int threads,
              u32 *challenges, u32 *finals, u32 *folded) {
    int D = tr->D;
    statement st;
    int rc = stmt_parse(&st, statement_text, nt, tnames, nc, cnames);
    if (rc) { stmt_free(&st); return rc; }
    if (degree < 0) degree = st.degree;
    int points = degree > 1 ? degree : 1;
    if (points > 16) { stmt_free(&st); return -3; }
    int blocks = K > 0 ? K : 1;
    threads = n_threads(threads);
    table *tabs = calloc((size_t)nt + 1, sizeof(table));
    for (int t = 0; t < nt; t++) {
        tabs[t].stride = strides[t]; tabs[t].size = (size_t)blocks << n;
        size_t words = tabs[t].size * (size_t)strides[t];
        tabs[t].e = malloc(4 * words + 4);
        for (size_t i = 0; i < words; i++) tabs[t].e[i] = tdata[t][i] % P; /* coerce-ext reduces, field.lisp:115-117 */
    }
    u8 hdr[300]; size_t hl = make_header(label, n, degree, (u32)blocks, hdr);
    orc_tr_absorb(tr, hdr, hl);
    u32 *sums = malloc(4 * (size_t)points * D);
    for (int j = 0; j < n; j++) {
        u32 *low, *high; size_t nlow, nhigh;
        if (K > 0) { /* :549-550 */
            low = weights(D, eq, j + 1, n); nlow = (size_t)1 << (n - j - 1);
            high = malloc(4 * (size_t)D * K); memcpy(high, bw, 4 * (size_t)D * K); nhigh = (size_t)K;
        } else { /* split-weights, :43-49 */
            int middle = (j + 1) + (n - (j + 1)) / 2;
            low = weights(D, eq, j + 1, middle); nlow = (size_t)1 << (middle - j - 1);
            high = weights(D, eq, middle, n); nhigh = (size_t)1 << (n - middle);
        }
        int base = nc == 0;
        for (int t = 0; t < nt; t++) base = base && tabs[t].stride == 1;
        round_sums(&st, D, points, tabs, cvals, low, nlow, high, nhigh, base, threads, sums);
        free(low); free(high);
        orc_tr_send(tr, sums, points, D);
        u32 r[MAXD]; orc_tr_challenge_base(tr, D, r);
        if (challenges) ecopy(D, r, challenges + D * j);
        for (int t = 0; t < nt; t++) fold_table(&tabs[t], D, r, threads);
    }
    for (int t = 0; t < nt; t++) {
        u32 e[MAXD];
        entry(&tabs[t], D, 0, e);
        if (finals) ecopy(D, e, finals + D * t);
        for (int b = 0; b < blocks; b++) { entry(&tabs[t], D, (size_t)b, e); if (folded) ecopy(D, e, folded + ((size_t)t * blocks + b) * D); }
        free(tabs[t].e);
    }
    free(tabs); free(sums); stmt_free(&st);
    return 0;
}

/* hypercube-sum (:112-127): the honest claim */
int orc_hypercube_sum(int D, int n, const char *statement_text, int nt, const char *const *tnames, const u32 *const *tdata,
                      const int *strides, const u32 *eq, int nc, const char *const *cnames, const u32 *cvals, u32 *out) {
    statement st; int rc = stmt_parse(&st, statement_text, nt, tnames, nc, cnames);
    if (rc) { stmt_free(&st); return rc; }
    u32 *w = weights(D, eq, 0, n);
    u32 *buf = malloc(4 * (size_t)(nt + 1) * D);
    const u32 **vals = malloc(sizeof(u32 *) * (size_t)(st.syms.n + 1));
    u32 sum[MAXD]; ezero(D, sum);
    for (size_t x = 0; x < ((size_t)1 << n); x++) {
        for (int t = 0; t < nt; t++) { ezero(D, buf + D * t); for (int c = 0; c < strides[t]; c++) buf[D * t + c] = tdata[t][strides[t] * x + c] % P; }
        for (int v = 0; v < st.syms.n; v++) { int s = st.slot_of_var[v]; vals[v] = s < nt ? buf + D * s : cvals + D * (s - nt); }
        u32 f[MAXD], term[MAXD]; eval_ext(st.root, D, vals, f); emul(D, w + D * x, f, term); eadd(D, sum, term, sum);
    }
    ecopy(D, sum, out); free(w); free(buf); free(vals); stmt_free(&st);
    return 0;
}

/* verify (:147-163) with next-claim (:137-145).  messages: n arrays (points, D), row-major, one
   after the other.  Returns 0 and writes the challenges (n*D) and the reduced claim (D). */
static int verify_on(orc_tr *tr, int D, int n, int degree, const u32 *claim_in, const u32 *eq,
                     int blocks, const char *label, const u32 *messages, u32 *challenges, u32 *reduced);
int orc_verify(const u8 *tr_label, int tr_label_len, int D, int n, int degree, const u32 *claim_in, const u32 *eq,
               int blocks, const char *label, const u32 *messages, u32 *challenges, u32 *reduced) {
    orc_tr *tr = orc_tr_new(tr_label, tr_label_len, D);
    int rc = verify_on(tr, D, n, degree, claim_in, eq, blocks, label, messages, challenges, reduced);
    orc_tr_free(tr);
    return rc;
}
/* the same on a transcript that already holds earlier messages (a caller's protocol around the sumcheck) */
int orc_verify_tr(orc_tr *tr, int n, int degree, const u32 *claim_in, const u32 *eq, int blocks, const char *label,
                  const u32 *messages, u32 *challenges, u32 *reduced) {
    return verify_on(tr, tr->D, n, degree, claim_in, eq, blocks, label, messages, challenges, reduced);
}
static int verify_on(orc_tr *tr, int D, int n, int degree, const u32 *claim_in, const u32 *eq,
                     int blocks, const char *label, const u32 *messages, u32 *challenges, u32 *reduced) {
    int points = degree > 1 ? degree : 1;
    u8 hdr[300]; size_t hl = make_header(label, n, degree, (u32)blocks, hdr);
    orc_tr_absorb(tr, hdr, hl);
    u32 claim[MAXD]; for (int c = 0; c < D; c++) claim[c] = claim_in[c] % P;
    for (int j = 0; j < n; j++) {
        const u32 *m = messages + (size_t)j * points * D;
        orc_tr_send(tr, m, points, D);
        u32 r[MAXD]; orc_tr_challenge_base(tr, D, r);
        u32 vals[(16 + 1) * MAXD], g1[MAXD];
        if (eq) { /* claim = (1 - r) g(0) + r g(1) */
            u32 one[MAXD], a[MAXD], b[MAXD], inv[MAXD];
            eone(D, one); esub(D, one, eq + D * j, a); emul(D, a, m, b); esub(D, claim, b, a);
            orc_ext_inv(D, eq + D * j, inv); emul(D, a, inv, g1);
        } else esub(D, claim, m, g1);
        ecopy(D, m, vals); ecopy(D, g1, vals + D);
        for (int x = 2; x <= points; x++) ecopy(D, m + D * (x - 1), vals + D * x);
        orc_lagrange(D, points + 1, vals, r, claim);
        ecopy(D, r, challenges + D * j);
    }
    ecopy(D, claim, reduced);
    return 0;
}

/* check-final (:165-172): the statement at the finals must be the reduced claim.  Returns 1/0. */
int orc_check_final(int D, const char *statement_text, int nt, const char *const *tnames, const u32 *finals,
                    int nc, const char *const *cnames, const u32 *cvals, const u32 *reduced) {
    statement st; int rc = stmt_parse(&st, statement_text, nt, tnames, nc, cnames);
    if (rc) { stmt_free(&st); return rc; }
    const u32 **vals = malloc(sizeof(u32 *) * (size_t)(st.syms.n + 1));
    for (int v = 0; v < st.syms.n; v++) { int s = st.slot_of_var[v]; vals[v] = s < nt ? finals + D * s : cvals + D * (s - nt); }
    u32 f[MAXD]; eval_ext(st.root, D, vals, f);
    int ok = memcmp(f, reduced, 4 * (size_t)D) == 0;
    free(vals); stmt_free(&st);
    return ok;
}

/* evaluate (src/forms.lisp:214-217): the statement's value at the given tables' and constants' values */
int orc_evaluate(int D, const char *statement_text, int nt, const char *const *tnames, const u32 *tvals,
                 int nc, const char *const *cnames, const u32 *cvals, u32 *out) {
    statement st; int rc = stmt_parse(&st, statement_text, nt, tnames, nc, cnames);
    if (rc) { stmt_free(&st); return rc; }
    const u32 **vals = malloc(sizeof(u32 *) * (size_t)(st.syms.n + 1));
    for (int v = 0; v < st.syms.n; v++) { int s = st.slot_of_var[v]; vals[v] = s < nt ? tvals + D * s : cvals + D * (s - nt); }
    eval_ext(st.root, D, vals, out);
    free(vals); stmt_free(&st);
    return 0;
}

/* One layer of a fraction tree (FRACTION-TREES, src/gkr.lisp:149-188): p/q = p0/q0 + p1/q1 entry
   by entry, so p = p0 q1 + p1 q0 and q = q0 q1.  COUNT entries of D words in each array. */
void orc_fraction_layer(int D, u64 count, const u32 *p0, const u32 *p1, const u32 *q0, const u32 *q1, u32 *p, u32 *q) {
#pragma omp parallel for schedule(static) if (count > 4096)
    for (u64 i = 0; i < count; i++) {
        u32 a[MAXD], b[MAXD];
        emul(D, p0 + D * i, q1 + D * i, a); emul(D, p1 + D * i, q0 + D * i, b);
        eadd(D, a, b, p + D * i);
        emul(D, q0 + D * i, q1 + D * i, a); ecopy(D, a, q + D * i);
    }
}

/* The seeded table generator shared with the device (splitmix64 of seed, table, coordinate and
   index, reduced mod p).  Not from the reference: it stands in for real inputs in benchmarks. */
static inline u64 splitmix64(u64 x) {
    x += 0x9E3779B97F4A7C15ull; x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull; x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
void orc_generate(u64 seed, int table_id, u64 first, u64 count, int stride, int nonzero, u32 *out) {
#pragma omp parallel for schedule(static) if (count > 65536)
    for (u64 i = 0; i < count; i++) {
        int all0 = 1;
        for (int c = 0; c < stride; c++) {
            u32 v = (u32)(splitmix64(seed ^ ((u64)table_id << 56) ^ ((u64)c << 48) ^ (first + i)) % P);
            out[i * stride + c] = v; all0 &= v == 0;
        }
        if (nonzero && all0) out[i * stride] = 1;
    }
}
