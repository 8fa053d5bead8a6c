// host.cpp -- part 2 of the C ABI: the host side of the prover for callers without a Lisp.
// It mirrors the reference's own host code for this path: forms as data (src/forms.lisp:28-106),
// the sequential BLAKE3 (src/blake3.lisp:44-155), the Fiat-Shamir transcript
// (src/transcript.lisp:24,95-176), the proof bytes (src/proofio.lisp:30-49) and PROVE itself
// (src/sumcheck.lisp:512-571), whose rounds run on the device through part 1 of the ABI.
#include <algorithm>
#include <cctype>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <set>
#include <memory>
#include <string>
#include <vector>

#include "../../include/sumcheck_b200.h"
#include "field.cuh"
#include "forms.h"
#include "part_workers.h"
#include "transcript.cuh"

using scf::u32;
using scf::u64;
typedef uint8_t u8;

using namespace scforms;

namespace {

// ------------------------------------------------------------------ BLAKE3 compression and the sequential mode

const u32 IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au, 0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
const u8 SIGMA[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
inline u32 ror(u32 x, int n) { return (x >> n) | (x << (32 - n)); }
inline void mix(u32 *v, int a, int b, int c, int d, u32 x, u32 y) {
    v[a] = v[a] + v[b] + x; v[d] = ror(v[d] ^ v[a], 16);
    v[c] = v[c] + v[d];     v[b] = ror(v[b] ^ v[c], 12);
    v[a] = v[a] + v[b] + y; v[d] = ror(v[d] ^ v[a], 8);
    v[c] = v[c] + v[d];     v[b] = ror(v[b] ^ v[c], 7);
}
// COMPRESS (src/blake3.lisp:44-88)
void compress(const u32 cv[8], const u32 block[16], u64 counter, u32 block_len, u32 flags, u32 out[16]) {
    u32 v[16], m[16];
    for (int i = 0; i < 8; i++) v[i] = cv[i];
    for (int i = 0; i < 4; i++) v[8 + i] = IV[i];
    v[12] = (u32)counter; v[13] = (u32)(counter >> 32); v[14] = block_len; v[15] = flags;
    for (int i = 0; i < 16; i++) m[i] = block[i];
    for (int round = 0;; round++) {
        mix(v, 0, 4, 8, 12, m[0], m[1]);  mix(v, 1, 5, 9, 13, m[2], m[3]);
        mix(v, 2, 6, 10, 14, m[4], m[5]); mix(v, 3, 7, 11, 15, m[6], m[7]);
        mix(v, 0, 5, 10, 15, m[8], m[9]); mix(v, 1, 6, 11, 12, m[10], m[11]);
        mix(v, 2, 7, 8, 13, m[12], m[13]); mix(v, 3, 4, 9, 14, m[14], m[15]);
        if (round == 6) break;
        u32 t[16];
        for (int i = 0; i < 16; i++) t[i] = m[SIGMA[i]];
        for (int i = 0; i < 16; i++) m[i] = t[i];
    }
    for (int i = 0; i < 8; i++) { out[i] = v[i] ^ v[i + 8]; out[i + 8] = v[i + 8] ^ cv[i]; }
}

// B3S (src/blake3.lisp:99-155): a chain over 64-byte blocks; the pending block is compressed
// only when more input arrives, and output comes from it with the flags CHUNK_END | ROOT.
struct B3S {
    u32 cv[8];
    u8 pending[64];
    int fill = 0;
    u64 blocks = 0;
    B3S() { memcpy(cv, IV, sizeof cv); memset(pending, 0, sizeof pending); }
    static void words(const u8 *b, u32 *w) { for (int i = 0; i < 16; i++) w[i] = (u32)b[4 * i] | (u32)b[4 * i + 1] << 8 | (u32)b[4 * i + 2] << 16 | (u32)b[4 * i + 3] << 24; }
    void update(const u8 *data, size_t len) {
        while (len) {
            if (fill == 64) {
                u32 w[16], o[16];
                words(pending, w);
                compress(cv, w, blocks++, 64, 0, o);
                memcpy(cv, o, sizeof cv);
                memset(pending, 0, sizeof pending);
                fill = 0;
            }
            const size_t take = std::min(len, (size_t)(64 - fill));
            memcpy(pending + fill, data, take);
            fill += (int)take; data += take; len -= take;
        }
    }
    void output(u8 *out, size_t n) const {
        u32 w[16], o[16];
        words(pending, w);
        u64 t = 0;
        for (size_t got = 0; got < n; t++) {
            compress(cv, w, t, (u32)fill, 2u | 8u, o);
            for (int i = 0; i < 64 && got < n; i++, got++) out[got] = (u8)(o[i >> 2] >> (8 * (i & 3)));
        }
    }
};

struct Message { u64 rows, cols; std::vector<u32> values; };

}  // namespace

// ------------------------------------------------------------------ the transcript (src/transcript.lisp)

struct sc_transcript {
    int degree;
    B3S state;
    std::vector<Message> messages;
    u64 sent_bytes = 0;
    void absorb(const u8 *data, u64 len) {   // u64 LE length, then the bytes (:95-100)
        u8 l[8];
        for (int i = 0; i < 8; i++) l[i] = (u8)(len >> (8 * i));
        state.update(l, 8);
        state.update(data, (size_t)len);
    }
    void squeeze(u8 *out, size_t n) {        // :152-157
        state.output(out, n);
        state.update((const u8 *)"squeeze", 7);
        state.update(out, std::min<size_t>(n, 32));
    }
    void challenge_base(int k, u32 *out) {   // :159-172
        int have = 0;
        std::vector<u8> buf;
        while (have < k) {
            const size_t n = 4 * ((size_t)(k - have) + 4);
            buf.resize(n);
            squeeze(buf.data(), n);
            for (size_t i = 0; i < n && have < k; i += 4) {
                const u32 w = ((u32)buf[i] | (u32)buf[i + 1] << 8 | (u32)buf[i + 2] << 16 | (u32)buf[i + 3] << 24) & 0x7FFFFFFFu;
                if (w < scf::P) out[have++] = w;
            }
        }
    }
    void send(const u32 *values, int rows, int cols) {   // record, then absorb the values as u32 LE (:116-135)
        Message m;
        m.rows = (u64)rows; m.cols = (u64)cols;
        m.values.assign(values, values + (size_t)rows * cols);
        std::vector<u8> bytes(4 * m.values.size());
        for (size_t i = 0; i < m.values.size(); i++) for (int b = 0; b < 4; b++) bytes[4 * i + b] = (u8)(m.values[i] >> (8 * b));
        sent_bytes += bytes.size();
        messages.push_back(std::move(m));
        absorb(bytes.data(), bytes.size());
    }
};

extern "C" sc_transcript *sc_transcript_new(const uint8_t *label, size_t label_len, int degree) {
    if (degree != 4 && degree != 8) return nullptr;   // CHECK-DEGREE, src/field.lisp:105-108
    sc_transcript *tr = new sc_transcript();
    tr->degree = degree;
    static const char domain[] = "LLM-SUMCHECK-v6-O|";   // *DOMAIN*, src/transcript.lisp:24
    tr->state.update((const u8 *)domain, sizeof domain - 1);
    if (label_len) tr->state.update(label, label_len);
    return tr;
}
extern "C" void sc_transcript_free(sc_transcript *tr) { delete tr; }
extern "C" int sc_transcript_degree(const sc_transcript *tr) { return tr ? tr->degree : 0; }
extern "C" int sc_transcript_state(const sc_transcript *tr, uint32_t cv[8], uint32_t pending[16], int *fill, uint64_t *blocks) {
    if (!tr || !cv || !pending || !fill || !blocks) return SC_EINVAL;
    memcpy(cv, tr->state.cv, sizeof tr->state.cv);
    B3S::words(tr->state.pending, pending);
    *fill = tr->state.fill;
    *blocks = tr->state.blocks;
    return SC_OK;
}
// The device's transcript code (transcript.cuh) run on the host from TR's present state: SEND of the ROWS x COLS
// values and CHALLENGE of TR's degree.  TR itself is not changed, so a test can make the same two steps on TR
// and compare the challenge and the state.
extern "C" int sc_transcript_device_round(const sc_transcript *tr, const uint32_t *values, int rows, int cols, uint32_t *state_out,
                                          uint32_t *challenge) {
    if (!tr || !values || rows < 1 || cols < 1 || rows * cols > SC_MAX_POINTS * 8) return SC_EINVAL;
    u32 state[sc::B3_STATE_WORDS] = {0}, pending[16];
    int fill = 0;
    uint64_t blocks = 0;
    sc_transcript_state(tr, state, pending, &fill, &blocks);
    memcpy(state + 8, pending, sizeof pending);
    state[24] = (u32)fill; state[25] = (u32)blocks; state[26] = (u32)(blocks >> 32);
    sc::TrWork work;
    sc::transcript_round(&work, state, values, rows * cols, tr->degree, state);
    if (state_out) memcpy(state_out, state, sizeof state);
    if (challenge) memcpy(challenge, work.chal, 4 * (size_t)tr->degree);
    return SC_OK;
}
extern "C" int sc_transcript_absorb(sc_transcript *tr, const uint8_t *data, uint64_t len) {
    if (!tr || (len && !data)) return SC_EINVAL;
    tr->absorb(data, len);
    return SC_OK;
}
extern "C" int sc_transcript_send(sc_transcript *tr, const uint32_t *values, int rows, int cols) {
    if (!tr || rows < 0 || cols < 0 || ((size_t)rows * cols && !values)) return SC_EINVAL;
    for (size_t i = 0; i < (size_t)rows * cols; i++) if (values[i] >= scf::P) return SC_EINVAL;
    tr->send(values, rows, cols);
    return SC_OK;
}
extern "C" int sc_transcript_challenge_base(sc_transcript *tr, int k, uint32_t *out) {
    if (!tr || k < 0 || (k && !out)) return SC_EINVAL;
    tr->challenge_base(k, out);
    return SC_OK;
}
extern "C" int sc_transcript_challenge_bits(sc_transcript *tr, int nbits, int k, uint64_t *out) {   // :186-190
    if (!tr || nbits < 1 || nbits > 64 || k < 0 || (k && !out)) return SC_EINVAL;
    std::vector<u8> buf(8 * (size_t)k);
    tr->squeeze(buf.data(), buf.size());
    for (int i = 0; i < k; i++) {
        u64 w = 0;
        for (int b = 0; b < 8; b++) w |= (u64)buf[8 * (size_t)i + b] << (8 * b);
        out[i] = nbits == 64 ? w : (w & ((1ull << nbits) - 1));
    }
    return SC_OK;
}
extern "C" int sc_transcript_digest(const sc_transcript *tr, uint8_t *out, size_t n) {
    if (!tr || (n && !out)) return SC_EINVAL;
    tr->state.output(out, n);
    return SC_OK;
}
extern "C" int sc_transcript_message_count(const sc_transcript *tr) { return tr ? (int)tr->messages.size() : 0; }
extern "C" int sc_transcript_message(const sc_transcript *tr, int index, uint64_t dims[2], uint32_t *values) {
    if (!tr || index < 0 || index >= (int)tr->messages.size()) return SC_EINVAL;
    const Message &m = tr->messages[index];
    if (dims) { dims[0] = m.rows; dims[1] = m.cols; }
    if (values && !m.values.empty()) memcpy(values, m.values.data(), 4 * m.values.size());
    return SC_OK;
}
extern "C" uint64_t sc_transcript_sent_bytes(const sc_transcript *tr) { return tr ? tr->sent_bytes : 0; }

// magic | u32 count | per field array: 1 | rank | u64 dims | u32 values  (src/proofio.lisp:1-9,30-49)
extern "C" uint64_t sc_transcript_encode(const sc_transcript *tr, const char magic[8], uint8_t *out, uint64_t cap) {
    if (!tr) return 0;
    u64 need = 12;
    for (auto &m : tr->messages) need += 2 + 16 + 4 * (u64)m.values.size();
    if (!out || cap < need) return need;
    u8 *p = out;
    memcpy(p, magic, 8); p += 8;
    const u32 count = (u32)tr->messages.size();
    for (int b = 0; b < 4; b++) *p++ = (u8)(count >> (8 * b));
    for (auto &m : tr->messages) {
        *p++ = 1; *p++ = 2;
        for (int b = 0; b < 8; b++) *p++ = (u8)(m.rows >> (8 * b));
        for (int b = 0; b < 8; b++) *p++ = (u8)(m.cols >> (8 * b));
        for (u32 v : m.values) for (int b = 0; b < 4; b++) *p++ = (u8)(v >> (8 * b));
    }
    return need;
}

// ------------------------------------------------------------------ the statement as a term table

struct LoweredTerm {
    std::vector<u32> coeff;     // D canonical words
    std::vector<int> tables;    // sorted, with multiplicity
};

// EXPAND and the lowering, without a limit on the number of terms
static int lower_terms(const char *statement, int D, int ntables, const char *const *table_names, int nconstants,
                       const char *const *constant_names, const uint32_t *constant_values, int *degree, std::vector<LoweredTerm> *out) {
    if (!statement || (D != 4 && D != 8) || ntables < 0 || nconstants < 0) return SC_EINVAL;
    Parser ps{statement};
    std::unique_ptr<Form> form = ps.form();
    ps.ws();
    if (!ps.ok || *ps.s) return SC_ESTATEMENT;
    std::map<std::string, int> table_of, constant_of;
    for (int t = 0; t < ntables; t++) table_of[lower(table_names[t])] = t;
    for (int c = 0; c < nconstants; c++) constant_of[lower(constant_names[c])] = c;
    // every variable written must be bound (COMPILE-FORM rejects free variables, src/forms.lisp:202-206)
    std::vector<std::string> vars;
    mentioned(*form, vars);
    for (auto &v : vars) if (!table_of.count(v) && !constant_of.count(v)) return SC_ESTATEMENT;

    const Poly poly = expand(*form);
    // monomials with the same tables share a term: coefficient = sum of c * product of the constants' values
    std::map<std::vector<int>, std::vector<u32>> terms;
    int deg = 0;
    for (auto &term : poly) {
        std::vector<int> tabs;
        std::vector<u32> c(D, 0);
        c[0] = term.second;
        for (auto &v : term.first) {
            auto it = table_of.find(v);
            if (it != table_of.end()) { tabs.push_back(it->second); continue; }
            ext_mul(D, c.data(), constant_values + (size_t)constant_of[v] * D, c.data());
        }
        std::sort(tabs.begin(), tabs.end());
        deg = std::max(deg, (int)tabs.size());   // FORM-DEGREE over the tables (src/forms.lisp:101-106)
        auto &slot = terms[tabs];
        if (slot.empty()) slot.assign(D, 0);
        for (int k = 0; k < D; k++) slot[k] = scf::fadd(slot[k], c[k]);
    }
    if (degree) *degree = deg;
    out->clear();
    for (auto &t : terms) {
        if (std::all_of(t.second.begin(), t.second.end(), [](u32 x) { return x == 0; })) continue;
        out->push_back(LoweredTerm{t.second, t.first});
    }
    return SC_OK;
}

// the terms as the flat arrays sc_set_statement takes; SC_EUNSUPPORTED beyond its capacities
static int flatten_terms(const std::vector<LoweredTerm> &terms, int D, int *nterms, uint32_t *coeffs, int32_t *term_ptr, int32_t *term_tables) {
    int count = 0, used = 0;
    for (auto &t : terms) {
        if (count >= SC_MAX_TERMS || (int)t.tables.size() > SC_MAX_FACTORS) return SC_EUNSUPPORTED;
        if (coeffs) memcpy(coeffs + (size_t)count * D, t.coeff.data(), 4 * (size_t)D);
        if (term_ptr) term_ptr[count] = used;
        for (int idx : t.tables) { if (term_tables) term_tables[used] = idx; used++; }
        count++;
    }
    if (term_ptr) term_ptr[count] = used;
    if (nterms) *nterms = count;
    return SC_OK;
}

extern "C" int sc_lower_statement(const char *statement, int D, int ntables, const char *const *table_names, int nconstants,
                                  const char *const *constant_names, const uint32_t *constant_values, int *degree, int *nterms,
                                  uint32_t *coeffs, int32_t *term_ptr, int32_t *term_tables) {
    std::vector<LoweredTerm> terms;
    int rc = lower_terms(statement, D, ntables, table_names, nconstants, constant_names, constant_values, degree, &terms);
    if (rc) return rc;
    return flatten_terms(terms, D, nterms, coeffs, term_ptr, term_tables);
}

// ------------------------------------------------------------------ statements wider than one kernel
//
// A round's sums are linear in the statement, so a statement with more tables or terms than one
// kernel takes is cut into parts -- groups of terms over at most four tables where that works --
// and part k runs on a context of its own (the caller's, then children of it) holding the part's
// tables; the host adds the parts' sums before it sends them.  A table that several parts use is
// uploaded to, and folded on, each of them.

static bool needs_parts(const std::vector<LoweredTerm> &terms, int ntables, int points) {
    if (ntables > SC_MAX_TABLES || (int)terms.size() > SC_MAX_TERMS) return true;
    std::set<int> used;
    for (auto &t : terms) used.insert(t.tables.begin(), t.tables.end());
    return points > 4 && used.size() > 4;   // above degree four the kernels take four tables
}

struct StatementPart {
    std::vector<int> tables;            // the part's tables (indices of the caller's), slot by slot
    std::vector<LoweredTerm> terms;     // over the part's slots
};

static int cut_into_parts(const std::vector<LoweredTerm> &terms, int ntables, std::vector<StatementPart> *parts) {
    parts->clear();
    std::set<int> current;
    std::vector<std::set<int>> sets;
    std::vector<std::vector<const LoweredTerm *>> members;
    for (auto &t : terms) {
        std::set<int> mine(t.tables.begin(), t.tables.end());
        if ((int)t.tables.size() > SC_MAX_FACTORS || mine.size() > (size_t)SC_MAX_TABLES) return SC_EUNSUPPORTED;
        // the first part this term fits: its tables joined with the part's stay within four (or within the term's own count)
        size_t at = sets.size();
        const size_t cap = std::max<size_t>(4, mine.size());
        for (size_t k = 0; k < sets.size(); k++) {
            std::set<int> joined = sets[k];
            joined.insert(mine.begin(), mine.end());
            if (joined.size() <= cap && members[k].size() < (size_t)SC_MAX_TERMS) { at = k; sets[k] = joined; break; }
        }
        if (at == sets.size()) { sets.push_back(mine); members.emplace_back(); }
        members[at].push_back(&t);
    }
    if (sets.empty()) { sets.emplace_back(); members.emplace_back(); }
    // tables outside the statement are only folded: they go where there is room
    std::set<int> placed;
    for (auto &st : sets) placed.insert(st.begin(), st.end());
    for (int t = 0; t < ntables; t++) {
        if (placed.count(t)) continue;
        size_t at = 0;
        while (at < sets.size() && sets[at].size() >= (size_t)SC_MAX_TABLES) at++;
        if (at == sets.size()) { sets.emplace_back(); members.emplace_back(); }
        sets[at].insert(t);
    }
    for (size_t k = 0; k < sets.size(); k++) {
        StatementPart pt;
        pt.tables.assign(sets[k].begin(), sets[k].end());
        std::map<int, int> slot;
        for (size_t i = 0; i < pt.tables.size(); i++) slot[pt.tables[i]] = (int)i;
        for (const LoweredTerm *t : members[k]) {
            LoweredTerm local{t->coeff, {}};
            for (int g : t->tables) local.tables.push_back(slot[g]);
            pt.terms.push_back(local);
        }
        parts->push_back(pt);
    }
    return SC_OK;
}

static int prove_in_parts(sc_ctx *ctx, sc_transcript *tr, int n, const std::vector<LoweredTerm> &lowered, int ntables,
                          const uint32_t *const *tables, const int *strides, const uint32_t *eq, const char *label, int blocks,
                          const uint32_t *block_weights, int degree, uint32_t *challenges, uint32_t *finals, uint32_t *folded) {
    const int D = tr->degree, points = std::max(degree, 1);
    int world = 1, rc;
    sc_comm_info(ctx, nullptr, &world);
    if (world > 1 || points > SC_MAX_POINTS) return SC_EUNSUPPORTED;   // parts run on one GPU
    if (!tables) return SC_EUNSUPPORTED;
    for (int t = 0; t < ntables; t++) if (!tables[t]) return SC_EUNSUPPORTED;   // a part may sit on another context: host tables only
    std::vector<StatementPart> parts;
    if ((rc = cut_into_parts(lowered, ntables, &parts))) return rc;
    std::vector<sc_ctx *> on(parts.size());
    for (size_t k = 0; k < parts.size(); k++) {
        on[k] = ctx;
        if (k && (rc = sc_child(ctx, (int)k - 1, &on[k]))) return rc;
        const StatementPart &pt = parts[k];
        int nterms = 0;
        std::vector<u32> coeffs((size_t)SC_MAX_TERMS * D);
        std::vector<int32_t> ptr(SC_MAX_TERMS + 1), idx((size_t)SC_MAX_TERMS * SC_MAX_FACTORS);
        if ((rc = flatten_terms(pt.terms, D, &nterms, coeffs.data(), ptr.data(), idx.data()))) return rc;
        if ((rc = sc_set_statement(on[k], D, points, (int)pt.tables.size(), nterms, coeffs.data(), ptr.data(), idx.data()))) return rc;
        for (size_t i = 0; i < pt.tables.size(); i++)
            if ((rc = sc_upload_table(on[k], (int)i, tables[pt.tables[i]], (u64)blocks << n, strides[pt.tables[i]]))) return rc;
        if ((rc = sc_begin(on[k], n, eq, blocks, block_weights))) return rc;
    }
    std::vector<u8> header(label, label + strlen(label));   // :24-27, :534
    header.push_back('|');
    header.push_back((u8)n); header.push_back((u8)(n >> 8));
    header.push_back((u8)degree); header.push_back((u8)(degree >> 8));
    for (int b = 0; b < 4; b++) header.push_back((u8)((u32)blocks >> (8 * b)));
    tr->absorb(header.data(), header.size());
    u32 sums[SC_MAX_POINTS * 8], r[8];
    sc::PartWorkers workers(on);   // the parts' rounds run side by side
    for (int j = 0; j < n; j++) {
        if ((rc = workers.round(sums))) return rc;
        for (size_t k = 1; k < parts.size(); k++)
            for (int w = 0; w < points * D; w++) sums[w] = scf::fadd(sums[w], workers.part(k)[w]);
        tr->send(sums, points, D);
        tr->challenge_base(D, r);
        if (challenges) memcpy(challenges + (size_t)j * D, r, 4 * (size_t)D);
        for (size_t k = 0; k < parts.size(); k++) if ((rc = sc_challenge(on[k], r))) return rc;
    }
    std::vector<bool> have((size_t)ntables, false);
    for (size_t k = 0; k < parts.size(); k++) {
        const StatementPart &pt = parts[k];
        std::vector<u32> out(pt.tables.size() * (size_t)blocks * D);
        if ((rc = sc_finish(on[k], out.data()))) return rc;
        for (size_t i = 0; i < pt.tables.size(); i++) {
            const int g = pt.tables[i];
            if (have[g]) continue;
            have[g] = true;
            if (folded) memcpy(folded + (size_t)g * blocks * D, out.data() + i * (size_t)blocks * D, 4 * (size_t)blocks * D);
            if (finals) memcpy(finals + (size_t)g * D, out.data() + i * (size_t)blocks * D, 4 * (size_t)D);
        }
    }
    return SC_OK;
}

// ------------------------------------------------------------------ PROVE (src/sumcheck.lisp:512-571)

extern "C" int sc_prove(sc_ctx *ctx, sc_transcript *tr, int n, const char *statement, int ntables,
                        const char *const *table_names, const uint32_t *const *tables, const int *strides, const uint32_t *eq,
                        int nconstants, const char *const *constant_names, const uint32_t *constant_values, const char *label,
                        int K, const uint32_t *block_weights, int degree, uint32_t *challenges, uint32_t *finals,
                        uint32_t *folded) {
    if (!ctx || !tr || !statement || n < 0 || ntables < 1 || ntables > SC_MAX_WIDE_TABLES) return SC_EINVAL;
    const int D = tr->degree;
    if (!label) label = "sc";
    const int blocks = block_weights ? K : 1;
    if (blocks < 1) return SC_EINVAL;

    int deg = 0, nterms = 0;
    std::vector<LoweredTerm> lowered;
    int rc = lower_terms(statement, D, ntables, table_names, nconstants, constant_names, constant_values, &deg, &lowered);
    if (rc) return rc;
    if (degree < 0) degree = deg;                       // :513
    const int points = std::max(degree, 1);             // :527
    if (needs_parts(lowered, ntables, points))
        return prove_in_parts(ctx, tr, n, lowered, ntables, tables, strides, eq, label, blocks, block_weights, degree, challenges, finals, folded);
    std::vector<u32> coeffs((size_t)SC_MAX_TERMS * D);
    std::vector<int32_t> ptr(SC_MAX_TERMS + 1), idx((size_t)SC_MAX_TERMS * SC_MAX_FACTORS);
    if ((rc = flatten_terms(lowered, D, &nterms, coeffs.data(), ptr.data(), idx.data()))) return rc;
    if ((rc = sc_set_statement(ctx, D, points, ntables, nterms, coeffs.data(), ptr.data(), idx.data()))) return rc;
    // with a communicator each rank passes its slice: entries [rank 2^n / world, (rank + 1) 2^n / world)
    int world = 1;
    sc_comm_info(ctx, nullptr, &world);
    if (world > 1 && (((u64)1 << n) < (u64)world)) return SC_EINVAL;
    for (int t = 0; t < ntables; t++)
        if (tables && tables[t] && (rc = sc_upload_table(ctx, t, tables[t], ((u64)blocks << n) / (u64)world, strides[t]))) return rc;
    const auto t_start = std::chrono::steady_clock::now();
    if ((rc = sc_begin(ctx, n, eq, blocks, block_weights))) return rc;
    const auto t_begun = std::chrono::steady_clock::now();
    // the last rounds may derive their challenges on the device from a copy of this transcript's state
    struct Attach { sc_ctx *c; ~Attach() { sc_attach_transcript(c, nullptr); } } attach{ctx};
    if ((rc = sc_attach_transcript(ctx, tr))) return rc;

    // header: label | "|" | n u16 | degree u16 | blocks u32 (:24-27, :534)
    std::vector<u8> header(label, label + strlen(label));
    header.push_back('|');
    header.push_back((u8)n); header.push_back((u8)(n >> 8));
    header.push_back((u8)degree); header.push_back((u8)(degree >> 8));
    for (int b = 0; b < 4; b++) header.push_back((u8)((u32)blocks >> (8 * b)));
    tr->absorb(header.data(), header.size());

    u32 sums[SC_MAX_POINTS * 8], r[8];
    const bool trace = getenv("SABLE_B200_TRACE") != nullptr;   // per-round host times on stderr
    auto now = [] { return std::chrono::steady_clock::now(); };
    auto us = [](std::chrono::steady_clock::time_point a, std::chrono::steady_clock::time_point b) {
        return std::chrono::duration<double, std::micro>(b - a).count();
    };
    for (int j = 0; j < n; j++) {                        // :547-563
        const auto t0 = now();
        if ((rc = sc_round(ctx, sums))) return rc;
        const auto t1 = now();
        tr->send(sums, points, D);
        tr->challenge_base(D, r);
        const auto t2 = now();
        if (challenges) memcpy(challenges + (size_t)j * D, r, 4 * (size_t)D);
        if ((rc = sc_challenge(ctx, r))) return rc;
        if (trace) fprintf(stderr, "round %d: device %.1f us, transcript %.1f us\n", j, us(t0, t1), us(t1, t2));
    }
    const auto t_rounds = now();
    std::vector<u32> out((size_t)ntables * blocks * D);
    if ((rc = sc_finish(ctx, out.data()))) return rc;   // :564-571
    if (trace) fprintf(stderr, "sc_prove: begin %.1f us, rounds %.1f us, finish %.1f us\n", us(t_start, t_begun), us(t_begun, t_rounds), us(t_rounds, now()));
    if (folded) memcpy(folded, out.data(), 4 * out.size());
    if (finals) for (int t = 0; t < ntables; t++) memcpy(finals + (size_t)t * D, out.data() + (size_t)t * blocks * D, 4 * (size_t)D);
    return SC_OK;
}
