// domain.cpp -- PROVE-DOMAIN (src/domain.lisp:336-372) on top of the device prover: a domain of K blocks of
// 2^n elements with base-field columns, zerocheck constraints and lookups is proved by one batched LogUp-GKR
// (sc_gkr_prove_upper) and one sumcheck over the halves of the columns (sc_prove), whose statement is one form
// built from the domain (DOMAIN-STATEMENT, :104-125) with the degree the reference's header states
// (DOMAIN-DEGREE, :127-156).  The forms stay on the host; the leaves of the lookups' trees and the tables of
// the sumcheck are made here from the columns and handed to the device.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/sumcheck_b200.h"
#include "field.cuh"
#include "forms.h"

using namespace scforms;

namespace {

enum { KIND_FULL = 0, KIND_ROW = 1, KIND_COL = 2 };

// One table of the sumcheck (DOMAIN-TABLES, :60-78): a column that depends on the top in-block variable has two,
// its halves; KIND and C say in which rounds the table varies.
struct Table {
    std::string symbol;
    int column;
    int half;   // 0, 1, or -1 for a column with one table
    int kind, c;
};

std::vector<Table> domain_tables(const sc_domain &d) {
    std::vector<Table> out;
    for (int i = 0; i < d.ncolumns; i++) {
        const sc_domain_column &col = d.columns[i];
        const std::string name = lower(col.name);
        const int c = col.kind == KIND_FULL ? 0 : col.c;
        if (col.kind == KIND_FULL || (col.kind == KIND_ROW && c < d.n)) {
            for (int h = 0; h < 2; h++) out.push_back({name + "@" + std::to_string(h), i, h, col.kind, c});
        } else if (col.kind == KIND_COL && c == d.n) {
            for (int h = 0; h < 2; h++) out.push_back({name + "@" + std::to_string(h), i, h, KIND_COL, d.n - 1});
        } else if (col.kind == KIND_ROW) {
            out.push_back({name, i, -1, KIND_ROW, d.n - 1});
        } else {
            out.push_back({name, i, -1, KIND_COL, c});
        }
    }
    return out;
}

std::unique_ptr<Form> parse(const char *text) {
    if (!text) return nullptr;
    Parser ps{text};
    std::unique_ptr<Form> f = ps.form();
    ps.ws();
    if (!ps.ok || *ps.s) return nullptr;
    return f;
}
std::string show(const Form &f) {
    switch (f.kind) {
    case Form::INT: return std::to_string(f.value);
    case Form::VAR: return f.name;
    default: break;
    }
    std::string out = f.kind == Form::ADD ? "(+" : f.kind == Form::SUB ? "(-" : f.kind == Form::MUL ? "(*" : "(expt";
    for (auto &a : f.args) out += " " + show(*a);
    return out + ")";
}
// FORM with each two-half column replaced by its table for HALF (AT-HALF, :80-85), as text
std::string at_half(const Form &f, const sc_domain &d, const std::vector<Table> &tables, int half) {
    if (f.kind == Form::VAR) {
        for (auto &t : tables)
            if (t.half == half && lower(d.columns[t.column].name) == f.name) return t.symbol;
        return f.name;
    }
    if (f.kind == Form::INT) return std::to_string(f.value);
    std::string out = f.kind == Form::ADD ? "(+" : f.kind == Form::SUB ? "(-" : f.kind == Form::MUL ? "(*" : "(expt";
    for (auto &a : f.args) out += " " + at_half(*a, d, tables, half);
    return out + ")";
}

struct Lookup {
    std::unique_ptr<Form> tag, num;
    std::vector<std::unique_ptr<Form>> values;
};
struct Parsed {
    std::vector<std::unique_ptr<Form>> constraints;
    std::vector<Lookup> lookups;
    int arity = 1;   // :92-94
};
int parse_domain(const sc_domain &d, Parsed *out) {
    for (int i = 0; i < d.nconstraints; i++) {
        out->constraints.push_back(parse(d.constraints[i]));
        if (!out->constraints.back()) return SC_ESTATEMENT;
    }
    for (int l = 0; l < d.nlookups; l++) {
        Lookup lk;
        lk.tag = parse(d.lookups[l].tag);
        if (!lk.tag) return SC_ESTATEMENT;
        for (int v = 0; v < d.lookups[l].nvalues; v++) {
            lk.values.push_back(parse(d.lookups[l].values[v]));
            if (!lk.values.back()) return SC_ESTATEMENT;
        }
        if (d.lookups[l].num) { lk.num = parse(d.lookups[l].num); if (!lk.num) return SC_ESTATEMENT; }
        out->arity = std::max(out->arity, d.lookups[l].nvalues);
        out->lookups.push_back(std::move(lk));
    }
    return SC_OK;
}

// q = Z - tag - sum_i beta_i v_i at HALF (DENOMINATOR-FORM, :96-102)
std::string denominator(const Lookup &lk, const sc_domain &d, const std::vector<Table> &tables, int half) {
    std::string out = "(- z " + at_half(*lk.tag, d, tables, half);
    for (size_t i = 0; i < lk.values.size(); i++) out += " (* beta" + std::to_string(i) + " " + at_half(*lk.values[i], d, tables, half) + ")";
    return out + ")";
}
// DOMAIN-STATEMENT (:104-125)
std::string statement_text(const sc_domain &d, const Parsed &p, const std::vector<Table> &tables) {
    std::string out = "(+";
    for (size_t l = 0; l < p.lookups.size(); l++) {
        const Lookup &lk = p.lookups[l];
        const std::string q0 = denominator(lk, d, tables, 0), q1 = denominator(lk, d, tables, 1), id = std::to_string(l);
        if (lk.num) out += " (* a" + id + " (+ (* " + at_half(*lk.num, d, tables, 0) + " " + q1 + ") (* " + at_half(*lk.num, d, tables, 1) + " " + q0 + ")))";
        else out += " (* a" + id + " (+ " + q0 + " " + q1 + "))";
        out += " (* al" + id + " " + q0 + " " + q1 + ")";
    }
    for (size_t i = 0; i < p.constraints.size(); i++) {
        out += " (* gam" + std::to_string(i) + " " + at_half(*p.constraints[i], d, tables, 0) + ")";
        out += " (* geta" + std::to_string(i) + " " + at_half(*p.constraints[i], d, tables, 1) + ")";
    }
    return out + ")";
}

// DOMAIN-DEGREE (:127-156): each polynomial piece counts, in each round, only the tables that vary in that round
int domain_degree(const sc_domain &d, const Parsed &p, const std::vector<Table> &tables, bool block_phase) {
    std::map<std::string, const Table *> by_symbol;
    for (auto &t : tables) by_symbol[t.symbol] = &t;
    auto varies = [&](const std::string &symbol, int round) {   // round -1: the block phase
        auto it = by_symbol.find(symbol);
        if (it == by_symbol.end()) return false;
        const Table &t = *it->second;
        if (round < 0) return d.columns[t.column].shared == 0;
        return t.kind == KIND_FULL ? true : (t.kind == KIND_COL ? round < t.c : round >= t.c);
    };
    auto piece = [&](const Form &f, int half) {
        std::unique_ptr<Form> g = parse(at_half(f, d, tables, half).c_str());
        const Poly poly = expand(*g);
        int best = 0;
        for (int round = block_phase ? -1 : 0; round < (block_phase ? 0 : d.n - 1); round++)
            for (auto &term : poly) {
                int count = 0;
                for (auto &v : term.first) count += varies(v, round);
                best = std::max(best, count);
            }
        return best;
    };
    int degree = 0;
    for (auto &lk : p.lookups) {
        int q[2];
        for (int h = 0; h < 2; h++) {
            q[h] = piece(*lk.tag, h);
            for (auto &v : lk.values) q[h] = std::max(q[h], piece(*v, h));
        }
        if (lk.num) degree = std::max({degree, piece(*lk.num, 0) + q[1], piece(*lk.num, 1) + q[0], q[0] + q[1]});
        else degree = std::max(degree, q[0] + q[1]);
    }
    for (auto &c : p.constraints) degree = std::max({degree, piece(*c, 0), piece(*c, 1)});
    return block_phase ? degree + 1 : degree;
}

// COLUMN-VALUE (:285-292) for every block and in-block index: K 2^n words
std::vector<u32> column_values(const sc_domain &d, const sc_domain_column &col) {
    const int n = d.n, K = d.blocks;
    const size_t size = (size_t)1 << n;
    std::vector<u32> out((size_t)K * size);
    const int c = col.kind == KIND_FULL ? 0 : col.c;
    for (int b = 0; b < K; b++)
        for (size_t x = 0; x < size; x++) {
            size_t at;
            if (col.kind == KIND_FULL) at = (size_t)b * size + x;
            else if (col.kind == KIND_ROW) at = (col.shared ? 0 : (size_t)b << (n - c)) + (x >> c);
            else at = (col.shared ? 0 : (size_t)b << c) + (x & (((size_t)1 << c) - 1));
            out[(size_t)b * size + x] = col.data[at] % scf::P;
        }
    return out;
}

// EVALUATE (src/forms.lisp:214-217) over F_p at every point of the domain: ENV maps a column to its values
std::vector<u32> eval_all(const Form &f, const std::map<std::string, std::vector<u32>> &env, size_t count, bool *ok) {
    std::vector<u32> out(count, 0);
    switch (f.kind) {
    case Form::INT: std::fill(out.begin(), out.end(), modp_ll(f.value)); break;
    case Form::VAR: {
        auto it = env.find(f.name);
        if (it == env.end()) { *ok = false; break; }
        out = it->second;
        break;
    }
    case Form::ADD: case Form::SUB:
        for (size_t i = 0; i < f.args.size(); i++) {
            const std::vector<u32> v = eval_all(*f.args[i], env, count, ok);
            const bool negate = f.kind == Form::SUB && (i > 0 || f.args.size() == 1);
            for (size_t k = 0; k < count; k++) out[k] = negate ? scf::fsub(out[k], v[k]) : scf::fadd(out[k], v[k]);
        }
        break;
    case Form::MUL:
        std::fill(out.begin(), out.end(), 1u);
        for (auto &a : f.args) {
            const std::vector<u32> v = eval_all(*a, env, count, ok);
            for (size_t k = 0; k < count; k++) out[k] = mulp(out[k], v[k]);
        }
        break;
    case Form::EXPT: {
        std::fill(out.begin(), out.end(), 1u);
        const std::vector<u32> v = eval_all(*f.args[0], env, count, ok);
        for (long long e = 0; e < f.args[1]->value; e++)
            for (size_t k = 0; k < count; k++) out[k] = mulp(out[k], v[k]);
        break;
    }
    }
    return out;
}

typedef std::vector<u32> E;
E e_add(const E &a, const E &b) { E o(a.size()); for (size_t c = 0; c < a.size(); c++) o[c] = scf::fadd(a[c], b[c]); return o; }
E e_sub(const E &a, const E &b) { E o(a.size()); for (size_t c = 0; c < a.size(); c++) o[c] = scf::fsub(a[c], b[c]); return o; }
E e_mul(const E &a, const E &b) { E o(a.size()); ext_mul((int)a.size(), a.data(), b.data(), o.data()); return o; }
E e_one(int D) { E o((size_t)D, 0u); o[0] = 1; return o; }
// EQ-TABLE (src/field.lisp:354-363): bit 0 of the index pairs with r_0
std::vector<E> eq_table(const std::vector<E> &r, int D) {
    std::vector<E> t{e_one(D)};
    for (const E &rb : r) {
        const size_t n = t.size();
        t.resize(2 * n);
        for (size_t i = 0; i < n; i++) { const E up = e_mul(t[i], rb); t[n + i] = up; t[i] = e_sub(t[i], up); }
    }
    return t;
}
// K challenges of degree D from D K consecutive base challenges (CHALLENGES, src/transcript.lisp:178-181)
int challenges(sc_transcript *tr, int k, int D, std::vector<E> *out) {
    std::vector<u32> flat((size_t)std::max(k, 1) * D);
    int rc = sc_transcript_challenge_base(tr, D * k, flat.data());
    if (rc) return rc;
    out->clear();
    for (int i = 0; i < k; i++) out->push_back(E(flat.begin() + (size_t)i * D, flat.begin() + (size_t)(i + 1) * D));
    return SC_OK;
}
// LABEL-NAME (src/transcript.lisp:219-230): the name without its layer prefixes ("12.mo" -> "mo")
std::string label_name(const std::string &name) {
    std::string out;
    size_t start = 0;
    for (;;) {
        const size_t bar = name.find('|', start);
        std::string segment = name.substr(start, bar == std::string::npos ? std::string::npos : bar - start);
        size_t digits = 0;
        while (digits < segment.size() && isdigit((unsigned char)segment[digits])) digits++;
        if (digits > 0 && digits < segment.size() && segment[digits] == '.') segment = segment.substr(digits + 1);
        out += segment;
        if (bar == std::string::npos) break;
        out += "|";
        start = bar + 1;
    }
    return out;
}

int check_domain(const sc_domain *d) {
    if (!d || !d->name || d->n < 2 || d->n > 30 || d->blocks < 1 || d->ncolumns < 1 || !d->columns) return SC_EINVAL;   // :44
    if (d->nconstraints < 0 || d->nlookups < 0 || (d->nconstraints && !d->constraints) || (d->nlookups && !d->lookups)) return SC_EINVAL;
    for (int i = 0; i < d->ncolumns; i++) {
        const sc_domain_column &c = d->columns[i];
        if (!c.name || c.kind < KIND_FULL || c.kind > KIND_COL) return SC_EINVAL;
        if (c.kind == KIND_FULL && c.shared) return SC_EINVAL;                     // :48-49
        if (c.kind != KIND_FULL && (c.c < 0 || c.c > d->n)) return SC_EINVAL;
    }
    return SC_OK;
}

}  // namespace

extern "C" int sc_domain_statement(const sc_domain *domain, char *statement, size_t cap, int *ntables, int *degree, int *block_degree) {
    int rc = check_domain(domain);
    if (rc) return rc;
    Parsed p;
    if ((rc = parse_domain(*domain, &p))) return rc;
    const std::vector<Table> tables = domain_tables(*domain);
    const std::string text = statement_text(*domain, p, tables);
    if (statement && cap) snprintf(statement, cap, "%s", text.c_str());
    if (ntables) *ntables = (int)tables.size();
    if (degree) *degree = domain_degree(*domain, p, tables, false);
    if (block_degree) *block_degree = domain_degree(*domain, p, tables, true);
    return statement && cap <= text.size() ? SC_EINVAL : SC_OK;
}

extern "C" int sc_prove_domain(sc_ctx *const *ctxs, int nctx, sc_transcript *tr, const sc_domain *domain, const uint32_t *z,
                               const uint32_t *betas, int nbetas, const char *label, int *point_len, uint32_t *points, int *value_rows,
                               uint32_t *values) {
    int rc = check_domain(domain);
    if (rc) return rc;
    if (!ctxs || !tr || !z || nctx < std::max(1, domain->nlookups)) return SC_EINVAL;
    for (int i = 0; i < domain->ncolumns; i++) if (!domain->columns[i].data) return SC_EINVAL;
    const sc_domain &d = *domain;
    const int D = sc_transcript_degree(tr), n = d.n, K = d.blocks, L = d.nlookups;
    if (D != 4 && D != 8) return SC_EINVAL;
    if (!label) label = "dom";
    Parsed p;
    if ((rc = parse_domain(d, &p))) return rc;
    if (L > 0 && (nbetas < p.arity || !betas)) return SC_EINVAL;
    int lk = 0;
    while ((1 << lk) < K) lk++;
    const std::vector<Table> tables = domain_tables(d);
    const int nt = (int)tables.size();
    if (nt > SC_MAX_WIDE_TABLES - 1) return SC_EUNSUPPORTED;
    const std::string statement = statement_text(d, p, tables);

    // the columns at every point of the domain, once
    const size_t size = (size_t)1 << n, count = (size_t)K * size;
    std::map<std::string, std::vector<u32>> env;
    for (int i = 0; i < d.ncolumns; i++) env[lower(d.columns[i].name)] = column_values(d, d.columns[i]);

    const std::string head = std::string(label) + label_name(d.name);
    if ((rc = sc_transcript_absorb(tr, (const uint8_t *)head.data(), head.size()))) return rc;

    // 1. the lookups' trees down to the leaves' parents (:345-348)
    std::vector<E> r, rb;
    if (L > 0) {
        // DOMAIN-LEAVES (:294-318): p the numerator (1 if absent), q = Z - tag - sum_i beta_i v_i
        std::vector<std::vector<u32>> lp(L), lq(L);
        bool ok = true;
        for (int l = 0; l < L; l++) {
            lp[l].assign(count * D, 0u); lq[l].assign(count * D, 0u);
            const Lookup &lookup = p.lookups[l];
            const std::vector<u32> tag = eval_all(*lookup.tag, env, count, &ok);
            std::vector<u32> num;
            if (lookup.num) num = eval_all(*lookup.num, env, count, &ok);
            for (size_t i = 0; i < count; i++) {
                lp[l][i * D] = lookup.num ? num[i] : 1u;
                for (int c = 0; c < D; c++) lq[l][i * D + c] = z[c] % scf::P;
                lq[l][i * D] = scf::fsub(lq[l][i * D], tag[i]);
            }
            for (size_t v = 0; v < lookup.values.size(); v++) {
                const std::vector<u32> val = eval_all(*lookup.values[v], env, count, &ok);
                for (size_t i = 0; i < count; i++)
                    for (int c = 0; c < D; c++) lq[l][i * D + c] = scf::fsub(lq[l][i * D + c], mulp(betas[v * D + c] % scf::P, val[i]));
            }
        }
        if (!ok) return SC_ESTATEMENT;   // a form names something that is not a column
        std::vector<const uint32_t *> pp(L), qp(L);
        for (int l = 0; l < L; l++) { pp[l] = lp[l].data(); qp[l] = lq[l].data(); }
        std::vector<u32> ri((size_t)std::max(n - 1, 1) * D), rbw((size_t)std::max(lk, 1) * D);
        if ((rc = sc_gkr_prove_upper(ctxs, L, tr, n, K, pp.data(), qp.data(), 0, "gkr", ri.data(), rbw.data(), nullptr, nullptr))) return rc;
        for (int j = 0; j < n - 1; j++) r.push_back(E(ri.begin() + (size_t)j * D, ri.begin() + (size_t)(j + 1) * D));
        for (int j = 0; j < lk; j++) rb.push_back(E(rbw.begin() + (size_t)j * D, rbw.begin() + (size_t)(j + 1) * D));
    } else {
        if ((rc = challenges(tr, n - 1, D, &r))) return rc;
        if ((rc = challenges(tr, lk, D, &rb))) return rc;
    }

    // 2. the challenges and constants of the statement (:158-175)
    std::vector<E> as, gams, lam1, eta1;
    if ((rc = challenges(tr, std::max(1, L), D, &as))) return rc;
    if ((rc = challenges(tr, 1, D, &lam1))) return rc;
    if ((rc = challenges(tr, std::max(1, d.nconstraints), D, &gams))) return rc;
    if ((rc = challenges(tr, 1, D, &eta1))) return rc;
    std::vector<std::string> cnames;
    std::vector<u32> cvals;
    auto constant = [&](const std::string &name, const E &value) { cnames.push_back(name); cvals.insert(cvals.end(), value.begin(), value.end()); };
    {
        E zz((size_t)D);
        for (int c = 0; c < D; c++) zz[c] = z[c] % scf::P;
        constant("z", zz);
        for (int i = 0; i < p.arity; i++) {
            E b((size_t)D, 0u);
            if (betas && i < nbetas) for (int c = 0; c < D; c++) b[c] = betas[(size_t)i * D + c] % scf::P;
            constant("beta" + std::to_string(i), b);
        }
        for (size_t l = 0; l < as.size(); l++) { constant("a" + std::to_string(l), as[l]); constant("al" + std::to_string(l), e_mul(as[l], lam1[0])); }
        for (size_t i = 0; i < gams.size(); i++) { constant("gam" + std::to_string(i), gams[i]); constant("geta" + std::to_string(i), e_mul(gams[i], eta1[0])); }
    }
    std::vector<const char *> cname_ptrs;
    for (auto &s : cnames) cname_ptrs.push_back(s.c_str());

    // 3. the sumcheck over the halves of the columns (:353-357); TABLE-VALUES (:320-330)
    std::vector<E> bw;                                  // BLOCK-WEIGHTS (src/gkr.lisp:73-77)
    if (rb.empty()) bw.push_back(e_one(D));
    else { const std::vector<E> e = eq_table(rb, D); bw.assign(e.begin(), e.begin() + K); }
    std::vector<u32> bwf;
    for (auto &w : bw) bwf.insert(bwf.end(), w.begin(), w.end());
    const size_t half = size / 2;
    std::vector<std::vector<u32>> tvals(nt, std::vector<u32>((size_t)K * half));
    for (int t = 0; t < nt; t++) {
        const std::vector<u32> &col = env[lower(d.columns[tables[t].column].name)];
        const size_t lo = tables[t].half > 0 ? half : 0;
        for (int b = 0; b < K; b++) memcpy(tvals[t].data() + (size_t)b * half, col.data() + (size_t)b * size + lo, half * 4);
    }
    std::vector<const char *> tnames(nt);
    std::vector<const uint32_t *> tptrs(nt);
    std::vector<int> strides(nt, 1);
    for (int t = 0; t < nt; t++) { tnames[t] = tables[t].symbol.c_str(); tptrs[t] = tvals[t].data(); }
    std::vector<u32> eq;
    for (auto &e : r) eq.insert(eq.end(), e.begin(), e.end());
    std::vector<u32> rho((size_t)std::max(n - 1, 1) * D), finals((size_t)nt * D), folded((size_t)nt * K * D);
    if ((rc = sc_prove(ctxs[0], tr, n - 1, statement.c_str(), nt, tnames.data(), tptrs.data(), strides.data(), eq.data(), (int)cnames.size(),
                       cname_ptrs.data(), cvals.data(), label, K, bwf.data(), domain_degree(d, p, tables, false), rho.data(), finals.data(),
                       folded.data())))
        return rc;

    // 4. the finals and the claims (:358-372, DOMAIN-CLAIMS :179-210)
    std::vector<E> rbn;
    std::vector<std::vector<E>> fin(nt);     // per table: one value (merged) or K (one for a shared column)
    if (d.merge) {
        if (lk > 0) {   // bind the block index: the blocks' values and weights, padded (a shared table with its value, the others with zero)
            const int KP = 1 << lk;
            std::vector<std::vector<u32>> padded(nt + 1, std::vector<u32>((size_t)KP * D, 0u));
            memcpy(padded[0].data(), bwf.data(), bwf.size() * 4);
            for (int t = 0; t < nt; t++) {
                memcpy(padded[t + 1].data(), folded.data() + (size_t)t * K * D, (size_t)K * D * 4);
                if (d.columns[tables[t].column].shared)
                    for (int b = K; b < KP; b++) memcpy(padded[t + 1].data() + (size_t)b * D, folded.data() + (size_t)t * K * D, (size_t)D * 4);
            }
            std::vector<const char *> bnames{"bw"};
            std::vector<const uint32_t *> bptrs{padded[0].data()};
            std::vector<int> bstrides(nt + 1, D);
            for (int t = 0; t < nt; t++) { bnames.push_back(tnames[t]); bptrs.push_back(padded[t + 1].data()); }
            const std::string blk_statement = "(* bw " + statement + ")", blk_label = std::string(label) + "-blk";
            std::vector<u32> rbw((size_t)lk * D), bfinals((size_t)(nt + 1) * D);
            if ((rc = sc_prove(ctxs[0], tr, lk, blk_statement.c_str(), nt + 1, bnames.data(), bptrs.data(), bstrides.data(), nullptr,
                               (int)cnames.size(), cname_ptrs.data(), cvals.data(), blk_label.c_str(), 1, nullptr,
                               domain_degree(d, p, tables, true), rbw.data(), bfinals.data(), nullptr)))
                return rc;
            for (int j = 0; j < lk; j++) rbn.push_back(E(rbw.begin() + (size_t)j * D, rbw.begin() + (size_t)(j + 1) * D));
            for (int t = 0; t < nt; t++) fin[t].push_back(E(bfinals.begin() + (size_t)(t + 1) * D, bfinals.begin() + (size_t)(t + 2) * D));
        } else {
            for (int t = 0; t < nt; t++) fin[t].push_back(E(finals.begin() + (size_t)t * D, finals.begin() + (size_t)(t + 1) * D));
        }
        for (int t = 0; t < nt; t++) if ((rc = sc_transcript_send(tr, fin[t][0].data(), 1, D))) return rc;
    } else {
        for (int t = 0; t < nt; t++) {
            const int rows = d.columns[tables[t].column].shared ? 1 : K;
            for (int b = 0; b < rows; b++) fin[t].push_back(E(folded.begin() + ((size_t)t * K + b) * D, folded.begin() + ((size_t)t * K + b + 1) * D));
            std::vector<u32> flat;
            for (auto &e : fin[t]) flat.insert(flat.end(), e.begin(), e.end());
            if ((rc = sc_transcript_send(tr, flat.data(), rows, D))) return rc;
        }
    }
    std::vector<E> tt1;
    if ((rc = challenges(tr, 1, D, &tt1))) return rc;
    const E &tt = tt1[0];
    std::vector<E> full;
    for (int j = 0; j < n - 1; j++) full.push_back(E(rho.begin() + (size_t)j * D, rho.begin() + (size_t)(j + 1) * D));
    std::vector<E> rho_only = full;
    full.push_back(tt);
    const size_t point_cap = (size_t)(n + lk) * D, value_cap = (size_t)K * D;
    for (int i = 0; i < d.ncolumns; i++) {
        const sc_domain_column &col = d.columns[i];
        const int c = col.kind == KIND_FULL ? 0 : col.c;
        int first = -1, last = -1;
        for (int t = 0; t < nt; t++) if (tables[t].column == i) { if (first < 0) first = t; last = t; }
        std::vector<E> point, value;
        if (last > first) {   // two halves: f0 + tt (f1 - f0) at (rho, tt), from c on for a :ROW column
            point.assign(full.begin() + (col.kind == KIND_ROW ? c : 0), full.end());
            for (size_t b = 0; b < fin[first].size(); b++) value.push_back(e_add(fin[first][b], e_mul(tt, e_sub(fin[last][b], fin[first][b]))));
        } else {
            if (col.kind == KIND_COL) point.assign(rho_only.begin(), rho_only.begin() + std::min(c, n - 1));
            value = fin[first];
        }
        if (d.merge && !col.shared) point.insert(point.end(), rbn.begin(), rbn.end());
        if (point_len) point_len[i] = (int)point.size();
        if (value_rows) value_rows[i] = (int)value.size();
        if (points) for (size_t k = 0; k < point.size(); k++) memcpy(points + (size_t)i * point_cap + k * D, point[k].data(), (size_t)D * 4);
        if (values) for (size_t k = 0; k < value.size(); k++) memcpy(values + (size_t)i * value_cap + k * D, value[k].data(), (size_t)D * 4);
    }
    return SC_OK;
}
