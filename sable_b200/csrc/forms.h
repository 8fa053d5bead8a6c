// forms.h -- statements as data, for the host side of the library: the reference's forms
// (src/forms.lisp:28-106: integers, symbols, (+ ..) (- ..) (* ..) (expt f k)), their expansion into a
// polynomial over F_p, and a few field helpers on canonical words.  Shared by the statement compiler
// (host.cpp) and the domain prover (domain.cpp).
#pragma once
#include <algorithm>
#include <cctype>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "field.cuh"

namespace scforms {

using scf::u32;
using scf::u64;

template <int D> inline void ext_mul_canon(const u32 *a, const u32 *b, u32 *o) {
    scf::Ext<D> x, y;
    for (int i = 0; i < D; i++) { x.v[i] = scf::to_mont(a[i]); y.v[i] = scf::to_mont(b[i]); }
    scf::Ext<D> z = scf::efrom_mont<D>(scf::emul<D>(x, y));
    for (int i = 0; i < D; i++) o[i] = z.v[i];
}
inline void ext_mul(int D, const u32 *a, const u32 *b, u32 *o) {
    u32 t[8];
    if (D == 4) ext_mul_canon<4>(a, b, t); else ext_mul_canon<8>(a, b, t);
    memcpy(o, t, 4 * (size_t)D);
}
inline u32 modp_ll(long long x) { long long r = x % (long long)scf::P; if (r < 0) r += scf::P; return (u32)r; }
inline u32 mulp(u32 a, u32 b) { return (u32)(((u64)a * b) % scf::P); }

// ------------------------------------------------------------------ forms as data (src/forms.lisp)

struct Form {
    enum Kind { INT, VAR, ADD, SUB, MUL, EXPT } kind = INT;
    long long value = 0;
    std::string name;
    std::vector<std::unique_ptr<Form>> args;
};

struct Parser {
    const char *s;
    bool ok = true;
    void ws() { while (*s && isspace((unsigned char)*s)) s++; }
    std::string token() {
        std::string t;
        while (*s && !isspace((unsigned char)*s) && *s != '(' && *s != ')') t.push_back((char)tolower((unsigned char)*s++));
        return t;
    }
    std::unique_ptr<Form> form() {
        auto f = std::make_unique<Form>();
        ws();
        if (*s == '(') {
            s++; ws();
            const std::string op = token();
            if (op == "+") f->kind = Form::ADD; else if (op == "-") f->kind = Form::SUB;
            else if (op == "*") f->kind = Form::MUL; else if (op == "expt") f->kind = Form::EXPT;
            else { ok = false; return f; }
            for (;;) {
                ws();
                if (*s == ')') { s++; break; }
                if (!*s) { ok = false; return f; }
                f->args.push_back(form());
                if (!ok) return f;
            }
            if (f->kind == Form::EXPT && (f->args.size() != 2 || f->args[1]->kind != Form::INT || f->args[1]->value < 0)) ok = false;
            if (f->kind == Form::SUB && f->args.empty()) ok = false;
            return f;
        }
        const std::string t = token();
        if (t.empty()) { ok = false; return f; }
        char *end = nullptr;
        const long long v = strtoll(t.c_str(), &end, 10);
        if (end && *end == 0) { f->kind = Form::INT; f->value = v; }
        else { f->kind = Form::VAR; f->name = t; }
        return f;
    }
};

// a polynomial: monomial (sorted variable names) -> coefficient in F_p
typedef std::vector<std::string> Monomial;
struct MonomialLess {   // graded order (monomial<, src/forms.lisp:31-36)
    bool operator()(const Monomial &a, const Monomial &b) const {
        if (a.size() != b.size()) return a.size() < b.size();
        return a < b;
    }
};
typedef std::map<Monomial, u32, MonomialLess> Poly;

inline void poly_add(Poly &p, const Monomial &m, u32 c) {
    u32 &slot = p[m];
    slot = scf::fadd(slot, c);
}
inline void poly_clean(Poly &p) {
    for (auto it = p.begin(); it != p.end();) it = it->second ? std::next(it) : p.erase(it);
}
inline Poly poly_mul(const Poly &a, const Poly &b) {
    Poly out;
    for (auto &x : a) for (auto &y : b) {
        Monomial m(x.first.size() + y.first.size());
        std::merge(x.first.begin(), x.first.end(), y.first.begin(), y.first.end(), m.begin());
        poly_add(out, m, mulp(x.second, y.second));
    }
    poly_clean(out);
    return out;
}
// EXPAND (src/forms.lisp:57-78)
inline Poly expand(const Form &f) {
    Poly p;
    switch (f.kind) {
    case Form::INT: poly_add(p, Monomial(), modp_ll(f.value)); break;
    case Form::VAR: poly_add(p, Monomial{f.name}, 1); break;
    case Form::ADD: case Form::SUB:
        for (size_t i = 0; i < f.args.size(); i++) {
            const bool negate = f.kind == Form::SUB && (i > 0 || f.args.size() == 1);
            for (auto &term : expand(*f.args[i])) poly_add(p, term.first, negate ? scf::fneg(term.second) : term.second);
        }
        break;
    case Form::MUL:
        poly_add(p, Monomial(), 1);
        for (auto &arg : f.args) p = poly_mul(p, expand(*arg));
        break;
    case Form::EXPT: {
        poly_add(p, Monomial(), 1);
        const Poly base = expand(*f.args[0]);
        for (long long k = 0; k < f.args[1]->value; k++) p = poly_mul(p, base);
        break;
    }
    }
    poly_clean(p);
    return p;
}
inline void mentioned(const Form &f, std::vector<std::string> &out) {
    if (f.kind == Form::VAR) out.push_back(f.name);
    const size_t count = f.kind == Form::EXPT ? 1 : f.args.size();
    for (size_t i = 0; i < count; i++) mentioned(*f.args[i], out);
}
inline std::string lower(const char *s) { std::string t; for (; *s; s++) t.push_back((char)tolower((unsigned char)*s)); return t; }

}  // namespace scforms
