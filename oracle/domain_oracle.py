"""TEST INFRASTRUCTURE ONLY: a CPU restatement of the reference's domains (src/domain.lisp) on top of
the sumcheck oracle (``oracle/pyoracle.py``) and the LogUp-GKR restatement (``oracle/gkr_oracle.py``).

The product never imports this file.  Every function cites the reference lines it follows.
Parity: the sumchecks inside are the pinned oracle's; the protocol around them has no golden vector
that can be read without running the reference (its frozen domain cases are made from SBCL's random
state), so it is held by the reference's own invariants (tests/tests.lisp:523-585): VERIFY-DOMAIN,
restated below, accepts what PROVE-DOMAIN sends and computes the same claims; a full column's claim
is its multilinear extension at the claimed point; a broken constraint and every forged message
are rejected.

Forms are nested lists of lower-case symbol strings and integers, e.g. ["*", "a", ["-", "a", 1]].
"""
import numpy as np

from . import gkr_oracle as gkr
from . import pyoracle as orc

P = 2130706433


# ------------------------------------------------------------------ forms as data

def parse(text):
    """Read one form from its text."""
    tokens = text.replace("(", " ( ").replace(")", " ) ").split()
    pos = 0

    def read():
        nonlocal pos
        tok = tokens[pos]
        pos += 1
        if tok == "(":
            out = []
            while tokens[pos] != ")":
                out.append(read())
            pos += 1
            return out
        try:
            return int(tok)
        except ValueError:
            return tok.lower()

    form = read()
    if pos != len(tokens):
        raise ValueError("trailing text after the form: %r" % text)
    return form


def show(form):
    if isinstance(form, list):
        return "(" + " ".join(show(f) for f in form) + ")"
    return str(form)


def sublis(mapping, form):
    """SUBLIS on symbols (not on operators in head position: column names never are)."""
    if isinstance(form, list):
        return [form[0]] + [sublis(mapping, f) for f in form[1:]] if form else form
    return mapping.get(form, form)


def eval_base(form, env):
    """EVALUATE (src/forms.lisp:214-217) over F_p, vectorised: ENV maps symbols to uint64 arrays (or ints)."""
    if isinstance(form, int):
        return np.uint64(form % P)
    if not isinstance(form, list):
        return env[form]
    op, args = form[0], form[1:]
    if op == "+":
        out = np.uint64(0)
        for a in args:
            out = (out + eval_base(a, env)) % P
        return out
    if op == "-":
        vals = [eval_base(a, env) for a in args]
        if len(vals) == 1:
            return (P - vals[0]) % P
        out = vals[0]
        for v in vals[1:]:
            out = (out + P - v) % P
        return out
    if op == "*":
        out = np.uint64(1)
        for a in args:
            out = (out * eval_base(a, env)) % P
        return out
    if op == "expt":
        base, out = eval_base(args[0], env), np.uint64(1)
        for _ in range(args[1]):
            out = (out * base) % P
        return out
    raise ValueError("operator %r" % op)


# ------------------------------------------------------------------ the domain (src/domain.lisp:32-53)

class Column:
    def __init__(self, name, kind="full", c=0, shared=False, data=None):
        if shared and kind == "full":
            raise ValueError("a full column is never shared")          # :48-49
        self.name, self.kind, self.c, self.shared = name.lower(), kind, (0 if kind == "full" else c), shared
        self.data = None if data is None else np.ascontiguousarray(data, dtype=np.uint32)


class Domain:
    def __init__(self, name, n, blocks=1, merge=False, columns=(), constraints=(), lookups=()):
        if n < 2:
            raise ValueError("n: at least 2")                           # :44
        self.name, self.n, self.blocks, self.merge = name, n, blocks, merge
        self.columns = list(columns)
        self.constraints = [parse(c) if isinstance(c, str) else c for c in constraints]
        self.lookups = []
        for lk in lookups:                                              # (:tag form :values (form ...) :num form)
            as_form = lambda f: parse(f) if isinstance(f, str) else f
            self.lookups.append({"tag": as_form(lk["tag"]), "values": [as_form(v) for v in lk.get("values", [])],
                                 "num": as_form(lk["num"]) if lk.get("num") is not None else None})


def domain_tables(domain):
    """:60-78: (symbol, column, half, kind, c) in the reference's order."""
    n, out = domain.n, []
    for col in domain.columns:
        if col.kind == "full" or (col.kind == "row" and col.c < n):
            out += [("%s@%d" % (col.name, h), col, h, col.kind, col.c) for h in range(2)]
        elif col.kind == "col" and col.c == n:
            out += [("%s@%d" % (col.name, h), col, h, "col", n - 1) for h in range(2)]
        elif col.kind == "row":
            out.append((col.name, col, None, "row", n - 1))
        else:
            out.append((col.name, col, None, "col", col.c))
    return out


def at_half(form, domain, half):
    """:80-85"""
    return sublis({col.name: sym for sym, col, h, _, _ in domain_tables(domain) if h == half}, form)


def arity(domain):
    """:92-94"""
    return max([1] + [len(lk["values"]) for lk in domain.lookups])


def denominator_form(lookup, domain, half):
    """:96-102: q = Z - tag - sum_i beta_i v_i at HALF."""
    return ["-", "z", at_half(lookup["tag"], domain, half)] + [["*", "beta%d" % i, at_half(v, domain, half)] for i, v in enumerate(lookup["values"])]


def domain_statement(domain):
    """:104-125"""
    terms = []
    for l, lookup in enumerate(domain.lookups):
        q0, q1, num = denominator_form(lookup, domain, 0), denominator_form(lookup, domain, 1), lookup["num"]
        inner = ["+", ["*", at_half(num, domain, 0), q1], ["*", at_half(num, domain, 1), q0]] if num is not None else ["+", q0, q1]
        terms += [["*", "a%d" % l, inner], ["*", "al%d" % l, q0, q1]]
    for i, constraint in enumerate(domain.constraints):
        terms += [["*", "gam%d" % i, at_half(constraint, domain, 0)], ["*", "geta%d" % i, at_half(constraint, domain, 1)]]
    return ["+"] + terms


def _variables(form, out):
    if isinstance(form, list):
        for f in form[1:]:
            _variables(f, out)
    elif isinstance(form, str) and form not in out:
        out.append(form)
    return out


def domain_degree(domain, block_phase=False):
    """:127-167"""
    n = domain.n
    tables = {sym: (col, kind, c) for sym, col, _, kind, c in domain_tables(domain)}
    rounds = ["block"] if block_phase else list(range(n - 1))

    def varies(symbol, rnd):
        col, kind, c = tables[symbol]
        if rnd == "block":
            return not col.shared
        return True if kind == "full" else (rnd < c if kind == "col" else rnd >= c)

    def piece(form):
        variables = _variables(form, [])
        monomials = orc.expand(show(form), variables) if variables else []
        best = 0
        for rnd in rounds:
            for idx, _ in monomials:
                best = max(best, sum(1 for i in idx if varies(variables[i], rnd)))
        return best

    def q(lookup, half):
        return max([piece(at_half(lookup["tag"], domain, half))] + [piece(at_half(v, domain, half)) for v in lookup["values"]])

    degree = 0
    for lookup in domain.lookups:
        q0, q1, num = q(lookup, 0), q(lookup, 1), lookup["num"]
        if num is not None:
            degree = max(degree, piece(at_half(num, domain, 0)) + q1, piece(at_half(num, domain, 1)) + q0, q0 + q1)
        else:
            degree = max(degree, q0 + q1)
    for constraint in domain.constraints:
        degree = max(degree, piece(at_half(constraint, domain, 0)), piece(at_half(constraint, domain, 1)))
    return degree + 1 if block_phase else degree


def domain_constants(domain, D, z, betas, a, lam, gams, eta):
    """:158-167"""
    out = [("z", list(z))] + [("beta%d" % i, list(betas[i])) for i in range(arity(domain))]
    for l, al in enumerate(a):
        out += [("a%d" % l, al), ("al%d" % l, orc.ext_mul(D, al, lam))]
    for i, g in enumerate(gams):
        out += [("gam%d" % i, g), ("geta%d" % i, orc.ext_mul(D, g, eta))]
    return out


def _challenges(tr, k, D):
    """CHALLENGES (src/transcript.lisp:178-181): K elements from D K consecutive base challenges."""
    flat = tr.challenge_base(D * k)
    return [flat[D * i:D * (i + 1)] for i in range(k)]


def domain_challenges(tr, domain, D):
    """:169-175"""
    a = _challenges(tr, max(1, len(domain.lookups)), D)
    lam = tr.challenge()
    gams = _challenges(tr, max(1, len(domain.constraints)), D)
    eta = tr.challenge()
    return a, lam, gams, eta


def domain_claims(domain, D, rho, rb, tt, finals):
    """:179-210: (name, point, value) per column; FINALS maps a table to one value (merged) or to a list of values."""
    n, tables, full = domain.n, domain_tables(domain), list(rho) + [tt]
    out = []
    for col in domain.columns:
        halves = [sym for sym, c, _, _, _ in tables if c is col]
        f0, f1 = finals[halves[0]], finals[halves[-1]]
        if len(halves) > 1:
            point = full[col.c:] if col.kind == "row" else full
            interpolate = lambda a, b: orc.ext_add(D, a, orc.ext_mul(D, tt, orc.ext_sub(D, b, a)))
            value = interpolate(f0, f1) if isinstance(f0[0], int) else [interpolate(a, b) for a, b in zip(f0, f1)]
        else:
            point = list(rho[:min(col.c, n - 1)]) if col.kind == "col" else []
            value = f0
        if domain.merge and not col.shared:
            point = point + list(rb)
        out.append((col.name, point, value))
    return out


def label_name(name):
    """LABEL-NAME (src/transcript.lisp:219-230): the name without its layer prefixes."""
    def strip(segment):
        digits = len(segment) - len(segment.lstrip("0123456789"))
        return segment[digits + 1:] if digits > 0 and digits < len(segment) and segment[digits] == "." else segment
    return "|".join(strip(s) for s in name.split("|"))


# ------------------------------------------------------------------ prover (:283-372)

def column_values(col, k, n):
    """COLUMN-VALUE (:285-292) for every block and in-block index: an array of shape (k, 2^n)."""
    size, x = 1 << n, np.arange(1 << n)
    if col.kind == "full":
        return col.data.reshape(k, size)
    per, index = (1 << (n - col.c), x >> col.c) if col.kind == "row" else (1 << col.c, x & ((1 << col.c) - 1))
    rows = col.data.reshape(1 if col.shared else k, per)[:, index]
    return np.broadcast_to(rows, (k, size)) if col.shared else rows


def domain_leaves(domain, D, z, betas):
    """:294-318: per lookup (p, q), arrays of shape (K 2^n, D)."""
    n, k = domain.n, domain.blocks
    env = {col.name: column_values(col, k, n).astype(np.uint64).reshape(-1) for col in domain.columns}
    count = k << n
    out = []
    for lookup in domain.lookups:
        p = np.zeros((count, D), dtype=np.uint64)
        p[:, 0] = eval_base(lookup["num"], env) if lookup["num"] is not None else 1
        q = np.tile(np.array(z, dtype=np.uint64), (count, 1))
        q[:, 0] = (q[:, 0] + P - np.broadcast_to(eval_base(lookup["tag"], env), (count,))) % P
        for v, beta in zip(lookup["values"], betas):
            vals = np.broadcast_to(eval_base(v, env), (count,)).astype(np.uint64)
            q = (q + P - (vals[:, None] * np.array(beta, dtype=np.uint64)[None, :]) % P) % P
        out.append((p.astype(np.uint32), q.astype(np.uint32)))
    return out


def table_values(table, k, n):
    """:320-330: a sumcheck table's K blocks of 2^(n-1) base elements."""
    _, col, half, _, _ = table
    v = column_values(col, k, n)
    lo = (half or 0) << (n - 1)
    return np.ascontiguousarray(v[:, lo:lo + (1 << (n - 1))]).reshape(-1).astype(np.uint32)


def prove_domain(tr, domain, z, betas, label="dom", threads=1):
    """:336-372.  Returns the column claims [(name, point, value)]."""
    D, n, k = tr.degree, domain.n, domain.blocks
    lk = gkr.block_bits(k)
    tables = domain_tables(domain)
    statement = show(domain_statement(domain))
    tr.absorb((label + label_name(domain.name)).encode())
    if domain.lookups:
        r, rb, _, _ = gkr.prove_upper(tr, n, k, domain_leaves(domain, D, z, betas), threads=threads)
    else:
        r, rb = _challenges(tr, n - 1, D), _challenges(tr, lk, D)
    a, lam, gams, eta = domain_challenges(tr, domain, D)
    constants = domain_constants(domain, D, z, betas, a, lam, gams, eta)
    bw = gkr.block_weights(D, rb, k)
    rho, finals, folded = orc.prove(tr, n - 1, statement, [(t[0], table_values(t, k, n)) for t in tables], eq=r, constants=constants,
                                    label=label, block_weights=bw, degree=domain_degree(domain), threads=threads)
    if domain.merge:
        rbn = []
        if lk > 0:
            pad = (1 << lk) - k
            padded = lambda values, shared: np.array(list(values) + [values[0] if shared else [0] * D] * pad, dtype=np.uint32)
            blk = [("bw", padded(bw, False))] + [(t[0], padded(folded[t[0]], t[1].shared)) for t in tables]
            rbn, finals, _ = orc.prove(tr, lk, "(* bw %s)" % statement, blk, constants=constants, label=label + "-blk",
                                       degree=domain_degree(domain, block_phase=True), threads=threads)
        finals = {t[0]: finals[t[0]] for t in tables}
        for t in tables:
            tr.send(np.array([finals[t[0]]], dtype=np.uint32))
        return domain_claims(domain, D, rho, rbn, tr.challenge(), finals)
    finals = {t[0]: (folded[t[0]][:1] if t[1].shared else folded[t[0]]) for t in tables}
    for t in tables:
        tr.send(np.array(finals[t[0]], dtype=np.uint32))
    return domain_claims(domain, D, rho, [], tr.challenge(), finals)


# ------------------------------------------------------------------ verifier (:212-281)

def verify_domain(tr_label, D, messages, domain, z, betas, label="dom"):
    """Returns (claims, roots); raises gkr.VerificationFailure."""
    rp = gkr._Replay(tr_label, D, messages)
    n, k = domain.n, domain.blocks
    lk = gkr.block_bits(k)
    lookups = len(domain.lookups)
    tables = domain_tables(domain)
    statement = show(domain_statement(domain))
    rp.tr.absorb((label + label_name(domain.name)).encode())
    roots, cp, cq = [], None, None
    if lookups:
        roots, r, rb, cp, cq = gkr.verify_upper_on(rp, n, k, lookups)
    else:
        r, rb = _challenges(rp.tr, n - 1, D), _challenges(rp.tr, lk, D)
    a, lam, gams, eta = domain_challenges(rp.tr, domain, D)
    constants = domain_constants(domain, D, z, betas, a, lam, gams, eta)
    claim = gkr.layer_claim(D, a, lam, cp, cq) if lookups else [0] * D
    bw = gkr.block_weights(D, rb, k)
    value = lambda finals: gkr._evaluate(D, statement, finals, constants)
    rho, reduced = gkr._verify(rp, n - 1, domain_degree(domain), claim, r, k, label)
    if domain.merge:
        rbn = []
        if lk > 0:
            rbn, reduced = gkr._verify(rp, lk, domain_degree(domain, block_phase=True), reduced, None, 1, label + "-blk")
        finals = [(t[0], rp.receive(1, D)[0].tolist()) for t in tables]
        if k > 1:
            weight = [0] * D
            for w, e in zip(bw, orc.eq_table(D, rbn)):
                weight = orc.ext_add(D, weight, orc.ext_mul(D, w, e))
        else:
            weight = bw[0]
        if reduced != orc.ext_mul(D, weight, value(finals)):
            raise gkr.VerificationFailure("%s: leaf/zerocheck sumcheck failed" % domain.name)
        claims = domain_claims(domain, D, rho, rbn, rp.tr.challenge(), dict(finals))
    else:
        finals = [(t[0], rp.receive(1 if t[1].shared else k, D).tolist()) for t in tables]
        total = [0] * D
        for b in range(k):
            block_finals = [(name, vals[b if len(vals) > 1 else 0]) for name, vals in finals]
            total = orc.ext_add(D, total, orc.ext_mul(D, bw[b], value(block_finals)))
        if reduced != total:
            raise gkr.VerificationFailure("%s: leaf/zerocheck sumcheck failed" % domain.name)
        claims = domain_claims(domain, D, rho, [], rp.tr.challenge(), dict(finals))
    if not rp.finished():
        raise gkr.VerificationFailure("messages left over")
    return claims, roots
