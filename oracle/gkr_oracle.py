"""TEST INFRASTRUCTURE ONLY: a CPU restatement of the reference's LogUp-GKR upper layers
(src/gkr.lisp), on top of the sumcheck oracle (``oracle/pyoracle.py``).

The product never imports this file.  Every function cites the reference lines it follows.
Parity: the sumchecks inside are the pinned oracle's; the protocol around them (order of the
messages and challenges, claims between the layers) has no golden vector that can be read
without running the reference (its frozen cases are made from SBCL's random state), so it is
held by the reference's own invariants instead (tests/tests.lisp:414-442): the verifier below,
written from VERIFY-UPPER, accepts what PROVE-UPPER sends and returns the prover's outputs; the
roots are the sums of the leaf fractions; the final claims are the leaves' parents at the point.

Data: a lookup's leaves are two arrays (p, q) of shape (K 2^n, D), block-major.
"""
import ctypes as C

import numpy as np

from . import pyoracle as orc

P = 2130706433


def block_bits(k):
    """:23-25"""
    return (k - 1).bit_length()


def layer_statement(lookups):
    """:30-41: the form, its tables in the proof's order, its constants."""
    tables, constants, terms = [], [], []
    for l in range(lookups):
        p0, p1, q0, q1, a, al = ("%s%d" % (nm, l) for nm in ("p0_", "p1_", "q0_", "q1_", "a", "al"))
        tables += [p0, p1, q0, q1]
        constants += [a, al]
        terms += ["(* %s %s %s)" % (a, p0, q1), "(* %s %s %s)" % (a, p1, q0), "(* %s %s %s)" % (al, q0, q1)]
    return "(+ %s)" % " ".join(terms), tables, constants


def layer_challenges(tr, lookups, D):
    """:43-51: a_l for each lookup, then lambda; returns the statement's constants, the a_l and lambda."""
    flat = tr.challenge_base(D * lookups)
    a = [flat[D * l:D * (l + 1)] for l in range(lookups)]
    lam = tr.challenge()
    constants = []
    for l in range(lookups):
        constants.append(("a%d" % l, a[l]))
        constants.append(("al%d" % l, orc.ext_mul(D, a[l], lam)))
    return constants, a, lam


def layer_claim(D, a, lam, cp, cq):
    """:53-55"""
    total = [0] * D
    for al, p, q in zip(a, cp, cq):
        total = orc.ext_add(D, total, orc.ext_mul(D, al, orc.ext_add(D, p, orc.ext_mul(D, lam, q))))
    return total


def fold_pair(D, lo, hi, r):
    """:65-66"""
    return orc.ext_add(D, lo, orc.ext_mul(D, r, orc.ext_sub(D, hi, lo)))


def next_claims(D, finals, lookups, tt):
    """:57-63"""
    cp = [fold_pair(D, finals["p0_%d" % l], finals["p1_%d" % l], tt) for l in range(lookups)]
    cq = [fold_pair(D, finals["q0_%d" % l], finals["q1_%d" % l], tt) for l in range(lookups)]
    return cp, cq


def padded_mass(D, rb, k):
    """:68-71"""
    total = [0] * D
    for e in orc.eq_table(D, rb)[k:]:
        total = orc.ext_add(D, total, e)
    return total


def block_weights(D, rb, k):
    """:73-77"""
    if not rb:
        return [[1] + [0] * (D - 1)]
    return orc.eq_table(D, rb)[:k].tolist()


def _fraction_layer(D, p0, p1, q0, q1):
    p0, p1, q0, q1 = (np.ascontiguousarray(a, dtype=np.uint32) for a in (p0, p1, q0, q1))
    p, q = np.zeros_like(p0), np.zeros_like(p0)
    orc.lib().orc_fraction_layer(C.c_int(D), C.c_uint64(len(p0)), orc._ptr(p0), orc._ptr(p1), orc._ptr(q0), orc._ptr(q1),
                                 orc._ptr(p), orc._ptr(q))
    return p, q


def halves_per_block(values, k, size):
    """:190-197: the lower and upper halves of K blocks of 2 SIZE entries."""
    v = values.reshape(k, 2, size, -1)
    return (np.ascontiguousarray(v[:, 0]).reshape(k * size, -1), np.ascontiguousarray(v[:, 1]).reshape(k * size, -1))


def fraction_trees(leaves, n, k):
    """:149-188: the in-block layers (index m: 2^m entries per block) and the top tree (index j: 2^j entries)."""
    D = leaves[0][0].shape[1]
    lk = block_bits(k)
    layers = [None] * (n + 1)
    layers[n] = [(np.ascontiguousarray(p, dtype=np.uint32) % P, np.ascontiguousarray(q, dtype=np.uint32) % P) for p, q in leaves]
    for m in range(n - 1, -1, -1):
        layers[m] = []
        for p, q in layers[m + 1]:
            p0, p1 = halves_per_block(p, k, 1 << m)
            q0, q1 = halves_per_block(q, k, 1 << m)
            layers[m].append(_fraction_layer(D, p0, p1, q0, q1))
    top = [None] * (lk + 1)
    pad = (1 << lk) - k
    one = np.zeros((pad, D), dtype=np.uint32)
    one[:, 0] = 1
    top[lk] = [(np.concatenate([p, np.zeros((pad, D), dtype=np.uint32)]), np.concatenate([q, one])) for p, q in layers[0]]
    for j in range(lk - 1, -1, -1):
        top[j] = []
        for p, q in top[j + 1]:
            h = 1 << j
            top[j].append(_fraction_layer(D, p[:h], p[h:], q[:h], q[h:]))
    return layers, top


def layer_tables(layer, tables, k, size):
    """:199-206"""
    out = []
    for l, (p, q) in enumerate(layer):
        p0, p1 = halves_per_block(p, k, size)
        q0, q1 = halves_per_block(q, k, size)
        out += [(tables[4 * l], p0), (tables[4 * l + 1], p1), (tables[4 * l + 2], q0), (tables[4 * l + 3], q1)]
    return out


def send_finals(tr, finals, tables):
    """:208-213"""
    for name in tables:
        tr.send(np.array([finals[name]], dtype=np.uint32))
    return tr.challenge()


def prove_upper(tr, n, k, leaves, label="gkr", threads=1):
    """:215-272.  Returns (ri, rb, cp, cq)."""
    D = tr.degree
    lookups = len(leaves)
    lk = block_bits(k)
    layers, top = fraction_trees(leaves, n, k)
    statement, tables, _ = layer_statement(lookups)
    for p, q in top[0]:
        tr.send(np.array([p[0], q[0]], dtype=np.uint32))
    cp = [p[0].tolist() for p, _ in top[0]]
    cq = [q[0].tolist() for _, q in top[0]]
    r = []
    for j in range(lk):
        constants, _, _ = layer_challenges(tr, lookups, D)
        rho, finals, _ = orc.prove(tr, j, statement, layer_tables(top[j + 1], tables, 1, 1 << j), eq=r if j > 0 else None,
                                   constants=constants, label=label + "-top", degree=2 if j > 0 else 0, threads=threads)
        tt = send_finals(tr, finals, tables)
        cp, cq = next_claims(D, finals, lookups, tt)
        r = rho + [tt]
    rb, ri = r, []
    if (1 << lk) != k:
        mass = padded_mass(D, rb, k)
        cq = [orc.ext_sub(D, q, mass) for q in cq]
    for layer in range(n - 1):
        constants, _, _ = layer_challenges(tr, lookups, D)
        bw = block_weights(D, rb, k)
        rho, finals, folded = orc.prove(tr, layer, statement, layer_tables(layers[layer + 1], tables, k, 1 << layer),
                                        eq=ri if layer > 0 else None, constants=constants, label=label,
                                        block_weights=bw, degree=2 if layer > 0 else 0, threads=threads)
        rbn = []
        if lk > 0:
            pad = [[0] * D] * ((1 << lk) - k)
            blk_tables = [("bw", np.array(bw + pad, dtype=np.uint32))]
            blk_tables += [(name, np.array(folded[name] + pad, dtype=np.uint32)) for name in tables]
            rbn, finals, _ = orc.prove(tr, lk, "(* bw %s)" % statement, blk_tables, constants=constants, label=label + "-blk",
                                       threads=threads)
        tt = send_finals(tr, finals, tables)
        cp, cq = next_claims(D, finals, lookups, tt)
        ri = rho + [tt]
        rb = rbn
    return ri, rb, cp, cq


class VerificationFailure(Exception):
    """The reference's VERIFICATION-FAILURE (src/conditions.lisp), with the step that failed."""


class _Replay:
    """A verifier's transcript: the proof's messages are absorbed in order as the protocol asks for them."""

    def __init__(self, label, D, messages):
        self.tr = orc.Transcript(label, D)
        self.messages = list(messages)
        self.at = 0

    def take(self, rows, cols):
        if self.at >= len(self.messages) or tuple(self.messages[self.at].shape) != (rows, cols):
            raise VerificationFailure("message %d: expected shape (%d, %d)" % (self.at, rows, cols))
        m = self.messages[self.at]
        self.at += 1
        return m

    def receive(self, rows, cols):
        m = self.take(rows, cols)
        self.tr.send(m)
        return m

    def finished(self):
        return self.at == len(self.messages)


def _verify(rp, n, degree, claim, eq, blocks, label):
    """VERIFY (src/sumcheck.lisp:147-163) on the running transcript."""
    D = rp.tr.degree
    points = max(degree, 1)
    msgs = [rp.take(points, D) for _ in range(n)]
    flat = np.ascontiguousarray(np.concatenate([m.reshape(-1) for m in msgs]) if n else np.zeros(1), dtype=np.uint32)
    eqa = np.ascontiguousarray(np.array(eq, dtype=np.uint32).reshape(-1, D)) if eq else None
    ch = np.zeros((max(n, 1), D), dtype=np.uint32)
    red = np.zeros(D, dtype=np.uint32)
    cl = np.array(claim, dtype=np.uint32)
    orc.lib().orc_verify_tr(rp.tr._h, C.c_int(n), C.c_int(degree), orc._ptr(cl), orc._ptr(eqa) if eqa is not None else None,
                            C.c_int(blocks), label.encode(), orc._ptr(flat), orc._ptr(ch), orc._ptr(red))
    return ch[:n].tolist(), red.tolist()


def _evaluate(D, statement, finals, constants):
    names = [f[0] for f in finals]
    vals = np.array([f[1] for f in finals], dtype=np.uint32).reshape(-1, D)
    cnames = [c[0] for c in constants]
    cvals = np.array([c[1] for c in constants], dtype=np.uint32).reshape(-1, D)
    out = np.zeros(D, dtype=np.uint32)
    rc = orc.lib().orc_evaluate(C.c_int(D), statement.encode(), C.c_int(len(names)), orc._strs(names), orc._ptr(vals),
                                C.c_int(len(cnames)), orc._strs(cnames), orc._ptr(cvals), orc._ptr(out))
    if rc:
        raise ValueError("evaluate: %d" % rc)
    return out.tolist()


def _receive_finals(rp, tables, D):
    """:84-89"""
    finals = [(name, rp.receive(1, D)[0].tolist()) for name in tables]
    return finals, rp.tr.challenge()


def verify_upper(tr_label, D, messages, n, k, lookups, label="gkr"):
    """:91-145.  Returns (roots, ri, rb, cp, cq); raises VerificationFailure."""
    rp = _Replay(tr_label, D, messages)
    out = verify_upper_on(rp, n, k, lookups, label)
    if not rp.finished():
        raise VerificationFailure("messages left over")
    return out


def verify_upper_on(rp, n, k, lookups, label="gkr"):
    """VERIFY-UPPER on a running verifier transcript (a caller such as VERIFY-DOMAIN goes on after it)."""
    D = rp.tr.degree
    lk = block_bits(k)
    roots = []
    for _ in range(lookups):
        m = rp.receive(2, D)
        roots.append((m[0].tolist(), m[1].tolist()))
    cp = [p for p, _ in roots]
    cq = [q for _, q in roots]
    statement, tables, _ = layer_statement(lookups)
    r = []
    for j in range(lk):
        constants, a, lam = layer_challenges(rp.tr, lookups, D)
        rho, reduced = _verify(rp, j, 2 if j > 0 else 0, layer_claim(D, a, lam, cp, cq), r if j > 0 else None, 1, label + "-top")
        finals, tt = _receive_finals(rp, tables, D)
        if reduced != _evaluate(D, statement, finals, constants):
            raise VerificationFailure("gkr-top: layer %d of the top tree" % j)
        cp, cq = next_claims(D, dict(finals), lookups, tt)
        r = rho + [tt]
    rb, ri = r, []
    if (1 << lk) != k:
        mass = padded_mass(D, rb, k)
        cq = [orc.ext_sub(D, q, mass) for q in cq]
    for layer in range(n - 1):
        constants, a, lam = layer_challenges(rp.tr, lookups, D)
        bw = block_weights(D, rb, k)
        rho, reduced = _verify(rp, layer, 2 if layer > 0 else 0, layer_claim(D, a, lam, cp, cq), ri if layer > 0 else None, k, label)
        rbn = []
        if lk > 0:
            rbn, reduced = _verify(rp, lk, 3, reduced, None, 1, label + "-blk")
        finals, tt = _receive_finals(rp, tables, D)
        if k > 1:
            weight = [0] * D
            for w, e in zip(bw, orc.eq_table(D, rbn)):
                weight = orc.ext_add(D, weight, orc.ext_mul(D, w, e))
        else:
            weight = bw[0]
        if reduced != orc.ext_mul(D, weight, _evaluate(D, statement, finals, constants)):
            raise VerificationFailure("gkr-layer: in-block layer %d" % layer)
        cp, cq = next_claims(D, dict(finals), lookups, tt)
        ri = rho + [tt]
        rb = rbn
    return roots, ri, rb, cp, cq
