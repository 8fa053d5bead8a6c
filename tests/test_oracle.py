"""The CPU oracle against every known-answer vector the reference holds for the prover path.

These are the pins that make the oracle trustworthy: reference tests/vectors.sexp, read through
tests/golden/vectors.json (see tests/golden/make_golden.py).  The checks follow the reference's own
tests (tests/tests.lisp:45-82 field, :154-184 B3S and transcript, :210-224 proof bytes, :264-282
sumcheck).
"""
import numpy as np
import pytest

from oracle import pyoracle as orc

P = orc.P


def test_ext_vectors(golden):
    assert len(golden["ext"]) == 24
    for v in golden["ext"]:
        d, a, b = v["d"], v["a"], v["b"]
        assert orc.ext_add(d, a, b) == v["add"]
        assert orc.ext_sub(d, a, b) == v["sub"]
        assert orc.ext_mul(d, a, b) == v["mul"]
        assert orc.ext_inv(d, a) == v["inv"]
        assert orc.ext_eq1(d, a, b) == v["eq1"]


def test_pow_vector(golden):
    for v in golden["pow"]:
        assert orc.fpow(v["a"], v["e"]) == v["res"]


def test_lagrange_vectors(golden):
    for v in golden["lagrange"]:
        assert orc.lagrange(v["d"], v["vals"], v["x"]) == v["res"]


def test_eq_vectors(golden):
    for v in golden["eq"]:
        d = v["d"]
        acc = [1] + [0] * (d - 1)
        for a, b in zip(v["a"] or [], v["b"] or []):
            acc = orc.ext_mul(d, acc, orc.ext_eq1(d, a, b))
        assert acc == v["res"]


def test_mle_vectors(golden):
    for v in golden["mle"]:
        d, r = v["d"], v["r"] or []
        assert orc.eq_table(d, r).tolist() == v["eqtab"]
        assert orc.mle_eval(d, np.array(v["base"], dtype=np.uint32), r) == v["base-res"]
        assert orc.mle_eval(d, np.array(v["ext"], dtype=np.uint32), r) == v["ext-res"]


def test_b3s_vectors(golden):
    assert len(golden["b3s"]) == 6
    for v in golden["b3s"]:
        chunks = [bytes.fromhex(c) for c in v["chunks"]]
        assert orc.b3s(chunks, 32).hex() == v["digest"]
        assert orc.b3s(chunks, len(v["xof"]) // 2).hex() == v["xof"]


def test_transcript_vector(golden):
    for v in golden["transcript"]:
        tr = orc.Transcript(bytes.fromhex(v["label"]), 8)
        for op in v["ops"]:
            kind = op[0]
            if kind == "absorb":
                tr.absorb(bytes.fromhex(op[1]))
            elif kind == "absorb-ext":
                tr.absorb(b"".join(int(x).to_bytes(4, "little") for x in op[1]))
            elif kind == "challenge-base":
                assert tr.challenge_base(op[1]) == op[2]
            elif kind == "challenge":
                assert tr.challenge(op[1]) == op[2]
            elif kind == "challenge-bits":
                assert tr.challenge_bits(op[1], op[2]) == op[3]
            elif kind == "digest":
                assert tr.digest(32).hex() == op[1]
            else:
                raise AssertionError(kind)


def test_proofio_field_arrays(golden):
    # the rank-2 field array of the vector, written by the encoder, appears byte for byte in the
    # reference's proof bytes
    v = golden["proofio"][0]
    raw = bytes.fromhex(v["bytes"])
    for kind, *spec in v["msgs"]:
        if kind == "array" and len(spec[0]) == 2 and spec[1]:
            tr = orc.Transcript(b"x", 4)
            tr.send(np.array(spec[1], dtype=np.uint32).reshape(spec[0]))
            enc = tr.proof(b"SABLEPF1")
            assert enc[:8] == b"SABLEPF1" and enc[8:12] == (1).to_bytes(4, "little")
            assert enc[12:] in raw


def test_poly_vector(golden):
    v = golden["poly"][0]
    form = "(- (+ (* (+ c0 3) (- c1 c0) c2) 7) (expt c0 2))"  # reference tests/tests.lisp:107
    terms = orc.expand(form, ["c0", "c1", "c2"])
    # the vector lists Python's term dictionary; the reference compares the polynomials (form=)
    assert sorted([ids, c] for ids, c in terms) == sorted(v["terms"])
    assert [len(ids) for ids, _ in terms] == sorted(len(ids) for ids, _ in terms)  # graded order
    assert orc.statement_degree(form, ["c0", "c1", "c2"]) == v["degree"]
    # a statement evaluated as written gives the vector's value: F at one point is the hypercube sum for n = 0
    vals = [("c0", np.array([11], dtype=np.uint32)), ("c1", np.array([P - 5], dtype=np.uint32)),
            ("c2", np.array([2 ** 30], dtype=np.uint32))]
    assert orc.hypercube_sum(4, 0, form, vals) == [v["eval"], 0, 0, 0]


def sumcheck_case(v):
    d, n = v["d"], v["n"]
    tables = [("t%d" % i, np.array(t, dtype=np.uint32)) for i, t in enumerate(v["tables"])]
    statement = "(* %s)" % " ".join(name for name, _ in tables)
    return d, n, tables, statement, v["eq-r"]


def test_sumcheck_vectors(golden):
    shapes = []
    for v in golden["sumcheck"]:
        d, n, tables, statement, eq = sumcheck_case(v)
        shapes.append((d, n, len(tables), bool(eq)))
        assert orc.hypercube_sum(d, n, statement, tables, eq=eq) == v["claim"]
        for threads in (1, 3):
            tr = orc.Transcript("sc-vec", d)
            rho, finals, _ = orc.prove(tr, n, statement, tables, eq=eq, threads=threads)
            assert rho == v["rho"]
            assert [finals[name] for name, _ in tables] == v["finals"]
            assert tr.proof(b"SABLEPF1").hex() == v["proof"]
        # the verifier replays the proof to the same challenges and reduced claim, and the final check holds
        vrho, reduced = orc.verify("sc-vec", d, n, len(tables), v["claim"], tr.messages(), eq=eq)
        assert vrho == v["rho"] and reduced == v["reduced"]
        assert orc.check_final(d, statement, [(name, finals[name]) for name, _ in tables], reduced)
    assert shapes == [(4, 4, 2, False), (8, 5, 3, True), (8, 3, 1, False), (4, 6, 4, True)]


def rand_ext(rng, d, count=None):
    if count is None:
        return rng.integers(0, P, size=d, dtype=np.uint32)
    return rng.integers(0, P, size=(count, d), dtype=np.uint32)


def test_base_tables_equal_their_lift():
    # reference tests/tests.lisp:329-346: base tables and their lift to F_p^D give the same proof
    for d in (4, 8):
        rng = np.random.default_rng(d)
        n = 4
        statement = "(+ (* t0 t1 t2) (* 7 t1))"
        base = [("t%d" % i, rng.integers(0, P, size=1 << n, dtype=np.uint32)) for i in range(3)]
        lifted = [(name, np.concatenate([a[:, None], np.zeros((1 << n, d - 1), dtype=np.uint32)], axis=1)) for name, a in base]
        eq = rand_ext(rng, d, n)
        out = []
        for tables in (base, lifted):
            tr = orc.Transcript("base", d)
            rho, finals, _ = orc.prove(tr, n, statement, tables, eq=eq)
            out.append((rho, finals, tr.proof()))
        assert out[0] == out[1]


def test_any_statement_is_accepted():
    # reference tests/tests.lisp:311-327: a constant beside the tables, no eq, accepted by the verifier
    d, n = 4, 3
    rng = np.random.default_rng(3)
    statement = "(+ (* alpha t0 t1) (* 3 t1) -2)"
    constants = [("alpha", rand_ext(rng, d))]
    tables = [("t0", rand_ext(rng, d, 1 << n)), ("t1", rand_ext(rng, d, 1 << n))]
    assert orc.statement_degree(statement, ["t0", "t1"], ["alpha"]) == 2
    claim = orc.hypercube_sum(d, n, statement, tables, constants=constants)
    tr = orc.Transcript("any", d)
    rho, finals, _ = orc.prove(tr, n, statement, tables, constants=constants)
    vrho, reduced = orc.verify("any", d, n, 2, claim, tr.messages())
    assert vrho == rho
    assert orc.check_final(d, statement, list(finals.items()), reduced, constants=constants)
    bad = [m.copy() for m in tr.messages()]
    bad[0][0, 0] = (int(bad[0][0, 0]) + 1) % P
    _, reduced_bad = orc.verify("any", d, n, 2, claim, bad)
    assert not orc.check_final(d, statement, list(finals.items()), reduced_bad, constants=constants)


def test_block_weights_and_zero_rounds():
    # n = 0: no round, finals are the entries themselves; block weights: K blocks summed with weights
    d = 4
    rng = np.random.default_rng(9)
    tr = orc.Transcript("z", d)
    t = [("a", rand_ext(rng, d, 1))]
    rho, finals, folded = orc.prove(tr, 0, "a", t, degree=0)
    assert rho == [] and finals["a"] == t[0][1][0].tolist() and tr.messages() == []
    K, n = 3, 3
    bw = rand_ext(rng, d, K)
    tabs = [("a", rand_ext(rng, d, K << n)), ("b", rng.integers(0, P, size=K << n, dtype=np.uint32))]
    eq = rand_ext(rng, d, n)
    tr = orc.Transcript("bw", d)
    rho, finals, folded = orc.prove(tr, n, "(* a b)", tabs, eq=eq, block_weights=bw)
    # the claim: sum_b bw_b sum_x eq(r, x) a b over block b
    claim = [0] * d
    for b in range(K):
        part = orc.hypercube_sum(d, n, "(* a b)", [(nm, a[b << n:(b + 1) << n]) for nm, a in tabs], eq=eq)
        claim = orc.ext_add(d, claim, orc.ext_mul(d, bw[b], part))
    vrho, reduced = orc.verify("bw", d, n, 2, claim, tr.messages(), eq=eq, blocks=K)
    assert vrho == rho
    # the reduced claim is sum_b bw_b F(folded_b)
    acc = [0] * d
    for b in range(K):
        acc = orc.ext_add(d, acc, orc.ext_mul(d, bw[b], orc.ext_mul(d, folded["a"][b], folded["b"][b])))
    assert acc == reduced
    # each folded value is the table's multilinear extension at the challenges
    for b in range(K):
        assert folded["a"][b] == orc.mle_eval(d, tabs[0][1][b << n:(b + 1) << n], rho)
        assert folded["b"][b] == orc.mle_eval(d, tabs[1][1][b << n:(b + 1) << n], rho)
