"""The host side of the library, without a GPU: the C ABI loads and exports what the header
declares, and the transcript, the statement compiler and the proof bytes agree with the
reference's vectors (tests/golden/vectors.json) and with the oracle."""
import ctypes
import os
import re

import numpy as np
import pytest

import sable_b200 as sb
from oracle import pyoracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
P = sb.P


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "sumcheck_b200.h")).read()
    declared = set(re.findall(r"\b(sc_[a-z0-9_]+)\s*\(", header))
    assert declared == set(sb.SYMBOLS)
    lib = sb.library()
    for name in sorted(declared):
        assert getattr(lib, name) is not None, name


def test_error_texts():
    lib = sb.library()
    assert lib.sc_strerror(0) == b"ok"
    for code in range(-7, 0):
        assert lib.sc_strerror(code) not in (b"ok", b"unknown error")
    assert lib.sc_strerror(-99) == b"unknown error"


def test_bad_extension_degree_is_rejected():
    # reference tests/tests.lisp:92: (make-transcript "x" 5) signals INVALID-PARAMETER
    with pytest.raises(sb.InvalidParameter):
        sb.Transcript("x", 5)


def test_transcript_vector(golden):
    for v in golden["transcript"]:
        tr = sb.Transcript(bytes.fromhex(v["label"]), 8)
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


def test_transcript_matches_oracle_on_random_traffic():
    rng = np.random.default_rng(5)
    for d in (4, 8):
        a, b = sb.Transcript("t", d), orc.Transcript("t", d)
        for step in range(40):
            if step % 3 == 0:
                data = rng.integers(0, 256, size=int(rng.integers(0, 200)), dtype=np.uint8).tobytes()
                a.absorb(data); b.absorb(data)
            elif step % 3 == 1:
                m = rng.integers(0, P, size=(int(rng.integers(1, 5)), d), dtype=np.uint32)
                a.send(m); b.send(m)
            else:
                assert a.challenge() == b.challenge()
        assert a.digest(64) == b.digest(64)
        assert a.proof() == b.proof()
        assert a.sent_bytes == b.sent_bytes()


def test_proof_bytes_of_the_sumcheck_vectors(golden):
    # replaying a vector's round messages through SEND reproduces its proof bytes and challenges
    for v in golden["sumcheck"]:
        d, n, k = v["d"], v["n"], len(v["tables"])
        raw = bytes.fromhex(v["proof"])
        words = np.frombuffer(raw[12:], dtype=np.uint8)
        tr = sb.Transcript("sc-vec", d)
        tr.absorb(b"sc|" + n.to_bytes(2, "little") + k.to_bytes(2, "little") + (1).to_bytes(4, "little"))
        pos, rho = 0, []
        for _ in range(n):
            pos += 18
            m = np.frombuffer(words[pos:pos + 4 * k * d].tobytes(), dtype="<u4").reshape(k, d)
            pos += 4 * k * d
            tr.send(m)
            rho.append(tr.challenge())
        assert rho == v["rho"]
        assert tr.proof(b"SABLEPF1") == raw


def test_send_rejects_values_not_below_p():
    tr = sb.Transcript("x", 4)
    with pytest.raises(sb.InvalidParameter):
        tr.send(np.array([[P, 0, 0, 0]], dtype=np.uint32))


def test_lowering_matches_the_poly_vector(golden):
    v = golden["poly"][0]
    form = "(- (+ (* (+ c0 3) (- c1 c0) c2) 7) (expt c0 2))"  # reference tests/tests.lisp:107
    degree, terms = sb.lower_statement(form, 4, ["c0", "c1", "c2"])
    assert degree == v["degree"]
    assert sorted([idx, c[0]] for c, idx in terms) == sorted(v["terms"])
    assert all(c[1:] == [0, 0, 0] for c, _ in terms)


def test_lowering_folds_constants_into_coefficients():
    rng = np.random.default_rng(1)
    alpha = rng.integers(0, P, size=4, dtype=np.uint32).tolist()
    degree, terms = sb.lower_statement("(+ (* alpha t0 t1) (* 3 t1) -2)", 4, ["t0", "t1"], [("alpha", alpha)])
    assert degree == 2
    assert sorted(terms, key=lambda t: t[1]) == [([P - 2, 0, 0, 0], []), ([alpha[0], alpha[1], alpha[2], alpha[3]], [0, 1]),
                                                ([3, 0, 0, 0], [1])]
    # powers repeat the table; a product of constants is one coefficient
    beta = rng.integers(0, P, size=4, dtype=np.uint32).tolist()
    degree, terms = sb.lower_statement("(- (* alpha beta (expt t0 2) t1) t1)", 4, ["t0", "t1"], [("alpha", alpha), ("beta", beta)])
    assert degree == 3
    ab = orc.ext_mul(4, alpha, beta)
    assert sorted(terms, key=lambda t: len(t[1])) == [([P - 1, 0, 0, 0], [1]), (ab, [0, 0, 1])]
    # terms that cancel disappear, but the degree is that of the form
    degree, terms = sb.lower_statement("(- (* 2 t0) t0 t0)", 4, ["t0"])
    assert (degree, terms) == (0, [])


def test_lowering_agrees_with_the_oracle_degree():
    cases = ["(* t0 t1 t2)", "(+ (* t0 t1 t2) (* 7 t1) -1)", "t0", "(- (expt t0 3) (* t0 t1))", "(* t0 t1 t2 t3)",
             "(+ (* t0 t3) (* t1 t2) (* lam t2 t3))", "(* (+ t0 1) (- t1 lam))"]
    for form in cases:
        tables = [t for t in ("t0", "t1", "t2", "t3") if t in form]
        consts = [("lam", [5, 6, 7, 8])] if "lam" in form else []
        degree, _ = sb.lower_statement(form, 4, tables, consts)
        assert degree == orc.statement_degree(form, tables, [c[0] for c in consts])


def test_bad_statements_are_rejected():
    for form in ["(/ a b)", "(* a", "(expt a -1)", "(* a b) c", ""]:
        with pytest.raises(sb.InvalidParameter):
            sb.lower_statement(form, 4, ["a", "b", "c"])
    with pytest.raises(sb.InvalidParameter):   # a free variable (reference tests/tests.lisp:139)
        sb.lower_statement("(* a b)", 4, ["a"])


def test_no_device_means_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(sb.SumcheckError):
        sb.Prover(0)


def test_gkr_and_helpers_reject_bad_arguments_without_a_device():
    # argument checks come before any CUDA call: no context, no lookups, no leaves, n < 1
    lib = sb.library()
    tr = sb.Transcript("x", 4)
    h = ctypes.c_void_p(tr._h)
    assert lib.sc_gkr_prove_upper(None, 1, h, 3, 1, None, None, 0, b"gkr", None, None, None, None) == -1
    ctxs = (ctypes.c_void_p * 1)(None)
    ptrs = (ctypes.POINTER(ctypes.c_uint32) * 1)()
    assert lib.sc_gkr_prove_upper(ctxs, 0, h, 3, 1, ptrs, ptrs, 0, b"gkr", None, None, None, None) == -1
    assert lib.sc_gkr_prove_upper(ctxs, 1, h, 0, 1, ptrs, ptrs, 0, b"gkr", None, None, None, None) == -1
    assert lib.sc_gkr_prove_upper(ctxs, 1, h, 3, 1, ptrs, ptrs, 0, b"gkr", None, None, None, None) == -1   # null context
    out = ctypes.c_void_p()
    assert lib.sc_borrow_table(None, 0, None, ctypes.c_uint64(4), 4) == -1
    assert lib.sc_reserve(None, 4, 3, 1, 4) == -1
    assert lib.sc_workspace(None, ctypes.c_uint64(16), ctypes.byref(out)) == -1
    assert lib.sc_child(None, 0, ctypes.byref(out)) == -1
    assert lib.sc_attach_transcript(None, h) == -1
    assert lib.sc_transcript_degree(h) == 4
    cv = (ctypes.c_uint32 * 8)(); pend = (ctypes.c_uint32 * 16)(); fill = ctypes.c_int(); blocks = ctypes.c_uint64()
    assert lib.sc_transcript_state(h, cv, pend, ctypes.byref(fill), ctypes.byref(blocks)) == 0
    assert 0 < fill.value <= 64 and blocks.value == 0          # "LLM-SUMCHECK-v6-O|x": 19 bytes pending, nothing compressed yet
    assert bytes(pend)[:fill.value] == b"LLM-SUMCHECK-v6-O|x"


def device_state(tr):
    """The transcript's hash state in the device's layout (32 words)."""
    lib = sb.library()
    cv = (ctypes.c_uint32 * 8)(); pend = (ctypes.c_uint32 * 16)(); fill = ctypes.c_int(); blocks = ctypes.c_uint64()
    assert lib.sc_transcript_state(ctypes.c_void_p(tr._h), cv, pend, ctypes.byref(fill), ctypes.byref(blocks)) == 0
    return list(cv) + list(pend) + [fill.value, blocks.value & 0xffffffff, blocks.value >> 32]


@pytest.mark.parametrize("d", [4, 8])
def test_device_transcript_code_follows_the_host_transcript(d):
    # the code the round kernels' last block runs (transcript.cuh), executed on the host: after any prefix, SEND of a
    # round message and CHALLENGE give the host transcript's challenge and leave the same hash state -- whatever
    # the byte offset inside the pending block, for every message size, over chains of rounds
    lib = sb.library()
    rng = np.random.default_rng(d)
    for trial in range(40):
        tr = sb.Transcript("dev-%d" % trial, d)
        tr.absorb(bytes(rng.integers(0, 256, size=int(rng.integers(0, 200)), dtype=np.uint8)))
        for rnd in range(12):
            rows = int(rng.integers(1, 9))
            values = rng.integers(0, P, size=(rows, d), dtype=np.uint32)
            state = (ctypes.c_uint32 * 32)()
            chal = (ctypes.c_uint32 * 8)()
            assert lib.sc_transcript_device_round(ctypes.c_void_p(tr._h), values.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)),
                                                  rows, d, state, chal) == 0
            tr.send(values)
            assert list(chal)[:d] == tr.challenge(), (trial, rnd)
            assert list(state)[:27] == device_state(tr), (trial, rnd)


def test_device_transcript_code_against_the_oracle_transcript():
    # the same through the oracle's transcript (pinned by the reference's :transcript and :b3s vectors)
    lib = sb.library()
    d = 4
    ta, tb = sb.Transcript("sc-vec", d), orc.Transcript("sc-vec", d)
    rng = np.random.default_rng(9)
    for rnd in range(30):
        values = rng.integers(0, P, size=(3, d), dtype=np.uint32)
        chal = (ctypes.c_uint32 * 8)()
        assert lib.sc_transcript_device_round(ctypes.c_void_p(ta._h), values.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), 3, d, None, chal) == 0
        ta.send(values); tb.send(values)
        want = tb.challenge()
        assert ta.challenge() == want and list(chal)[:d] == want


def toy_columns(n, k, seed=5):
    """The reference's toy domain (tests/tests.lisp:487-512): every kind of column."""
    rng = np.random.default_rng(seed)
    size = 1 << n
    a = rng.integers(0, 2, size=k * size, dtype=np.uint32)
    b = rng.integers(0, P, size=k * size, dtype=np.uint32)
    c = ((a.astype(np.uint64) * b) % P).astype(np.uint32)
    return [("a", "full", 0, False, a), ("b", "full", 0, False, b), ("c", "full", 0, False, c),
            ("m", "row", 1, True, rng.integers(0, P, size=1 << (n - 1), dtype=np.uint32)),
            ("s", "col", n, True, rng.integers(0, 2, size=size, dtype=np.uint32)),
            ("kb", "row", n, False, rng.integers(0, P, size=k, dtype=np.uint32)),
            ("w", "col", 2, False, rng.integers(0, P, size=k * 4, dtype=np.uint32))]


TOY_CONSTRAINTS = ["(* a (- a 1))", "(- c (* a b))", "(* s (- s 1) m)"]
TOY_LOOKUPS = [dict(tag="5", values=["a", "b"]), dict(tag="7", values=["c", "m", "w"], num="(+ s 2)"), dict(tag="9", values=["kb"])]


@pytest.mark.parametrize("n,k,merge,lookups,constraints", [(3, 3, False, True, True), (2, 1, True, True, True), (4, 4, True, True, False),
                                                         (3, 2, False, False, True), (5, 3, False, True, True)])
def test_domain_statement_and_degree_match_the_oracle(n, k, merge, lookups, constraints):
    # DOMAIN-STATEMENT, DOMAIN-TABLES and DOMAIN-DEGREE (reference src/domain.lisp:60-156): the library's text and degrees
    # against the oracle's restatement, form for form
    from oracle import domain_oracle as dom
    cols = toy_columns(n, k)
    mine = sb.Domain("12.toy", n, k, merge, cols, TOY_CONSTRAINTS if constraints else [], TOY_LOOKUPS if lookups else [])
    theirs = dom.Domain("12.toy", n, k, merge, [dom.Column(nm, kind, c, sh, data) for nm, kind, c, sh, data in cols],
                        TOY_CONSTRAINTS if constraints else [], TOY_LOOKUPS if lookups else [])
    text, ntables, degree, block_degree = mine.statement()
    assert text == dom.show(dom.domain_statement(theirs))
    assert ntables == len(dom.domain_tables(theirs))
    assert degree == dom.domain_degree(theirs) and block_degree == dom.domain_degree(theirs, block_phase=True)


def test_domain_arguments_are_checked():
    cols = toy_columns(3, 2)
    with pytest.raises(sb.InvalidParameter):          # n at least 2 (reference src/domain.lisp:44)
        sb.Domain("d", 1, 2, False, cols, [], []).statement()
    with pytest.raises(sb.InvalidParameter):          # a :full column is never shared (:48-49)
        sb.Domain("d", 3, 2, False, [("a", "full", 0, True, cols[0][4])], [], []).statement()
    with pytest.raises(sb.InvalidParameter):          # a form that does not read
        sb.Domain("d", 3, 2, False, cols, ["(* a (- a 1)"], []).statement()
