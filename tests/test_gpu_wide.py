"""Statements wider than one kernel (more than 8 tables, more than 16 terms, or more than four tables
above degree four): sc_prove cuts them into groups of terms on child contexts and adds the groups'
sums per round.  The proof must be the oracle's, byte for byte (the oracle evaluates the statement as
written, whatever its width)."""
import numpy as np
import pytest

import sable_b200 as sb
from oracle import pyoracle as orc

pytestmark = pytest.mark.gpu
P = 2130706433


def run(d, n, statement, names, base=(), constants=(), with_eq=True, blocks=None, seed=0):
    rng = np.random.default_rng(seed)
    K = blocks or 1
    tables = [(nm, rng.integers(0, P, size=(K << n) if nm in base else (K << n, d), dtype=np.uint32)) for nm in names]
    eq = rng.integers(0, P, size=(n, d), dtype=np.uint32) if with_eq else None
    bw = rng.integers(0, P, size=(K, d), dtype=np.uint32) if blocks else None
    consts = [(c, rng.integers(0, P, size=d, dtype=np.uint32).tolist()) for c in constants]
    ta, tb = sb.Transcript("wide", d), orc.Transcript("wide", d)
    got = sb.prove(ta, n, statement, tables, eq=eq, constants=consts, block_weights=bw)
    want = orc.prove(tb, n, statement, tables, eq=eq, constants=consts, block_weights=bw.tolist() if blocks else None)
    assert got[0] == want[0] and got[1] == want[1] and got[2] == want[2]
    assert ta.proof() == tb.proof()


def layer_statement(lookups):
    terms, tables, constants = [], [], []
    for l in range(lookups):
        p0, p1, q0, q1, a, al = ("%s%d" % (nm, l) for nm in ("p0_", "p1_", "q0_", "q1_", "a", "al"))
        tables += [p0, p1, q0, q1]
        constants += [a, al]
        terms += ["(* %s %s %s)" % (a, p0, q1), "(* %s %s %s)" % (a, p1, q0), "(* %s %s %s)" % (al, q0, q1)]
    return "(+ %s)" % " ".join(terms), tables, constants


@pytest.mark.parametrize("lookups,d,n", [(3, 4, 10), (4, 8, 6), (5, 4, 14)])
def test_gkr_layer_statements_of_many_lookups(lookups, d, n):
    statement, tables, constants = layer_statement(lookups)      # 12, 16 and 20 tables (reference src/gkr.lisp:30-41)
    run(d, n, statement, tables, constants=constants, seed=lookups)


def test_ten_tables_mixed():
    names = ["t%d" % i for i in range(10)]
    run(8, 7, "(+ (* t0 t1) (* t2 t3 t4) (* 5 t5 t6) (* t7 t8 t9) (* c t0 t9) t4 -2)", names, base=("t1", "t5", "t8"), constants=("c",), seed=1)


def test_more_than_sixteen_terms():
    names = ["t%d" % i for i in range(6)]
    pairs = ["(* %d t%d t%d)" % (3 + i + 7 * j, i, j) for i in range(6) for j in range(i, 6)]     # 21 terms
    run(4, 9, "(+ %s)" % " ".join(pairs), names, base=("t0",), seed=2)


def test_tables_outside_the_statement_are_folded():
    names = ["t%d" % i for i in range(11)]
    run(4, 8, "(* t1 t7 t10)", names, base=("t7", "t3"), seed=3)


def test_degree_six_over_six_tables():
    names = ["t%d" % i for i in range(6)]
    run(4, 8, "(+ (* t0 t1 t2 t3 t0 t1) (* 9 t4 t5 t4 t5 t4) (* t2 t5))", names, base=("t4",), seed=4)


def test_wide_with_block_weights_and_no_eq():
    statement, tables, constants = layer_statement(3)
    run(4, 5, statement, tables, constants=constants, blocks=3, seed=5)
    run(4, 6, statement, tables, constants=constants, with_eq=False, seed=6)
