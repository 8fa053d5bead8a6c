"""The domain restatement (oracle/domain_oracle.py) against the reference's own invariants
(tests/tests.lisp:523-585): the verifier accepts the prover's messages and computes the same claims,
a full column's claim is its multilinear extension at the claimed point, a constraint that does not
hold is rejected, and so is every forged message."""
import numpy as np
import pytest

from oracle import domain_oracle as dom
from oracle import gkr_oracle as gkr
from oracle import pyoracle as orc

P = 2130706433
CASES = [dict(n=3, k=3), dict(n=2, k=1), dict(n=3, k=3, merge=True), dict(n=4, k=4, merge=True), dict(n=3, k=2, lookups=False),
         dict(n=3, k=2, constraints=False), dict(n=2, k=1, merge=True)]          # tests/tests.lisp:524-525


def toy_domain(n=3, k=3, merge=False, lookups=True, constraints=True, seed=5, broken=False):
    """tests/tests.lisp:487-512: every kind of column."""
    rng = np.random.default_rng(seed)
    size = 1 << n
    a = rng.integers(0, 2, size=k * size, dtype=np.uint32)
    b = rng.integers(0, P, size=k * size, dtype=np.uint32)
    c = ((a.astype(np.uint64) * b) % P).astype(np.uint32)
    if broken:
        c[1] = (c[1] + 1) % P
    cols = [dom.Column("a", data=a), dom.Column("b", data=b), dom.Column("c", data=c),
            dom.Column("m", "row", 1, True, rng.integers(0, P, size=1 << (n - 1), dtype=np.uint32)),
            dom.Column("s", "col", n, True, rng.integers(0, 2, size=size, dtype=np.uint32)),
            dom.Column("kb", "row", n, False, rng.integers(0, P, size=k, dtype=np.uint32)),
            dom.Column("w", "col", 2, False, rng.integers(0, P, size=k * 4, dtype=np.uint32))]
    return dom.Domain("12.toy-merged" if merge else "12.toy", n, k, merge, cols,
                      ["(* a (- a 1))", "(- c (* a b))", "(* s (- s 1) m)"] if constraints else [],
                      [dict(tag="5", values=["a", "b"]), dict(tag="7", values=["c", "m", "w"], num="(+ s 2)"), dict(tag="9", values=["kb"])]
                      if lookups else [])


def challenges(d, seed):
    rng = np.random.default_rng(1000 + seed)
    return rng.integers(0, P, size=d, dtype=np.uint32).tolist(), rng.integers(0, P, size=(8, d), dtype=np.uint32).tolist()


def proof(domain, d, z, betas):
    tr = orc.Transcript("dom-test", d)
    claims = dom.prove_domain(tr, domain, z, betas)
    return tr.messages(), claims


def test_the_statement_and_its_degree():
    domain = toy_domain()
    names = [t[0] for t in dom.domain_tables(domain)]
    assert names == ["a@0", "a@1", "b@0", "b@1", "c@0", "c@1", "m@0", "m@1", "s@0", "s@1", "kb", "w"]
    assert dom.domain_degree(domain) == 3 and dom.domain_degree(domain, block_phase=True) == 3
    assert dom.label_name("12.toy") == "toy" and dom.label_name("3.oproj|3.rqo") == "oproj|rqo" and dom.label_name("plain") == "plain"
    text = dom.show(dom.domain_statement(domain))
    assert text.startswith("(+ (* a0 (+ (- z 5 (* beta0 a@0) (* beta1 b@0)) (- z 5 (* beta0 a@1) (* beta1 b@1)))) (* al0 ")
    assert "(* gam2 (* s@0 (- s@0 1) m@0)) (* geta2 (* s@1 (- s@1 1) m@1))" in text


@pytest.mark.parametrize("d", [4, 8])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join("%s%s" % kv for kv in c.items()))
def test_roundtrip(case, d):
    domain = toy_domain(seed=d + case["n"] + case["k"], **case)
    z, betas = challenges(d, d)
    messages, proved = proof(domain, d, z, betas)
    claims, _ = dom.verify_domain("dom-test", d, messages, domain, z, betas)
    assert claims == proved
    n, k = domain.n, domain.blocks
    for (name, point, value), col in zip(claims, domain.columns):
        if col.kind != "full":
            continue
        blocks = col.data.reshape(k, 1 << n)
        if domain.merge:
            weights = orc.eq_table(d, point[n:]).tolist() if k > 1 else [[1] + [0] * (d - 1)]
            total = [0] * d
            for b in range(k):
                total = orc.ext_add(d, total, orc.ext_mul(d, weights[b], orc.mle_eval(d, blocks[b], point[:n])))
            assert value == total
        else:
            for b in range(k):
                assert value[b] == orc.mle_eval(d, blocks[b], point)


@pytest.mark.parametrize("merge", [False, True])
def test_rejects(merge):
    d = 4
    z, betas = challenges(d, 3)
    broken = toy_domain(merge=merge, seed=3, broken=True)
    with pytest.raises(gkr.VerificationFailure):
        dom.verify_domain("dom-test", d, proof(broken, d, z, betas)[0], broken, z, betas)
    domain = toy_domain(merge=merge, seed=4)
    messages, _ = proof(domain, d, z, betas)
    for i, m in enumerate(messages):
        forged = [x.copy() for x in messages]
        forged[i].reshape(-1)[0] = (int(forged[i].reshape(-1)[0]) + 1) % P
        with pytest.raises(gkr.VerificationFailure):
            dom.verify_domain("dom-test", d, forged, domain, z, betas)
