"""PROVE-DOMAIN on the device (sc_prove_domain: the LogUp-GKR of the lookups, then the sumcheck over the halves of
the columns) against the oracle's restatement of the reference prover (oracle/domain_oracle.py): the same messages,
the same claims, and a proof the restated VERIFY-DOMAIN accepts.  The cases are the reference's
(tests/tests.lisp:523-585) and larger ones."""
import numpy as np
import pytest

import sable_b200 as sb
from oracle import domain_oracle as dom
from oracle import gkr_oracle as gkr
from oracle import pyoracle as orc

from test_host import TOY_CONSTRAINTS, TOY_LOOKUPS, toy_columns

pytestmark = pytest.mark.gpu
P = sb.P
CASES = [dict(n=3, k=3), dict(n=2, k=1), dict(n=3, k=3, merge=True), dict(n=4, k=4, merge=True), dict(n=3, k=2, lookups=False),
         dict(n=3, k=2, constraints=False), dict(n=2, k=1, merge=True), dict(n=9, k=5, merge=True), dict(n=11, k=2)]


def both(case, d, seed):
    n, k, merge = case["n"], case["k"], case.get("merge", False)
    cols = toy_columns(n, k, seed)
    constraints = TOY_CONSTRAINTS if case.get("constraints", True) else []
    lookups = TOY_LOOKUPS if case.get("lookups", True) else []
    rng = np.random.default_rng(77 + seed)
    z, betas = rng.integers(0, P, size=d, dtype=np.uint32).tolist(), rng.integers(0, P, size=(8, d), dtype=np.uint32).tolist()
    mine = sb.Domain("12.toy", n, k, merge, cols, constraints, lookups)
    theirs = dom.Domain("12.toy", n, k, merge, [dom.Column(nm, kind, c, sh, data) for nm, kind, c, sh, data in cols], constraints, lookups)
    ta, tb = sb.Transcript("dom-test", d), orc.Transcript("dom-test", d)
    got = sb.prove_domain(ta, mine, z, betas)
    want = dom.prove_domain(tb, theirs, z, betas, threads=0)
    return got, want, ta, tb, theirs, z, betas


@pytest.mark.parametrize("d", [4, 8])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join("%s%s" % kv for kv in c.items()))
def test_device_domain_proof_is_the_oracle_s(case, d):
    got, want, ta, tb, theirs, z, betas = both(case, d, d + case["n"] + case["k"])
    assert got == want, "claims"
    assert ta.proof() == tb.proof() and ta.digest(32) == tb.digest(32)
    claims, _ = dom.verify_domain("dom-test", d, ta.messages, theirs, z, betas)      # the restated verifier accepts the device's proof
    assert claims == got


def test_forged_device_proofs_are_rejected():
    d = 4
    got, want, ta, tb, theirs, z, betas = both(dict(n=3, k=3, merge=True), d, 4)
    messages = ta.messages
    for i in range(len(messages)):
        forged = [m.copy() for m in messages]
        forged[i].reshape(-1)[0] = (int(forged[i].reshape(-1)[0]) + 1) % P
        with pytest.raises(gkr.VerificationFailure):
            dom.verify_domain("dom-test", d, forged, theirs, z, betas)
