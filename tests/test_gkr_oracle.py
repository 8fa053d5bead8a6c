"""The LogUp-GKR restatement (oracle/gkr_oracle.py) against the reference's own invariants
(tests/tests.lisp:414-462): the verifier accepts the prover's messages and returns the prover's
outputs, the roots are the sums of the leaf fractions, the final claims are the leaves' parents at
the returned point, and every forged message is rejected."""
import numpy as np
import pytest

from oracle import gkr_oracle as gkr
from oracle import pyoracle as orc

P = 2130706433
CASES = [(3, 1, 1, 4), (3, 3, 2, 4), (2, 4, 1, 8), (4, 5, 2, 4), (1, 2, 1, 4), (1, 1, 2, 8), (2, 2, 3, 4)]   # tests.lisp:415


def random_leaves(lookups, n, k, d, seed):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(lookups):
        p = rng.integers(0, P, size=(k << n, d), dtype=np.uint32)
        q = rng.integers(0, P, size=(k << n, d), dtype=np.uint32)
        q[:, 0] |= 1          # nonzero denominators
        out.append((p, q))
    return out


def prove(n, k, leaves, d):
    tr = orc.Transcript("gkr-test", d)
    outputs = gkr.prove_upper(tr, n, k, leaves)
    return tr.messages(), outputs


@pytest.mark.parametrize("n,k,lookups,d", CASES)
def test_roundtrip(n, k, lookups, d):
    leaves = random_leaves(lookups, n, k, d, n + k + lookups + d)
    messages, outputs = prove(n, k, leaves, d)
    roots, ri, rb, cp, cq = gkr.verify_upper("gkr-test", d, messages, n, k, lookups)
    assert (ri, rb, cp, cq) == tuple(outputs)
    for (p, q), (rp, rq) in zip(leaves, roots):      # LogUp: each root is the sum of its leaf fractions
        total = [0] * d
        for a, b in zip(p, q):
            total = orc.ext_add(d, total, orc.ext_mul(d, a, orc.ext_inv(d, b)))
        assert orc.ext_mul(d, rp, orc.ext_inv(d, rq)) == total
    layers, _ = gkr.fraction_trees(leaves, n, k)      # the claims are on the leaves' parents
    size = 1 << (n - 1)
    weights = orc.eq_table(d, rb) if rb else np.array([[1] + [0] * (d - 1)], dtype=np.uint32)
    for (p, q), claim_p, claim_q in zip(layers[n - 1], cp, cq):
        for values, claim in ((p, claim_p), (q, claim_q)):
            total = [0] * d
            for b in range(k):
                total = orc.ext_add(d, total, orc.ext_mul(d, weights[b], orc.mle_eval(d, values[b * size:(b + 1) * size], ri)))
            assert total == claim


def test_forgeries_are_rejected():
    n, k, lookups, d = 3, 3, 2, 4                     # tests.lisp:444-462
    messages, _ = prove(n, k, random_leaves(lookups, n, k, d, 9), d)
    assert gkr.verify_upper("gkr-test", d, messages, n, k, lookups)
    for i, m in enumerate(messages):
        forged = [x.copy() for x in messages]
        forged[i].reshape(-1)[0] = (int(forged[i].reshape(-1)[0]) + 1) % P
        with pytest.raises(gkr.VerificationFailure):
            gkr.verify_upper("gkr-test", d, forged, n, k, lookups)
