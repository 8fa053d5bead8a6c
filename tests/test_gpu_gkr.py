"""LogUp-GKR upper layers on the device (sc_gkr_prove_upper) against the CPU restatement
(oracle/gkr_oracle.py): same messages byte for byte, same outputs, and the restated verifier
accepts the device's proof.  Cases of the reference's round trip (tests/tests.lisp:414-442) and
larger ones that reach the split weights, several blocks per SM and the resident last rounds."""
import numpy as np
import pytest

import sable_b200 as sb
from oracle import gkr_oracle as gkr
from oracle import pyoracle as orc

pytestmark = pytest.mark.gpu
P = 2130706433


def random_leaves(lookups, n, k, d, seed):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(lookups):
        p = rng.integers(0, P, size=(k << n, d), dtype=np.uint32)
        q = rng.integers(0, P, size=(k << n, d), dtype=np.uint32)
        q[:, 0] |= 1
        out.append((p, q))
    return out


def both(n, k, lookups, d, seed, threads=1):
    leaves = random_leaves(lookups, n, k, d, seed)
    ta = sb.Transcript("gkr-test", d)
    got = sb.gkr_prove_upper(ta, n, k, leaves)
    tb = orc.Transcript("gkr-test", d)
    want = gkr.prove_upper(tb, n, k, leaves, threads=threads)
    return leaves, ta, got, tb, want


@pytest.mark.parametrize("n,k,lookups,d", [(3, 1, 1, 4), (3, 3, 2, 4), (2, 4, 1, 8), (4, 5, 2, 4), (1, 2, 1, 4), (1, 1, 2, 8),
                                            (2, 2, 3, 4), (9, 1, 1, 4), (7, 6, 2, 8), (14, 3, 2, 4)])
def test_device_proof_is_the_oracles(n, k, lookups, d):
    leaves, ta, got, tb, want = both(n, k, lookups, d, n + k + lookups + d)
    assert got == tuple(want)
    assert ta.proof() == tb.proof()
    roots, ri, rb, cp, cq = gkr.verify_upper("gkr-test", d, ta.messages(), n, k, lookups)
    assert (ri, rb, cp, cq) == got


def test_large_layers_reach_the_bandwidth_kernels():
    # 2^21 leaves per block: the upper layers run the split eq weights and full grids
    n, k, lookups, d = 21, 1, 1, 4
    leaves, ta, got, tb, want = both(n, k, lookups, d, 5, threads=0)
    assert got == tuple(want)
    assert ta.proof() == tb.proof()


def test_words_above_p_are_reduced():
    n, k, d = 4, 2, 4
    leaves = random_leaves(1, n, k, d, 3)
    raised = [(p + np.uint32(P) * (p < 2**32 - P).astype(np.uint32), q) for p, q in leaves]   # the same residues, larger words
    ta, tb = sb.Transcript("gkr-test", d), sb.Transcript("gkr-test", d)
    assert sb.gkr_prove_upper(ta, n, k, leaves) == sb.gkr_prove_upper(tb, n, k, raised)
    assert ta.proof() == tb.proof()
