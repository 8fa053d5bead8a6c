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
    roots, ri, rb, cp, cq = gkr.verify_upper("gkr-test", d, ta.messages, n, k, lookups)
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


def test_leaves_on_the_device_give_the_same_proof():
    import torch
    n, k, lookups, d = 10, 3, 2, 4
    leaves = random_leaves(lookups, n, k, d, 11)
    dev = [(torch.from_numpy(p.view(np.int32)).cuda(), torch.from_numpy(q.view(np.int32)).cuda()) for p, q in leaves]
    ta, tb = sb.Transcript("gkr-test", d), sb.Transcript("gkr-test", d)
    assert sb.gkr_prove_upper(ta, n, k, leaves) == sb.gkr_prove_upper(tb, n, k, dev)
    assert ta.proof() == tb.proof()
    for (p, q), (dp, dq) in zip(leaves, dev):      # the caller's leaves are only read
        assert (dp.cpu().numpy().view(np.uint32) == p).all() and (dq.cpu().numpy().view(np.uint32) == q).all()


def test_borrowed_tables_prove_like_uploaded_ones():
    # sc_borrow_table: round 0 reads the caller's device memory where it lies; the proof is the uploaded tables' proof
    import torch
    d, n = 4, 13
    rng = np.random.default_rng(8)
    tables = [("t%d" % i, rng.integers(0, P, size=(1 << n, d), dtype=np.uint32)) for i in range(4)]
    eq = rng.integers(0, P, size=(n, d), dtype=np.uint32)
    statement = "(+ (* t0 t3) (* t1 t2) (* 7 t2 t3))"
    prover = sb.Prover(0)
    try:
        ta = sb.Transcript("borrow", d)
        want = sb.prove(ta, n, statement, tables, eq=eq, prover=prover)
        dev = [torch.from_numpy(t.view(np.int32)).cuda() for _, t in tables]
        torch.cuda.synchronize()
        for rep in range(2):                         # twice: the borrowed tables are left as they were
            for slot, t in enumerate(dev):
                prover.borrow_table(slot, t.data_ptr(), 1 << n, d)
            tb = sb.Transcript("borrow", d)
            got = sb.prove(tb, n, statement, [(nm, sb.DeviceTable(d)) for nm, _ in tables], eq=eq, prover=prover)
            assert got == want and tb.proof() == ta.proof()
        for (_, t), dt in zip(tables, dev):
            assert (dt.cpu().numpy().view(np.uint32) == t).all()
        prover.upload_table(0, tables[0][1])         # a slot goes back to memory of the context's own
        tb = sb.Transcript("borrow", d)
        assert sb.prove(tb, n, statement, [(nm, sb.DeviceTable(d)) for nm, _ in tables], eq=eq, prover=prover) == want
    finally:
        prover.close()


def test_one_lookup_with_the_device_transcript():
    # with one lookup every layer's rounds are enqueued at once, the kernels drawing the challenges themselves
    prover = sb.Prover(0)
    prover.set_device_transcript(True)
    try:
        for n, k, d in ((9, 1, 4), (6, 3, 8), (16, 1, 4)):
            leaves = random_leaves(1, n, k, d, 21 + n)
            ta, tb = sb.Transcript("gkr-test", d), orc.Transcript("gkr-test", d)
            got = sb.gkr_prove_upper(ta, n, k, leaves, provers=[prover])
            want = gkr.prove_upper(tb, n, k, leaves, threads=0)
            assert got == tuple(want)
            assert ta.proof() == tb.proof()
    finally:
        prover.close()


def test_device_roots_are_the_sums_of_the_leaf_fractions():
    # reference tests/tests.lisp:423-427 on the device's messages: each root is the sum of its leaf fractions
    n, k, lookups, d = 4, 3, 2, 4
    leaves = random_leaves(lookups, n, k, d, 31)
    ta = sb.Transcript("gkr-test", d)
    sb.gkr_prove_upper(ta, n, k, leaves)
    roots = [(m[0].tolist(), m[1].tolist()) for m in ta.messages[:lookups]]
    for (p, q), (rp, rq) in zip(leaves, roots):
        total = [0] * d
        for a, b in zip(p, q):
            total = orc.ext_add(d, total, orc.ext_mul(d, a.tolist(), orc.ext_inv(d, b.tolist())))
        assert orc.ext_mul(d, rp, orc.ext_inv(d, rq)) == total


@pytest.mark.parametrize("n,k,lookups,d", [(3, 3, 2, 4), (4, 1, 1, 8)])
def test_forged_device_proofs_are_rejected(n, k, lookups, d):
    # reference tests/tests.lisp:444-462 (test-gkr-rejects-forgeries) on the device's messages: one changed word in any message and the verifier rejects
    leaves = random_leaves(lookups, n, k, d, 41)
    ta = sb.Transcript("gkr-test", d)
    sb.gkr_prove_upper(ta, n, k, leaves)
    messages = ta.messages
    gkr.verify_upper("gkr-test", d, messages, n, k, lookups)
    for i in range(len(messages)):
        forged = [m.copy() for m in messages]
        forged[i].reshape(-1)[0] = (int(forged[i].reshape(-1)[0]) + 1) % P
        with pytest.raises(gkr.VerificationFailure):
            gkr.verify_upper("gkr-test", d, forged, n, k, lookups)
