"""The CPU port on the benchmark's smallest workload at its own size: the recorded proof hash (the one the
device is held to in tests/test_gpu_parity.py)."""
import hashlib

import numpy as np

import bench
from oracle import pyoracle as orc


def test_c1_proof_hash():
    n, d = 20, 4
    tables = [("t%d" % t, orc.generate(bench.SEED, t, 0, 1 << n, 1)) for t in range(2)]
    eq = np.array([bench.seeded_ext(bench.EQ_ID, i, d) for i in range(n)], dtype=np.uint32)
    tr = orc.Transcript("bench", d)
    orc.prove(tr, n, "(* t0 t1)", tables, eq=eq, threads=0)
    assert hashlib.sha256(tr.proof()).hexdigest() == "d486796f96c2cb854fa7bad8a0cc8eafc68aeee6aaa6ba8a90ead994060a8744"
