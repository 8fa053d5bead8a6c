"""sc_round_sums_static: one round's sums with nothing allocated, against sc_round and the oracle.

Some callers may not allocate device memory where they run (a stream capture in progress, a
memory pool already handed out in full, a plug-in without an allocator).  For them the library has
one entry point whose only scratch is a fixed array inside the library.  This test calls it
through the C ABI on tables that live in torch tensors, twice in a row (the second call finds
the array as the first one left it), and checks every word against the context's own
sc_round on the same tables, statement and (absent) eq weights, and against the first round
message of the CPU oracle's proof of the same inputs.  The results are integers: the comparison
is exact.  It runs alone in a fresh process as well as after the other tests.
"""
import numpy as np
import pytest

import sable_b200 as sb
from oracle import pyoracle as orc

pytestmark = pytest.mark.gpu
P = sb.P


def reference_sums(prover, d, statement, names, tables, n):
    degree, terms = sb.lower_statement(statement, d, names)
    prover.set_statement(d, max(degree, 1), len(names), terms)
    for slot, t in enumerate(tables):
        prover.upload_table(slot, t)
    prover.begin(n, eq=None)
    return prover.round(), max(degree, 1), terms


@pytest.mark.parametrize("d,n,statement,strides", [
    (4, 18, "(+ (* t0 t3) (* t1 t2) (* 5 t2 t3))", [1, 1, 4, 4]),
    (4, 9, "(* t0 t1 t2)", [1, 1, 1]),
    (8, 12, "(+ (* 7 t0 t1) t1 -3)", [8, 1]),
    # five and seven tables run the kernels built for six and eight: the spare position must point at a real table
    (4, 10, "(+ (* t0 t1) (* t1 t2) (* t2 t3) (* t3 t4) (* 3 t4 t0))", [1, 4, 4, 1, 4]),
    (4, 10, "(+ (* t0 t1) (* t2 t3) (* t4 t5) (* t6 t0) -1)", [4, 1, 4, 4, 1, 4, 4]),
    (4, 20, "(* t0 t1)", [1, 1]),      # more chunks of pairs than blocks: every block sums several
])
def test_static_round_equals_the_context_round(d, n, statement, strides):
    import torch
    prover = sb.Prover(0)
    try:
        names = ["t%d" % i for i in range(len(strides))]
        stream = torch.cuda.current_stream().cuda_stream
        for call in range(2):      # two calls in a row share the scratch array
            rng = np.random.default_rng(100 * n + call)
            tables = [rng.integers(0, P, size=(1 << n) if s == 1 else (1 << n, s), dtype=np.uint32) for s in strides]
            want, points, terms = reference_sums(prover, d, statement, names, tables, n)
            dev = [torch.from_numpy(t.view(np.int32)).cuda() for t in tables]
            out = torch.full((points * d,), -1, dtype=torch.int32, device="cuda")
            torch.cuda.synchronize()
            sb.round_sums_static(d, points, [t.data_ptr() for t in dev], strides, 1 << n, terms, out.data_ptr(), stream)
            torch.cuda.synchronize()
            got = out.cpu().numpy().view(np.uint32).reshape(points, d)
            assert got.tolist() == want.tolist(), "call %d" % call
            tr = orc.Transcript("static", d)
            orc.prove(tr, n, statement, list(zip(names, tables)), threads=0)
            assert got.tolist() == tr.messages()[0].tolist(), "call %d against the oracle" % call
    finally:
        prover.close()


def test_static_round_refuses_what_its_scratch_cannot_hold():
    import torch
    t = torch.zeros(16, dtype=torch.int32, device="cuda")
    out = torch.zeros(8, dtype=torch.int32, device="cuda")
    terms = [([1, 0, 0, 0], [0, 1])]
    with pytest.raises(sb.InvalidParameter) as e:     # 2^29 entries: beyond the 2^28 the fixed array covers
        sb.round_sums_static(4, 2, [t.data_ptr(), t.data_ptr()], [1, 1], 1 << 29, terms, out.data_ptr())
    assert e.value.code == -1 and "268435456" in str(e.value)      # the message names the limit
    with pytest.raises(sb.InvalidParameter):          # an odd number of entries has no pairs
        sb.round_sums_static(4, 2, [t.data_ptr(), t.data_ptr()], [1, 1], 7, terms, out.data_ptr())


def test_static_round_refuses_misaligned_tables_without_launching():
    import torch
    buf = torch.zeros(64, dtype=torch.int32, device="cuda")
    out = torch.full((8,), -1, dtype=torch.int32, device="cuda")
    terms = [([1, 0, 0, 0], [0, 1])]
    with pytest.raises(sb.InvalidParameter) as e:     # a table that starts 4 bytes into an allocation
        sb.round_sums_static(4, 2, [buf.data_ptr() + 4, buf.data_ptr()], [1, 1], 16, terms, out.data_ptr())
    assert "16-byte" in str(e.value)
    with pytest.raises(sb.InvalidParameter):          # sums at an odd address
        sb.round_sums_static(4, 2, [buf.data_ptr(), buf.data_ptr()], [1, 1], 16, terms, out.data_ptr() + 2)
    torch.cuda.synchronize()
    assert (out.cpu().numpy() == -1).all()            # nothing ran
