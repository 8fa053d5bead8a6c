"""One rank of the multi-GPU parity test (run by tests/test_gpu_multi.py, one process per GPU).

usage: multi_gpu_worker.py RANK WORLD ID_FILE OUT_FILE
Each rank holds its slice of every table (the top log2(WORLD) variables select the rank), proves
through the C ABI with an NCCL communicator, and rank 0 compares with the oracle on the whole tables.
"""
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import sable_b200 as sb  # noqa: E402

P = sb.P
CASES = [
    # d, n, statement, table strides (1 base, 0 extension), constants, eq
    (4, 12, "(+ (* t0 t3) (* t1 t2) (* lam t2 t3))", [1, 1, 0, 0], ["lam"], True),
    (4, 9, "(* t0 t1 t2)", [1, 1, 1], [], True),
    (8, 7, "(+ (* alpha t0 t1) (* 3 t1) -2)", [0, 1], ["alpha"], False),
    (4, 3, "(* t0 t1)", [0, 0], [], True),
    (4, 17, "(+ (* t0 t3) (* t1 t2) (* lam t2 t3))", [1, 1, 0, 0], ["lam"], True),   # sharded rounds before the gather
    (4, 23, "(* t0 t1 t2)", [1, 1, 1], [], True),   # large enough for the small-value rounds on every rank
    (4, 24, "(* t0 t1)", [1, 1], [], True),         # degree two: three small-value rounds on two ranks, two on four
    (8, 23, "(* t0 t1 t2)", [1, 1, 1], [], True),   # 128 words of small-value accumulators per rank
]


def lost_rank(prover, rank, out_file, withheld=False):
    """Rank 1 leaves between two rounds (or, WITHHELD, stays but never runs its next round); rank 0's next
    exchange must end with SC_ECOMM, not hang."""
    d, n = 4, 20
    rng = np.random.default_rng(3)
    size = (1 << n) // 2
    tables = [rng.integers(0, P, size=1 << n, dtype=np.uint32)[rank * size:(rank + 1) * size] for _ in range(2)]
    degree, terms = sb.lower_statement("(* a b)", d, ["a", "b"])
    prover.set_statement(d, 2, 2, terms)
    for slot, t in enumerate(tables):
        prover.upload_table(slot, t)
    prover.begin(n, eq=rng.integers(0, P, size=(n, d), dtype=np.uint32))
    tr = sb.Transcript("lost", d)
    for _ in range(2):
        tr.send(prover.round())
        prover.challenge(tr.challenge())
    if rank == 1 and withheld:
        # alive, its mailbox still there, but no round: rank 0's kernel runs out of polls.  Leave only once rank 0
        # has reported (it has closed its view of this rank's memory by then)
        other = out_file.replace("out1", "out0")
        deadline = time.time() + 90
        while not os.path.exists(other) and time.time() < deadline:
            time.sleep(0.05)
        json.dump({"withheld": True}, open(out_file, "w"))
        os._exit(0)
    if rank == 1:
        json.dump({"left": True}, open(out_file, "w"))
        os._exit(0)      # between rounds, nothing of this rank in flight
    result = {"code": 0}
    t0 = time.time()
    try:
        prover.round()
    except sb.SumcheckError as e:
        result = {"code": e.code, "seconds": time.time() - t0, "text": str(e)}
    # the context is usable again, on its own GPU
    small = [rng.integers(0, P, size=16, dtype=np.uint32) for _ in range(2)]
    tr2 = sb.Transcript("after", d)
    sb.prove(tr2, 4, "(* a b)", [("a", small[0]), ("b", small[1])], prover=prover)
    result["after"] = len(tr2.messages)
    prover.close()
    with open(out_file + ".tmp", "w") as f:
        json.dump(result, f)
    os.rename(out_file + ".tmp", out_file)


def main():
    rank, world, id_file, out_file = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    logw = world.bit_length() - 1
    prover = sb.Prover(rank)
    if rank == 0:
        with open(id_file + ".tmp", "wb") as f:
            f.write(sb.comm_unique_id())
        os.rename(id_file + ".tmp", id_file)
    deadline = time.time() + 60
    while not os.path.exists(id_file):
        if time.time() > deadline:
            raise SystemExit("no communicator id after 60 s")
        time.sleep(0.05)
    prover.comm_init(open(id_file, "rb").read(), rank, world)
    if len(sys.argv) > 5 and sys.argv[5] in ("lost-rank", "withheld-round"):
        return lost_rank(prover, rank, out_file, withheld=sys.argv[5] == "withheld-round")
    results = []
    for d, n, statement, strides, consts, with_eq in CASES + [(4, logw, "(* t0 t1)", [1, 0], [], True)]:
        rng = np.random.default_rng(1000 + n)     # the same stream on every rank
        full = [("t%d" % t, rng.integers(0, P, size=1 << n, dtype=np.uint32) if s == 1 else rng.integers(0, P, size=(1 << n, d), dtype=np.uint32))
                for t, s in enumerate(strides)]
        constants = [(c, rng.integers(0, P, size=d, dtype=np.uint32).tolist()) for c in consts]
        eq = rng.integers(0, P, size=(n, d), dtype=np.uint32) if with_eq else None
        size = (1 << n) >> logw
        mine = [(name, a[rank * size:(rank + 1) * size]) for name, a in full]
        tr = sb.Transcript("multi", d)
        # the Python face checks table sizes against n; the slices go through the device layer
        degree, terms = sb.lower_statement(statement, d, [nm for nm, _ in full], constants)
        points = max(degree, 1)
        prover.set_statement(d, points, len(full), terms)
        for slot, (_, a) in enumerate(mine):
            prover.upload_table(slot, a)
        prover.begin(n, eq=eq)
        prover.attach_transcript(tr)      # used only when the device carries the transcript (SABLE_B200_DEVICE_TRANSCRIPT=1)
        tr.absorb(b"sc|" + n.to_bytes(2, "little") + degree.to_bytes(2, "little") + (1).to_bytes(4, "little"))
        rho = []
        for _ in range(n):
            sums = prover.round()
            tr.send(sums)
            r = tr.challenge()
            rho.append(r)
            prover.challenge(r)
        finals = prover.finish(len(full))[:, 0, :].tolist()
        prover.attach_transcript(None)
        if rank == 0:
            from oracle import pyoracle as orc
            tb = orc.Transcript("multi", d)
            want = orc.prove(tb, n, statement, full, eq=eq, constants=constants, threads=0)
            ok = rho == want[0] and finals == [want[1][nm] for nm, _ in full] and tr.proof() == tb.proof()
            results.append({"case": statement, "n": n, "d": d, "ok": bool(ok)})
        else:
            results.append({"proof": tr.proof().hex(), "finals": finals})
    # block weights: every rank holds its slice of every block, block after block (reference :block-weights,
    # src/sumcheck.lisp:519-525, 549-551); sharded rounds before the gather at n = 16, the gather at once at n = 6
    for d, K, n in ((4, 3, 16), (8, 2, 6)):
        rng = np.random.default_rng(2000 + n)
        statement, names = "(+ (* a b) (* lam b c))", ["a", "b", "c"]
        full = [("a", rng.integers(0, P, size=(K << n, d), dtype=np.uint32)), ("b", rng.integers(0, P, size=K << n, dtype=np.uint32)),
                ("c", rng.integers(0, P, size=(K << n, d), dtype=np.uint32))]
        constants = [("lam", rng.integers(0, P, size=d, dtype=np.uint32).tolist())]
        eq = rng.integers(0, P, size=(n, d), dtype=np.uint32)
        bw = rng.integers(0, P, size=(K, d), dtype=np.uint32)
        size = (1 << n) >> logw
        mine = [np.concatenate([a[(b << n) + rank * size:(b << n) + (rank + 1) * size] for b in range(K)]) for _, a in full]
        tr = sb.Transcript("multi", d)
        degree, terms = sb.lower_statement(statement, d, names, constants)
        prover.set_statement(d, max(degree, 1), len(full), terms)
        for slot, a in enumerate(mine):
            prover.upload_table(slot, np.ascontiguousarray(a))
        prover.begin(n, eq=eq, block_weights=bw)
        prover.attach_transcript(tr)
        tr.absorb(b"sc|" + n.to_bytes(2, "little") + degree.to_bytes(2, "little") + K.to_bytes(4, "little"))
        rho = []
        for _ in range(n):
            tr.send(prover.round())
            rho.append(tr.challenge())
            prover.challenge(rho[-1])
        folded = prover.finish(len(full), K).tolist()
        prover.attach_transcript(None)
        if rank == 0:
            from oracle import pyoracle as orc
            tb = orc.Transcript("multi", d)
            want = orc.prove(tb, n, statement, full, eq=eq, constants=constants, block_weights=bw, threads=0)
            ok = rho == want[0] and folded == [want[2][nm] for nm in names] and tr.proof() == tb.proof()
            results.append({"case": statement + " with %d blocks" % K, "n": n, "d": d, "ok": bool(ok)})
        else:
            results.append({"proof": tr.proof().hex(), "finals": folded})
    with open(out_file, "w") as f:
        json.dump(results, f)
    prover.close()


if __name__ == "__main__":
    main()
