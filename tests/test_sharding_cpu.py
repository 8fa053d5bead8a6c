"""The partition used across GPUs, checked on CPU ranks (gloo, world size 2).

Rank k holds entries [k N/W, (k+1) N/W) of every table.  For the first n - log2(W) rounds each
rank sums its own pairs with the eq weights of its local variables, multiplies by
eq(r[n-w..n), k), and the ranks' words are all-gathered and added mod p; then every rank has one
entry per table, these are gathered, and the last log2(W) rounds run alike on every rank.  The
arithmetic of each rank is the oracle's; what is tested is the partition and the exchange.  The
messages, challenges and finals must be those of the unsharded prover.
"""
import os
import sys

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
P = 2130706433


def _rank(rank, world, port, out):
    import torch
    from oracle import pyoracle as orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d, n, statement = 4, 6, "(+ (* alpha t0 t1) (* 3 t1))"
        logw = world.bit_length() - 1
        rng = np.random.default_rng(5)
        full = [("t0", rng.integers(0, P, size=1 << n, dtype=np.uint32)), ("t1", rng.integers(0, P, size=(1 << n, d), dtype=np.uint32))]
        constants = [("alpha", rng.integers(0, P, size=d, dtype=np.uint32).tolist())]
        eq = rng.integers(0, P, size=(n, d), dtype=np.uint32)
        size = (1 << n) >> logw
        lift = lambda a: a if a.ndim == 2 else np.concatenate([a[:, None], np.zeros((len(a), d - 1), dtype=np.uint32)], axis=1)
        cur = [(nm, lift(a[rank * size:(rank + 1) * size])) for nm, a in full]
        weight = orc.eq_table(d, eq[n - logw:])[rank].tolist()     # eq(r[n-w..n), rank)
        tr = orc.Transcript("shard", d)
        tr.absorb(b"sc|" + n.to_bytes(2, "little") + (2).to_bytes(2, "little") + (1).to_bytes(4, "little"))
        rho, messages = [], []

        def first_message(tables, nvars, eqs):
            t = orc.Transcript("scratch", d)
            orc.prove(t, nvars, statement, tables, eq=eqs, constants=constants)
            return t.messages()[0]

        def fold(tables, r):
            return [(nm, np.array([orc.ext_add(d, a[2 * i], orc.ext_mul(d, r, orc.ext_sub(d, a[2 * i + 1], a[2 * i]))) for i in range(len(a) // 2)],
                                  dtype=np.uint32)) for nm, a in tables]

        for j in range(n - logw):
            local = first_message(cur, n - logw - j, eq[j:n - logw])
            mine = np.array([orc.ext_mul(d, weight, row) for row in local.tolist()], dtype=np.int64)
            gathered = [torch.zeros(mine.shape, dtype=torch.int64) for _ in range(world)]
            dist.all_gather(gathered, torch.from_numpy(mine))
            total = (sum(g.numpy() for g in gathered) % P).astype(np.uint32)
            messages.append(total.tolist())
            tr.send(total)
            r = tr.challenge()
            rho.append(r)
            cur = fold(cur, r)
        # one entry per table and rank: gather them, finish alike everywhere
        tables = []
        for nm, a in cur:
            gathered = [torch.zeros((1, d), dtype=torch.int64) for _ in range(world)]
            dist.all_gather(gathered, torch.from_numpy(a.astype(np.int64)))
            tables.append((nm, np.concatenate([g.numpy() for g in gathered]).astype(np.uint32)))
        for j in range(n - logw, n):
            msg = first_message(tables, n - j, eq[j:])
            messages.append(msg.tolist())
            tr.send(msg)
            r = tr.challenge()
            rho.append(r)
            tables = fold(tables, r)
        tb = orc.Transcript("shard", d)
        want = orc.prove(tb, n, statement, full, eq=eq, constants=constants)
        ok = rho == want[0] and [a[0].tolist() for _, a in tables] == [want[1]["t0"], want[1]["t1"]] and tr.proof() == tb.proof()
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_reproduce_the_unsharded_proof():
    world = 2
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as manager:
        out = manager.dict()
        mp.spawn(_rank, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}


def _rank_blocks(rank, world, port, out):
    """The same with block weights: every rank holds its slice of every block, block after block; the gather is per block."""
    import torch
    from oracle import pyoracle as orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d, n, K, statement, names = 4, 5, 3, "(+ (* a b) (* lam b c))", ["a", "b", "c"]
        logw = world.bit_length() - 1
        rng = np.random.default_rng(11)
        lift = lambda a: a if a.ndim == 2 else np.concatenate([a[:, None], np.zeros((len(a), d - 1), dtype=np.uint32)], axis=1)
        full = [("a", rng.integers(0, P, size=(K << n, d), dtype=np.uint32)), ("b", rng.integers(0, P, size=K << n, dtype=np.uint32)),
                ("c", rng.integers(0, P, size=(K << n, d), dtype=np.uint32))]
        constants = [("lam", rng.integers(0, P, size=d, dtype=np.uint32).tolist())]
        eq = rng.integers(0, P, size=(n, d), dtype=np.uint32)
        bw = rng.integers(0, P, size=(K, d), dtype=np.uint32)
        size = (1 << n) >> logw
        cur = [(nm, lift(np.concatenate([a[(b << n) + rank * size:(b << n) + (rank + 1) * size] for b in range(K)]))) for nm, a in full]
        weight = orc.eq_table(d, eq[n - logw:])[rank].tolist()
        tr = orc.Transcript("shard", d)
        tr.absorb(b"sc|" + n.to_bytes(2, "little") + (2).to_bytes(2, "little") + K.to_bytes(4, "little"))
        rho = []

        def first_message(tables, nvars, eqs):
            t = orc.Transcript("scratch", d)
            orc.prove(t, nvars, statement, tables, eq=eqs, constants=constants, block_weights=bw)
            return t.messages()[0]

        def fold(tables, r):
            return [(nm, np.array([orc.ext_add(d, a[2 * i], orc.ext_mul(d, r, orc.ext_sub(d, a[2 * i + 1], a[2 * i]))) for i in range(len(a) // 2)],
                                  dtype=np.uint32)) for nm, a in tables]

        for j in range(n - logw):
            local = first_message(cur, n - logw - j, eq[j:n - logw])
            mine = np.array([orc.ext_mul(d, weight, row) for row in local.tolist()], dtype=np.int64)
            gathered = [torch.zeros(mine.shape, dtype=torch.int64) for _ in range(world)]
            dist.all_gather(gathered, torch.from_numpy(mine))
            total = (sum(g.numpy() for g in gathered) % P).astype(np.uint32)
            tr.send(total)
            rho.append(tr.challenge())
            cur = fold(cur, rho[-1])
        # one entry per table, block and rank: gathered block by block (a block's slices in rank order are the block)
        tables = []
        for nm, a in cur:
            gathered = [torch.zeros((K, d), dtype=torch.int64) for _ in range(world)]
            dist.all_gather(gathered, torch.from_numpy(a.astype(np.int64)))
            per_rank = [g.numpy() for g in gathered]
            tables.append((nm, np.concatenate([np.stack([per_rank[r][b] for r in range(world)]) for b in range(K)]).astype(np.uint32)))
        for j in range(n - logw, n):
            msg = first_message(tables, n - j, eq[j:])
            tr.send(msg)
            rho.append(tr.challenge())
            tables = fold(tables, rho[-1])
        tb = orc.Transcript("shard", d)
        want = orc.prove(tb, n, statement, full, eq=eq, constants=constants, block_weights=bw)
        ok = rho == want[0] and [a.tolist() for _, a in tables] == [want[2][nm] for nm in names] and tr.proof() == tb.proof()
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_two_cpu_ranks_with_block_weights():
    world = 2
    port = 31500 + os.getpid() % 2000
    with mp.Manager() as manager:
        out = manager.dict()
        mp.spawn(_rank_blocks, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: True, 1: True}
