#!/usr/bin/env python3
"""Benchmark of the sumcheck prover: Mentries/s of a whole proof, with the HBM roofline of its round kernel.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C4] [--degree 4] [--impl reference]

One step is one whole proof (every round, host transcript included) of a BASELINE workload on
seeded synthetic tables: value = 2^n / (time per proof) / 10^6, the tables resident in HBM when
the clock starts.  `e2e` is the same proof through the public call with the tables in pinned host
memory, uploaded inside the timed region.  `roofline` is the fused round kernel's algorithmic
bytes over its measured launch time against the measured HBM copy bandwidth.  `cpu_baseline` is
the CPU oracle (a port of the reference prover) on the box's host cores, on a bounded sample.

With N > 1 (one process per GPU under torch.distributed.run) the hypercube of the same n is cut
on its top log2(N) variables: total work is fixed, so the scaling is strong.

`--impl reference` times the CPU port alone, with all host threads, on a bounded sample.
"""
import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

P = 2130706433
MASK = (1 << 64) - 1

# BASELINE.json configs: statement, n, tables (name, stride: 1 base, 0 extension, nonzero), constants
CONFIGS = {
    "C1": dict(n=20, statement="(* t0 t1)", tables=[("t0", 1, False), ("t1", 1, False)], constants=[]),
    "C2": dict(n=24, statement="(* t0 t1 t2)", tables=[("t0", 1, False), ("t1", 1, False), ("t2", 1, False)], constants=[]),
    "C3": dict(n=26, statement="(+ (* alpha t0 t1) (* 3 t1))", tables=[("t0", 1, False), ("t1", 1, False)], constants=["alpha"]),
    "C4": dict(n=28, statement="(+ (* t0 t3) (* t1 t2) (* lam t2 t3))",
               tables=[("t0", 1, False), ("t1", 1, False), ("t2", 0, True), ("t3", 0, True)], constants=["lam"]),
    "C5": dict(n=30, statement="(* t0 t1 t2)", tables=[("t0", 1, False), ("t1", 1, False), ("t2", 1, False)], constants=[]),
}
SEED = 1
EQ_ID, CONST_ID = 255, 254
# DRAM bytes per algorithmic byte of the fused round kernel, from an ncu capture of the C4 workload at n = 24
# (rounds 1 and 2: dram__bytes_read.sum equal to the tables read to 0.1 %, dram__bytes_write.sum 0.91 and 0.81 of
# the folded tables written, the rest still in L2 when the kernel ended).  `roofline.traffic` is SCALED from
# that capture, not measured in this run: the read ratio times the bytes read plus the round-1 write ratio
# times the bytes written, over the launches that move more than twice the L2 (the others are left out of both
# `traffic` and `traffic_basis`).
NCU_READ_RATIO, NCU_WRITE_RATIO = 1.0, 0.91
L2_BYTES = 126 << 20


def splitmix64(x):
    x = (x + 0x9E3779B97F4A7C15) & MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK
    return x ^ (x >> 31)


def seeded_ext(table_id, index, D):
    return [splitmix64(SEED ^ (table_id << 56) ^ (c << 48) ^ index) % P for c in range(D)]


def algorithmic_bytes(cfg, n, D):
    """Whole-proof bytes: the inputs read twice (round 0, then the first fold) and every folded table written and read once."""
    total = 0
    sizes = [4 * (1 if stride == 1 else D) << n for _, stride, _ in cfg["tables"]]
    total += sum(sizes)                      # round 0 reads T_0
    prev = sizes
    for j in range(1, n + 1):                # the kernel of round j reads T_{j-1} and writes T_j (the last fold: j = n)
        cur = [4 * D << (n - j) for _ in sizes]
        total += sum(prev) + sum(cur)
        prev = cur
    return total


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 50 ms from the first timed step to the last end-to-end step."""
    FIELDS = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 8 and parts[0] == str(self.index):
                self.rows.append(parts)

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": float(self.rows[0][2]) if self.rows else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def host_cores():
    """The host cores this process may run on (not OMP_NUM_THREADS, which a launcher may have set to 1)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def bind_near_gpu(index):
    """Run this process on the host cores next to GPU INDEX, so that the pinned buffers it allocates from now on lie on
    that GPU's NUMA node (first touch).  Returns (the affinity before, the NUMA node or None)."""
    before = None
    try:
        import torch
        before = os.sched_getaffinity(0)
        p = torch.cuda.get_device_properties(index)
        base = "/sys/bus/pci/devices/%04x:%02x:%02x.0/" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        cpus = set()
        for part in open(base + "local_cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        node = int(open(base + "numa_node").read().strip())
        cpus &= before
        if cpus:
            os.sched_setaffinity(0, cpus)
        return before, node
    except (OSError, ValueError, AttributeError, RuntimeError):
        return before, None


def cpu_port(cfg, D, n_sample, steps, warmup, threads=0):
    """The CPU oracle (a port of the reference prover) on a bounded sample of the workload: Mentries/s."""
    from oracle import pyoracle as orc
    tables = [(name, orc.generate(SEED, t, 0, 1 << n_sample, 1 if stride == 1 else D, nonzero=nz)) for t, (name, stride, nz) in enumerate(cfg["tables"])]
    eq = [seeded_ext(EQ_ID, i, D) for i in range(n_sample)]
    constants = [(c, seeded_ext(CONST_ID, i, D)) for i, c in enumerate(cfg["constants"])]
    cores = host_cores() if threads == 0 else threads
    times = []
    for step in range(warmup + steps):
        tr = orc.Transcript("bench", D)
        t0 = time.perf_counter()
        orc.prove(tr, n_sample, cfg["statement"], tables, eq=eq, constants=constants, threads=cores)
        dt = time.perf_counter() - t0
        if step >= warmup:
            times.append(dt)
    mean = sum(times) / len(times)
    return (1 << n_sample) / mean / 1e6, mean, cores, tr.proof()


def gkr_bench(args):
    """LogUp-GKR upper layers (sc_gkr_prove_upper): one step is one whole PROVE-UPPER of LOOKUPS trees of
    K blocks of 2^n leaf fractions, trees and host transcript included; value = leaves / time."""
    import numpy as np
    import torch
    import sable_b200 as sb
    D, n, K, L = args.degree, args.n or 22, args.blocks, args.gkr
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda").manual_seed(SEED)
    leaves = []
    for _ in range(L):
        p = torch.randint(0, P, ((K << n), D), generator=gen, device="cuda", dtype=torch.int64).to(torch.int32)
        q = torch.randint(0, P, ((K << n), D), generator=gen, device="cuda", dtype=torch.int64).to(torch.int32)
        q[:, 0] |= 1
        leaves.append((p.contiguous(), q.contiguous()))
    provers = [sb.Prover(0) for _ in range(L)]
    for p in provers:
        p.set_device_transcript(args.transcript == "device")

    def run(lv):
        tr = sb.Transcript("bench", D)
        out = sb.gkr_prove_upper(tr, n, K, lv, provers=provers)
        return tr, out

    def timed(lv, steps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            tr, _ = run(lv)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / steps, tr

    for _ in range(args.warmup):
        run(leaves)
    before = sum(p.launches for p in provers)
    sampler = ClockSampler(0)
    sampler.start()
    mean, tr = timed(leaves, args.steps)
    launches = sum(p.launches for p in provers) - before   # over the timed region, as in the sumcheck line
    e2e = None
    if not args.no_e2e:
        host = [(p.cpu().numpy().view(np.uint32), q.cpu().numpy().view(np.uint32)) for p, q in leaves]
        run(host)
        emean, etr = timed(host, max(1, args.steps // 2))
        assert etr.proof() == tr.proof()
        e2e = {"value": L * (K << n) / emean / 1e6, "unit": "Mleaves/s", "ms_per_step": emean * 1e3,
               "h2d_bytes_per_step": 2 * L * (K << n) * D * 4, "d2h_bytes_per_step": len(tr.proof())}
    clocks = sampler.stop()
    # bytes the layers must move: the tree pass reads a layer and writes the one above (3/2 of a layer); the
    # layer's sumcheck reads its tables in rounds 0 and 1 and a geometric tail of folded tables after (4 x in all)
    entry = 4 * D
    tree = sum(2 * L * (K << m) * entry * 3 // 2 for m in range(1, n + 1))
    proofs = sum(2 * L * (K << m) * entry * 4 for m in range(1, n))
    cpu = None
    if not args.no_cpu:
        from oracle import gkr_oracle as gkr, pyoracle as orc
        ns = min(n, 18)
        rng = np.random.default_rng(SEED)
        lv = []
        for _ in range(L):
            p = rng.integers(0, P, size=(K << ns, D), dtype=np.uint32)
            q = rng.integers(0, P, size=(K << ns, D), dtype=np.uint32)
            q[:, 0] |= 1
            lv.append((p, q))
        t0 = time.perf_counter()
        gkr.prove_upper(orc.Transcript("bench", D), ns, K, lv, threads=0)
        dt = time.perf_counter() - t0
        cpu = {"value": L * (K << ns) / dt / 1e6, "unit": "Mleaves/s", "cores": orc.max_threads(), "kind": "port",
               "sample": "the same trees at n=%d, all host threads in the sumchecks" % ns}
    print(json.dumps({
        "metric": "gkr prove-upper Mleaves/s", "value": L * (K << n) / mean / 1e6, "unit": "Mleaves/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32",
        "data": "synthetic", "config": {"workload": "LogUp-GKR upper layers: %d lookups, K=%d blocks of 2^%d leaf fractions, D=%d" % (L, K, n, D),
                                        "l2": "inputs larger than L2" if 2 * L * (K << n) * entry > (126 << 20) else "inputs fit L2"},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": (tree + proofs) / mean / 1e9, "peak": measured_peak()[0], "unit": "GB/s",
                     "frac": (tree + proofs) / mean / 1e9 / measured_peak()[0], "traffic": None,
                     "note": "whole PROVE-UPPER: algorithmic bytes of all tree passes and all layers' sumchecks over wall time, %d rounds of latency included" % (n * (n - 1) // 2)},
        "cpu_baseline": cpu, "proof_sha256": hashlib.sha256(tr.proof()).hexdigest(),
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="C4", choices=sorted(CONFIGS))
    ap.add_argument("--degree", type=int, default=4, choices=(4, 8))
    ap.add_argument("--n", type=int, default=None, help="override the config's n (smaller runs)")
    ap.add_argument("--impl", default="sable", choices=("sable", "reference"))
    ap.add_argument("--cpu-n", type=int, default=24, help="n of the CPU sample")
    ap.add_argument("--verify", action="store_true", help="one proof at the config's own n on the device and on the CPU port (all host threads): the proof bytes must be equal")
    ap.add_argument("--transcript", default="host", choices=("host", "device"),
                    help="device: a one-block kernel behind each round kernel carries the BLAKE3 transcript on and every round is enqueued at once (an option of the library; the default is the reference's host transcript)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-device-transcript", action="store_true", help="skip the second figure with the transcript on the device")
    ap.add_argument("--gkr", type=int, default=0, metavar="LOOKUPS", help="time LogUp-GKR PROVE-UPPER of this many lookups instead (one GPU; --n leaf bits, default 22)")
    ap.add_argument("--blocks", type=int, default=1, help="K of --gkr")
    args = ap.parse_args()
    if args.gkr:
        return gkr_bench(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = CONFIGS[args.config]
    D = args.degree
    n = args.n if args.n is not None else cfg["n"]
    workload = "%s: %s, n=%d, D=%d, eq mode, %s" % (args.config, cfg["statement"], n, D,
                                                      ", ".join("%s %s" % (nm, "base" if s == 1 else "ext") for nm, s, _ in cfg["tables"]))
    metric = "sumcheck prove Mentries/s"

    if args.impl == "reference":
        if rank != 0:
            return
        n_sample = min(n, args.cpu_n)
        value, mean, cores, _ = cpu_port(cfg, D, n_sample, max(args.steps, 1), args.warmup)
        sample = "the same statement at n=%d (one whole proof per step), %d host threads" % (n_sample, cores)
        # the reference itself is single-threaded: one proof on one thread beside it, on a smaller sample
        n_one = min(n_sample, 20)
        one_value, one_mean, _, _ = cpu_port(cfg, D, n_one, 1, 0, threads=1)
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": value, "unit": "Mentries/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u32", "data": "synthetic",
            "config": {"workload": workload, "sample": sample},
            "cpu_baseline": {"value": value, "unit": "Mentries/s", "cores": cores, "kind": "port", "sample": sample,
                             "one_thread": {"value": one_value, "unit": "Mentries/s", "cores": 1,
                                            "sample": "one proof of the same statement at n=%d on one thread (%.2f s)" % (n_one, one_mean)}},
            "e2e": {"value": value, "unit": "Mentries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "the reference is Common Lisp (SBCL) and no Lisp is installed; this is the C port of its prover, pinned by the reference's own vectors",
        }))
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    import sable_b200 as sb

    if world > 1:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
    assert world & (world - 1) == 0 and (1 << n) >= world, "the world must be a power of two"
    logw = world.bit_length() - 1
    n_loc = n - logw
    prover = sb.Prover(local_rank)
    prover.set_device_transcript(args.transcript == "device")
    if world > 1:
        ids = [sb.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        prover.comm_init(ids[0], rank, world)

    # the tables of this rank's slice, generated on the device
    first = rank << n_loc
    strides = []
    for slot, (name, stride, nz) in enumerate(cfg["tables"]):
        st = 1 if stride == 1 else D
        strides.append(st)
        prover.generate_table(slot, SEED, slot, 1 << n_loc, st, first=first, nonzero=nz)
    eq = np.array([seeded_ext(EQ_ID, i, D) for i in range(n)], dtype=np.uint32)
    constants = [(c, seeded_ext(CONST_ID, i, D)) for i, c in enumerate(cfg["constants"])]
    resident = [(name, sb.DeviceTable(strides[slot])) for slot, (name, _, _) in enumerate(cfg["tables"])]

    def one_proof(tables):
        tr = sb.Transcript("bench", D)
        out = sb.prove(tr, n, cfg["statement"], tables, eq=eq, constants=constants, prover=prover)
        return tr, out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(tables, steps):
        barrier()
        launches0 = prover.launches
        prover.timer_start()
        t0 = time.perf_counter()
        for _ in range(steps):
            tr, out = one_proof(tables)
        ms = prover.timer_stop()
        wall = (time.perf_counter() - t0) * 1e3
        barrier()
        ms = max(ms, 0.0)
        if world > 1:
            t = torch.tensor([ms, wall], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms, wall = t.tolist()
        return ms, wall, prover.launches - launches0, tr, out

    if args.verify:
        # the device against the CPU port at full size, once: same seeded tables (generated on the device here, by the
        # identical generator on the host there), same transcript, the proof bytes and the finals compared
        t0 = time.perf_counter()
        tr, out = one_proof(resident)
        torch.cuda.synchronize()
        gpu_s = time.perf_counter() - t0
        record = {"verify": args.config, "n": n, "D": D, "n_gpus": world, "device_s": round(gpu_s, 4), "proof_bytes": len(tr.proof()),
                  "proof_sha256": hashlib.sha256(tr.proof()).hexdigest()}
        if rank == 0:
            from oracle import pyoracle as orc
            t0 = time.perf_counter()
            tables = [(name, orc.generate(SEED, t, 0, 1 << n, 1 if stride == 1 else D, nonzero=nz)) for t, (name, stride, nz) in enumerate(cfg["tables"])]
            gen_s = time.perf_counter() - t0
            otr = orc.Transcript("bench", D)
            t0 = time.perf_counter()
            want = orc.prove(otr, n, cfg["statement"], tables, eq=eq, constants=constants, threads=host_cores())
            record.update({"cpu_s": round(time.perf_counter() - t0, 2), "cpu_generate_s": round(gen_s, 2), "cpu_threads": host_cores(),
                           "cpu_proof_sha256": hashlib.sha256(otr.proof()).hexdigest(),
                           "equal": otr.proof() == tr.proof() and want[0] == out[0] and want[1] == out[1]})
            print(json.dumps(record))
            assert record["equal"], "the device proof differs from the CPU port's"
        if world > 1:
            dist.destroy_process_group()
        return

    for _ in range(args.warmup):
        one_proof(resident)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, wall, launches, tr, out = timed(resident, args.steps)
    ms_per_step = ms / args.steps
    value = (1 << n) / (ms_per_step * 1e-3) / 1e6
    proof_bytes = tr.proof()

    # the round kernels, one by one (a separate pass, straight after the timed proofs: the events cost a little)
    prover.enable_timing(True)
    one_proof(resident)
    stats = prover.round_stats()
    prover.enable_timing(False)
    # the same proofs with the transcript carried on the device (the library's option), as a second figure
    other = None
    if args.transcript == "host" and not args.no_device_transcript:
        prover.set_device_transcript(True)
        for _ in range(min(args.warmup, 3)):
            one_proof(resident)
        oms, _, olaunches, otr, oout = timed(resident, args.steps)
        prover.set_device_transcript(False)
        other = {"transcript": "device (a one-block kernel behind each round kernel hashes the sums and draws the challenge; all rounds enqueued at once)",
                 "value": (1 << n) / (oms / args.steps * 1e-3) / 1e6, "unit": "Mentries/s", "ms_per_step": oms / args.steps,
                 "gpu_launches": olaunches, "same_proof": otr.proof() == proof_bytes and oout == out}

    peak, peak_kind = measured_peak()
    fused = stats[1:] if len(stats) > 1 else stats
    fused_bytes = sum(s[1] for s in fused)
    fused_ms = sum(s[0] for s in fused)
    achieved = fused_bytes / (fused_ms * 1e-3) / 1e9 if fused_ms > 0 else 0.0
    rounds = [{"round": j, "ms": round(s[0], 4), "GB/s": round(s[1] / (s[0] * 1e-3) / 1e9, 1)} for j, s in enumerate(stats) if s[1] >= (128 << 20) and s[0] > 0]
    traffic = traffic_basis = None
    if args.config == "C4" and D == 4:      # the workload the ncu capture was taken on
        traffic = traffic_basis = 0
        for j, st in enumerate(stats):
            if j == 0 or st[1] < 2 * L2_BYTES:
                continue
            read = sum(4 * (1 if (stride == 1 and j == 1) else D) << (n_loc - j + 1) for _, stride, _ in cfg["tables"])
            write = st[1] - read
            traffic += int(read * NCU_READ_RATIO + write * NCU_WRITE_RATIO)
            traffic_basis += st[1]
    roofline = {"bound": "hbm", "kernel": "round_kernel<D=%d,points,tables,fold> (rounds 1..n-1: fold by the previous challenge + round sums)" % D,
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                "traffic": traffic, "traffic_basis": traffic_basis,
                "traffic_note": "scaled from an ncu capture of the same kernel at n=24 (per-launch DRAM bytes over algorithmic bytes), launches above twice the L2 only; not measured in this run",
                "launches": len(fused), "bytes_per_step": fused_bytes, "ms_per_step": fused_ms, "rounds": rounds,
                "whole_proof_frac": algorithmic_bytes(cfg, n_loc, D) / (ms_per_step * 1e-3) / 1e9 / peak}

    clocks = sampler.stop() if rank == 0 else None   # over the proofs with resident tables (timed region, per-round pass, device-transcript leg)

    # end to end: the tables start in pinned host memory and are uploaded inside the timed region
    e2e = None
    affinity_before, numa_node = None, None
    if not args.no_e2e:
        affinity_before, numa_node = bind_near_gpu(local_rank)      # the pinned buffers below: on this GPU's NUMA node
        host = []
        for slot, (name, _, _) in enumerate(cfg["tables"]):
            words = strides[slot] << n_loc
            t = torch.empty(words, dtype=torch.int32, pin_memory=True)
            prover.fetch_pointer(slot, t.data_ptr(), words)
            a = t.numpy().view(np.uint32)
            host.append((name, a if strides[slot] == 1 else a.reshape(-1, D), t))
        host_tables = [(nm, a) for nm, a, _ in host]
        e2e_steps = max(1, min(args.steps, 3))
        one_proof(host_tables)
        ems, ewall, _, etr, eout = timed(host_tables, e2e_steps)
        assert etr.proof() == proof_bytes and eout == out, "the end-to-end proof differs from the resident one"
        h2d = sum(4 * (strides[s] << n_loc) for s in range(len(strides))) + eq.nbytes + 4 * D * len(constants)
        d2h = 4 * D * (n * max(len(tr.messages[0]) if n else 1, 1) + len(strides))
        # the uploads alone, per rank (all ranks at once, as in the proof): the slowest rank's rate
        barrier()
        t0 = time.perf_counter()
        for slot, (_, _, t) in enumerate(host):
            prover.upload_pointer(slot, t.data_ptr(), 1 << n_loc, strides[slot])
        torch.cuda.synchronize()
        up_s = time.perf_counter() - t0
        up_gbs = sum(4 * (strides[s] << n_loc) for s in range(len(strides))) / up_s / 1e9
        if world > 1:
            t = torch.tensor([up_gbs], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            up_gbs = t.item()
        e2e = {"value": (1 << n) / (ewall / e2e_steps * 1e-3) / 1e6, "unit": "Mentries/s", "h2d_bytes_per_step": h2d * world,
               "d2h_bytes_per_step": d2h, "steps": e2e_steps, "ms_per_step": ewall / e2e_steps,
               "h2d_gbs_slowest_rank": round(up_gbs, 2), "pinned_on_numa_node": numa_node}
        if affinity_before:
            os.sched_setaffinity(0, affinity_before)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        n_sample = min(n, args.cpu_n)
        v, mean, cores, cpu_proof = cpu_port(cfg, D, n_sample, 1, 0)
        n_one = min(n_sample, 20)
        v1, mean1, _, _ = cpu_port(cfg, D, n_one, 1, 0, threads=1)
        cpu = {"value": v, "unit": "Mentries/s", "cores": cores, "kind": "port",
               "sample": "one proof of the same statement at n=%d on %d host threads (%.2f s)" % (n_sample, cores, mean),
               "one_thread": {"value": v1, "unit": "Mentries/s", "cores": 1,
                              "sample": "one proof of the same statement at n=%d on one thread (%.2f s)" % (n_one, mean1)}}
        if n_sample == n:
            assert cpu_proof == proof_bytes, "the device proof differs from the CPU port's"
            cpu["verified"] = "the device's proof bytes equal the CPU port's at n=%d" % n

    if rank == 0:
        print(json.dumps({
            "metric": metric, "value": value, "unit": "Mentries/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "wall_ms_per_step": wall / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "u32", "data": "synthetic",
            "config": {"workload": workload, "sharding": "top %d variables over %d GPUs" % (logw, world),
                       "transcript": "host (BLAKE3)" if args.transcript == "host" else "device (BLAKE3 in the round kernels' last block)",
                       "l2": "inputs larger than L2 (%.1f GiB per rank per proof)" % (sum(4 * (strides[s] << n_loc) for s in range(len(strides))) / 2 ** 30)},
            "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "transcript_on_device": other,
            "proof_bytes": len(proof_bytes), "proof_sha256": hashlib.sha256(proof_bytes).hexdigest(),
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
