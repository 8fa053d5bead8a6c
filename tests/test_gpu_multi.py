"""Several GPUs: the hypercube cut on its top variables, one process per GPU, sums combined by an
NCCL all-gather and a sum mod p, tables gathered for the last rounds.  The proof must be the
single-GPU (and the oracle's) proof, bit for bit.  Skipped with fewer than two GPUs."""
import json
import os
import subprocess
import sys
import tempfile

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def gpu_count():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("world,gather_bits,device_transcript", [(2, None, False), (2, 0, False), (4, None, False), (8, 2, False),
                                                                  (2, None, True), (4, None, True), (8, None, True)])
def test_sharded_proof_equals_the_oracle(world, gather_bits, device_transcript):
    # gather_bits: the slice size (log2) at which the ranks gather their tables; 0 keeps every round but the last sharded
    if gpu_count() < world:
        pytest.skip("needs %d GPUs" % world)
    with tempfile.TemporaryDirectory() as tmp:
        env = dict(os.environ, NCCL_NVLS_ENABLE="0")
        if device_transcript:                 # every rank's round kernels hash the summed words themselves
            env["SABLE_B200_DEVICE_TRANSCRIPT"] = "1"
        if gather_bits is not None:
            env["SABLE_B200_GATHER_BITS"] = str(gather_bits)
            env["SABLE_B200_P2P"] = "0"       # these runs carry the sums with NCCL, the others with peer stores
        procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "multi_gpu_worker.py"), str(r), str(world),
                                   os.path.join(tmp, "id"), os.path.join(tmp, "out%d.json" % r)], env=env,
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=300)
            except subprocess.TimeoutExpired:
                for q in procs:
                    q.kill()
                raise
            outs.append(out)
        for r, p in enumerate(procs):
            assert p.returncode == 0, "rank %d failed:\n%s" % (r, outs[r][-3000:])
        res = [json.load(open(os.path.join(tmp, "out%d.json" % r))) for r in range(world)]
        assert all(c["ok"] for c in res[0]), res[0]
        # every rank ends with the same transcript and the same finals
        for r in range(2, world):
            assert res[r] == res[1]


def run_two_ranks(mode, env_extra):
    with tempfile.TemporaryDirectory() as tmp:
        env = dict(os.environ, NCCL_NVLS_ENABLE="0", **env_extra)
        procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "multi_gpu_worker.py"), str(r), "2",
                                   os.path.join(tmp, "id"), os.path.join(tmp, "out%d.json" % r), mode], env=env,
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=150)
            except subprocess.TimeoutExpired:
                for q in procs:
                    q.kill()
                raise
            outs.append(out)
        assert procs[0].returncode == 0, outs[0][-3000:]
        return json.load(open(os.path.join(tmp, "out0.json")))


def test_a_rank_that_leaves_is_reported_not_waited_for():
    # failure detection on the host: rank 1 exits between two rounds; rank 0's next exchange (an NCCL all-gather:
    # with peer stores switched off no kernel touches the memory of the process that left) runs into the time
    # limit, the communicator is aborted, the call returns SC_ECOMM and the context works again alone
    if gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = run_two_ranks("lost-rank", {"SABLE_B200_COMM_TIMEOUT_S": "3", "SABLE_B200_P2P": "0"})
    assert res["code"] == -6, res
    assert res["seconds"] < 30 and res["after"] == 4, res


def test_a_rank_that_withholds_a_round_runs_the_mailbox_wait_out():
    # the bounded wait inside the round kernel: rank 1 stays alive (its mailbox stays mapped) but does not run
    # its next round; rank 0's last block polls its mailbox a limited number of times, gives up and posts the
    # failure, and the host returns SC_ECOMM with the context usable again
    if gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    res = run_two_ranks("withheld-round", {"SABLE_B200_MAIL_POLLS": "200000"})
    assert res["code"] == -6 and "never arrived" in res["text"], res
    assert res["seconds"] < 30 and res["after"] == 4, res
