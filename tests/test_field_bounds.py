"""The 64-bit running sums of the kernels, checked on the host: csrc/field.cuh is host/device code, so the sums the
small-value passes, round 0 and the three-challenge bind carry without reducing are replayed here with the largest
operands (every word p - 1) against exact 128-bit arithmetic: they must not wrap, must stay in the range the final
reduction takes, and must reduce to the exact value."""
import os
import subprocess
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_running_sums_stay_in_range_and_reduce_exactly():
    src = os.path.join(ROOT, "tests", "native", "field_bounds.cpp")
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "field_bounds")
        build = subprocess.run(["g++", "-O2", "-std=c++17", "-o", exe, src], capture_output=True, text=True)
        assert build.returncode == 0, build.stderr[-2000:]
        run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
        assert run.returncode == 0 and run.stdout.strip() == "ok", run.stdout[-2000:] + run.stderr[-2000:]
