"""Build libsumcheck_b200.so (sm_100a) in-tree with nvcc.

    python -m sable_b200.build [--force]

The translation units compile side by side; an object is rebuilt when its source or any header is
newer.  The library links the CUDA runtime statically and loads NCCL at run time only when a
communicator is asked for, so it has no other dependency than the driver.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libsumcheck_b200.so")
UNITS = ["round_d4.cu", "round_d8.cu", "round_base.cu", "round_tail.cu", "round_sv.cu", "round_sv3.cu", "round_d4w.cu", "round_d8w.cu", "round_d4h.cu", "round_d8h.cu", "aux_kernels.cu", "context.cu", "gkr.cu", "host.cpp", "domain.cpp"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC",
         "-ccbin", "g++"] + os.environ.get("SC_NVCC_EXTRA", "").split()


def _headers():
    out = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    out.append(os.path.join(os.path.dirname(HERE), "include", "sumcheck_b200.h"))
    return out


def _compile(unit, force, verbose):
    src = os.path.join(CSRC, unit)
    obj = os.path.join(OBJ, os.path.splitext(unit)[0] + ".o")
    newest = max(os.path.getmtime(p) for p in [src] + _headers())
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= newest:
        return obj, False
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode:
        raise RuntimeError("nvcc failed on %s:\n%s\n%s" % (unit, res.stdout, res.stderr))
    if verbose:
        sys.stderr.write(res.stderr)
    return obj, True


def build(force=False, verbose=False):
    """Compile what is out of date and link the shared library; returns its path."""
    os.makedirs(OBJ, exist_ok=True)
    with ThreadPoolExecutor(max_workers=len(UNITS)) as pool:
        results = list(pool.map(lambda u: _compile(u, force, verbose), UNITS))
    objs = [o for o, _ in results]
    if any(changed for _, changed in results) or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-ccbin", "g++", "-o", LIB] + objs + ["-ldl"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode:
            raise RuntimeError("link failed:\n%s\n%s" % (res.stdout, res.stderr))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
