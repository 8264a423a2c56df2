"""In-tree build of libternary_b200.so for sm_100a with nvcc (no torch involvement).

    python -m reimagined_b200.build [--force] [--verbose]

The shared library lands beside this file so it travels with the source tree.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libternary_b200.so")
SOURCES = ["api.cu", "quantize.cu", "gemv_stream.cu", "gemv_generic.cu", "gemv_strip.cu", "gemv_chain.cu",
           "gemm_tcgen05.cu", "gemm_widen.cu", "moe.cu", "glue.cu", "decode.cu", "packer.cpp", "edge_pack.cpp"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# IEEE division/sqrt and no fast-math: the fp32 epilogue and the quantiser scale are part of the
# bit-exact contract.  -lineinfo keeps profiler source correlation.
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
         "--prec-div=true", "--prec-sqrt=true", "--fmad=true", "-Xcompiler", "-fPIC",
         "-Xptxas", "-v"]


STAMP = LIB + ".sources"


def _digest() -> str:
    """SHA-256 over the sources, the public header and the flags: what the library was built from."""
    h = hashlib.sha256(" ".join(FLAGS).encode())
    deps = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC))
    deps.append(os.path.join(HERE, "..", "include", "ternary_b200.h"))
    for d in deps:
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale() -> bool:
    # by content, not by time stamp: a copy of the tree (another machine, a fresh checkout) keeps the library valid
    if not os.path.exists(LIB) or not os.path.exists(STAMP):
        return True
    with open(STAMP) as f:
        return f.read().strip() != _digest()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    # one builder at a time: several ranks of one job may get here together
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    with open(os.path.join(HERE, "build", "lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if force or _stale():
                _compile(verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB


def _compile(verbose: bool) -> None:
    objs = []
    procs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for src in SOURCES:
        obj = os.path.join(HERE, "build", src + ".o")
        objs.append(obj)
        cmd = [NVCC, *FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = []
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        log.append(f"==== {src}\n{out}")
        failed |= p.returncode != 0
    with open(os.path.join(HERE, "build", "ptxas.log"), "w") as f:
        f.write("\n".join(log))
    if verbose or failed:
        print("\n".join(log))
    if failed:
        raise RuntimeError("nvcc failed; see output above")
    # link beside the target and rename: a process that is loading the old library never sees a half-written file
    tmp = LIB + ".tmp"
    subprocess.run([NVCC, "-shared", "-o", tmp, *objs, "-lcudart"], check=True)
    os.replace(tmp, LIB)
    with open(STAMP, "w") as f:
        f.write(_digest())


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
