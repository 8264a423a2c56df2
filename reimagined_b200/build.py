"""In-tree build of libternary_b200.so for sm_100a with nvcc (no torch involvement).

    python -m reimagined_b200.build [--force] [--verbose]

The shared library lands beside this file so it travels with the source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libternary_b200.so")
SOURCES = ["api.cu", "quantize.cu", "gemv_stream.cu", "gemv_generic.cu", "gemv_strip.cu", "gemv_chain.cu",
           "gemm_tcgen05.cu", "moe.cu", "glue.cu", "decode.cu", "packer.cpp", "edge_pack.cpp"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# IEEE division/sqrt and no fast-math: the fp32 epilogue and the quantiser scale are part of the
# bit-exact contract.  -lineinfo keeps profiler source correlation.
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
         "--prec-div=true", "--prec-sqrt=true", "--fmad=true", "-Xcompiler", "-fPIC",
         "-Xptxas", "-v"]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "ternary_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
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
    subprocess.run([NVCC, "-shared", "-o", LIB, *objs, "-lcudart"], check=True)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
