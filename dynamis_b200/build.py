"""Builds dynamis_b200/libdynb.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m dynamis_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The host parts of the .cu files are compiled with
-ffp-contract=off: the host cell geometry must round exactly as plain float arithmetic does.
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SO = os.path.join(HERE, "libdynb.so")
SOURCES = ["lib.cu", "radius_graph.cu", "sfc.cu", "halo.cu", "exchange.cu", "state_ops.cu", "integrators.cu", "kdtree.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-ffp-contract=off,-O2", "-ccbin", "/usr/bin/g++",
]


def _deps():
    out = [os.path.join(HERE, "..", "include", "dynb.h")]
    for f in os.listdir(CSRC):
        if f.endswith((".cu", ".cuh")):
            out.append(os.path.join(CSRC, f))
    return out


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    if not force and os.path.exists(SO) and all(os.path.getmtime(d) <= os.path.getmtime(SO) for d in _deps()):
        return SO
    objs = []
    procs = []
    for s in srcs:
        o = s[:-3] + ".o"
        cmd = [NVCC, *FLAGS, "-c", s, "-o", o] + (["-Xptxas", "-v"] if verbose else [])
        procs.append((s, o, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, o, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed for {s}:\n{out}\n")
        elif verbose:
            sys.stderr.write(out)
        objs.append(o)
    if failed:
        raise RuntimeError("nvcc compilation failed")
    subprocess.run([NVCC, "-shared", "-o", SO, *objs, "-lcudart", "-ccbin", "/usr/bin/g++"], check=True)
    return SO


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
