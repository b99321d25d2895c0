"""TEST INFRASTRUCTURE ONLY — compiles the reference's own CUDA sources for the hot path into
oracle/_ref/libdynamis_ref.so (git-ignored), for use as the parity oracle on a GPU.

The reference .cu files of the path (radius graph, SFC, halo ops, KD-tree, integrators) are compiled where they lie (nothing is copied), with nvcc for
compute_100 exactly as the reference's own CMake does (plain SIMT, default FMA contraction),
against this image's libtorch headers, together with ref_shim.cpp (ours) which registers them as
torch ops in the ``dynamis_ref`` namespace.  The reference's build system is not run.

    python oracle/build_ref.py [--reference DIR]      (default: $DYNB_REFERENCE, else /root/reference)
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SO = os.path.join(OUT, "libdynamis_ref.so")
REF_SOURCES = [
    "dynamis_state/src/csrc/graph/radius_graph_kernels.cu",
    "dynamis_state/src/csrc/partition/sfc_kernels.cu",
    "dynamis_state/src/csrc/graph/dist_graph_ops_kernels.cu",
    "dynamis_state/src/csrc/partition/kdtree_kernels.cu",
    "dynamis_integrator/src/csrc/euler_integrator.cu",
    "dynamis_integrator/src/csrc/verlet_integrator.cu",
    "dynamis_integrator/src/csrc/langevin_integrator.cu",
]
SHIMS = ["ref_shim.cpp", "ref_shim_integrators.cpp"]
DEFAULT_REFERENCE = os.environ.get("DYNB_REFERENCE", "/root/reference")

# What the reference's CMake writes from dynamis_state/include/dynamis_state/timing_config.hpp.in with
# its timing option OFF (dynamis_state/CMakeLists.txt:17-19): the integrator sources include it.
TIMING_CONFIG = "#pragma once\n/* #undef DYNAMIS_TIMING */\n"


def build(reference: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    if not os.path.isdir(reference):
        return SO if os.path.exists(SO) else None
    if os.path.exists(SO) and not force:
        return SO
    import torch
    from torch.utils import cpp_extension as ce

    import sysconfig

    gen = os.path.join(OUT, "include", "dynamis_state")
    os.makedirs(gen, exist_ok=True)
    with open(os.path.join(gen, "timing_config.hpp"), "w") as f:
        f.write(TIMING_CONFIG)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{reference}/dynamis_state/include",
                                                            f"-I{reference}/dynamis_integrator/include",
                                                            f"-I{os.path.join(OUT, 'include')}",
                                                            f"-I{sysconfig.get_paths()['include']}"]
    common = ["-std=c++17", "-O2", "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objs, procs = [], []
    for rel in REF_SOURCES:
        o = os.path.join(OUT, os.path.basename(rel) + ".o")
        cmd = [nvcc, "-gencode", "arch=compute_100,code=sm_100", "-lineinfo", *common, *inc, "-Xcompiler", "-fPIC",
               "-ccbin", "/usr/bin/g++", "--expt-relaxed-constexpr", "-c", os.path.join(reference, rel), "-o", o]
        procs.append((rel, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(o)
    for shim in SHIMS:
        o = os.path.join(OUT, shim[:-4] + ".o")
        cmd = ["/usr/bin/g++", *common, *inc, "-fPIC", "-c", os.path.join(HERE, shim), "-o", o]
        procs.append((shim, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(o)
    for rel, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            sys.stderr.write(f"compile failed for {rel}:\n{out[-4000:]}\n")
            return None
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["/usr/bin/g++", "-shared", "-o", SO, *objs, f"-L{libdir}", "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda",
           "-ltorch_cuda", "-L/usr/local/cuda/lib64", "-lcudart", f"-Wl,-rpath,{libdir}"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout[-4000:])
        return None
    return SO


def load():
    """Registers torch.ops.dynamis_ref.* ; returns False when the library was never built."""
    if not os.path.exists(SO):
        return False
    import torch

    torch.ops.load_library(SO)
    return True


if __name__ == "__main__":
    ref = sys.argv[sys.argv.index("--reference") + 1] if "--reference" in sys.argv else DEFAULT_REFERENCE
    print(build(ref, force="--force" in sys.argv))
