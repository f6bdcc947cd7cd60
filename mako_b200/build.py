"""Builds the native parts in-tree: the CUDA library (sm_100a only) and the synthetic-input generator.

    python -m mako_b200.build            # build what is out of date
    python -m mako_b200.build --force

nvcc cross-compiles without a GPU. The shared objects land next to this file so that they travel with the tree.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmako_b200.so")
SYNTH = os.path.join(HERE, "libmk_synth.so")

CUDA_SOURCES = ["row_pipeline.cu", "aux_kernels.cu", "capi.cu", "row_sampler.cu"]
CUDA_DEPS = ["row_pipeline.h", "device_expf.cuh", "ptx.cuh", "exp2_table.inc", "../../include/mako_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default", "--shared", "-cudart", "shared",
]


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def _run(cmd: list[str]) -> None:
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build(force: bool = False, verbose_ptxas: bool = False) -> None:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cu = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    deps = cu + [os.path.join(CSRC, d) for d in CUDA_DEPS]
    if force or _stale(LIB, deps):
        flags = list(NVCC_FLAGS)
        if verbose_ptxas:
            flags += ["-Xptxas", "-v"]
        _run([nvcc, *flags, "-o", LIB, *cu])
    synth_src = os.path.join(CSRC, "synth.cpp")
    if force or _stale(SYNTH, [synth_src]):
        cxx = os.environ.get("CXX", "g++")
        _run([cxx, "-std=c++17", "-O2", "-fPIC", "-shared", "-pthread", "-o", SYNTH, synth_src])


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose_ptxas="-v" in sys.argv)
