"""Builds ``libaf3k.so`` in-tree with nvcc for sm_100a.

Usage: ``python -m af3_kernels_b200.build [--force]``.  nvcc cross-compiles, so this works on a
host without a GPU; the resulting library needs a compute-capability-10.x device to run.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "libaf3k.so")
SOURCES = [os.path.join(CSRC, "af3k_capi.cu")]
HEADERS = [
    os.path.join(CSRC, "attn_sm100.cuh"),
    os.path.join(CSRC, "pair_bias_sm100.cuh"),
    os.path.join(CSRC, "proj_sm100.cuh"),
    os.path.join(CSRC, "ptx_sm100.cuh"),
    os.path.join(_HERE, "..", "include", "af3k.h"),
]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "-cudart", "shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libaf3k.so cannot be built")
    return exe


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(f) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library when it is missing or older than its sources; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH] + SOURCES
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libaf3k.so")
    return LIB_PATH


PROBE_SRC = os.path.join(CSRC, "xu_pipe_probe.cu")
PROBE_PATH = os.path.join(_HERE, "xu_pipe_probe")


def build_probe() -> str:
    """Compiles the stand-alone instruction-pipe probe (csrc/xu_pipe_probe.cu): the measurements
    behind the softmax loop's formulation.  Not part of the library."""
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-o", PROBE_PATH, PROBE_SRC]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building xu_pipe_probe")
    return PROBE_PATH


if __name__ == "__main__":
    if "--probe" in sys.argv:
        print(build_probe())
    else:
        print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
