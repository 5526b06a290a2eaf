"""Build librq_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Usage: ``python rotorquant-vllm_b200/csrc/build.py [--verbose]``.  The library is
written next to the Python package that loads it
(``rotorquant-vllm_b200/rotorquant_vllm/librq_b200.so``).
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

CSRC = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(os.path.dirname(CSRC), "rotorquant_vllm")
LIB = os.path.join(PKG, "librq_b200.so")
SOURCES = ["rq_api.cu", "rq_compress.cu", "rq_decode.cu", "rq_peer.cu", "rq_prefill.cu", "rq_probe.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; librq_b200.so cannot be built")
    return exe


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))]
    deps.append(os.path.join(os.path.dirname(os.path.dirname(CSRC)), "include", "rq_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every ``.cu`` file into one shared library; returns its path."""
    srcs = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    if not force and not _stale():
        return LIB
    cmd = [_nvcc(), "-O3", "-std=c++17", *ARCH, "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
           "--threads", "0", "-o", LIB, *srcs]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build_library(force=True, verbose="--verbose" in sys.argv))
