"""Builds libbtp_sm100.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

    python -m spear_b200.build [--force] [--verbose]

The result lands next to this file as spear_b200/lib/libbtp_sm100.so.  nvcc cross-compiles, so no
GPU is needed to build.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libbtp_sm100.so")
SOURCES = [os.path.join(CSRC, "btp_sm100.cu")]
HEADERS = [
    os.path.join(CSRC, "btp_kernels.cuh"),
    os.path.join(CSRC, "btp_decode.cuh"),
    os.path.join(CSRC, "btp_gated.cuh"),
    os.path.join(CSRC, "btp_gated_bwd.cuh"),
    os.path.join(CSRC, "btp_ptx.cuh"),
    os.path.join(os.path.dirname(HERE), "include", "btp_sm100.h"),
]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(p) > built for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile for sm_100a only.  Returns the path of the shared library."""
    if not force and not is_stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [
        nvcc_path(),
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-O3", "-std=c++17", "-lineinfo",
        "-Xcompiler", "-fPIC", "-shared",
        "-Xptxas", "-v" if verbose else "-O3",
        "-o", LIB_PATH,
    ] + SOURCES
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
