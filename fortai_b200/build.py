"""Builds the backend shared library in-tree with nvcc for sm_100a.

    python -m fortai_b200.build [--force]

Output: fortai_b200/lib/libfortai_cuda_b200.so (git-ignored; it is the file that
the reference's link line would name instead of its own backend object).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
# FORTAI_B200_LIB names another build of the same sources (e.g. with other -D tuning
# constants); it must exist, it is never rebuilt
LIB_PATH = os.environ.get("FORTAI_B200_LIB") or os.path.join(LIB_DIR, "libfortai_cuda_b200.so")
SOURCES = ["backend_abi.cu", "gguf_reader.cpp"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-lcuda",
]


def _newest_source_mtime() -> float:
    newest = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for name in os.listdir(root):
            if name.endswith((".cu", ".cuh", ".h", ".cpp")):
                newest = max(newest, os.path.getmtime(os.path.join(root, name)))
    return newest


def build(force: bool = False, verbose: bool = False) -> str:
    if os.environ.get("FORTAI_B200_LIB"):
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"FORTAI_B200_LIB={LIB_PATH} does not exist")
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest_source_mtime():
        return LIB_PATH
    command = [NVCC, *FLAGS, "-o", LIB_PATH, *[os.path.join(CSRC, s) for s in SOURCES]]
    if verbose:
        command.insert(1, "-Xptxas")
        command.insert(2, "-v")
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + result.stdout + result.stderr)
    if verbose:
        print(result.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
