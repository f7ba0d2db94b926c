"""Compile the CUDA sources under ``csrc/`` into ``liblf_b200.so`` next to this file.

The library is built in-tree with plain ``nvcc`` for sm_100a only; there is no other
back end and no fallback: a missing or stale library is an error at first use.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
LIB_PATH = os.path.join(_HERE, "liblf_b200.so")
SOURCES = sorted(glob.glob(os.path.join(_HERE, "csrc", "*.cu")))
HEADERS = sorted(glob.glob(os.path.join(_HERE, "csrc", "*.cuh"))) + \
    sorted(glob.glob(os.path.join(_ROOT, "include", "*.h")))

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-shared",
    "-I", os.path.join(_ROOT, "include"),
    "-I", os.path.join(_HERE, "csrc"),
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


BUILD_ID_PATH = os.path.join(_HERE, "liblf_b200.build_id")


def source_id() -> str:
    """sha256 over the contents of every source and header the library is built from."""
    import hashlib
    h = hashlib.sha256()
    for f in SOURCES + HEADERS:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def is_stale() -> bool:
    """True when the library is missing or was built from other sources than the ones on disk
    (compared by content: file times do not survive a copy of the tree)."""
    if not os.path.isfile(LIB_PATH):
        return True
    if not os.path.isfile(BUILD_ID_PATH):
        return False   # a library that came without its build record: nothing to compare with
    with open(BUILD_ID_PATH) as f:
        return f.read().strip() != source_id()


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    """(Re)build the shared library when a source is newer than it; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [find_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + \
        ["-o", LIB_PATH + ".tmp"] + SOURCES
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if ptxas_info or verbose:
        sys.stderr.write(res.stderr)
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    with open(BUILD_ID_PATH, "w") as f:
        f.write(source_id() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(LIB_PATH)
