"""Builds libfta.so (the C-ABI library of hand-written sm_100a kernels) in-tree with nvcc.

Run as `python -m flash_tree_attn_b200.build`.  nvcc cross-compiles without a GPU.  The
translation units are torch-free and compile in parallel; the library lands next to this
file so that it is found by `_lib.py` and loaded with ctypes.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libfta.so")

SOURCES = [
    "fta_api.cu",
    "fta_stage2.cu",
    "fta_commit.cu",
    "fta_stage1_umma.cu",
    "fta_stage1_mma_d32.cu",
    "fta_stage1_mma_d64.cu",
    "fta_stage1_mma_d128.cu",
    "fta_stage1_mma_d256.cu",
]

EXTRA = os.environ.get("FTA_EXTRA_NVCC_FLAGS", "").split()

NVCC_FLAGS = EXTRA + [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--use_fast_math",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libfta.so cannot be built")
    return exe


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(os.path.relpath(p, HERE).encode())  # relative: the stamp stays valid when the tree is copied elsewhere
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _all_inputs():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    files.append(os.path.join(HERE, "..", "include", "fta.h"))
    return [os.path.normpath(f) for f in files if os.path.isfile(f)]


def _compile(src: str) -> str:
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(obj + ".log", "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
    return obj


def build(force: bool = False, verbose: bool = True) -> str:
    """Compile every CUDA translation unit for sm_100a and link libfta.so."""
    os.makedirs(OBJ, exist_ok=True)
    stamp = os.path.join(OBJ, "stamp.txt")
    digest = _digest(_all_inputs())
    if not force and os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read() == digest:
        if verbose:
            print(f"[fta build] up to date: {LIB}")
        return LIB
    with cf.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(_compile, SOURCES))
    cmd = [_nvcc(), "-shared", "-o", LIB, *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as f:
        f.write(digest)
    if verbose:
        print(f"[fta build] built {LIB}")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv)
