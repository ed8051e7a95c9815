"""Builds libattn_b200.so (the C-ABI library of include/attn_b200.h) in-tree with nvcc for sm_100a.

    python -m attention_autotuner_b200.build [--force] [--benchmarks]

--benchmarks also compiles the standalone C++ micro-benchmarks under benchmarks/.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
LIB_PATH = os.environ.get("ATTN_B200_LIB", os.path.join(CSRC, "libattn_b200.so"))  # override: a library built elsewhere
NVCC = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "--shared", "-Xcompiler", "-fPIC",
]


def _sources():
    out = []
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            out.append(os.path.join(CSRC, name))
    out.append(os.path.join(CSRC, "..", "..", "include", "attn_b200.h"))
    return out


def source_hash() -> str:
    """Hash of every source the library is compiled from (file names and contents)."""
    import hashlib
    h = hashlib.sha1()
    for path in _sources():
        if os.path.exists(path):
            with open(path, "rb") as f:
                h.update(os.path.basename(path).encode() + b"\0" + f.read() + b"\0")
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _stamp_path() -> str:
    return LIB_PATH + ".srchash"


def is_stale() -> bool:
    """True when the library is missing or was built from other sources than the ones present now. Decided by a
    hash of the sources stored beside the library, not by file times (a fresh checkout has arbitrary ones)."""
    if not os.path.exists(LIB_PATH):
        return True
    try:
        with open(_stamp_path()) as f:
            return f.read().strip() != source_hash()
    except OSError:
        return True


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compiles csrc/attn_b200.cu into csrc/libattn_b200.so; returns the library path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [NVCC, *NVCC_FLAGS, "-o", LIB_PATH, os.path.join(CSRC, "attn_b200.cu")]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    with open(_stamp_path(), "w") as f:
        f.write(source_hash() + "\n")
    return LIB_PATH


BENCH_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "benchmarks")
BENCH_PROGRAMS = {"attention_bench": "attention.cu", "retnet_bench": "retnet.cu"}


def _bench_hash() -> str:
    import hashlib
    h = hashlib.sha1(source_hash().encode())
    for name in sorted(os.listdir(BENCH_DIR)):
        if name.endswith((".cu", ".cuh")):
            with open(os.path.join(BENCH_DIR, name), "rb") as f:
                h.update(name.encode() + b"\0" + f.read())
    return h.hexdigest()


def build_benchmarks(force: bool = False) -> list:
    """Compiles the standalone C++ micro-benchmarks (benchmarks/attention.cu, benchmarks/retnet.cu) into
    benchmarks/attention_bench and benchmarks/retnet_bench; returns the program paths. Rebuilt when the hash of
    the kernel and benchmark sources changes."""
    stamp = os.path.join(BENCH_DIR, ".srchash")
    paths = [os.path.join(BENCH_DIR, exe) for exe in BENCH_PROGRAMS]
    want = _bench_hash()
    try:
        with open(stamp) as f:
            fresh = f.read().strip() == want
    except OSError:
        fresh = False
    if not force and fresh and all(os.path.exists(p) for p in paths):
        return paths
    for exe, src in BENCH_PROGRAMS.items():
        cmd = [NVCC, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
               "-o", os.path.join(BENCH_DIR, exe), os.path.join(BENCH_DIR, src)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + res.stdout + res.stderr)
    with open(stamp, "w") as f:
        f.write(want + "\n")
    return paths


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--benchmarks" in sys.argv:
        print("\n".join(build_benchmarks(force="--force" in sys.argv)))
