"""Builds libattn_b200.so (the C-ABI library of include/attn_b200.h) in-tree with nvcc for sm_100a.

    python -m attention_autotuner_b200.build [--force]
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


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
