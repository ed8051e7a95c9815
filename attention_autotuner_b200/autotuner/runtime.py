"""Compile one tile configuration into its own shared library and call it through ctypes.

Same surface as the reference's python/autotuner/runtime.py (``Runtime(arch, config, tmp_dir, libname)``,
``.compile(timeout)``, ``.apply(torch_array, device)``, ``compile_parallel``). Differences that matter:
the library handle is cached per process instead of re-opened on every call (runtime.py:79 of the
reference), the device comes from the tensors, launch errors raise, and ``apply`` accepts the knobs the
reference hard-codes (scale, causal, stream, LSE output).
"""
from __future__ import annotations

import ctypes
import importlib.util
import os
import shutil
import subprocess
import threading
from concurrent.futures import ThreadPoolExecutor

import torch

from ..arch import Arch
from .configs import BaseConfig

NVCC_EXE = os.environ.get("NVCC", shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc")
PKG_DIR = os.path.normpath(os.path.join(os.path.dirname(__file__), ".."))
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
DEFAULT_JIT_DIR = os.environ.get("ATTN_B200_JIT_DIR", os.path.join(PKG_DIR, "_jit"))

_source_tag_cache = None


def source_tag() -> str:
    """Short hash of the kernel sources; part of every per-config library name, so that libraries built
    from older sources are never picked up."""
    global _source_tag_cache
    if _source_tag_cache is None:
        import hashlib
        h = hashlib.sha1()
        for root, _dirs, files in sorted(os.walk(CSRC_DIR)):
            for name in sorted(files):
                if name.endswith((".cuh", ".cu", ".h", ".py")):
                    with open(os.path.join(root, name), "rb") as f:
                        h.update(name.encode() + b"\0" + f.read())
        _source_tag_cache = h.hexdigest()[:10]
    return _source_tag_cache


def prune_stale(jit_dir: str = None) -> int:
    """Delete per-config sources and libraries whose name carries another source hash than the current one
    (they can never be selected again). Returns the number of files removed."""
    jit_dir = jit_dir or DEFAULT_JIT_DIR
    if not os.path.isdir(jit_dir):
        return 0
    keep = "_" + source_tag()
    removed = 0
    for name in os.listdir(jit_dir):
        stem, ext = os.path.splitext(name)
        if ext in (".cu", ".so") and not stem.endswith(keep):
            os.remove(os.path.join(jit_dir, name))
            removed += 1
    return removed


_handles: dict = {}
_built: dict = {}  # (directory, config name) -> library file name
_handles_lock = threading.Lock()


class KernelError(RuntimeError):
    pass


def _entry_module(config):
    path = os.path.join(config.template_dir, "profile_code.py")
    spec = importlib.util.spec_from_file_location("EntryCode_" + config.operation, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _create_entry_code(config) -> str:
    return _entry_module(config).kernel_code.format_map(config.substitution_map())


def nvcc_command(arch: Arch, src: str, out: str) -> list:
    cc = arch.compute_capability
    if not str(cc).startswith("100"):
        raise KernelError(f"these kernels are written for sm_100a only; arch reports compute_capability={cc}")
    return [NVCC_EXE, "-std=c++17", "-O3", "-lineinfo", "--disable-warnings", "--compiler-options", "-fPIC", "--shared",
            src, f"-gencode=arch=compute_{cc},code=sm_{cc}", f"-I{CSRC_DIR}", "-o", out]


def _load(path: str):
    with _handles_lock:
        lib = _handles.get(path)
        if lib is None:
            lib = ctypes.CDLL(path)
            lib.kernel_entry.restype = ctypes.c_int
            lib.kernel_entry_ex.restype = ctypes.c_int
            lib.profile.restype = ctypes.c_float
            lib.profile_ex.restype = ctypes.c_float
            lib.last_error.restype = ctypes.c_char_p
            lib.device_status.restype = ctypes.c_int
            _handles[path] = lib
    return lib


class Runtime:
    def __init__(self, arch: Arch, config: BaseConfig, tmp_dir=None, libname=None):
        self.arch = arch
        self.config = config
        self.tmp_dir = tmp_dir if tmp_dir is not None else DEFAULT_JIT_DIR
        self.libname = libname
        if self.libname is None:
            key = (self.tmp_dir, str(config))
            self.libname = _built.get(key)  # built or found earlier in this process: no file-system calls per launch
            if self.libname is None:
                os.makedirs(self.tmp_dir, exist_ok=True)
                self.libname = self.compile()
                if self.libname is None:
                    raise KernelError(f"nvcc failed for config {config!r} (see {self.tmp_dir})")
                _built[key] = self.libname

    def compile(self, timeout: float = None):
        """Writes <str(config)>.cu and builds <str(config)>.so in tmp_dir (skipped if it exists).
        Returns the library file name, or None if nvcc failed or timed out."""
        config = self.config
        filename = str(config) + "_" + source_tag() + ".cu"
        lib_name = str(config) + "_" + source_tag() + ".so"
        lib_path = os.path.join(self.tmp_dir, lib_name)
        if os.path.exists(lib_path):
            return lib_name
        src_path = os.path.join(self.tmp_dir, filename)
        with open(src_path, "w") as f:
            f.write(_create_entry_code(config))
        tmp_out = lib_path + f".{os.getpid()}.{threading.get_ident()}.tmp"
        command = nvcc_command(self.arch, src_path, tmp_out)
        try:
            ret = subprocess.run(command, timeout=timeout, capture_output=True, text=True)
        except subprocess.TimeoutExpired:
            return None
        if ret.returncode != 0:
            with open(os.path.join(self.tmp_dir, str(config) + ".log"), "w") as f:
                f.write(" ".join(command) + "\n" + ret.stdout + ret.stderr)
            return None
        os.replace(tmp_out, lib_path)
        return lib_name

    @property
    def lib_path(self) -> str:
        return os.path.join(self.tmp_dir, self.libname)

    def _lib(self):
        return _load(self.lib_path)

    def apply(self, torch_array: list, device=None, *, scale=None, causal=False, stream=None, extra_ptrs=(),
              decay=None):
        """Launches the kernel on the tensors in the operation's fixed order
        (attention: [q,k,v,o]; retnet: [q,k,v,mask,o,r]; retnet bwd: [q,k,v,mask,do,r,dq,dk,dv,dq_accum], the last one
        optional scratch of any dtype: with a mask tensor the backward keeps a transposed copy of the mask there).
        scale=None keeps the reference's constants through the legacy ``kernel_entry`` symbol when no other
        option is used. Raises KernelError on a non-zero status."""
        t0 = torch_array[0]
        dev = t0.device if device is None else torch.device(device)
        if dev.type != "cuda":
            raise KernelError("tensors must live on a CUDA device; there is no CPU path")
        batch_size, nheads, seqlen_q = t0.shape[0], t0.shape[1], t0.shape[2]
        seqlen_k = torch_array[1].shape[2]
        lib = self._lib()
        ptrs = [ctypes.c_void_p(arr.data_ptr() if arr is not None else 0) for arr in torch_array]
        dims = [ctypes.c_int(batch_size), ctypes.c_int(nheads), ctypes.c_int(seqlen_k), ctypes.c_int(seqlen_q)]
        with torch.cuda.device(dev):
            if scale is None and not causal and stream is None and not extra_ptrs and decay is None:
                ret = lib.kernel_entry(*ptrs, *dims)
            else:
                if stream is None:
                    stream = torch.cuda.current_stream(dev).cuda_stream
                op = self.config.operation
                default_scale = 0.125 if op == "attn" else 1.0
                args = [*ptrs, *[ctypes.c_void_p(p) for p in extra_ptrs], *dims,
                        ctypes.c_float(default_scale if scale is None else scale)]
                if op == "attn":
                    if not extra_ptrs:  # no LSE output requested
                        args.insert(len(ptrs), ctypes.c_void_p(0))
                    args.append(ctypes.c_int(1 if causal else 0))
                else:
                    args.append(ctypes.c_void_p(decay.data_ptr()) if decay is not None else ctypes.c_void_p(0))
                    args.append(ctypes.c_int(1 if causal else 0))
                args.append(ctypes.c_void_p(stream))
                if op == "ret_bwd":
                    # the scratch tensor (the reference's dq_accum slot, last in the array) goes with its size in bytes
                    acc = torch_array[9] if len(torch_array) > 9 else None
                    args.append(ctypes.c_size_t(acc.numel() * acc.element_size() if acc is not None else 0))
                ret = lib.kernel_entry_ex(*args)
        if ret != 0:
            raise KernelError(f"{self.libname}: status {ret}: {lib.last_error().decode()}")
        return ret

    def device_status(self, clear=True) -> int:
        return self._lib().device_status(1 if clear else 0)


def compile_parallel(configs: list, arch, tmp_dir=None):
    def _func(cc):
        try:
            return Runtime(arch, cc, tmp_dir=tmp_dir).libname
        except KernelError:
            return None
    with ThreadPoolExecutor(max_workers=os.cpu_count()) as executor:
        lib_names = executor.map(_func, configs)
    return list(lib_names)
