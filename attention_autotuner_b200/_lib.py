"""ctypes binding of libattn_b200.so (include/attn_b200.h). No CPU fallback: a missing library or a
non-zero status raises."""
from __future__ import annotations

import ctypes
import os
import threading

from .build import LIB_PATH

F16, BF16 = 0, 1

_lock = threading.Lock()
_lib = None


class AttnB200Error(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"libattn_b200 error {code}: {text}")
        self.code = code


def _declare(lib):
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.attn_b200_last_error.restype = ctypes.c_char_p
    lib.attn_b200_last_error.argtypes = []
    lib.attn_b200_device_status.restype = ci
    lib.attn_b200_device_status.argtypes = [ci]
    lib.attn_b200_abi_version.restype = ci
    lib.attn_b200_abi_version.argtypes = []
    fa = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, cf, ci, vp]
    lib.attn_b200_fa_fwd.restype = ci
    lib.attn_b200_fa_fwd.argtypes = fa
    lib.attn_b200_fa_fwd_profile.restype = cf
    lib.attn_b200_fa_fwd_profile.argtypes = fa
    fb = [vp] * 9 + [ci] * 6 + [cf, ci, vp]
    lib.attn_b200_fa_bwd.restype = ci
    lib.attn_b200_fa_bwd.argtypes = fb
    lib.attn_b200_fa_bwd_profile.restype = cf
    lib.attn_b200_fa_bwd_profile.argtypes = fb
    rf = [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, cf, vp, ci, vp]
    lib.attn_b200_ret_fwd.restype = ci
    lib.attn_b200_ret_fwd.argtypes = rf
    lib.attn_b200_ret_fwd_profile.restype = cf
    lib.attn_b200_ret_fwd_profile.argtypes = rf
    rb = [vp] * 10 + [ci] * 7 + [cf, vp, ci, vp]
    lib.attn_b200_ret_bwd.restype = ci
    lib.attn_b200_ret_bwd.argtypes = rb
    lib.attn_b200_ret_bwd_profile.restype = cf
    lib.attn_b200_ret_bwd_profile.argtypes = rb
    lib.attn_b200_ret_bwd_ws.restype = ci
    lib.attn_b200_ret_bwd_ws.argtypes = [vp] * 10 + [ctypes.c_size_t] + [ci] * 7 + [cf, vp, ci, vp]
    lib.attn_b200_ret_bwd_noalloc.restype = ci
    lib.attn_b200_ret_bwd_noalloc.argtypes = [vp] * 9 + [ci] * 7 + [cf, vp, ci, vp]
    lib.attn_b200_ret_bwd_noalloc_max_bytes.restype = ctypes.c_size_t
    lib.attn_b200_ret_bwd_noalloc_max_bytes.argtypes = []
    lib.attn_b200_ret_bwd_workspace_bytes.restype = ctypes.c_size_t
    lib.attn_b200_ret_bwd_workspace_bytes.argtypes = [ci, ci, ci]
    lib.attn_b200_selftest_gemm_ss.restype = ci
    lib.attn_b200_selftest_gemm_ss.argtypes = [vp, vp, vp, ci, ci, ci, vp]
    lib.attn_b200_selftest_gemm_ts.restype = ci
    lib.attn_b200_selftest_gemm_ts.argtypes = [vp, vp, vp, ci, ci, vp]
    lib.attn_b200_selftest_pair.restype = ci
    lib.attn_b200_selftest_pair.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, vp]
    lib.attn_b200_ret_chunk_fwd.restype = ci
    lib.attn_b200_ret_chunk_fwd.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, cf, vp]
    lib.attn_b200_ret_chunk_workspace_bytes.restype = ctypes.c_size_t
    lib.attn_b200_ret_chunk_workspace_bytes.argtypes = [ci, ci, ci, ci, ci, ci]
    lib.attn_b200_ret_chunk_fwd_ws.restype = ci
    lib.attn_b200_ret_chunk_fwd_ws.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.c_size_t, ci, ci, ci, ci, ci, ci, ci, cf, vp]
    lib.attn_b200_selftest_wait.restype = ci
    lib.attn_b200_selftest_wait.argtypes = [ci, ci, vp]
    for name, sig in _OPTIONAL.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = sig


_OPTIONAL: dict = {}


def load():
    """Returns the loaded library; raises if it has not been built (python -m attention_autotuner_b200.build)."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python -m attention_autotuner_b200.build` "
                    "(needs nvcc with sm_100a support). There is no CPU fallback.")
            lib = ctypes.CDLL(LIB_PATH)
            _declare(lib)
            _lib = lib
    return _lib


def check(code: int):
    if code != 0:
        raise AttnB200Error(code, load().attn_b200_last_error().decode())


def device_status(clear: bool = True) -> int:
    return load().attn_b200_device_status(1 if clear else 0)
