"""Brute-force tile-configuration search: enumerate -> feasibility filter -> compile every candidate in
parallel -> time each through its ``profile`` symbol -> argmin -> log + JSON cache.

Same method and the same public names as the reference's python/autotuner/base_tunner.py
(``BaseTunner.tune / get_tuned_configs / compile / compile_parallel / profile / check_cache`` and the
``validate_*`` / ``generate_configs`` hooks). The log keeps the reference's text format (alternating
``repr(config)`` / latency lines, then "best config:" and "search time", base_tunner.py:178-188) and a
JSON twin with TFLOPS and the fraction of the tensor peak is written next to it.
"""
from __future__ import annotations

import ctypes
import json
import os
import pprint
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor

import torch

from .configs import BaseConfig, supported_configs
from .runtime import DEFAULT_JIT_DIR, KernelError, Runtime, _load

PKG_DIR = os.path.normpath(os.path.join(os.path.dirname(__file__), ".."))


class CompileResult:
    def __init__(self, config: BaseConfig, lib_name) -> None:
        self.config = config
        self.lib_name = lib_name  # absolute path of the library, or None when the build failed


def _compile(config, arch, temp_dir: str, timeout: float = None):
    try:
        rt = Runtime(arch, config, tmp_dir=temp_dir, libname="pending")
        name = rt.compile(timeout=timeout)
    except (KernelError, OSError):
        name = None
    return CompileResult(config, os.path.join(temp_dir, name) if name else None)


def _dtype_name(t: torch.Tensor) -> str:
    return "bf16" if t.dtype == torch.bfloat16 else "fp16"


_CACHE_MEMO: dict = {}  # cache file path -> (mtime_ns, parsed configuration or None)


class BaseTunner:
    def __init__(self, arch, torch_array: list, op_name, *, scale=None, causal=False, decay=None):
        self.arch = arch
        self.torch_array = torch_array
        # rows per CTA (128 per query tile) and keys per block the sm_100a kernels are built for
        self.Br_list = [128, 256]
        self.Bc_list = [128]
        self.op_name = op_name
        self.cache_path = os.environ.get("ATTN_B200_CACHE_DIR", os.path.join(PKG_DIR, "cache"))
        self.problem_key = {
            "dim_qk": torch_array[0].shape[-1],
            "dim_v": torch_array[2].shape[-1],
        }
        self.dtype = _dtype_name(torch_array[0])
        self.scale = scale
        self.causal = bool(causal)
        self.decay = decay
        self.last_results = None

    # ------------------------------------------------------------------ compile
    def compile(self, configs: list, temp_dir: str, timeout: float = None):
        return [_compile(config, self.arch, temp_dir, timeout) for config in configs]

    def compile_parallel(self, configs: list, temp_dir: str, timeout: float = None):
        arch = self.arch
        with ThreadPoolExecutor(max_workers=os.cpu_count()) as executor:
            libs = executor.map(_compile, configs, [arch] * len(configs), [temp_dir] * len(configs),
                                [timeout] * len(configs))
        return list(libs)

    # ------------------------------------------------------------------ profile
    def _profile_args(self):
        """(pointer list, extra args after the sizes) for profile_ex of this operation."""
        raise NotImplementedError

    def profile(self, libname, device=None) -> float:
        """ms per launch of the library's kernel on this tuner's tensors; 1e8 on any failure."""
        torch_array = self.torch_array
        t0 = torch_array[0]
        dev = t0.device if device is None else torch.device(device)
        batch_size, nheads, seqlen_q = t0.shape[0], t0.shape[1], t0.shape[2]
        seqlen_k = torch_array[1].shape[2]
        try:
            lib = _load(libname)
            ptrs, tail = self._profile_args()
            with torch.cuda.device(dev):
                latency = lib.profile_ex(*ptrs, ctypes.c_int(batch_size), ctypes.c_int(nheads), ctypes.c_int(seqlen_q),
                                         ctypes.c_int(seqlen_k), *tail)
        except (OSError, AttributeError):
            return 1e8
        if latency < 0:
            latency = 1e8
        return latency

    # ------------------------------------------------------------------ search space
    def get_tuned_configs(self):
        dim_qk = self.problem_key["dim_qk"]
        dim_v = self.problem_key["dim_v"]
        configs = []
        for Br in self.Br_list:
            for Bc in self.Bc_list:
                for cur_config in self.generate_configs(Br, Bc, dim_qk, dim_v):
                    if self.validate_kernel(cur_config):
                        configs.append(cur_config)
        return configs

    def default_config(self):
        """The configuration used when no cache entry exists and searching is disabled."""
        raise NotImplementedError

    def flops(self) -> float:
        return 0.0

    # ------------------------------------------------------------------ tune
    def problem(self) -> dict:
        """Problem description the cost model works on."""
        t = self.torch_array
        B, H, Lq, dqk = (int(x) for x in t[0].shape)
        return dict(B=B, H=H, Lq=Lq, Lkv=int(t[1].shape[2]), dqk=dqk, dv=int(t[2].shape[3]), causal=self._cost_model_causal())

    def _cost_model_causal(self) -> bool:
        return self.causal

    def tune(self, log_path=None, *, search=None, top_k=None, force=False):
        """Returns the best configuration: from the JSON cache if present (unless ``force``); otherwise by searching
        (default, as in the reference) or, when ``search`` is False / ATTN_B200_AUTOTUNE=0 / nvcc is missing,
        the built-in default. ``top_k`` (or ATTN_B200_TUNE_TOPK) prunes the search with the cost model
        (autotuner/cost_model.py): only the k candidates it predicts fastest are compiled and timed. Without
        pruning the log records what pruning to five candidates would have picked and at what regret."""
        st = time.time()
        dim_qk = self.problem_key["dim_qk"]
        dim_v = self.problem_key["dim_v"]

        best_config = None if force else self.check_cache()
        if best_config is not None:
            return best_config
        if search is None:
            search = os.environ.get("ATTN_B200_AUTOTUNE", "1") != "0"
        if not search or not torch.cuda.is_available():
            return self.default_config()

        configs = self.get_tuned_configs()
        n_candidates = len(configs)
        if top_k is None and os.environ.get("ATTN_B200_TUNE_TOPK"):
            top_k = int(os.environ["ATTN_B200_TUNE_TOPK"])
        predicted = {}
        try:
            from . import cost_model
            op = configs[0].operation if configs else None
            prob = self.problem()
            predicted = {c: cost_model.predict_ms(op, c.__dict__, prob) for c in configs}
            if top_k is not None and 0 < top_k < len(configs):
                configs = cost_model.rank(op, configs, prob)[:top_k]
        except (OSError, KeyError, ValueError) as e:  # no weights file, or no weights for this operation: search everything
            print("cost model unavailable (%s): exhaustive search" % e)
            predicted = {}
        print("Configs to be tuned: ")
        for config in configs:
            pprint.pprint(config)

        t_compile = time.time()
        cresults = self.compile_parallel(configs, DEFAULT_JIT_DIR, timeout=300)
        t_compile = time.time() - t_compile
        profile_dict = {}
        latency = 1e8
        best_config = None
        # Every candidate is timed twice and the second figure kept: loading a library leaves the GPU idle long enough
        # to cool, and a 100 ms timing loop started on a cool chip reads up to 10 % faster than the same loop on a chip
        # at its power limit, which favoured whatever was timed first or after a slow load.
        twice = os.environ.get("ATTN_B200_TUNE_CONFIRM", "1") != "0"
        for cresult in cresults:
            if cresult is None or cresult.lib_name is None:
                continue
            lib_latency = self.profile(cresult.lib_name)
            if twice and lib_latency != 1e8:
                lib_latency = self.profile(cresult.lib_name)
            if lib_latency == 1e8:
                pprint.pprint(cresult.config)
                print("profile runtime error")
            if lib_latency < latency:
                latency = lib_latency
                best_config = cresult.config
            profile_dict[cresult.config] = lib_latency
        # Confirmation pass. A timing loop of 100 ms is long enough for the GPU to reach its power limit, so the
        # candidates timed first (on a cooler chip) look up to several per cent faster than they are. The candidates
        # within 4 % of the best (at most six) are therefore timed twice more, in the opposite and then the original
        # order, and ranked by the median of their three measurements. (The reference times every candidate once,
        # python/autotuner/base_tunner.py:148-160.)
        confirm = {}
        if best_config is not None and os.environ.get("ATTN_B200_TUNE_CONFIRM", "1") != "0":
            close = sorted((c for c, ms in profile_dict.items() if ms <= 1.04 * latency), key=lambda c: profile_dict[c])[:6]
            if len(close) > 1:
                lib_of = {cr.config: cr.lib_name for cr in cresults if cr is not None and cr.lib_name is not None}
                confirm = {c: [profile_dict[c]] for c in close}
                for order in (list(reversed(close)), close):
                    for c in order:
                        confirm[c].append(self.profile(lib_of[c]))
                med = {c: sorted(v)[len(v) // 2] for c, v in confirm.items()}
                best_config = min(close, key=lambda c: med[c])
                latency = med[best_config]
        end = time.time()
        self.last_results = profile_dict
        if best_config is None:
            print("no configuration could be built and run; using the default")
            return self.default_config()

        print("##########################################################")
        print("Operation type: ", best_config.operation)
        print("Best config: ")
        pprint.pprint(best_config)
        print("Latency: ", latency)

        if log_path is None:
            log_path = os.environ.get("ATTN_B200_LOG_DIR", os.path.join(PKG_DIR, "logs"))
        os.makedirs(log_path, exist_ok=True)
        stem = "profile_result_{}_{}_{}".format(best_config.operation, dim_qk, dim_v) + self._key_suffix()
        with open(os.path.join(log_path, stem + ".txt"), "w") as f:
            for config in profile_dict:
                f.write(repr(config) + "\n")
                f.write(str(profile_dict[config]) + "\n")
            f.write("\n")
            f.write("best config: \n")
            f.write(repr(best_config) + "\n")
            f.write(str(latency) + "\n")
            f.write("\nsearch time: " + str(end - st) + "s")
        fl = self.flops()
        peak = getattr(self.arch, "dense_tflops", 0.0)
        with open(os.path.join(log_path, stem + ".json"), "w") as f:
            json.dump({
                "operation": best_config.operation, "shape": [int(x) for x in self.torch_array[0].shape],
                "seqlen_k": int(self.torch_array[1].shape[2]), "dim_qk": int(dim_qk), "dim_v": int(dim_v),
                "dtype": self.dtype, "causal": self.causal, "flops": fl, "peak_tflops": peak,
                "results": [{"config": repr(c), "ms": ms,
                             "tflops": (fl / ms / 1e9 if ms < 1e8 else 0.0),
                             "frac_of_peak": (fl / ms / 1e9 / peak if ms < 1e8 and peak else 0.0),
                             "predicted_ms": predicted.get(c), "confirm_ms": confirm.get(c)}
                            for c, ms in profile_dict.items()],
                "best": repr(best_config), "best_ms": latency, "search_time_s": end - st,
                "compile_time_s": t_compile,
                "cost_model": self._cost_model_record(profile_dict, predicted, n_candidates, top_k, t_compile, end - st)},
                f, indent=1)

        os.makedirs(self.cache_path, exist_ok=True)
        with open(self._cache_file(), "w") as f:
            json.dump(best_config.to_dict(), f)
        if os.environ.get("ATTN_B200_REFERENCE_FILES", "0") == "1":
            # the reference's own file names (python/autotuner/base_tunner.py:178-193): one log and one cache entry per
            # (operation, dqk, dv), whatever the dtype or mask form; same text format, so old and new logs diff
            import shutil
            shutil.copyfile(os.path.join(log_path, stem + ".txt"),
                            os.path.join(log_path, "profile_result_{}_{}_{}.txt".format(best_config.operation, dim_qk, dim_v)))
            with open(os.path.join(self.cache_path, "best_config_{}_{}_{}.json".format(self.op_name, dim_qk, dim_v)), "w") as f:
                json.dump(best_config.to_dict(), f)
        return best_config

    @staticmethod
    def _cost_model_record(profile_dict, predicted, n_candidates, top_k, t_compile, t_search, k_report=5):
        """What the cost model did (pruned search) or would have done (exhaustive search) for this problem."""
        rec = {"candidates": n_candidates, "timed": len(profile_dict), "pruned_to_top_k": top_k}
        timed = [(c, ms) for c, ms in profile_dict.items() if ms < 1e8 and predicted.get(c) is not None]
        if len(timed) >= 2 and (top_k is None or top_k >= n_candidates):
            order = sorted(timed, key=lambda t: predicted[t[0]])
            k = min(k_report, len(order))
            best_all = min(ms for _c, ms in timed)
            best_k = min(ms for _c, ms in order[:k])
            rec.update({"what_if_top_k": k, "what_if_best_ms": best_k, "what_if_regret": best_k / best_all - 1.0,
                        "rank_of_measured_best": 1 + [ms for _c, ms in order].index(best_all),
                        # compilation dominates the search and is spread over the cores: k of n candidates cost about k/n
                        "what_if_search_time_s": t_search - t_compile * (1.0 - k / len(order))})
        return rec

    # ------------------------------------------------------------------ cache
    def _key_suffix(self) -> str:
        cc = str(getattr(self.arch, "compute_capability", ""))
        return f"_sm{cc}_{self.dtype}" + ("_causal" if self.causal else "")

    def _cache_file(self) -> str:
        return os.path.join(self.cache_path, "best_config_{}_{}_{}{}.json".format(
            self.op_name, self.problem_key["dim_qk"], self.problem_key["dim_v"], self._key_suffix()))

    def check_cache(self):
        """Best configuration from cache/best_config_<op>_<dqk>_<dv>_sm<cc>_<dtype>[_causal].json; the
        reference's coarser key (base_tunner.py:192,202: op, dqk, dv only) is read as a fallback when it holds
        a configuration of this package."""
        old_style = os.path.join(self.cache_path, "best_config_{}_{}_{}.json".format(
            self.op_name, self.problem_key["dim_qk"], self.problem_key["dim_v"]))
        for path in (self._cache_file(), old_style):
            try:
                mtime = os.stat(path).st_mtime_ns
            except OSError:
                continue
            memo = _CACHE_MEMO.get(path)
            if memo is None or memo[0] != mtime:
                # parsed once per file version: the operators look the configuration up on every call
                try:
                    with open(path, "r") as f:
                        d = json.load(f)
                    memo = (mtime, supported_configs[d["operation"]].from_dict(d))
                except (OSError, ValueError, KeyError):
                    memo = (mtime, None)
                _CACHE_MEMO[path] = memo
            cfg = memo[1]
            if cfg is not None and hasattr(cfg, "dv_chunk") and cfg.dtype == self.dtype:
                return cfg
        return None

    # ------------------------------------------------------------------ hooks
    def validate_shared_fuse(self, config):
        return self.validate_kernel(config)

    def validate_register_fuse(self, config):
        return self.validate_kernel(config)

    def validate_kernel(self, config):
        return False

    def generate_configs(self, Br: int, Bc: int, dim_qk: int, dim_v: int):
        return []
