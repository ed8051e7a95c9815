"""Per-operation search spaces and feasibility checks (reference: python/autotuner/tunner.py).

The knobs are Blackwell's: query tiles per CTA, depth of the TMA-fed K/V ring, V columns per CTA.
Feasibility = shared memory per CTA <= arch.smem_cap and tensor-memory columns <= arch.tmem_columns,
which replace the reference's shared-memory and accumulator-register checks (tunner.py:102-151)."""
import ctypes

from .base_tunner import BaseTunner, CompileResult  # noqa: F401
from .configs import AttnConfig, RetBwdConfig, RetConfig  # noqa: F401
from .configs.base_config import dv_chunk_for, find_best_pair, find_factor_pairs  # noqa: F401
from .configs.retnet import pair_ok


def _flops_fwd(t, causal):
    B, H, Lq, dqk = t[0].shape
    Lkv, dv = t[2].shape[2], t[2].shape[3]
    pairs = Lq * Lkv
    if causal:
        shift = Lkv - Lq
        pairs = sum(max(0, min(Lkv, i + shift + 1)) for i in range(Lq))
    return 2.0 * B * H * pairs * (dqk + dv)


class AttnTunner(BaseTunner):
    def __init__(self, arch, torch_array: list, *, scale=None, causal=False):
        super().__init__(arch, torch_array, "attention", scale=scale, causal=causal)

    def validate_kernel(self, config):
        if config.Kd % 64 != 0 or config.D % 64 != 0 or config.D % config.dv_chunk != 0:
            return False
        if config.smem_bytes() > self.arch.smem_cap:
            return False
        if config.tmem_columns() > getattr(self.arch, "tmem_columns", 512):
            return False
        if config.dv_chunk > 256 or config.kv_stages < 2:
            return False
        if config.softmax_split == 2 and (config.q_tiles != 2 or config.dv_chunk % 64 != 0):
            return False
        if config.mma_warps == 2 and config.q_tiles != 2:
            return False
        if getattr(config, "exp_h2", 0) and (config.dtype != "fp16" or config.softmax_split != 1 or config.exp_emu != 0
                                              or config.cta_pair or not 0 < config.exp_h2 <= 4):
            return False
        if config.cta_pair and (config.q_tiles != 2 or config.dv_chunk != 128 or config.softmax_split != 1
                                or config.exp_emu != 0 or config.mma_warps != 1):
            return False
        persistent = getattr(config, "persistent", -1)
        if persistent not in (-1, 0, 1):
            return False
        if persistent == 1 and (config.q_tiles != 2 or config.dv_chunk > 128 or config.softmax_split != 1 or config.exp_emu != 0
                                or config.mma_warps != 1 or config.cta_pair or getattr(config, "exp_h2", 0)):
            return False
        return True

    def generate_configs(self, Br: int, Bc: int, dim_qk: int, dim_v: int):
        configs = []
        q_tiles = Br // 128
        chunks = [c for c in (256, 128, 64) if dim_v % c == 0]
        for dv_chunk in chunks[:2]:
            for kv_stages in (2, 3, 4, 5, 6):
                configs.append(AttnConfig(Br, Bc, dim_qk, dim_v, q_tiles=q_tiles, kv_stages=kv_stages,
                                          dv_chunk=dv_chunk, dtype=self.dtype))
            if q_tiles == 2:
                # second-order knobs around the usual ring depth: two softmax warpgroups per tile, part of the
                # exponentials on the FMA pipes, two MMA-issuing warps taking turns
                for split, emu, mw in ((2, 0, 1), (2, 2, 1), (1, 2, 1), (1, 0, 2), (2, 0, 2)):
                    configs.append(AttnConfig(Br, Bc, dim_qk, dim_v, q_tiles=2, kv_stages=4, dv_chunk=dv_chunk,
                                              softmax_split=split, exp_emu=emu, mma_warps=mw, dtype=self.dtype))
                # packed half-precision exponentials (two per MUFU operation) for a quarter / half / all of the scores
                if self.dtype == "fp16":
                    for h2 in (1, 2, 3, 4):
                        for stages in (4, 5):
                            configs.append(AttnConfig(Br, Bc, dim_qk, dim_v, q_tiles=2, kv_stages=stages, dv_chunk=dv_chunk,
                                                      exp_h2=h2, dtype=self.dtype))
                # the form of the grid, forced either way (the default picks per call by the length of the work items)
                if dv_chunk <= 128:
                    for form in (0, 1):
                        for stages in (4, 5):
                            configs.append(AttnConfig(Br, Bc, dim_qk, dim_v, q_tiles=2, kv_stages=stages, dv_chunk=dv_chunk,
                                                      persistent=form, dtype=self.dtype))
                # CTA pairs (cta_group::2): 512 query rows per cluster
                for stages in (3, 4):
                    configs.append(AttnConfig(Br, Bc, dim_qk, dim_v, q_tiles=2, kv_stages=stages, dv_chunk=dv_chunk,
                                              cta_pair=1, dtype=self.dtype))
        return configs

    def default_config(self):
        dqk, dv = self.problem_key["dim_qk"], self.problem_key["dim_v"]
        best = None
        for q_tiles in (2, 1):
            for kv_stages in (4, 6, 3, 2):
                cfg = AttnConfig(128 * q_tiles, 128, dqk, dv, q_tiles=q_tiles, kv_stages=kv_stages,
                                 dv_chunk=dv_chunk_for(dv), dtype=self.dtype)
                if self.validate_kernel(cfg):
                    best = cfg
                    break
            if best is not None:
                break
        if best is None:
            raise ValueError(f"no feasible attention tile for dqk={dqk}, dv={dv}")
        return best

    def flops(self):
        return _flops_fwd(self.torch_array, self.causal)

    def _profile_args(self):
        q, k, v, o = self.torch_array[:4]
        ptrs = [ctypes.c_void_p(t.data_ptr()) for t in (q, k, v, o)] + [ctypes.c_void_p(0)]
        scale = 0.125 if self.scale is None else self.scale
        tail = [ctypes.c_float(scale), ctypes.c_int(1 if self.causal else 0), ctypes.c_void_p(0)]
        return ptrs, tail


def _chunks(d):
    return [c for c in (256, 128, 64) if d % c == 0]


class _RetBase(BaseTunner):
    def _tail(self):
        scale = 1.0 if self.scale is None else self.scale
        dec = ctypes.c_void_p(self.decay.data_ptr()) if self.decay is not None else ctypes.c_void_p(0)
        return [ctypes.c_float(scale), dec, ctypes.c_int(1 if self.causal else 0), ctypes.c_void_p(0)]

    def _ptrs(self, n):
        return [ctypes.c_void_p(t.data_ptr() if t is not None else 0) for t in self.torch_array[:n]]

    def _key_suffix(self) -> str:
        if self.decay is not None:
            # a decay mask is lower triangular whatever ``causal`` says: one cache entry for both
            cc = str(getattr(self.arch, "compute_capability", ""))
            return f"_sm{cc}_{self.dtype}_decay"
        return super()._key_suffix()

    def _pairs_causal(self):
        return self.causal or self.decay is not None

    def _cost_model_causal(self) -> bool:
        return self._pairs_causal()


class RetTunner(_RetBase):
    """Forward search space: columns of V per CTA. torch_array = [q, k, v, mask, o, r] (mask may be None
    when ``decay`` is given)."""

    def __init__(self, arch, torch_array: list, *, scale=None, causal=False, decay=None):
        super().__init__(arch, torch_array, "retnet", scale=scale, causal=causal, decay=decay)

    def validate_kernel(self, config):
        if config.cta_pair and not pair_ok(config.dv_chunk):
            return False
        return (config.Kd % 64 == 0 and config.D % config.dv_chunk == 0 and config.dv_chunk <= 256
                and config.smem_bytes() <= self.arch.smem_cap + 1024
                and config.tmem_columns() <= getattr(self.arch, "tmem_columns", 512) and config.ring_slots() >= 3)

    def generate_configs(self, Br: int, Bc: int, dim_qk: int, dim_v: int):
        if Br != 128:
            return []
        from .configs import RetConfig
        return [RetConfig(Br, Bc, dim_qk, dim_v, dv_chunk=c, cta_pair=pr, dtype=self.dtype)
                for c in _chunks(dim_v) for pr in ((0, 1) if pair_ok(c) else (0,))]

    def default_config(self):
        from .configs import RetConfig
        return RetConfig(128, 128, self.problem_key["dim_qk"], self.problem_key["dim_v"], dtype=self.dtype)

    def flops(self):
        return _flops_fwd(self.torch_array, self._pairs_causal())

    def _profile_args(self):
        return self._ptrs(6), self._tail()


class RetBwdTunner(_RetBase):
    """Backward search space: output columns per CTA of the dV kernel and of the dK / dQ kernels.
    torch_array = [q, k, v, mask, do, r, dq, dk, dv, dq_accum]."""

    def __init__(self, arch, torch_array: list, *, scale=None, causal=False, decay=None):
        super().__init__(arch, torch_array, "retnet_bwd", scale=scale, causal=causal, decay=decay)

    def validate_kernel(self, config):
        if config.cta_pair and not pair_ok(config.dv_chunk, config.dq_chunk):
            return False
        return (config.Kd % 64 == 0 and config.D % 64 == 0 and config.D <= 512 and config.D % config.dv_chunk == 0
                and config.Kd % config.dq_chunk == 0 and config.smem_bytes() <= self.arch.smem_cap + 1024
                and config.tmem_columns() <= getattr(self.arch, "tmem_columns", 512) and config.ring_slots() >= 3)

    def generate_configs(self, Br: int, Bc: int, dim_qk: int, dim_v: int):
        if Br != 128:
            return []
        from .configs import RetBwdConfig
        return [RetBwdConfig(Br, Bc, dim_qk, dim_v, dv_chunk=cv, dq_chunk=cq, cta_pair=pr, dtype=self.dtype)
                for cv in _chunks(dim_v) for cq in _chunks(dim_qk) for pr in ((0, 1) if pair_ok(cv, cq) else (0,))]

    def default_config(self):
        from .configs import RetBwdConfig
        return RetBwdConfig(128, 128, self.problem_key["dim_qk"], self.problem_key["dim_v"], dtype=self.dtype)

    def flops(self):
        t = self.torch_array
        B, H, Lq, dqk = t[0].shape
        Lkv, dv = t[2].shape[2], t[2].shape[3]
        pairs = Lq * Lkv
        if self._pairs_causal():
            pairs = sum(max(0, min(Lkv, i + 1)) for i in range(Lq))
        return 2.0 * B * H * pairs * (3 * dqk + 2 * dv)

    def _profile_args(self):
        acc = self.torch_array[9] if len(self.torch_array) > 9 else None
        nbytes = acc.numel() * acc.element_size() if acc is not None else 0
        return self._ptrs(10), self._tail() + [ctypes.c_size_t(nbytes)]  # the scratch tensor's size in bytes comes last
