import os

from .base_config import BaseConfig, dv_chunk_for
from .retnet import CSRC_DIR, _chain_smem, pair_ok


class RetBwdConfig(BaseConfig):
    """RetNet parallel backward tile configuration (reference: python/autotuner/configs/retnet_bwd.py).

    Three kernels, each owning its output tile: dV (128 keys x dv_chunk columns, contraction over dqk),
    dK and dQ (128 rows x dq_chunk columns, contraction over dv). The reference's warp-grid arguments
    are accepted and ignored."""

    def __init__(self, Br, Bc, Kd, D, mmawarpsN=None, mmawarpsN_dv=None, mmawarpsN_dk=None, mmawarpsN_dq=None,
                 Nthreads=256, unrollLastIter: bool = True, BlockKSmem=256, num_stages_qk=1, num_stages_mask=1,
                 num_stages_dv=1, num_stages_ds=1, num_stages_dq=1, *, dv_chunk=None, dq_chunk=None,
                 cta_pair=None, dtype: str = "fp16") -> None:
        super().__init__(Br, Bc, Kd, D, BlockKSmem, num_stages_qk, Nthreads, unrollLastIter, dtype=dtype)
        self.num_stages_mask = num_stages_mask
        self.mmawarpsN = mmawarpsN
        self.mmawarpsN_dv = mmawarpsN_dv
        self.mmawarpsN_dk = mmawarpsN_dk
        self.mmawarpsN_dq = mmawarpsN_dq
        self.num_stages_dv = num_stages_dv
        self.num_stages_ds = num_stages_ds
        self.num_stages_dq = num_stages_dq
        self.dv_chunk = dv_chunk if dv_chunk is not None else dv_chunk_for(D)
        self.dq_chunk = dq_chunk if dq_chunk is not None else dv_chunk_for(Kd)
        # cta_pair: all three kernels as CTA pairs on 256-row tiles (needs both chunks in {128, 256})
        self.cta_pair = int(pair_ok(self.dv_chunk, self.dq_chunk) if cta_pair is None else cta_pair)
        self.Br = 128
        self.Bc = 128
        self.Nthreads = 384
        self.operation = "ret_bwd"

    def smem_bytes(self) -> int:
        return max(_chain_smem(self.Kd)[0], _chain_smem(self.D)[0])

    def ring_slots(self) -> int:
        return min(_chain_smem(self.Kd)[1], _chain_smem(self.D)[1])

    def tmem_columns(self) -> int:
        return 256 + max(self.dv_chunk, self.dq_chunk)

    def __repr__(self) -> str:
        return "RetBwdConfig(Br={}, Bc={}, Kd={}, D={}, dv_chunk={}, dq_chunk={}, cta_pair={}, dtype={})".format(
            self.Br, self.Bc, self.Kd, self.D, self.dv_chunk, self.dq_chunk, self.cta_pair, self.dtype)

    def __str__(self) -> str:
        return f"{self.operation}_{self.Br}_{self.Bc}_{self.Kd}_{self.D}_{self.dv_chunk}_{self.dq_chunk}_{self.cta_pair}_{self.dtype}"
