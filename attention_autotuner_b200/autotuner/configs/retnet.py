import os

from .base_config import BaseConfig, dv_chunk_for

CSRC_DIR = os.path.normpath(os.path.join(os.path.dirname(__file__), "..", "..", "csrc"))


def _chain_smem(k1: int) -> int:
    """Shared memory of one chain-kernel CTA: the resident 128 x k1 tile plus the largest ring of 32 KB
    items that fits (capped at 6), as ChainConfig in csrc/chain_sm100.cuh computes it."""
    r_bytes = 128 * k1 * 2
    nslot = min(6, (232448 - 1024 - 2048 - r_bytes) // 32768)
    return 1024 + r_bytes + nslot * 32768 + 2048, nslot


def pair_ok(*chunks) -> bool:
    """The CTA-pair chain kernel splits the streamed T tile by columns between the two CTAs in 64-column
    boxes: every output chunk must be 128 or 256 columns wide."""
    return all(c in (128, 256) for c in chunks)


class RetConfig(BaseConfig):
    """RetNet parallel forward tile configuration (reference: python/autotuner/configs/retnet.py).

    One CTA owns a 128-row query tile and ``dv_chunk`` columns of V / O; when D > dv_chunk the score tile
    is recomputed by each of the D / dv_chunk CTAs of a query tile (tensor memory holds 512 columns:
    2 x 128 for the double-buffered scores + dv_chunk for O)."""

    def __init__(self, Br, Bc, Kd, D, BlockKSmem=256, BlockKSmem2=64, num_stages_qk=1, num_stages_mask=1,
                 num_stages_v=1, Nthreads=256, unrollLastIter: bool = True, warps_mma1_n=None, warps_mma_n=None, *,
                 dv_chunk=None, cta_pair=None, dtype: str = "fp16") -> None:
        super().__init__(Br, Bc, Kd, D, BlockKSmem, num_stages_qk, Nthreads, unrollLastIter, dtype=dtype)
        self.BlockKSmem2 = BlockKSmem2
        self.num_stages_v = num_stages_v
        self.num_stages_mask = num_stages_mask
        if warps_mma1_n is not None:
            self.warps_mma1_n = warps_mma1_n
        if warps_mma_n is not None:
            self.warps_mma_n = warps_mma_n
        self.dv_chunk = dv_chunk if dv_chunk is not None else dv_chunk_for(D)
        # cta_pair: two CTAs (one cluster, the two SMs of a TPC) share a 256-row tile with cta_group::2 MMAs;
        # needs dv_chunk in {128, 256}. Default: on whenever the chunk allows it.
        self.cta_pair = int(pair_ok(self.dv_chunk) if cta_pair is None else cta_pair)
        self.Br = 128
        self.Bc = 128
        self.Nthreads = 384
        self.operation = "ret"

    def smem_bytes(self) -> int:
        return _chain_smem(self.Kd)[0]

    def ring_slots(self) -> int:
        return _chain_smem(self.Kd)[1]

    def tmem_columns(self) -> int:
        return 256 + self.dv_chunk

    def __repr__(self) -> str:
        return "Config(fuse_type={}, Br={}, Bc={}, Kd={}, D={}, dv_chunk={}, cta_pair={}, dtype={})".format(
            self.fuse_type, self.Br, self.Bc, self.Kd, self.D, self.dv_chunk, self.cta_pair, self.dtype)

    def __str__(self) -> str:
        return f"ret_{self.fuse_type}_{self.Br}_{self.Bc}_{self.Kd}_{self.D}_{self.dv_chunk}_{self.cta_pair}_{self.dtype}"
