import os

from .base_config import BaseConfig, dv_chunk_for

CSRC_DIR = os.path.normpath(os.path.join(os.path.dirname(__file__), "..", "..", "csrc"))


class AttnConfig(BaseConfig):
    """Flash-attention forward tile configuration (reference: python/autotuner/configs/attention.py).

    Blackwell knobs (keyword-only):
      q_tiles    query tiles of 128 rows per CTA (1, or 2 ping-ponging); Br = 128 * q_tiles
      kv_stages  depth of the shared-memory ring of K / V tiles fed by TMA
      dv_chunk   columns of V / O per CTA (grid y = D / dv_chunk)
      softmax_split  softmax warpgroups per query tile (1, or 2: two threads share a score row; needs q_tiles == 2)
      mma_warps  MMA-issuing warps: 1, or 2 taking strict turns, one per query tile (needs q_tiles == 2)
      exp_emu    of every 8 pairs of scores, how many use the FMA-pipe exp2 polynomial instead of MUFU (0..8)
      exp_h2     of every 4 groups of 8 scores, how many use the packed fp16 exponential (two results per MUFU
                 operation; fp16 only, needs softmax_split == 1 and exp_emu == 0; the rescale threshold drops to 2^4)
      persistent form of the grid: -1 chosen per call by the length of the work items (the default), 0 one CTA per
                 256 query rows, 1 one CTA per SM walking a work list (needs q_tiles == 2, dv_chunk <= 128 and the
                 other second-order knobs at their defaults)
      cta_pair   1: clusters of two CTAs with cta_group::2 MMAs (512 query rows per pair, each CTA streams half of K and V);
                 needs q_tiles == 2, dv_chunk == 128 and the other second-order knobs at their defaults;
                 kv_stages then counts full K/V tiles as before (the ring holds twice as many half tiles)
    """

    def __init__(self, Br, Bc, Kd, D, BlockKSmem=256, BlockKSmem2=64, num_stages_qk=1, num_stages_v=1,
                 Nthreads=256, unrollLastIter: bool = True, warps_mma1_n=None, warps_mma_n=None, *,
                 q_tiles=None, kv_stages=None, dv_chunk=None, softmax_split=1, exp_emu=0, mma_warps=1, cta_pair=0,
                 exp_h2=0, persistent=-1, dtype: str = "fp16") -> None:
        super().__init__(Br, Bc, Kd, D, BlockKSmem, num_stages_qk, Nthreads, unrollLastIter, dtype=dtype)
        self.BlockKSmem2 = BlockKSmem2
        self.num_stages_v = num_stages_v
        if warps_mma1_n is not None:
            self.warps_mma1_n = warps_mma1_n
        if warps_mma_n is not None:
            self.warps_mma_n = warps_mma_n
        self.dv_chunk = dv_chunk if dv_chunk is not None else dv_chunk_for(D)
        self.q_tiles = q_tiles if q_tiles is not None else (2 if Br >= 256 else 1)
        self.kv_stages = kv_stages if kv_stages is not None else max(2, num_stages_qk + num_stages_v)
        self.softmax_split = softmax_split
        self.exp_emu = exp_emu
        self.mma_warps = mma_warps
        self.exp_h2 = int(exp_h2)
        self.persistent = int(persistent)
        self.cta_pair = int(cta_pair)
        self.Br = 128 * self.q_tiles
        self.Bc = 128
        self.Nthreads = 128 * self.q_tiles * self.softmax_split + 128
        self.operation = "attn"

    # ---- resources (bytes / columns), used by the tuner's feasibility check
    def smem_bytes(self) -> int:
        q = self.q_tiles * 128 * self.Kd * 2
        slot = max(128 * self.Kd * 2, 128 * self.dv_chunk * 2)
        if self.cta_pair:
            return q + 2 * self.kv_stages * (slot // 2) + 1024 + 512
        return q + self.kv_stages * slot + 1024 + 256 + (self.q_tiles * 3072 if self.softmax_split == 2 else 0)

    def tmem_columns(self) -> int:
        return self.q_tiles * (128 + self.dv_chunk)

    def substitution_map(self) -> dict:
        d = super().substitution_map()
        if self.cta_pair:
            d["cfg_type"] = "FaPairConfig<{}, {}, {}>".format(self.Kd, 2 * self.kv_stages, d["bf16"])
            d["launcher"] = "fa_fwd_pair_launch"
        else:
            d["cfg_type"] = "FaFwdConfig<{}, {}, {}, {}, {}, {}, {}, {}, {}>".format(
                self.Kd, self.dv_chunk, self.q_tiles, self.kv_stages, d["bf16"], self.exp_emu, self.softmax_split,
                self.mma_warps, self.exp_h2)
            d["launcher"] = {-1: "fa_fwd_launch_auto", 0: "fa_fwd_launch", 1: "fa_fwd_persist_launch"}[self.persistent]
        return d

    def __repr__(self) -> str:
        return ("Config(fuse_type={}, Br={}, Bc={}, Kd={}, D={}, q_tiles={}, kv_stages={}, dv_chunk={}, softmax_split={}, "
                "exp_emu={}, mma_warps={}, cta_pair={}, exp_h2={}, persistent={}, dtype={})".format(
                    self.fuse_type, self.Br, self.Bc, self.Kd, self.D, self.q_tiles, self.kv_stages, self.dv_chunk,
                    self.softmax_split, self.exp_emu, self.mma_warps, self.cta_pair, self.exp_h2, self.persistent, self.dtype))

    def __str__(self) -> str:
        return (f"attn_{self.fuse_type}_{self.Br}_{self.Bc}_{self.Kd}_{self.D}_{self.q_tiles}_{self.kv_stages}_{self.dv_chunk}_"
                f"{self.softmax_split}_{self.exp_emu}_{self.mma_warps}_{self.cta_pair}_"
                + (f"h{self.exp_h2}_" if self.exp_h2 else "") + (f"p{self.persistent}_" if self.persistent >= 0 else "")
                + f"{self.dtype}")
