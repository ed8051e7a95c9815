"""Tile-configuration records of the tuner. Same roles as the reference's
python/autotuner/configs/base_config.py: ``__str__`` is the on-disk library name, ``__repr__`` the log
line, ``__dict__`` the JSON cache entry and the substitution map of the generated launch code.

What a "tile configuration" means changed with the hardware. On sm_100a the accumulators live in tensor
memory and one elected thread issues 128-row tcgen05 MMAs, so the reference's warp grids, register/shared
fusion styles and cp.async K-splits have no counterpart. The reference's positional arguments are still
accepted so that code constructing configs the old way keeps working; the fields that no longer steer
anything are stored and otherwise ignored (listed in LEGACY_FIELDS).
"""

import os

CSRC_DIR = os.path.normpath(os.path.join(os.path.dirname(__file__), "..", "..", "csrc"))
TEMPLATE_SUBDIR = {"attn": ("attention",), "ret": ("retnet",), "ret_bwd": ("retnet", "bwd")}

LEGACY_FIELDS = ("BlockKSmem", "BlockKSmem2", "num_stages_qk", "num_stages_v", "num_stages_mask", "unrollLastIter",
                 "warps_mma1_n", "warps_mma_n", "mmawarpsN", "mmawarpsN_dv", "mmawarpsN_dk", "mmawarpsN_dq",
                 "num_stages_dv", "num_stages_ds", "num_stages_dq")


def find_factors(n: int):
    return [i for i in range(1, n + 1) if n % i == 0]


def find_factor_pairs(n: int):
    return [(i, n // i) for i in range(1, n + 1) if n % i == 0]


def find_best_pair(pair_list: list, target_pair: tuple):
    """Warp-grid heuristic of the reference (base_config.py:17-28): the factor pair whose aspect ratio is
    closest to the tile's. Kept for API compatibility; tcgen05 kernels have no warp grid."""
    min_cost = 1.0
    best_pair = None
    for pair in pair_list:
        cost = abs(pair[0] * target_pair[1] / (pair[1] * target_pair[0] + pair[0] * target_pair[1]) - 0.5)
        if target_pair[1] % (pair[1] * 16) != 0 or target_pair[0] % (pair[0] * 16) != 0:
            continue
        if cost < min_cost:
            min_cost = cost
            best_pair = pair
    return best_pair


def dv_chunk_for(D: int) -> int:
    """Columns of V (and O) one CTA owns: the largest of 256/128/64 dividing D. One tcgen05.mma covers
    at most N = 256 and tensor memory has 512 columns."""
    return 256 if D % 256 == 0 else 128 if D % 128 == 0 else 64


class BaseConfig:
    def __init__(self, Br, Bc, Kd, D, BlockKSmem=256, num_stages_qk=1, Nthreads=256, unrollLastIter: bool = True,
                 *, dtype: str = "fp16") -> None:
        self.Br = Br              # query rows per CTA (128 per query tile)
        self.Bc = Bc              # keys per KV block
        self.Kd = Kd              # head dim of q, k
        self.D = D                # head dim of v, o
        self.BlockKSmem = BlockKSmem
        self.num_stages_qk = num_stages_qk
        self.Nthreads = Nthreads
        self.unrollLastIter = int(unrollLastIter)
        self.warps_mma1_n = 1
        self.warps_mma_n = 1
        self.dtype = dtype        # "fp16" | "bf16"
        self.fuse_type = "tmem"   # the reference's "register"/"shared" styles both map onto tensor memory
        self.operation = None

    def set_fuse_type(self, fuse_type):
        """Accepted for compatibility ("register", "shared"); accumulators always live in tensor memory."""
        self.fuse_type = "tmem"

    @property
    def template_dir(self) -> str:
        """Directory of this operation's launch-shim template (profile_code.py). Always derived from ``operation``
        and the location of the installed package; never stored, so cache files written on one machine load on
        any other (the reference stores an absolute path, python/autotuner/configs/attention.py:25)."""
        return os.path.join(CSRC_DIR, "kernels", *TEMPLATE_SUBDIR[self.operation])

    def to_dict(self) -> dict:
        """JSON-serialisable fields of the record: what the tuner writes to its cache file."""
        return {k: v for k, v in self.__dict__.items() if k != "template_dir"}

    @property
    def bf16(self) -> int:
        return 1 if self.dtype == "bf16" else 0

    def substitution_map(self) -> dict:
        d = dict(self.__dict__)
        d["bf16"] = "true" if self.dtype == "bf16" else "false"
        d["cta_pair_bool"] = "true" if getattr(self, "cta_pair", 0) else "false"
        return d

    def __eq__(self, other):
        return type(self) is type(other) and str(self) == str(other)

    def __hash__(self):
        return hash(str(self))

    @classmethod
    def from_dict(cls, dd: dict):
        cc = cls.__new__(cls)
        # a path read from a file must never decide which template gets executed: drop it, template_dir is derived
        cc.__dict__.update({k: v for k, v in dd.items() if k != "template_dir"})
        cc.__dict__.setdefault("dtype", "fp16")
        cc.__dict__.setdefault("fuse_type", "tmem")
        if cc.__dict__.get("operation") == "attn":
            cc.__dict__.setdefault("softmax_split", 1)
            cc.__dict__.setdefault("exp_emu", 0)
            cc.__dict__.setdefault("mma_warps", 1)
            cc.__dict__.setdefault("cta_pair", 0)
            cc.__dict__.setdefault("exp_h2", 0)
            cc.__dict__.setdefault("persistent", -1)  # entries cached before the knob existed: chosen per call
        if cc.__dict__.get("operation") in ("ret", "ret_bwd"):
            cc.__dict__.setdefault("cta_pair", 0)  # entries cached before the knob existed were single-CTA
        return cc
