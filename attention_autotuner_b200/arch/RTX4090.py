from .arch_base import Arch


class RTX4090(Arch):
    """Kept for import compatibility with the reference (python/arch/RTX4090.py); not a build target."""

    def __init__(self):
        super().__init__()
        self.reg_cap = 65536
        self.smem_cap = 100 * 1024
        self.compute_max_core = 128
        self.warp_size = 32
        self.sm_partition = 4
        self.transaction_size = [32, 128]
        self.max_smem_usage = 100 * 1024
        self.bandwidth = [1008, 0]
        self.platform = "CUDA"
        self.compute_capability = "89"
        self.cutlass_mma = [16, 8, 16]
        self.register_per_thread = 255
