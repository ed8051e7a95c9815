class Arch:
    """Static hardware description consumed by the tuner's feasibility checks and by the runtime's
    ``-gencode`` flag. Field names follow the reference (python/arch/arch_base.py:1-13)."""

    def __init__(self) -> None:
        self.reg_cap = 0
        self.smem_cap = 0
        self.compute_max_core = 0
        self.warp_size = 0
        self.sm_partition = 0
        self.transaction_size = [0, 0]
        self.max_smem_usage = 0
        self.bandwidth = [0, 0]
        self.platform = "unknown"
        self.compute_capability = "unknown"
        self.register_per_thread = 0
