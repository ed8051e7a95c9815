import json
import os

from .arch_base import Arch


class B200(Arch):
    """NVIDIA B200 (sm_100a). Beyond the reference's fields it carries the Blackwell limits the tuner's
    feasibility checks need: tensor-memory columns, the tcgen05 instruction shape, SM count and the dense
    16-bit tensor peak (measured value when a MEASURED_PEAKS.json sits in the working tree, else nominal)."""

    def __init__(self):
        super().__init__()
        self.reg_cap = 65536
        self.smem_cap = 227 * 1024          # max dynamic shared memory per CTA (232448 B)
        self.compute_max_core = 148         # SMs
        self.warp_size = 32
        self.sm_partition = 4
        self.transaction_size = [32, 128]
        self.max_smem_usage = 228 * 1024
        self.bandwidth = [7700, 0]          # HBM3e GB/s (nominal)
        self.platform = "CUDA"
        self.compute_capability = "100a"
        self.register_per_thread = 255
        # Blackwell additions
        self.tmem_columns = 512             # 32-bit columns x 128 lanes per SM
        self.tmem_lanes = 128
        self.umma_shape = [128, 256, 16]    # max M, max N, K of one tcgen05.mma (16-bit inputs, 1 CTA)
        self.cutlass_mma = self.umma_shape  # the name the reference's validators read
        self.l2_bytes = 126 * 1024 * 1024
        self.hbm_bytes = 180 * 10**9
        self.dense_tflops_nominal = 2250.0  # fp16/bf16 dense
        self.dense_tflops = self._measured("bf16_tflops", self.dense_tflops_nominal)
        self.hbm_gbs = self._measured("hbm_gbs", 7700.0)

    @staticmethod
    def _measured(key, default):
        for root in (os.environ.get("ATTN_B200_PEAKS_DIR", ""), os.getcwd(),
                     os.path.join(os.path.dirname(__file__), "..", "..")):
            path = os.path.join(root, "MEASURED_PEAKS.json") if root else ""
            if path and os.path.exists(path):
                try:
                    with open(path) as f:
                        return float(json.load(f)[key])
                except (OSError, ValueError, KeyError):
                    pass
        return default
