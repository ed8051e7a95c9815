"""Registers this package's sub-packages under the reference's top-level import names, so that code
written for the reference (``PYTHONPATH=attention_autotuner/python``) runs unchanged:

    import attention_autotuner_b200.compat; attention_autotuner_b200.compat.install()
    from ops.attention_interface import flash_attn_func
    from arch import B200
"""
import importlib
import sys

_NAMES = ("arch", "autotuner", "ops", "utils")


def install():
    for name in _NAMES:
        mod = importlib.import_module(f"attention_autotuner_b200.{name}")
        sys.modules.setdefault(name, mod)
    for sub in ("autotuner.runtime", "autotuner.tunner", "autotuner.base_tunner", "autotuner.configs",
                "ops.attention_interface", "ops.retnet_interface", "utils.ref_op", "utils.misc"):
        try:
            mod = importlib.import_module(f"attention_autotuner_b200.{sub}")
        except ImportError:
            continue
        sys.modules.setdefault(sub, mod)
