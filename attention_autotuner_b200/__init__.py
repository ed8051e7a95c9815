"""B200 (sm_100a) fused attention / RetNet kernels behind the attention_autotuner operator API.

Sub-packages mirror the reference's import roots (``python/`` in the reference):
``arch``, ``autotuner``, ``ops``, ``utils``. ``attention_autotuner_b200.compat.install()`` registers them
under the reference's top-level names so ``from ops.attention_interface import flash_attn_func`` works
unchanged.
"""
__version__ = "0.1.0"
