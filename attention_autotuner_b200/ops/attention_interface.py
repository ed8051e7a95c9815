"""``flash_attn_func``: same entry point as the reference's python/ops/attention_interface.py:60.

    o = flash_attn_func(q, k, v, device_type, causal=False, softmax_scale=None, return_lse=False)

q [B,H,Lq,dqk], k [B,H,Lkv,dqk], v [B,H,Lkv,dv], fp16 or bf16 CUDA tensors. ``softmax_scale=None`` keeps
the reference's fixed 0.125 (attention_interface.py / ref_op.py:3). The reference accepts ``causal`` and
ignores it (csrc/kernels/attention/regfuse/regfuse.h:59-60); here it masks key j > i + (Lkv - Lq).
Backward is not implemented in the reference (attention_interface.py:38-39) and raises here instead of
silently returning None.
"""
import torch

from ..arch import Arch
from ..autotuner.runtime import Runtime
from ..autotuner.tunner import AttnTunner


class MultiHeadAttnFunc(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, device_type: Arch, causal=False, softmax_scale=None, return_lse=False):
        q, k, v = [x.contiguous() for x in [q, k, v]]
        batch_size, nheads, seqlen_q, key_dim = q.shape
        head_dim = v.shape[-1]
        assert q.dtype in (torch.float16, torch.bfloat16) and k.dtype == q.dtype and v.dtype == q.dtype
        assert head_dim % 64 == 0 and head_dim <= 512
        assert key_dim % 64 == 0 and key_dim <= 256

        o = torch.empty(batch_size, nheads, seqlen_q, head_dim, device=q.device, dtype=q.dtype)
        lse = torch.empty(batch_size, nheads, seqlen_q, device=q.device, dtype=torch.float32) if return_lse else None

        cc = AttnTunner(arch=device_type, torch_array=[q, k, v, o], scale=softmax_scale, causal=causal).tune()
        extra = (lse.data_ptr(),) if lse is not None else ()
        Runtime(device_type, cc).apply([q, k, v, o], scale=0.125 if softmax_scale is None else softmax_scale,
                                       causal=bool(causal), extra_ptrs=extra)
        ctx.save_for_backward(q, k, v)
        ctx.device_type = device_type
        ctx.mark_non_differentiable(*([lse] if lse is not None else []))
        if return_lse:
            return o, lse
        return o

    @staticmethod
    def backward(ctx, do, *unused):
        raise NotImplementedError("attention backward is not part of this operator (nor of the reference)")


def flash_attn_func(q, k, v, device_type, causal=False, softmax_scale=None, return_lse=False):
    return MultiHeadAttnFunc.apply(q, k, v, device_type, causal, softmax_scale, return_lse)
