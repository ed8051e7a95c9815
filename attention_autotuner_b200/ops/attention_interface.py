"""``flash_attn_func``: same entry point as the reference's python/ops/attention_interface.py:60.

    o = flash_attn_func(q, k, v, device_type, causal=False, softmax_scale=None, return_lse=False)

q [B,H,Lq,dqk], k [B,H,Lkv,dqk], v [B,H,Lkv,dv], fp16 or bf16 CUDA tensors. ``softmax_scale=None`` keeps
the reference's fixed 0.125 (attention_interface.py / ref_op.py:3). The reference accepts ``causal`` and
ignores it (csrc/kernels/attention/regfuse/regfuse.h:59-60); here it masks key j > i + (Lkv - Lq).
Backward is empty in the reference (attention_interface.py:38-39: autograd gets None). Here it runs the
flash-attention backward kernels (csrc/fa_bwd_kv_sm100.cuh, csrc/fa_bwd_sm100.cuh) when q, k and v share a head dimension of 64 or 128, and
raises for every other shape instead of returning None.
"""
import ctypes

import torch

from .. import _lib
from ._checks import check_like, check_qkv
from ..arch import Arch
from ..autotuner.runtime import Runtime
from ..autotuner.tunner import AttnTunner


class MultiHeadAttnFunc(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, device_type: Arch, causal=False, softmax_scale=None, return_lse=False):
        check_qkv("flash_attn_func", q, k, v)
        q, k, v = [x.contiguous() for x in [q, k, v]]
        batch_size, nheads, seqlen_q, key_dim = q.shape
        head_dim = v.shape[-1]

        o = torch.empty(batch_size, nheads, seqlen_q, head_dim, device=q.device, dtype=q.dtype)
        needs_grad = any(ctx.needs_input_grad[:3])
        lse = (torch.empty(batch_size, nheads, seqlen_q, device=q.device, dtype=torch.float32)
               if (return_lse or needs_grad) else None)

        cc = AttnTunner(arch=device_type, torch_array=[q, k, v, o], scale=softmax_scale, causal=causal).tune()
        extra = (lse.data_ptr(),) if lse is not None else ()
        Runtime(device_type, cc).apply([q, k, v, o], scale=0.125 if softmax_scale is None else softmax_scale,
                                       causal=bool(causal), extra_ptrs=extra)
        if needs_grad:
            ctx.save_for_backward(q, k, v, o, lse)
        ctx.device_type = device_type
        ctx.scale = 0.125 if softmax_scale is None else float(softmax_scale)
        ctx.causal = bool(causal)
        if return_lse:
            ctx.mark_non_differentiable(lse)
            return o, lse
        return o

    @staticmethod
    def backward(ctx, do, *unused):
        q, k, v, o, lse = ctx.saved_tensors
        B, H, Lq, d = q.shape
        Lkv = k.shape[2]
        if not (k.shape[3] == d and v.shape[3] == d and d in (64, 128)):
            raise NotImplementedError(f"attention backward needs one head dimension of 64 or 128 for q, k and v "
                                      f"(got {d}, {k.shape[3]}, {v.shape[3]})")
        if ctx.causal and Lq != Lkv:
            raise NotImplementedError("causal attention backward needs Lq == Lkv")
        check_like("flash_attn_func backward", "dO", do, o.shape, o.dtype, o.device)
        do = do.contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        with torch.cuda.device(q.device):
            stream = ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
            _lib.check(_lib.load().attn_b200_fa_bwd(P(q), P(k), P(v), P(o), P(do), P(lse), P(dq), P(dk), P(dv), B, H, Lq, Lkv,
                                                    d, 0 if q.dtype == torch.float16 else 1, ctx.scale, int(ctx.causal),
                                                    stream))
        return dq, dk, dv, None, None, None, None


def flash_attn_func(q, k, v, device_type, causal=False, softmax_scale=None, return_lse=False):
    return MultiHeadAttnFunc.apply(q, k, v, device_type, causal, softmax_scale, return_lse)
