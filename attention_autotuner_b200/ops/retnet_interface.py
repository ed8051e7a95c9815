"""``RetNetAttnFunc``: same entry point as the reference's python/ops/retnet_interface.py:57.

    o = RetNetAttnFunc(q, k, v, mask, device_type, causal=False, scale=None, decay=None)
    o.backward(do)            # dq, dk, dv; no gradient for mask, r is a constant (ref_op.py:11)

q, k [B,H,L,dqk], v [B,H,Lkv,dv], mask [H,Lq,Lkv], all fp16 (bf16 also accepted). ``scale=None`` keeps the
reference's unscaled scores. ``decay`` (tensor of H per-head gammas) replaces the mask tensor by
M[h,i,j] = gamma_h^(i-j) (i >= j) built inside the kernel; ``mask`` may then be None. With a mask
tensor, ``causal=True`` declares it lower triangular so the kernels skip the blocks above the diagonal
(the reference accepts the argument and ignores it)."""
import torch

from ..arch import Arch
from ._checks import check_like, check_mask_decay, check_qkv
from ..autotuner.runtime import Runtime
from ..autotuner.tunner import RetBwdTunner, RetTunner


def retnet_forward(q, k, v, mask, device_type: Arch, causal=False, scale=None, decay=None):
    """The forward launch without autograd: returns (o, r, mask, decay) with mask / decay as the kernels took them
    (contiguous, decay as fp32 on the device). r = max(sum_j |S~|, 1) per row is what the backward needs."""
    check_qkv("RetNetAttnFunc", q, k, v)
    check_mask_decay("RetNetAttnFunc", q, k, mask, decay)
    q, k, v = [x.contiguous() for x in [q, k, v]]
    batch_size, nheads, seqlen_q, key_dim = q.shape
    head_dim = v.shape[-1]
    maskr = None
    if mask is not None:
        maskr = mask.detach().contiguous()
    decayr = None
    if decay is not None:
        decayr = decay.detach().to(device=q.device, dtype=torch.float32).contiguous().reshape(-1)
    o = torch.empty(batch_size, nheads, seqlen_q, head_dim, device=q.device, dtype=q.dtype)
    r = torch.empty(batch_size, nheads, seqlen_q, device=q.device, dtype=torch.float32)
    arr = [q, k, v, maskr, o, r]
    cc = RetTunner(arch=device_type, torch_array=arr, scale=scale, causal=causal, decay=decayr).tune()
    Runtime(device_type, cc).apply(arr, scale=1.0 if scale is None else scale, causal=causal, decay=decayr)
    return o, r, maskr, decayr


def retnet_backward(q, k, v, mask, do, r, device_type: Arch, causal=False, scale=None, decay=None):
    """The backward launches without autograd: (dq, dk, dv) from the tensors of retnet_forward. r is a constant
    (python/utils/ref_op.py:11 detaches it)."""
    check_qkv("RetNetAttnFunc backward", q, k, v)
    check_mask_decay("RetNetAttnFunc backward", q, k, mask, decay)
    check_like("RetNetAttnFunc backward", "dO", do, (*q.shape[:3], v.shape[3]), q.dtype, q.device)
    check_like("RetNetAttnFunc backward", "r", r, q.shape[:3], torch.float32, q.device)
    do = do.contiguous()
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    # The last slot is the reference's dq_accum scratch (python/ops/retnet_interface.py:48-54). Nothing is accumulated
    # in it here (each output tile has one owner); with a mask tensor it gives the dV / dK kernels room for a transposed
    # copy of the mask (H * Lq * Lkv values), which they read by rows instead of transposing columns in registers.
    scratch = None
    if mask is not None and q.shape[2] % 8 == 0:
        scratch = torch.empty(mask.shape[0] * q.shape[2] * k.shape[2], dtype=q.dtype, device=q.device)
    arr = [q, k, v, mask, do, r, dq, dk, dv, scratch]
    cc = RetBwdTunner(arch=device_type, torch_array=arr, scale=scale, causal=causal, decay=decay).tune()
    Runtime(device_type, cc).apply(arr, scale=1.0 if scale is None else scale, causal=causal, decay=decay)
    return dq, dk, dv


class RetNetAttn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, mask, device_type: Arch, *opts):
        causal = bool(opts[0]) if len(opts) > 0 else False
        scale = opts[1] if len(opts) > 1 else None
        decay = opts[2] if len(opts) > 2 else None
        q, k, v = [x.contiguous() for x in [q, k, v]]
        o, r, maskr, decayr = retnet_forward(q, k, v, mask, device_type, causal, scale, decay)
        ctx.save_for_backward(q, k, v, maskr, r, decayr)
        ctx.device_type = device_type
        ctx.opts = (causal, scale)
        ctx.n_extra = len(opts)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, mask, r, decay = ctx.saved_tensors
        causal, scale = ctx.opts
        dq, dk, dv = retnet_backward(q, k, v, mask, do, r, ctx.device_type, causal, scale, decay)
        return (dq, dk, dv, None, None) + (None,) * ctx.n_extra


def retnet_chunkwise(q, k, v, decay, device_type: Arch = None, scale=None):
    """Chunkwise (recurrent-state) RetNet forward: o[i] = scale * sum_{j <= i} decay_h^(i-j) (q_i . k_j) v_j, the
    unnormalised retention of the reference's recurrent kernel (csrc/kernels/retnet/recurrent/recurrent.h:427-463),
    evaluated chunk by chunk with the state in tensor memory: the cost grows with L, not L^2. Forward only.
    q, k [B,H,L,dqk] (dqk 128 or 256), v [B,H,L,dv], fp16 or bf16 on one CUDA device; ``decay``: H per-head gammas.
    With few (batch, head) slices and a long sequence the library cuts the sequence into segments that run at once
    (attn_b200_ret_chunk_fwd_ws); the scratch for the segment states is allocated here."""
    import ctypes

    from .. import _lib
    check_qkv("retnet_chunkwise", q, k, v)
    check_mask_decay("retnet_chunkwise", q, k, None, decay)
    if k.shape[2] != q.shape[2]:
        raise ValueError(f"retnet_chunkwise: q and k must have the same length, got {q.shape[2]} and {k.shape[2]}")
    if q.shape[3] not in (128, 256):
        raise ValueError(f"retnet_chunkwise: head dimension of q/k must be 128 or 256, got {q.shape[3]}")
    q, k, v = [x.contiguous() for x in [q, k, v]]
    B, H, L, dqk = q.shape
    dv = v.shape[3]
    lib = _lib.load()
    decayd = decay.detach().to(device=q.device, dtype=torch.float32).contiguous().reshape(-1)
    o = torch.empty(B, H, L, dv, device=q.device, dtype=q.dtype)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    with torch.cuda.device(q.device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
        ws_bytes = int(lib.attn_b200_ret_chunk_workspace_bytes(B, H, L, dqk, dv, 0))
        ws = torch.empty(ws_bytes, device=q.device, dtype=torch.uint8) if ws_bytes else None
        _lib.check(lib.attn_b200_ret_chunk_fwd_ws(P(q), P(k), P(v), P(decayd), P(o), P(ws) if ws_bytes else None, ws_bytes, 0,
                                                  B, H, L, dqk, dv, 0 if q.dtype == torch.float16 else 1,
                                                  1.0 if scale is None else float(scale), stream))
    return o


def RetNetAttnFunc(q, k, v, mask, device_type, causal=False, scale=None, decay=None):
    if scale is None and decay is None:
        if causal is False:
            return RetNetAttn.apply(q, k, v, mask, device_type)
        return RetNetAttn.apply(q, k, v, mask, device_type, causal)
    return RetNetAttn.apply(q, k, v, mask, device_type, causal, scale, decay)
