"""Plain PyTorch formulas of the two operators, in whatever dtype / device the inputs have.
Same names and semantics as the reference's python/utils/ref_op.py, plus optional keyword arguments
whose defaults reproduce it. Used by demos and tests; never by the operators themselves."""
import torch
import torch.nn.functional as F


def attention_ref(q, k, v, softmax_scale=0.125, causal=False):
    attn = q @ k.transpose(-1, -2)
    attn = attn * softmax_scale
    if causal:
        Lq, Lkv = attn.shape[-2], attn.shape[-1]
        i = torch.arange(Lq, device=attn.device)[:, None]
        j = torch.arange(Lkv, device=attn.device)[None, :]
        attn = attn.masked_fill(j > i + (Lkv - Lq), float("-inf"))
    return F.softmax(attn, dim=-1) @ v


def retnet_ref(q, k, v, mask, scale=1.0):
    attn = q @ k.transpose(-1, -2)
    qkm = attn * mask if scale == 1.0 else attn * scale * mask
    r_ref = qkm.detach().abs().sum(dim=-1, keepdim=True).clamp(min=1.0)
    return (qkm / r_ref) @ v
