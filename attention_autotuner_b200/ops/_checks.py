"""Argument checks shared by the operators. The kernels index raw pointers from q's batch / head counts and the
configured head dimensions, so every tensor is checked against q BEFORE anything is launched: a mismatched call
(fewer k/v heads, another head dimension, a tensor on another device) raises ValueError instead of reading
past an allocation. The reference checks nothing but two head-dimension asserts
(python/ops/attention_interface.py:23-24)."""
import torch

_DTYPES = (torch.float16, torch.bfloat16)


def _fail(msg):
    raise ValueError(msg)


def check_qkv(op: str, q, k, v):
    """q [B,H,Lq,dqk], k [B,H,Lkv,dqk], v [B,H,Lkv,dv]: CUDA tensors of one 16-bit dtype on one device."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor) or t.dim() != 4:
            _fail(f"{op}: {name} must be a 4-d tensor [batch, heads, length, head_dim]")
    if q.dtype not in _DTYPES:
        _fail(f"{op}: dtype must be float16 or bfloat16, got {q.dtype}")
    for name, t in (("k", k), ("v", v)):
        if t.device != q.device:
            _fail(f"{op}: {name} is on {t.device}, q on {q.device}")
        if t.dtype != q.dtype:
            _fail(f"{op}: {name} has dtype {t.dtype}, q has {q.dtype}")
        if tuple(t.shape[:2]) != tuple(q.shape[:2]):
            _fail(f"{op}: {name} has batch/heads {tuple(t.shape[:2])}, q has {tuple(q.shape[:2])} "
                  "(grouped or multi-query k/v must be expanded by the caller)")
    if k.shape[3] != q.shape[3]:
        _fail(f"{op}: k has head dimension {k.shape[3]}, q has {q.shape[3]}")
    if v.shape[2] != k.shape[2]:
        _fail(f"{op}: v has {v.shape[2]} keys, k has {k.shape[2]}")
    if min(q.shape) <= 0 or min(k.shape) <= 0 or min(v.shape) <= 0:
        _fail(f"{op}: empty tensors are not supported (shapes {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)})")
    dqk, dv = q.shape[3], v.shape[3]
    if q.device.type != "cuda":
        _fail(f"{op}: tensors must live on a CUDA device (there is no CPU path); q is on {q.device}")
    if dqk % 64 != 0 or dqk > 256:
        _fail(f"{op}: head dimension of q/k must be a multiple of 64 up to 256, got {dqk}")
    if dv % 64 != 0 or dv > 512:
        _fail(f"{op}: head dimension of v must be a multiple of 64 up to 512, got {dv}")


def check_like(op: str, name: str, t, shape, dtype, device):
    """A tensor that must have exactly this shape, dtype and device (dO against O, r against [B,H,Lq], ...)."""
    if not isinstance(t, torch.Tensor):
        _fail(f"{op}: {name} must be a tensor")
    if tuple(t.shape) != tuple(shape):
        _fail(f"{op}: {name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
    if t.dtype != dtype:
        _fail(f"{op}: {name} has dtype {t.dtype}, expected {dtype}")
    if t.device != device:
        _fail(f"{op}: {name} is on {t.device}, expected {device}")


def check_mask_decay(op: str, q, k, mask, decay):
    """Exactly one of mask [H,Lq,Lkv] (dtype and device of q) / decay (H gammas, any float dtype, any device)."""
    if (mask is None) == (decay is None):
        _fail(f"{op}: give either a mask tensor or per-head decay, not both and not neither")
    H, Lq, Lkv = q.shape[1], q.shape[2], k.shape[2]
    if mask is not None:
        check_like(op, "mask", mask, (H, Lq, Lkv), q.dtype, q.device)
        if Lkv % 8 != 0:
            _fail(f"{op}: a mask tensor needs a key length that is a multiple of 8, got {Lkv}")
    else:
        if not isinstance(decay, torch.Tensor) or decay.numel() != H or not decay.dtype.is_floating_point:
            _fail(f"{op}: decay must be a floating-point tensor of {H} per-head values")
