"""CPU fp32 oracle for the two hot paths. TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference legs may import this
module, and only as the checker or the timed CPU baseline. The product path (the CUDA kernels behind
attention_autotuner_b200) never routes through it.

Parity status: PINNED. tests/golden/ holds outputs of the reference's own formulas
(python/utils/ref_op.py, imported unmodified by tests/golden/make_golden.py) on seeded inputs;
tests/test_oracle.py checks every function below against them.

Each function restates the reference formula it cites, evaluated in fp32 on the storage-dtype-rounded
inputs, with the knobs the reference lacks (explicit scale, causal masking, decay-mask builder) added
as arguments whose defaults reproduce the reference.
"""
from __future__ import annotations

import math
import os

import torch

SEED0 = 20240229

# (name -> dict) shapes of the benchmark configurations the parity tests and bench.py use.
CONFIGS = {
    "C1": dict(op="attn", B=2, H=4, Lq=512, Lkv=512, dqk=64, dv=64, dtype="fp16", causal=False),
    "C2": dict(op="attn", B=8, H=16, Lq=4096, Lkv=4096, dqk=128, dv=128, dtype="fp16", causal=False),
    "C3": dict(op="ret", B=8, H=8, Lq=2048, Lkv=2048, dqk=256, dv=512, dtype="fp16"),
    "C4": dict(op="ret_bwd", B=8, H=8, Lq=2048, Lkv=2048, dqk=256, dv=512, dtype="fp16"),
    "C5sq": dict(op="attn", B=16, H=32, Lq=16384, Lkv=16384, dqk=128, dv=128, dtype="bf16", causal=False),
    "C5dec": dict(op="attn", B=16, H=32, Lq=1024, Lkv=16384, dqk=128, dv=128, dtype="bf16", causal=False),
}
_CFG_INDEX = {"C1": 1, "C2": 2, "C3": 3, "C4": 4, "C5sq": 5, "C5dec": 6}


def torch_dtype(name: str) -> torch.dtype:
    return {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}[name]


def slice_inputs(cfg_name: str, b: int, h: int, H: int, Lq: int, Lkv: int, dqk: int, dv: int,
                 dtype: torch.dtype, with_do: bool = False):
    """Seeded N(0,1) q, k, v (and dO) of ONE (batch, head) slice, rounded to the storage dtype.

    Per-slice seeding makes every shard reproducible on any rank without communication (the
    reference draws randn on the GPU with one global seed, python/tests/test_runtime.py:97-103,
    which cannot be reproduced on a CPU)."""
    g = torch.Generator("cpu").manual_seed(SEED0 + 1000 * _CFG_INDEX.get(cfg_name, 0) + b * H + h)
    q = torch.randn(Lq, dqk, generator=g, dtype=torch.float32).to(dtype)
    k = torch.randn(Lkv, dqk, generator=g, dtype=torch.float32).to(dtype)
    v = torch.randn(Lkv, dv, generator=g, dtype=torch.float32).to(dtype)
    if with_do:
        do = torch.randn(Lq, dv, generator=g, dtype=torch.float32).to(dtype)
        return q, k, v, do
    return q, k, v


def decay_gammas(H: int) -> torch.Tensor:
    """gamma_h = 1 - 2^(-5-h), h = 0..H-1 (RetNet's per-head decay)."""
    return 1.0 - torch.pow(2.0, -5.0 - torch.arange(H, dtype=torch.float64))


def decay_mask(H: int, Lq: int, Lkv: int, gammas: torch.Tensor | None = None) -> torch.Tensor:
    """M[h,i,j] = gamma_h^(i-j) for i >= j, else 0, in fp32 (computed in fp64)."""
    if gammas is None:
        gammas = decay_gammas(H)
    i = torch.arange(Lq, dtype=torch.float64)[:, None]
    j = torch.arange(Lkv, dtype=torch.float64)[None, :]
    diff = i - j
    m = torch.pow(gammas.to(torch.float64)[:, None, None], diff.clamp(min=0)[None])
    m = torch.where(diff[None] >= 0, m, torch.zeros_like(m))
    return m.to(torch.float32)


def attention_fwd(q, k, v, scale: float = 0.125, causal: bool = False):
    """o = softmax(q k^T * scale) v and lse, fp32.  python/utils/ref_op.py:2-6 (scale fixed at 0.125
    there, no causal option). causal masks key j for query i when j > i + (Lkv - Lq)."""
    q, k, v = (t.to(torch.float32) for t in (q, k, v))
    s = (q @ k.transpose(-1, -2)) * scale
    if causal:
        Lq, Lkv = s.shape[-2], s.shape[-1]
        i = torch.arange(Lq)[:, None]
        j = torch.arange(Lkv)[None, :]
        s = s.masked_fill(j > i + (Lkv - Lq), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.softmax(s, dim=-1) @ v
    return o, lse


def attention_bwd(q, k, v, do, scale: float = 0.125, causal: bool = False):
    """Closed-form gradients of attention_fwd (the derivative of python/utils/ref_op.py:2-6; the reference's own
    backward is empty, python/ops/attention_interface.py:38-39). Returns (dq, dk, dv) in fp32.
        P = softmax(S),  dV = P^T dO,  dP = dO V^T,  dS = P .* (dP - rowsum(dO .* O)) * scale,  dQ = dS K,  dK = dS^T Q"""
    q, k, v, do = (t.to(torch.float32) for t in (q, k, v, do))
    s = (q @ k.transpose(-1, -2)) * scale
    if causal:
        Lq, Lkv = s.shape[-2], s.shape[-1]
        i = torch.arange(Lq)[:, None]
        j = torch.arange(Lkv)[None, :]
        s = s.masked_fill(j > i + (Lkv - Lq), float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = p @ v
    dv = p.transpose(-1, -2) @ do
    dp = do @ v.transpose(-1, -2)
    delta = (do * o).sum(dim=-1, keepdim=True)
    ds = p * (dp - delta) * scale
    return ds @ k, ds.transpose(-1, -2) @ q, dv


def attention_bwd_autograd(q, k, v, do, scale: float = 0.125, causal: bool = False):
    """Same gradients through torch.autograd on attention_fwd."""
    q, k, v = (t.to(torch.float32).clone().requires_grad_(True) for t in (q, k, v))
    o, _ = attention_fwd(q, k, v, scale, causal)
    o.backward(do.to(torch.float32))
    return q.grad, k.grad, v.grad


def retnet_fwd(q, k, v, mask, scale: float = 1.0):
    """o = ((q k^T * scale * mask) / r) v with r = clamp(sum_j |.|, min=1), fp32.
    python/utils/ref_op.py:8-13 (no scale there). mask is [H,Lq,Lkv] (or [Lq,Lkv] for one slice),
    broadcast over batch. Returns (o, r) with r of shape [..., Lq]."""
    q, k, v, mask = (t.to(torch.float32) for t in (q, k, v, mask))
    qkm = (q @ k.transpose(-1, -2)) * scale * mask
    r = qkm.abs().sum(dim=-1, keepdim=True).clamp(min=1.0)
    o = (qkm / r) @ v
    return o, r.squeeze(-1)


def retnet_bwd(q, k, v, mask, do, scale: float = 1.0):
    """Closed-form gradients of retnet_fwd with r treated as a constant (python/utils/ref_op.py:11
    detaches it; the reference kernel does the same, csrc/kernels/retnet/bwd/bwd_colblock.h:541-550).
    Returns (dq, dk, dv) in fp32. No gradient for mask."""
    q, k, v, mask, do = (t.to(torch.float32) for t in (q, k, v, mask, do))
    qkm = (q @ k.transpose(-1, -2)) * scale * mask
    r = qkm.abs().sum(dim=-1, keepdim=True).clamp(min=1.0)
    p = qkm / r
    dv = p.transpose(-1, -2) @ do
    dp = do @ v.transpose(-1, -2)
    g = (dp / r) * mask * scale
    dk = g.transpose(-1, -2) @ q
    dq = g @ k
    return dq, dk, dv


def retnet_bwd_autograd(q, k, v, mask, do, scale: float = 1.0):
    """Same gradients through torch.autograd on the formula of ref_op.py:8-13 (r detached)."""
    q, k, v = (t.to(torch.float32).clone().requires_grad_(True) for t in (q, k, v))
    mask = mask.to(torch.float32)
    qkm = (q @ k.transpose(-1, -2)) * scale * mask
    r = qkm.detach().abs().sum(dim=-1, keepdim=True).clamp(min=1.0)
    o = (qkm / r) @ v
    o.backward(do.to(torch.float32))
    return q.grad, k.grad, v.grad


def retnet_recurrent(q, k, v, gammas, scale: float = 1.0):
    """The recurrent form, position by position, in fp32: state_t = gamma * state_{t-1} + k_t^T v_t (a [dqk, dv] matrix
    per slice), o_t = scale * q_t state_t. Restates the reference's scan (csrc/kernels/retnet/recurrent/recurrent.h:
    110-114 combines (decay, k*v) pairs as state = decay * state + k*v; :262-275 multiply the scanned state by q and
    sum over the k dimension) for a per-head constant decay. No normalisation, no r. q, k [B,H,L,dqk], v [B,H,L,dv],
    gammas [H]. Parity status of THIS function: unpinned - the reference's kernel cannot be built here and its Python
    package has no formula for the recurrent form; it is pinned only against retnet_retention below (same
    function, evaluated over all pairs)."""
    q, k, v = (t.to(torch.float32) for t in (q, k, v))
    B, H, L, dqk = q.shape
    dv = v.shape[-1]
    g = gammas.to(torch.float32).view(1, H, 1, 1)
    state = torch.zeros(B, H, dqk, dv)
    out = torch.empty(B, H, L, dv)
    for t in range(L):
        state = g * state + k[:, :, t, :, None] * v[:, :, t, None, :]
        out[:, :, t] = torch.einsum("bhk,bhkv->bhv", q[:, :, t], state) * scale
    return out


def retnet_retention(q, k, v, gammas, scale: float = 1.0):
    """The same function over all (i, j) pairs: o = ((q k^T * scale) .* D) v with D[h,i,j] = gamma_h^(i-j) for i >= j.
    This is retnet_fwd without the division by r (python/utils/ref_op.py:9-12 minus line 11)."""
    q, k, v = (t.to(torch.float32) for t in (q, k, v))
    H, L = q.shape[1], q.shape[2]
    d = decay_mask(H, L, L, gammas)
    return ((q @ k.transpose(-1, -2)) * scale * d) @ v


def flops_ret_chunk(B, H, L, dqk, dv) -> int:
    """Chunkwise algorithm, chunks of 128: per chunk Q K^T, W V, Q S and K^T V."""
    nchunk = (L + 127) // 128
    per_chunk = 2 * 128 * 128 * dqk + 2 * 128 * 128 * dv + 2 * 2 * 128 * dqk * dv
    return B * H * nchunk * per_chunk


# ------------------------------------------------------------------------------------------------
# FLOP model (algorithmic; recomputation forced by tiling is not counted)
# ------------------------------------------------------------------------------------------------
def pairs(Lq: int, Lkv: int, causal: bool) -> int:
    if not causal:
        return Lq * Lkv
    shift = Lkv - Lq
    return sum(max(0, min(Lkv, i + shift + 1)) for i in range(Lq))


def flops_fwd(B, H, Lq, Lkv, dqk, dv, causal=False) -> int:
    return 2 * B * H * pairs(Lq, Lkv, causal) * (dqk + dv)


def flops_attn_bwd(B, H, Lq, Lkv, d, causal=False) -> int:
    """Five GEMMs over the (query, key) pairs that are not masked: S, dP, dV, dQ, dK."""
    return 5 * 2 * B * H * pairs(Lq, Lkv, causal) * d


def flops_ret_bwd(B, H, Lq, Lkv, dqk, dv, causal=False) -> int:
    return 2 * B * H * pairs(Lq, Lkv, causal) * (3 * dqk + 2 * dv)


# ------------------------------------------------------------------------------------------------
# Tolerances (absolute, against this fp32 oracle)
# ------------------------------------------------------------------------------------------------
TOL = {
    # fp16 outputs
    "fp16": dict(max_abs=2e-3, mean_abs=2e-4),
    # bf16 has 3 fewer mantissa bits: 8x
    "bf16": dict(max_abs=1.6e-2, mean_abs=1.6e-3),
}


def error_stats(x: torch.Tensor, ref: torch.Tensor) -> dict:
    d = (x.to(torch.float32) - ref.to(torch.float32)).abs()
    denom = ref.abs().max().clamp(min=1e-30)
    return dict(max_abs=d.max().item(), mean_abs=d.mean().item(), max_rel_to_peak=(d.max() / denom).item(),
                ref_peak=denom.item())


def report(name: str, stats: dict, dtype_name: str = "fp16", scale_by_peak: bool = False) -> bool:
    """Prints one line with the error figures of a compared tensor (max-abs, mean-abs, max-abs relative to the
    reference's peak, the peak, and which bound gates it), appends the record to the JSON-lines file named by the
    environment variable ATTN_B200_PARITY_LOG when it is set, and returns within(...)."""
    ok = within(stats, dtype_name, scale_by_peak)
    gate = "peak-scaled" if (scale_by_peak and stats["ref_peak"] > 1.0) else "absolute"
    t = TOL[dtype_name]
    print(f"[parity] {name}: max_abs={stats['max_abs']:.3e} mean_abs={stats['mean_abs']:.3e} "
          f"max_rel_to_peak={stats['max_rel_to_peak']:.3e} ref_peak={stats['ref_peak']:.3e} "
          f"bound={gate} ({t['max_abs']:.1e}/{t['mean_abs']:.1e} {dtype_name}) {'ok' if ok else 'FAIL'}")
    path = os.environ.get("ATTN_B200_PARITY_LOG")
    if path:
        import json
        with open(path, "a") as f:
            f.write(json.dumps(dict(name=name, dtype=dtype_name, gate=gate, ok=ok, **stats)) + "\n")
    return ok


def within(stats: dict, dtype_name: str, scale_by_peak: bool = False) -> bool:
    """scale_by_peak: gate on error relative to max(1, |ref| peak): gradients that sum thousands of
    terms have magnitudes well above 1, where an absolute 2e-3 is below the output dtype's own spacing."""
    t = TOL[dtype_name]
    s = max(1.0, stats["ref_peak"]) if scale_by_peak else 1.0
    return stats["max_abs"] <= t["max_abs"] * s and stats["mean_abs"] <= t["mean_abs"] * s and math.isfinite(stats["max_abs"])
