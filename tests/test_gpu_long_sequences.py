"""Long-sequence bf16 attention (B=16, H=32, d=128: 512 (batch, head) slices; Lq = Lkv = 16384 non-causal and causal,
and Lq = 1024 against Lkv = 16384): whole slices against the fp32 oracle, launched on the full-size tensors so that
element offsets pass 2^31 (each tensor has 2^30 elements; the reference indexes with 32-bit ints,
csrc/kernels/attention/regfuse/regfuse.h:62-65), and checksums of the outputs that must not depend on how the
slices are split into launches (what a rank count changes).

Tolerance: bf16 max-abs <= 1.6e-2 and mean-abs <= 1.6e-3 against the fp32 oracle (8x the fp16 bound)."""
import ctypes

import pytest
import torch

from attention_autotuner_b200 import _lib, sharding
from oracle import oracle

pytestmark = pytest.mark.gpu

D = 128
SCALE = D ** -0.5


def P(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _launch(lib, q, k, v, o, causal, lse=None):
    B, H, Lq, _ = q.shape
    Lkv = k.shape[2]
    _lib.check(lib.attn_b200_fa_fwd(P(q), P(k), P(v), P(o), P(lse), B, H, Lq, Lkv, D, D, 1, SCALE, int(causal), None))


def _gen(B, H, L, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = torch.empty(B, H, L, D, device="cuda", dtype=torch.bfloat16)
    for b in range(B):   # batch entry by batch entry: the fp32 randn of the whole tensor would need 4 GB
        out[b] = torch.randn(H, L, D, device="cuda", generator=g).to(torch.bfloat16)
    return out


def _check_slice(tag, o, lse, q, k, v, b, h, causal):
    oref, lref = oracle.attention_fwd(q[b, h].cpu(), k[b, h].cpu(), v[b, h].cpu(), SCALE, causal)
    st = oracle.error_stats(o[b, h].cpu(), oref)
    assert oracle.report(f"{tag} slice ({b},{h}) o", st, "bf16"), (tag, b, h, st)
    if lse is not None:
        assert (lse[b, h].cpu() - lref).abs().max().item() < 1e-3


@pytest.mark.parametrize("causal", [False, True])
def test_square_16384_full_size_first_and_last_slice(lib, causal):
    B, H, L = 16, 32, 16384
    q, k, v = _gen(B, H, L, 1), _gen(B, H, L, 2), _gen(B, H, L, 3)
    assert q.numel() == 2 ** 30
    o = torch.full((B, H, L, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    lse = torch.full((B, H, L), float("nan"), device="cuda", dtype=torch.float32)
    _launch(lib, q, k, v, o, causal, lse)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    _check_slice("L=16384" + (" causal" if causal else ""), o, lse, q, k, v, 0, 0, causal)
    _check_slice("L=16384" + (" causal" if causal else ""), o, lse, q, k, v, B - 1, H - 1, causal)   # offsets beyond 2^31
    assert not torch.isnan(o[B // 2]).any()


def test_decode_like_1024_by_16384_full_size(lib):
    B, H, Lq, Lkv = 16, 32, 1024, 16384
    q, k, v = _gen(B, H, Lq, 4), _gen(B, H, Lkv, 5), _gen(B, H, Lkv, 6)
    o = torch.full((B, H, Lq, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    lse = torch.full((B, H, Lq), float("nan"), device="cuda", dtype=torch.float32)
    _launch(lib, q, k, v, o, False, lse)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    for b, h in ((0, 0), (7, 13), (B - 1, H - 1)):
        _check_slice("Lq=1024 Lkv=16384", o, lse, q, k, v, b, h, False)
    assert not torch.isnan(o).any()


@pytest.mark.parametrize("causal", [False, True])
def test_output_checksums_do_not_depend_on_the_number_of_ranks(lib, causal):
    """Rank r of N runs slices sharding.slice_range(r, N, n) as its own launch. Emulated on one GPU for N = 1, 2, 4,
    8 (one launch per rank, one after the other): every slice's output must be bit-identical whichever launch,
    batch position or grid computed it, so the per-slice checksums (sums of the 16-bit patterns) are equal."""
    n, L = 16, 4096
    q, k, v = _gen(n, 1, L, 11), _gen(n, 1, L, 12), _gen(n, 1, L, 13)

    def sums_for(world):
        o = torch.full((n, 1, L, D), float("nan"), device="cuda", dtype=torch.bfloat16)
        for r in range(world):
            lo, hi = sharding.slice_range(r, world, n)
            _launch(lib, q[lo:hi], k[lo:hi], v[lo:hi], o[lo:hi], causal)
        torch.cuda.synchronize()
        return o.view(torch.int16).reshape(n, -1).to(torch.int64).sum(dim=1).cpu(), o
    base, o1 = sums_for(1)
    for world in (2, 4, 8):
        s, ow = sums_for(world)
        assert torch.equal(s, base), world
        assert torch.equal(ow.view(torch.int16), o1.view(torch.int16))
    _check_slice("rank-count invariance", o1, None, q, k, v, n - 1, 0, causal)
    assert _lib.device_status() == 0
