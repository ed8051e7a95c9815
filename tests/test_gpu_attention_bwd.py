"""Flash-attention backward on the GPU, through the C ABI and through autograd on the Python operator, against
the CPU fp32 oracle and golden gradients of the reference's formula.

Tolerances (absolute, vs the fp32 oracle evaluated on the same 16-bit inputs, with the forward's o and lse taken
from the GPU forward): fp16 max-abs <= 2e-3 and mean-abs <= 2e-4 relative to max(1, peak |gradient|); bf16 8x."""
import ctypes

import pytest
import torch

from attention_autotuner_b200 import _lib
from attention_autotuner_b200.arch import B200
from oracle import oracle

pytestmark = pytest.mark.gpu


def P(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def run_fwd_bwd(lib, q, k, v, do, scale, causal):
    B, H, Lq, d = q.shape
    Lkv = k.shape[2]
    code = 0 if q.dtype == torch.float16 else 1
    qd, kd, vd, dod = (t.cuda() for t in (q, k, v, do))
    o = torch.full((B, H, Lq, d), float("nan"), device="cuda", dtype=q.dtype)
    lse = torch.full((B, H, Lq), float("nan"), device="cuda")
    _lib.check(lib.attn_b200_fa_fwd(P(qd), P(kd), P(vd), P(o), P(lse), B, H, Lq, Lkv, d, d, code, scale, int(causal), None))
    dq = torch.full_like(qd, float("nan"))
    dk = torch.full_like(kd, float("nan"))
    dv = torch.full_like(vd, float("nan"))
    _lib.check(lib.attn_b200_fa_bwd(P(qd), P(kd), P(vd), P(o), P(dod), P(lse), P(dq), P(dk), P(dv), B, H, Lq, Lkv, d, code,
                                    scale, int(causal), None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return dq.cpu(), dk.cpu(), dv.cpu()


def rand_case(seed, B, H, Lq, Lkv, d, dt):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, H, Lq, d, generator=g).to(dt), torch.randn(B, H, Lkv, d, generator=g).to(dt),
            torch.randn(B, H, Lkv, d, generator=g).to(dt), torch.randn(B, H, Lq, d, generator=g).to(dt))


def check(grads, q, k, v, do, scale, causal, dtype_name):
    ref = oracle.attention_bwd(q, k, v, do, scale, causal)
    for got, want, name in zip(grads, ref, ("dq", "dk", "dv")):
        st = oracle.error_stats(got, want)
        assert oracle.within(st, dtype_name, scale_by_peak=True), (name, st)


@pytest.mark.parametrize("name", ["attn_bwd_d128_ragged", "attn_bwd_d64"])
def test_golden_gradients_of_the_reference_formula(lib, golden, name):
    g = golden(name)
    q, k, v, do = (torch.from_numpy(g[x]) for x in ("q", "k", "v", "do"))
    grads = run_fwd_bwd(lib, q, k, v, do, 0.125, False)
    for got, key in zip(grads, ("dq", "dk", "dv")):
        st = oracle.error_stats(got, torch.from_numpy(g[key]))
        assert oracle.within(st, "fp16", scale_by_peak=True), (key, st)


@pytest.mark.parametrize("dtype_name", ["fp16", "bf16"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
def test_square_medium(lib, dtype_name, causal, d):
    dt = torch.float16 if dtype_name == "fp16" else torch.bfloat16
    q, k, v, do = rand_case(3, 2, 3, 640, 640, d, dt)
    scale = d ** -0.5
    check(run_fwd_bwd(lib, q, k, v, do, scale, causal), q, k, v, do, scale, causal, dtype_name)


@pytest.mark.parametrize("Lq,Lkv,causal", [(1, 1, False), (1, 300, False), (127, 129, False), (129, 127, False),
                                           (300, 1, False), (200, 200, True), (1, 1, True), (513, 513, True)])
def test_ragged_and_rectangular(lib, Lq, Lkv, causal):
    q, k, v, do = rand_case(5, 1, 2, Lq, Lkv, 128, torch.float16)
    check(run_fwd_bwd(lib, q, k, v, do, 0.125, causal), q, k, v, do, 0.125, causal, "fp16")


def test_many_slices_deterministic_and_linear_in_dout(lib):
    """More (batch, head) slices than SMs (several work items per CTA); two runs agree bit for bit; the gradients are
    linear in dO (doubling dO doubles them up to 16-bit rounding in the subnormal range)."""
    q, k, v, do = rand_case(7, 4, 48, 384, 384, 128, torch.float16)
    do = do * 0.25
    a = run_fwd_bwd(lib, q, k, v, do, 0.125, True)
    b = run_fwd_bwd(lib, q, k, v, do, 0.125, True)
    c = run_fwd_bwd(lib, q, k, v, do * 2, 0.125, True)
    for x, y, z in zip(a, b, c):
        assert torch.equal(x, y)
        assert (x.float() * 2 - z.float()).abs().max().item() < 1e-3
    ref = oracle.attention_bwd(q[:1, :4], k[:1, :4], v[:1, :4], do[:1, :4], 0.125, True)
    for got, want in zip(a, ref):
        assert oracle.within(oracle.error_stats(got[:1, :4], want), "fp16", scale_by_peak=True)


@pytest.mark.parametrize("split", ["0", "1"])
def test_more_query_blocks_than_the_delta_cache_holds(lib, monkeypatch, split):
    """The three-kernel form's dK kernel caches delta for the first 32 query blocks of a slice; 33 blocks exercise both
    of its paths (and many ring turns of the fused kernel)."""
    monkeypatch.setenv("ATTN_B200_FA_BWD_SPLIT", split)
    q, k, v, do = rand_case(17, 1, 2, 4224, 256, 64, torch.float16)
    check(run_fwd_bwd(lib, q, k, v, do, 0.125, False), q, k, v, do, 0.125, False, "fp16")


@pytest.mark.parametrize("split", ["1", "0"])
@pytest.mark.parametrize("d,causal", [(128, False), (64, True)])
def test_three_kernel_form_and_fused_form(lib, monkeypatch, split, d, causal):
    """dK and dV come from one fused kernel by default; ATTN_B200_FA_BWD_SPLIT=1 selects the form with one kernel per
    gradient (also taken for very short query sequences). Both are checked against the oracle."""
    monkeypatch.setenv("ATTN_B200_FA_BWD_SPLIT", split)
    q, k, v, do = rand_case(23, 1, 3, 520, 520 if causal else 300, d, torch.float16)
    check(run_fwd_bwd(lib, q, k, v, do, 0.1, causal), q, k, v, do, 0.1, causal, "fp16")


@pytest.mark.parametrize("dtype_name,mag", [("fp16", 1.0 / 64), ("fp16", 512.0), ("bf16", 1e-4), ("bf16", 1e4)])
def test_small_and_large_output_gradients(lib, dtype_name, mag):
    """The fused kernel folds -lse / scale and -delta into its GEMMs as sums of three 16-bit pieces; gradients far from
    unit size (loss scaling, tiny learning signals) must keep their relative accuracy. Errors are judged on
    gradients / mag."""
    dt = torch.float16 if dtype_name == "fp16" else torch.bfloat16
    q, k, v, do = rand_case(29, 1, 2, 384, 448, 128, dt)
    do = (do.float() * mag).to(dt)
    grads = run_fwd_bwd(lib, q, k, v, do, 0.09, False)
    ref = oracle.attention_bwd(q, k, v, do, 0.09, False)
    for got, want, name in zip(grads, ref, ("dq", "dk", "dv")):
        st = oracle.error_stats(got.float() / mag, want / mag)
        assert oracle.within(st, dtype_name, scale_by_peak=True), (name, mag, st)


def test_short_query_sequences_take_the_three_kernel_form(lib):
    """Fewer than 16 queries at d = 64: the dq buffer cannot hold a block of per-query terms."""
    q, k, v, do = rand_case(31, 2, 2, 9, 200, 64, torch.float16)
    check(run_fwd_bwd(lib, q, k, v, do, 0.125, False), q, k, v, do, 0.125, False, "fp16")


def test_argument_errors(lib):
    q, k, v, do = (t.cuda() for t in rand_case(9, 1, 1, 128, 256, 128, torch.float16))
    o = torch.empty_like(q)
    lse = torch.empty(1, 1, 128, device="cuda")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    args = lambda d, causal, scale: (P(q), P(k), P(v), P(o), P(do), P(lse), P(dq), P(dk), P(dv), 1, 1, 128, 256, d, 0, scale,
                                     causal, None)
    assert lib.attn_b200_fa_bwd(*args(96, 0, 0.1)) == 2      # head dimension not built
    assert lib.attn_b200_fa_bwd(*args(128, 1, 0.1)) == 2     # causal with Lq != Lkv
    assert lib.attn_b200_fa_bwd(*args(128, 0, 0.0)) == 1     # scale
    assert lib.attn_b200_fa_bwd(P(q), P(k), P(v), None, P(do), P(lse), P(dq), P(dk), P(dv), 1, 1, 128, 256, 128, 0, 0.1, 0,
                                None) == 1                   # null pointer


def test_autograd_through_the_python_operator(lib):
    from attention_autotuner_b200.ops.attention_interface import flash_attn_func
    q, k, v, do = rand_case(13, 2, 4, 512, 512, 128, torch.float16)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = flash_attn_func(qd, kd, vd, B200(), True, 0.1)
    o.backward(do.cuda())
    torch.cuda.synchronize()
    check((qd.grad.cpu(), kd.grad.cpu(), vd.grad.cpu()), q, k, v, do, 0.1, True, "fp16")
    # unsupported shapes raise instead of returning silently
    q2, k2, v2 = (torch.randn(1, 1, 128, dd, device="cuda", dtype=torch.float16, requires_grad=True) for dd in (64, 64, 128))
    o2 = flash_attn_func(q2, k2, v2, B200())
    with pytest.raises(Exception):
        o2.sum().backward()
