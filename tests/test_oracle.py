"""The CPU oracle against the golden vectors produced by the reference's own formulas
(tests/golden/make_golden.py imports python/utils/ref_op.py of the reference), plus internal consistency
of the knobs the reference lacks (scale, causal, decay mask, closed-form backward)."""
import math

import pytest
import torch

from oracle import oracle


def T(a):
    return torch.from_numpy(a)


@pytest.mark.parametrize("name", ["attn_d64", "attn_d128_ragged", "attn_d256_128_demo_scaling"])
def test_attention_matches_reference_golden(golden, name):
    g = golden(name)
    o, lse = oracle.attention_fwd(T(g["q"]), T(g["k"]), T(g["v"]))  # defaults = reference: scale 0.125, non-causal
    assert torch.allclose(o, T(g["o"]), rtol=1e-5, atol=1e-6)
    assert torch.isfinite(lse).all()


@pytest.mark.parametrize("name", ["ret_randmask", "ret_demo_scaling", "ret_decay"])
def test_retnet_matches_reference_golden(golden, name):
    g = golden(name)
    q, k, v, mask, do = (T(g[x]) for x in ("q", "k", "v", "mask", "do"))
    o, r = oracle.retnet_fwd(q, k, v, mask)
    assert torch.allclose(o, T(g["o"]), rtol=1e-5, atol=1e-6)
    assert (r >= 1.0).all()
    for grads in (oracle.retnet_bwd(q, k, v, mask, do), oracle.retnet_bwd_autograd(q, k, v, mask, do)):
        for got, key in zip(grads, ("dq", "dk", "dv")):
            ref = T(g[key])
            assert torch.allclose(got, ref, rtol=1e-4, atol=1e-4 * max(1.0, ref.abs().max().item())), key


@pytest.mark.parametrize("name", ["attn_bwd_d128_ragged", "attn_bwd_d64"])
def test_attention_backward_matches_reference_golden(golden, name):
    """Closed-form gradients against autograd through the reference's attention formula (golden), and against
    autograd through the oracle's own forward, with and without the causal mask."""
    g = golden(name)
    q, k, v, do = (T(g[x]) for x in ("q", "k", "v", "do"))
    dq, dk, dv = oracle.attention_bwd(q, k, v, do, 0.125, False)
    for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert (got - T(g[key])).abs().max().item() < 2e-5, key
    Lmin = min(q.shape[2], k.shape[2])
    qs, dos, ks, vs = q[:, :, :Lmin], do[:, :, :Lmin], k[:, :, :Lmin], v[:, :, :Lmin]
    for causal, scale in ((True, 0.125), (False, 0.3)):
        a = oracle.attention_bwd(qs, ks, vs, dos, scale, causal)
        b = oracle.attention_bwd_autograd(qs, ks, vs, dos, scale, causal)
        for x, y in zip(a, b):
            assert (x - y).abs().max().item() < 2e-5


def test_lse_and_scale_and_causal():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(2, 3, 40, 16, generator=g) for _ in range(3))
    o, lse = oracle.attention_fwd(q, k, v, scale=0.3, causal=True)
    s = (q @ k.transpose(-1, -2)) * 0.3
    for i in range(40):
        row = s[..., i, : i + 1]
        p = torch.softmax(row, -1)
        assert torch.allclose(o[..., i, :], (p.unsqueeze(-2) @ v[..., : i + 1, :]).squeeze(-2), atol=1e-5)
        assert torch.allclose(lse[..., i], torch.logsumexp(row, -1), atol=1e-5)
    # rectangular causal is bottom-right aligned
    o2, _ = oracle.attention_fwd(q[..., 30:, :], k, v, scale=0.3, causal=True)
    assert torch.allclose(o2, o[..., 30:, :], atol=1e-5)


def test_decay_mask_and_scaled_retnet():
    H, L = 3, 50
    m = oracle.decay_mask(H, L, L)
    gam = oracle.decay_gammas(H)
    assert m.shape == (H, L, L)
    assert m[1, 7, 3].item() == pytest.approx(float(gam[1]) ** 4, rel=1e-6)
    assert m[2, 3, 7].item() == 0.0 and m[0, 5, 5].item() == 1.0
    g = torch.Generator().manual_seed(2)
    q, k = (torch.randn(2, H, L, 8, generator=g) for _ in range(2))
    v = torch.randn(2, H, L, 12, generator=g)
    o1, r1 = oracle.retnet_fwd(q, k, v, m, scale=0.25)
    o2, r2 = oracle.retnet_fwd(q * 0.25, k, v, m)  # the reference has no scale: pre-scaling q is equivalent
    assert torch.allclose(o1, o2, atol=1e-6) and torch.allclose(r1, r2, atol=1e-6)
    do = torch.randn(2, H, L, 12, generator=g)
    a = oracle.retnet_bwd(q, k, v, m, do, scale=0.25)
    b = oracle.retnet_bwd_autograd(q, k, v, m, do, scale=0.25)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, rtol=1e-4, atol=1e-5)


def test_flop_model():
    assert oracle.flops_fwd(2, 4, 512, 512, 64, 64) == 2 * 8 * 512 * 512 * 128
    assert oracle.pairs(4096, 4096, True) == 4096 * 4097 // 2
    assert oracle.pairs(2, 5, True) == 4 + 5
    assert oracle.flops_ret_bwd(1, 1, 8, 8, 4, 6) == 2 * 64 * (12 + 12)
    # B=8 H=16 L=4096 d=128 forward: 1.0995 TFLOP
    assert math.isclose(oracle.flops_fwd(8, 16, 4096, 4096, 128, 128), 1.0995e12, rel_tol=1e-3)


def test_slice_inputs_reproducible():
    a = oracle.slice_inputs("C1", 1, 2, 4, 64, 64, 16, 16, torch.float16)
    b = oracle.slice_inputs("C1", 1, 2, 4, 64, 64, 16, 16, torch.float16)
    c = oracle.slice_inputs("C1", 1, 3, 4, 64, 64, 16, 16, torch.float16)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert not torch.equal(a[0], c[0])


def test_recurrent_form_equals_the_all_pairs_form():
    """The position-by-position recurrence (the reference's scan operator, csrc/kernels/retnet/recurrent/recurrent.h:
    110-114) and the all-pairs evaluation with the decay mask are the same function; where r = 1 it is also what
    retnet_fwd (pinned to the reference's retnet_ref) returns."""
    g = torch.Generator().manual_seed(3)
    B, H, L, dqk, dv = 2, 3, 70, 16, 24
    q, k, v = (torch.randn(B, H, L, d, generator=g) for d in (dqk, dqk, dv))
    gam = oracle.decay_gammas(H)
    a = oracle.retnet_recurrent(q, k, v, gam, 0.3)
    b = oracle.retnet_retention(q, k, v, gam, 0.3)
    assert torch.allclose(a, b, atol=1e-4, rtol=1e-5)
    tiny = 1e-5
    c, r = oracle.retnet_fwd(q, k, v, oracle.decay_mask(H, L, L, gam), tiny)
    assert (r == 1).all()
    assert torch.allclose(c, oracle.retnet_retention(q, k, v, gam, tiny), atol=1e-9, rtol=1e-5)
    assert oracle.flops_ret_chunk(1, 1, 128, 256, 512) == 2 * 128 * 128 * 256 + 2 * 128 * 128 * 512 + 4 * 128 * 256 * 512
