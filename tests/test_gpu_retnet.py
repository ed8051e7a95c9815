"""RetNet parallel forward + backward on the GPU, through the C ABI and the Python operator, against the
CPU fp32 oracle (r detached in the backward, exactly as the reference's retnet_ref, python/utils/ref_op.py:11)
and the golden vectors produced by the reference's own formula + torch.autograd.

Tolerance: fp16 max-abs <= 2e-3, mean-abs <= 2e-4 against the fp32 oracle, scaled by max(1, peak |ref|) for
tensors whose magnitude exceeds 1 (gradients sum hundreds of terms; fp16's spacing at 8 is already 7.8e-3)."""
import ctypes

import pytest
import torch

from attention_autotuner_b200 import _lib
from attention_autotuner_b200.arch import B200
from oracle import oracle

pytestmark = pytest.mark.gpu


def P(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def run_fwd_bwd(lib, q, k, v, do, mask=None, decay=None, scale=1.0, causal=0):
    B, H, Lq, dqk = q.shape
    Lkv, dv = v.shape[2], v.shape[3]
    code = 0 if q.dtype == torch.float16 else 1
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    md = mask.cuda() if mask is not None else None
    dd = decay.float().cuda() if decay is not None else None
    nan = float("nan")
    o = torch.full((B, H, Lq, dv), nan, device="cuda", dtype=q.dtype)
    r = torch.full((B, H, Lq), nan, device="cuda")
    _lib.check(lib.attn_b200_ret_fwd(P(qd), P(kd), P(vd), P(md), P(o), P(r), B, H, Lq, Lkv, dqk, dv, code, scale,
                                     P(dd), causal, None))
    dq = torch.full((B, H, Lq, dqk), nan, device="cuda", dtype=q.dtype)
    dk = torch.full((B, H, Lkv, dqk), nan, device="cuda", dtype=q.dtype)
    dvo = torch.full((B, H, Lkv, dv), nan, device="cuda", dtype=q.dtype)
    _lib.check(lib.attn_b200_ret_bwd(P(qd), P(kd), P(vd), P(md), P(dod), P(r), P(dq), P(dk), P(dvo), None, B, H, Lq,
                                     Lkv, dqk, dv, code, scale, P(dd), causal, None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return o.cpu(), r.cpu(), dq.cpu(), dk.cpu(), dvo.cpu()


def rand_case(seed, B, H, Lq, Lkv, dqk, dv, dt=torch.float16, mscale=0.5):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, Lq, dqk, generator=g).to(dt)
    k = torch.randn(B, H, Lkv, dqk, generator=g).to(dt)
    v = torch.randn(B, H, Lkv, dv, generator=g).to(dt)
    do = torch.randn(B, H, Lq, dv, generator=g).to(dt)
    mask = (mscale * torch.randn(H, Lq, Lkv, generator=g)).to(dt)
    return q, k, v, do, mask


def check_all(got, q, k, v, do, maskf, scale, dtype_name="fp16", tag=None):
    o, r, dq, dk, dv = got
    oref, rref = oracle.retnet_fwd(q, k, v, maskf, scale)
    if tag:
        assert oracle.report(f"{tag} o", oracle.error_stats(o, oref), dtype_name, scale_by_peak=True)
    assert oracle.within(oracle.error_stats(o, oref), dtype_name, scale_by_peak=True)
    assert ((r - rref).abs() / rref).max().item() < 1e-4
    gq, gk, gv = oracle.retnet_bwd(q, k, v, maskf, do, scale)
    for name, a, b in (("dq", dq, gq), ("dk", dk, gk), ("dv", dv, gv)):
        st = oracle.error_stats(a, b)
        if tag:
            oracle.report(f"{tag} {name}", st, dtype_name, scale_by_peak=True)
        assert oracle.within(st, dtype_name, scale_by_peak=True), (name, st)


@pytest.mark.parametrize("name", ["ret_randmask", "ret_demo_scaling", "ret_decay"])
def test_golden_vectors_of_the_reference_formula(lib, golden, name):
    g = golden(name)
    q, k, v, mask, do = (torch.from_numpy(g[x]) for x in ("q", "k", "v", "mask", "do"))
    o, r, dq, dk, dv = run_fwd_bwd(lib, q, k, v, do, mask=mask)   # reference semantics: no scale, mask tensor
    for key, got in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
        st = oracle.error_stats(got, torch.from_numpy(g[key]))
        assert oracle.within(st, "fp16", scale_by_peak=True), (key, st)


@pytest.mark.parametrize("dqk,dv", [(64, 64), (64, 128), (128, 128), (128, 256), (256, 256), (256, 512)])
def test_general_mask_head_dims(lib, dqk, dv):
    q, k, v, do, mask = rand_case(dqk + dv, 1, 2, 384, 384, dqk, dv)
    scale = 0.5 * dqk ** -0.5
    check_all(run_fwd_bwd(lib, q, k, v, do, mask=mask, scale=scale), q, k, v, do, mask.float(), scale)


@pytest.mark.parametrize("dqk,dv", [(64, 64), (128, 256), (256, 512)])
def test_decay_head_dims(lib, dqk, dv):
    H, L = 4, 640
    q, k, v, do, _ = rand_case(7, 1, H, L, L, dqk, dv)
    gam = oracle.decay_gammas(H)
    scale = dqk ** -0.5
    got = run_fwd_bwd(lib, q, k, v, do, decay=gam, scale=scale)
    check_all(got, q, k, v, do, oracle.decay_mask(H, L, L, gam), scale)


@pytest.mark.parametrize("Lq,Lkv", [(1, 8), (128, 128), (200, 328), (129, 136), (640, 256), (256, 640)])
def test_ragged_lengths_general_mask(lib, Lq, Lkv):
    q, k, v, do, mask = rand_case(Lq * 7 + Lkv, 2, 2, Lq, Lkv, 64, 128)
    check_all(run_fwd_bwd(lib, q, k, v, do, mask=mask, scale=0.2), q, k, v, do, mask.float(), 0.2)


@pytest.mark.parametrize("Lq,Lkv", [(1, 1), (100, 100), (333, 200), (200, 333), (512, 512)])
def test_ragged_lengths_decay(lib, Lq, Lkv):
    H = 3
    q, k, v, do, _ = rand_case(Lq + Lkv, 1, H, Lq, Lkv, 64, 128)
    gam = oracle.decay_gammas(H)
    got = run_fwd_bwd(lib, q, k, v, do, decay=gam, scale=0.125)
    check_all(got, q, k, v, do, oracle.decay_mask(H, Lq, Lkv, gam), 0.125)


def test_lower_triangular_hint_equals_full_evaluation(lib):
    """causal=1 with a mask tensor only skips blocks whose mask entries are zero: same bits as causal=0."""
    q, k, v, do, mask = rand_case(5, 1, 2, 512, 512, 128, 128)
    mask = torch.tril(mask)
    a = run_fwd_bwd(lib, q, k, v, do, mask=mask, scale=0.1, causal=0)
    b = run_fwd_bwd(lib, q, k, v, do, mask=mask, scale=0.1, causal=1)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    check_all(b, q, k, v, do, mask.float(), 0.1)


def test_decay_path_matches_materialised_mask_path(lib):
    """gamma close to one: the fp16-rounded mask tensor and the in-register decay agree to fp16 accuracy."""
    H, L = 2, 384
    q, k, v, do, _ = rand_case(9, 1, H, L, L, 128, 128)
    gam = torch.tensor([0.999, 0.9995], dtype=torch.float64)
    m = oracle.decay_mask(H, L, L, gam)
    a = run_fwd_bwd(lib, q, k, v, do, decay=gam, scale=0.09)
    check_all(a, q, k, v, do, m, 0.09)
    b = run_fwd_bwd(lib, q, k, v, do, mask=m.half(), scale=0.09)
    check_all(b, q, k, v, do, m.half().float(), 0.09)


def test_bf16(lib):
    H, L = 2, 512
    q, k, v, do, mask = rand_case(11, 1, H, L, L, 128, 128, dt=torch.bfloat16)
    check_all(run_fwd_bwd(lib, q, k, v, do, mask=mask, scale=0.1), q, k, v, do, mask.float(), 0.1, "bf16")


def test_unnormalised_scores_above_fp16_range_are_reported_not_silently_clamped(lib):
    """The forward keeps S~ unnormalised in 16 bits until the epilogue (the reference divides by the running r before
    its fp16 cast and cannot leave the fp16 range, csrc/kernels/retnet/regfuse/regfuse.h:306-316). Scores beyond
    65504 cannot be held in fp16: the kernel must say so (status 2, then every launcher refuses until it is
    cleared) instead of returning a clamped, wrong output. The same inputs in bf16, whose range is fp32's, must
    simply be right."""
    q, k, v, do, mask = rand_case(13, 1, 1, 256, 256, 64, 64)
    q40, k40 = (q.float() * 40).half(), (k.float() * 40).half()
    sref = (q40.float() @ k40.float().transpose(-1, -2)) * mask.float()
    assert sref.abs().max().item() > 65504                      # the case really leaves the fp16 range
    qd, kd, vd, md = q40.cuda(), k40.cuda(), v.cuda(), mask.cuda()
    o = torch.zeros(1, 1, 256, 64, device="cuda", dtype=torch.float16)
    r = torch.zeros(1, 1, 256, device="cuda")
    args = (P(qd), P(kd), P(vd), P(md), P(o), P(r), 1, 1, 256, 256, 64, 64, 0, 1.0, None, 0, None)
    assert _lib.device_status() == 0
    assert lib.attn_b200_ret_fwd(*args) == 0
    torch.cuda.synchronize()
    assert lib.attn_b200_ret_fwd(*args) == 4                    # ATTN_B200_ERR_DEVICE: noticed before the next launch
    assert "fp16 range" in lib.attn_b200_last_error().decode()
    assert lib.attn_b200_device_status(1) == 2 and "65504" in lib.attn_b200_last_error().decode()
    assert lib.attn_b200_device_status(0) == 0
    assert torch.isfinite(o.float()).all() and torch.isfinite(r).all()
    # r is accumulated in fp32 from the unclamped values and stays right even then
    _, rref = oracle.retnet_fwd(q40, k40, v, mask.float(), 1.0)
    assert ((r.cpu() - rref).abs() / rref).max().item() < 1e-3
    # inputs just inside the range raise nothing
    q5, k5 = (q.float() * 5).half(), (k.float() * 5).half()
    got = run_fwd_bwd(lib, q5, k5, v, do, mask=mask, scale=1.0)
    check_all(got, q5, k5, v, do, mask.float(), 1.0)
    # bf16 holds the same unnormalised scores without clamping: right answer, no status
    qb, kb, vb, dob, mb = (t.float().bfloat16() for t in (q40, k40, v, do, mask))
    gotb = run_fwd_bwd(lib, qb, kb, vb, dob, mask=mb, scale=1.0)
    oref, rref = oracle.retnet_fwd(qb, kb, vb, mb.float(), 1.0)
    assert oracle.report("bf16 forward with scores above the fp16 range", oracle.error_stats(gotb[0], oref), "bf16",
                         scale_by_peak=True)


def test_linearity_and_determinism_at_config3_size(lib):
    """The RetNet benchmark shape at full size (B=8 H=8 L=2048 dqk=256 dv=512 fp16, scale 1/16, decay mask): two runs
    bit-identical (no atomics anywhere), O linear in V, sampled slices against the oracle."""
    c = oracle.CONFIGS["C4"]
    B, H, L, dqk, dv = c["B"], c["H"], c["Lq"], c["dqk"], c["dv"]
    gam = oracle.decay_gammas(H)
    g = torch.Generator(device="cuda").manual_seed(3)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g).half()
    q, k, v, do = mk(B, H, L, dqk), mk(B, H, L, dqk), mk(B, H, L, dv), mk(B, H, L, dv)
    dd = gam.float().cuda()
    outs = []
    for rep in range(2):
        o = torch.empty(B, H, L, dv, device="cuda", dtype=torch.float16)
        r = torch.empty(B, H, L, device="cuda")
        dq, dk, dvo = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _lib.check(lib.attn_b200_ret_fwd(P(q), P(k), P(v), None, P(o), P(r), B, H, L, L, dqk, dv, 0, 1 / 16, P(dd), 0, None))
        _lib.check(lib.attn_b200_ret_bwd(P(q), P(k), P(v), None, P(do), P(r), P(dq), P(dk), P(dvo), None, B, H, L, L,
                                         dqk, dv, 0, 1 / 16, P(dd), 0, None))
        torch.cuda.synchronize()
        outs.append((o, r, dq, dk, dvo))
    for x, y in zip(*outs):
        assert torch.equal(x, y)
    assert _lib.device_status() == 0
    o, r, dq, dk, dvo = outs[0]
    mfull = oracle.decay_mask(H, L, L, gam)
    for (b, h) in ((0, 0), (B - 1, H - 1)):
        sl = lambda t: t[b, h].cpu()
        check_all((sl(o), sl(r), sl(dq), sl(dk), sl(dvo)), sl(q), sl(k), sl(v), sl(do), mfull[h], 1 / 16)


@pytest.mark.parametrize("form", ["decay", "mask"])
def test_config4_every_slice_against_the_oracle(lib, form):
    """B=8 H=8 L=2048 dqk=256 dv=512 fp16, scale 1/16, the decay mask given as per-head gammas and as the reference's
    materialised [H, L, L] fp16 mask tensor (its own call form): O, r, dQ, dK, dV of all 64 (batch, head) slices
    against the fp32 oracle (r detached in the backward, as python/utils/ref_op.py:11). O is a convex-like combination
    of rows of V (sum_j |S~_ij| / r <= 1), so |O| <= max |V| (about 4 for N(0,1) values) and it is held to the ABSOLUTE
    2e-3 / 2e-4 bound; the gradients sum thousands of terms (peaks of 7 to 16) and are gated relative to their peak.
    The worst figures over the slices are printed for every tensor."""
    c = oracle.CONFIGS["C4"]
    B, H, L, dqk, dv = c["B"], c["H"], c["Lq"], c["dqk"], c["dv"]
    scale = 1 / 16
    gam = oracle.decay_gammas(H)
    mfull = oracle.decay_mask(H, L, L, gam)
    q, k = torch.empty(B, H, L, dqk, dtype=torch.float16), torch.empty(B, H, L, dqk, dtype=torch.float16)
    v, do = torch.empty(B, H, L, dv, dtype=torch.float16), torch.empty(B, H, L, dv, dtype=torch.float16)
    for b in range(B):
        for h in range(H):
            q[b, h], k[b, h], v[b, h], do[b, h] = oracle.slice_inputs("C4", b, h, H, L, L, dqk, dv, torch.float16, with_do=True)
    if form == "mask":
        mask16 = mfull.half()
        got = run_fwd_bwd(lib, q, k, v, do, mask=mask16, scale=scale, causal=1)
        mref = mask16.float()
    else:
        got = run_fwd_bwd(lib, q, k, v, do, decay=gam, scale=scale)
        mref = mfull
    names = ("o", "dq", "dk", "dv")
    worst = {n: dict(max_abs=0.0, mean_abs=0.0, max_rel_to_peak=0.0, ref_peak=0.0) for n in names}
    o, r, dq, dk, dvo = got
    for b in range(B):
        oref, rref = oracle.retnet_fwd(q[b], k[b], v[b], mref, scale)          # the 8 heads of one batch entry at once
        gq, gk, gv = oracle.retnet_bwd(q[b], k[b], v[b], mref, do[b], scale)
        assert ((r[b] - rref).abs() / rref).max().item() < 1e-4
        for n, a, ref in (("o", o[b], oref), ("dq", dq[b], gq), ("dk", dk[b], gk), ("dv", dvo[b], gv)):
            for h in range(H):
                st = oracle.error_stats(a[h], ref[h])
                assert oracle.within(st, "fp16", scale_by_peak=True), (n, b, h, st)
                worst[n] = {key: max(worst[n][key], st[key]) for key in st}
    for n in names:
        assert oracle.report(f"C4 ({form}) worst of 64 slices {n}", worst[n], "fp16", scale_by_peak=True)
    # O meets the absolute bound (no scaling by its peak)
    assert oracle.within(worst["o"], "fp16", scale_by_peak=False), worst["o"]


@pytest.mark.parametrize("Lq,Lkv,dqk,dv", [(512, 512, 128, 128), (200, 328, 64, 128), (456, 456, 256, 512), (136, 640, 64, 64)])
def test_backward_with_scratch_for_the_transposed_mask(lib, Lq, Lkv, dqk, dv):
    """With a mask tensor the kernels that own keys (dV, dK) need columns of the mask. Given scratch memory
    (attn_b200_ret_bwd_ws, or the reference's dq_accum slot of attn_b200_ret_bwd when it is large enough) the mask is
    transposed once and read by rows; without it the columns are transposed in registers. Same bits either way, and
    right against the oracle."""
    B, H = 2, 2
    q, k, v, do, mask = rand_case(Lq + Lkv + dqk, B, H, Lq, Lkv, dqk, dv)
    base = run_fwd_bwd(lib, q, k, v, do, mask=mask, scale=0.2)            # no scratch
    check_all(base, q, k, v, do, mask.float(), 0.2)
    qd, kd, vd, dod, md, rd = q.cuda(), k.cuda(), v.cuda(), do.cuda(), mask.cuda(), base[1].cuda()
    need = lib.attn_b200_ret_bwd_workspace_bytes(H, Lq, Lkv)
    assert need == H * Lq * Lkv * 2
    outs = []
    for mode in ("ws", "dq_accum"):
        dq = torch.full((B, H, Lq, dqk), float("nan"), device="cuda", dtype=torch.float16)
        dk = torch.full((B, H, Lkv, dqk), float("nan"), device="cuda", dtype=torch.float16)
        dvo = torch.full((B, H, Lkv, dv), float("nan"), device="cuda", dtype=torch.float16)
        if mode == "ws":
            ws = torch.empty(need + 64, dtype=torch.uint8, device="cuda")
            _lib.check(lib.attn_b200_ret_bwd_ws(P(qd), P(kd), P(vd), P(md), P(dod), P(rd), P(dq), P(dk), P(dvo), P(ws), ws.numel(),
                                                B, H, Lq, Lkv, dqk, dv, 0, 0.2, None, 0, None))
        else:  # the reference's call form: a pre-zeroed fp32 [B, H, Lq, dqk] tensor (large enough only when 2*B*dqk >= Lkv)
            acc = torch.zeros(B, H, Lq, dqk, device="cuda", dtype=torch.float32)
            _lib.check(lib.attn_b200_ret_bwd(P(qd), P(kd), P(vd), P(md), P(dod), P(rd), P(dq), P(dk), P(dvo), P(acc), B, H, Lq, Lkv,
                                             dqk, dv, 0, 0.2, None, 0, None))
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        outs.append((dq.cpu(), dk.cpu(), dvo.cpu()))
    for got in outs:
        for a, b in zip(got, base[2:]):
            assert torch.equal(a, b)
    # a workspace that is too small is simply not used
    small = torch.empty(64, dtype=torch.uint8, device="cuda")
    dq = torch.empty(B, H, Lq, dqk, device="cuda", dtype=torch.float16)
    dk, dvo = torch.empty_like(kd), torch.empty_like(vd)
    _lib.check(lib.attn_b200_ret_bwd_ws(P(qd), P(kd), P(vd), P(md), P(dod), P(rd), P(dq), P(dk), P(dvo), P(small), 64, B, H, Lq, Lkv,
                                        dqk, dv, 0, 0.2, None, 0, None))
    torch.cuda.synchronize()
    assert torch.equal(dq.cpu(), base[2]) and torch.equal(dk.cpu(), base[3])


def test_python_operator_forward_backward(lib):
    from attention_autotuner_b200.ops.retnet_interface import RetNetAttnFunc
    q, k, v, do, mask = rand_case(17, 2, 2, 256, 256, 64, 64)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = RetNetAttnFunc(qd, kd, vd, mask.cuda(), B200())          # reference call form
    o.backward(do.cuda())
    got = (o.detach().cpu(), None, qd.grad.cpu(), kd.grad.cpu(), vd.grad.cpu())
    oref, _ = oracle.retnet_fwd(q, k, v, mask.float())
    assert oracle.within(oracle.error_stats(got[0], oref), "fp16", scale_by_peak=True)
    for a, b in zip(got[2:], oracle.retnet_bwd_autograd(q, k, v, mask.float(), do)):
        assert oracle.within(oracle.error_stats(a, b), "fp16", scale_by_peak=True)
    # decay form, scaled, through the same operator
    H = 2
    gam = oracle.decay_gammas(H)
    qd2, kd2, vd2 = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o2 = RetNetAttnFunc(qd2, kd2, vd2, None, B200(), True, scale=0.125, decay=gam)
    o2.backward(do.cuda())
    m = oracle.decay_mask(H, 256, 256, gam)
    oref2, _ = oracle.retnet_fwd(q, k, v, m, 0.125)
    assert oracle.within(oracle.error_stats(o2.detach().cpu(), oref2), "fp16", scale_by_peak=True)
    for a, b in zip((qd2.grad, kd2.grad, vd2.grad), oracle.retnet_bwd(q, k, v, m, do, 0.125)):
        assert oracle.within(oracle.error_stats(a.cpu(), b), "fp16", scale_by_peak=True)


@pytest.mark.parametrize("pair", [0, 1])
def test_cta_pair_knob_through_the_tuner_runtime(pair, tmp_path):
    """The same problem through per-config libraries with and without CTA pairs (cta_group::2 on 256-row
    tiles): both must meet the oracle; lengths are not multiples of 256, so the second CTA of the last pair
    owns a partly (forward: 72 rows) filled tile."""
    from attention_autotuner_b200.autotuner.configs import RetBwdConfig, RetConfig
    from attention_autotuner_b200.autotuner.runtime import Runtime
    B, H, L, dqk, dv = 1, 2, 456, 128, 256
    q, k, v, do, _ = rand_case(23, B, H, L, L, dqk, dv)
    gam = oracle.decay_gammas(H)
    qd, kd, vd, dod = (t.cuda() for t in (q, k, v, do))
    o = torch.full((B, H, L, dv), float("nan"), device="cuda", dtype=torch.float16)
    r = torch.full((B, H, L), float("nan"), device="cuda")
    dq, dk, dvo = torch.full_like(qd, float("nan")), torch.full_like(kd, float("nan")), torch.full_like(vd, float("nan"))
    dec = gam.float().cuda()
    fwd = Runtime(B200(), RetConfig(128, 128, dqk, dv, dv_chunk=128, cta_pair=pair), tmp_dir=str(tmp_path))
    bwd = Runtime(B200(), RetBwdConfig(128, 128, dqk, dv, dv_chunk=256, dq_chunk=128, cta_pair=pair), tmp_dir=str(tmp_path))
    fwd.apply([qd, kd, vd, None, o, r], scale=0.1, causal=True, decay=dec)
    bwd.apply([qd, kd, vd, None, dod, r, dq, dk, dvo, None], scale=0.1, causal=True, decay=dec)
    torch.cuda.synchronize()
    assert fwd.device_status() == 0 and bwd.device_status() == 0
    m = oracle.decay_mask(H, L, L, gam)
    check_all((o.cpu(), r.cpu(), dq.cpu(), dk.cpu(), dvo.cpu()), q, k, v, do, m, 0.1)


def test_argument_errors(lib):
    x = torch.zeros(1, 1, 128, 64, device="cuda", dtype=torch.float16)
    r = torch.zeros(1, 1, 128, device="cuda")
    m = torch.zeros(1, 128, 128, device="cuda", dtype=torch.float16)
    d = torch.ones(1, device="cuda")
    args = lambda mask, dec, dqk=64: (P(x), P(x), P(x), P(mask), P(x), P(r), 1, 1, 128, 128, dqk, 64, 0, 1.0, P(dec), 0, None)
    assert lib.attn_b200_ret_fwd(*args(None, None)) == 1        # neither mask nor decay
    assert lib.attn_b200_ret_fwd(*args(m, d)) == 1              # both
    assert lib.attn_b200_ret_fwd(*args(m, None, 96)) == 2       # head dim not built
    assert lib.attn_b200_ret_fwd(*args(m, None)) == 0
    torch.cuda.synchronize()


def test_host_buffer_operator_forward_backward():
    """retnet_host: host tensors in, (o, dq, dk, dv) on the host out, batch entries pipelined through three
    streams; bit-identical to the device operator on the whole batch."""
    from attention_autotuner_b200.ops.host_interface import retnet_host
    from attention_autotuner_b200.ops.retnet_interface import RetNetAttnFunc
    B, H, L, dqk, dv = 3, 2, 256, 64, 128
    q, k, v, do, _ = rand_case(41, B, H, L, L, dqk, dv)
    q, k, v, do = (t.pin_memory() for t in (q, k, v, do))
    gam = oracle.decay_gammas(H)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = RetNetAttnFunc(qd, kd, vd, None, B200(), True, scale=0.125, decay=gam)
    o.backward(do.cuda())
    ref = [t.detach().cpu() for t in (o, qd.grad, kd.grad, vd.grad)]
    got = retnet_host(q, k, v, B200(), decay=gam, causal=True, scale=0.125, dout=do)
    for a, b in zip(got, ref):                # no device synchronisation: the results are complete on return
        assert torch.equal(a, b)
    fwd_only = retnet_host(q, k, v, B200(), decay=gam, causal=True, scale=0.125, chunks=2)
    assert torch.equal(fwd_only, ref[0])
    m = oracle.decay_mask(H, L, L, gam)
    oref, _ = oracle.retnet_fwd(q, k, v, m, 0.125)
    assert oracle.within(oracle.error_stats(got[0], oref), "fp16", scale_by_peak=True)
