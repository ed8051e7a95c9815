"""Flash-attention forward on the GPU, through the C ABI and through the Python operator, against the
CPU fp32 oracle and the golden vectors of the reference's formula.

Tolerances (absolute, vs the fp32 oracle evaluated on the same 16-bit inputs): fp16 max-abs <= 2e-3 and
mean-abs <= 2e-4; bf16 8x those (three fewer mantissa bits in P and O). LSE is fp32: 1e-3."""
import ctypes

import pytest
import torch

from attention_autotuner_b200 import _lib
from attention_autotuner_b200.arch import B200
from oracle import oracle

pytestmark = pytest.mark.gpu

DT = {"fp16": (torch.float16, 0), "bf16": (torch.bfloat16, 1)}


def P(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def run_capi(lib, q, k, v, scale, causal, want_lse=True):
    B, H, Lq, dqk = q.shape
    Lkv, dv = v.shape[2], v.shape[3]
    code = 0 if q.dtype == torch.float16 else 1
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.full((B, H, Lq, dv), float("nan"), device="cuda", dtype=q.dtype)
    lse = torch.full((B, H, Lq), float("nan"), device="cuda") if want_lse else None
    _lib.check(lib.attn_b200_fa_fwd(P(qd), P(kd), P(vd), P(o), P(lse), B, H, Lq, Lkv, dqk, dv, code, scale,
                                    int(causal), None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return o.cpu(), (lse.cpu() if want_lse else None)


def rand_qkv(seed, B, H, Lq, Lkv, dqk, dv, dt):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, H, Lq, dqk, generator=g).to(dt), torch.randn(B, H, Lkv, dqk, generator=g).to(dt),
            torch.randn(B, H, Lkv, dv, generator=g).to(dt))


def check(o, lse, q, k, v, scale, causal, dtype_name):
    oref, lref = oracle.attention_fwd(q, k, v, scale, causal)
    st = oracle.error_stats(o, oref)
    assert oracle.within(st, dtype_name), st
    if lse is not None:
        assert (lse - lref).abs().max().item() < 1e-3


@pytest.mark.parametrize("name", ["attn_d64", "attn_d128_ragged", "attn_d256_128_demo_scaling"])
def test_golden_vectors_of_the_reference_formula(lib, golden, name):
    g = golden(name)
    q, k, v = (torch.from_numpy(g[x]) for x in ("q", "k", "v"))
    o, _ = run_capi(lib, q, k, v, 0.125, False)
    st = oracle.error_stats(o, torch.from_numpy(g["o"]))
    # the demo-scaling case has |o| up to 12, where fp16's own spacing (2^-7) exceeds the absolute bound:
    # the bound scales with max(1, peak |o|)
    assert oracle.within(st, "fp16", scale_by_peak=True), st


def test_config1_full(lib):
    """The small benchmark shape B=2 H=4 L=512 d=64 fp16 non-causal scale 1/8, every slice."""
    c = oracle.CONFIGS["C1"]
    qs, ks, vs = [], [], []
    for b in range(c["B"]):
        for h in range(c["H"]):
            q, k, v = oracle.slice_inputs("C1", b, h, c["H"], c["Lq"], c["Lkv"], c["dqk"], c["dv"], torch.float16)
            qs.append(q), ks.append(k), vs.append(v)
    shape = lambda xs, L, d: torch.stack(xs).view(c["B"], c["H"], L, d)
    q, k, v = shape(qs, 512, 64), shape(ks, 512, 64), shape(vs, 512, 64)
    o, lse = run_capi(lib, q, k, v, 0.125, False)
    check(o, lse, q, k, v, 0.125, False, "fp16")


@pytest.mark.parametrize("dtype_name", ["fp16", "bf16"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dqk,dv", [(64, 64), (128, 128)])
def test_square_medium(lib, dtype_name, causal, dqk, dv):
    dt, _ = DT[dtype_name]
    q, k, v = rand_qkv(3, 2, 3, 1024, 1024, dqk, dv, dt)
    scale = dqk ** -0.5
    o, lse = run_capi(lib, q, k, v, scale, causal)
    check(o, lse, q, k, v, scale, causal, dtype_name)


@pytest.mark.parametrize("Lq,Lkv,causal", [(1, 1, False), (1, 300, False), (127, 129, False), (129, 127, False),
                                           (200, 333, True), (333, 200, True), (384, 640, True), (257, 256, True),
                                           (128, 128, True), (256, 2048, False)])
def test_ragged_and_rectangular(lib, Lq, Lkv, causal):
    """Lengths that are not tile multiples, single rows, Lq != Lkv (causal is bottom-right aligned; rows
    with no visible key give zeros and lse = -inf, as the oracle's softmax of an empty row would not)."""
    q, k, v = rand_qkv(5, 1, 2, Lq, Lkv, 128, 128, torch.float16)
    scale = 128 ** -0.5
    o, lse = run_capi(lib, q, k, v, scale, causal)
    oref, lref = oracle.attention_fwd(q, k, v, scale, causal)
    if causal and Lkv < Lq:
        empty = torch.arange(Lq) + (Lkv - Lq) < 0
        assert (o[:, :, empty] == 0).all() and torch.isinf(lse[:, :, empty]).all()
        o, oref, lse, lref = o[:, :, ~empty], oref[:, :, ~empty], lse[:, :, ~empty], lref[:, :, ~empty]
    st = oracle.error_stats(o, oref)
    assert oracle.within(st, "fp16"), st
    assert (lse - lref).abs().max().item() < 1e-3


@pytest.mark.parametrize("form", ["grid", "persistent"])
@pytest.mark.parametrize("B,H,Lq,Lkv,dqk,dv,causal", [
    (1, 2, 1, 300, 128, 128, False), (1, 2, 129, 127, 128, 128, False), (2, 3, 640, 640, 128, 128, True),
    (1, 2, 300, 900, 128, 128, True), (1, 2, 900, 300, 128, 128, True), (3, 70, 520, 520, 64, 64, True),
    (1, 4, 1300, 1300, 64, 128, False), (2, 2, 768, 768, 128, 64, True)])
def test_both_forms_of_the_forward_kernel(lib, monkeypatch, form, B, H, Lq, Lkv, dqk, dv, causal):
    """The forward exists as a grid of one CTA per 256 query rows and as a persistent grid walking a work list (chosen
    automatically: persistent under a causal mask); ATTN_B200_FA_FWD_FORM forces one of them. Cases: a single query,
    ragged lengths, more keys than queries and fewer (causal rows without any visible key), more work items than
    SMs (several items per CTA, tiles past the end of Q), V narrower and wider than Q."""
    monkeypatch.setenv("ATTN_B200_FA_FWD_FORM", form)
    q, k, v = rand_qkv(41, B, H, Lq, Lkv, dqk, dv, torch.float16)
    scale = dqk ** -0.5
    if B * H > 16:   # the oracle on a few slices only
        o, lse = run_capi(lib, q, k, v, scale, causal)
        check(o[:1, :4], lse[:1, :4], q[:1, :4], k[:1, :4], v[:1, :4], scale, causal, "fp16")
        check(o[-1:, -4:], lse[-1:, -4:], q[-1:, -4:], k[-1:, -4:], v[-1:, -4:], scale, causal, "fp16")
    else:
        o, lse = run_capi(lib, q, k, v, scale, causal)
        if causal and Lkv < Lq:   # rows without a visible key: zeros and lse = -inf; the rest against the oracle
            oref, lref = oracle.attention_fwd(q, k, v, scale, causal)
            empty = torch.arange(Lq) + (Lkv - Lq) < 0
            assert (o[:, :, empty] == 0).all() and torch.isinf(lse[:, :, empty]).all()
            assert oracle.within(oracle.error_stats(o[:, :, ~empty], oref[:, :, ~empty]), "fp16")
            assert (lse[:, :, ~empty] - lref[:, :, ~empty]).abs().max().item() < 1e-3
        else:
            check(o, lse, q, k, v, scale, causal, "fp16")


@pytest.mark.parametrize("causal", [False, True])
def test_both_forms_give_the_same_bits(lib, monkeypatch, causal):
    """Same tile, same order of operations: the persistent and the grid form agree bit for bit (ragged lengths, several
    work items per CTA)."""
    q, k, v = rand_qkv(43, 2, 90, 700, 700, 128, 128, torch.float16)
    out = {}
    for form in ("grid", "persistent"):
        monkeypatch.setenv("ATTN_B200_FA_FWD_FORM", form)
        out[form] = run_capi(lib, q, k, v, 0.09, causal)
    assert torch.equal(out["grid"][0], out["persistent"][0])
    assert torch.equal(out["grid"][1], out["persistent"][1])


@pytest.mark.parametrize("dqk,dv", [(256, 256), (256, 128), (128, 512), (64, 192), (128, 64), (256, 64), (64, 256)])
def test_head_dim_matrix(lib, dqk, dv):
    """The reference's head-dim range: dqk % 64 == 0 <= 256, dv % 64 == 0 <= 512
    (python/ops/attention_interface.py:23-24), including its test shapes (256,256), (256,128), (128,128)."""
    q, k, v = rand_qkv(7, 1, 2, 512, 512, dqk, dv, torch.float16)
    o, lse = run_capi(lib, q, k, v, 0.125, False)
    check(o, lse, q, k, v, 0.125, False, "fp16")


def test_large_scores_trigger_rescale(lib):
    """Keys whose scores grow along the sequence force the running maximum to move by far more than the
    lazy-rescale threshold in every block."""
    q, k, v = rand_qkv(9, 1, 1, 256, 1024, 64, 64, torch.float16)
    ramp = torch.linspace(0.2, 4.0, 1024)[None, None, :, None]
    k = (k.float() * ramp).half()
    o, lse = run_capi(lib, q, k, v, 0.5, False)
    check(o, lse, q, k, v, 0.5, False, "fp16")


def test_reference_test_shape_and_scalings(lib):
    """(B,H,L)=(4,8,2048) as python/tests/test_runtime.py:16 with one head kept, and the demo input scalings
    key = 3*randn, value = 3*randn (python/tests/attntuner_demo.py:45-48), fixed 0.125 scale."""
    q, k, v = rand_qkv(11, 1, 1, 2048, 2048, 128, 128, torch.float16)
    k, v = (k.float() * 3).half(), (v.float() * 3).half()
    o, _ = run_capi(lib, q, k, v, 0.125, False, want_lse=False)
    oref, _ = oracle.attention_fwd(q, k, v, 0.125, False)
    st = oracle.error_stats(o, oref)
    # |v| is 3x larger here; scale the absolute bound with the output's peak
    assert oracle.within(st, "fp16", scale_by_peak=True), st


def test_deterministic_and_linear_in_v(lib):
    """Size-independent properties: two runs are bit-identical; O is linear in V."""
    q, k, v = rand_qkv(13, 1, 2, 1024, 1024, 128, 128, torch.float16)
    o1, _ = run_capi(lib, q, k, v, 0.09, True)
    o2, _ = run_capi(lib, q, k, v, 0.09, True)
    assert torch.equal(o1, o2)
    o3, _ = run_capi(lib, q, k, (v.float() * 2).half(), 0.09, True)
    assert torch.allclose(o3.float(), 2 * o1.float(), atol=2e-3)


def test_config2_full_size_properties(lib):
    """The headline benchmark shape at full size (B=8 H=16 L=4096 d=128, fp16 and bf16, causal and not): two sampled
    (batch, head) slices against the oracle, and softmax rows summing to one (V = ones gives O = 1)."""
    c = oracle.CONFIGS["C2"]
    B, H, L, d = c["B"], c["H"], c["Lq"], c["dqk"]
    scale = d ** -0.5
    for dtype_name in ("fp16", "bf16"):
        dt, code = DT[dtype_name]
        g = torch.Generator(device="cuda").manual_seed(17)
        q = torch.randn(B, H, L, d, device="cuda", generator=g).to(dt)
        k = torch.randn(B, H, L, d, device="cuda", generator=g).to(dt)
        v = torch.randn(B, H, L, d, device="cuda", generator=g).to(dt)
        ones = torch.ones_like(v)
        o = torch.empty_like(q)
        for causal in (False, True):
            _lib.check(lib.attn_b200_fa_fwd(P(q), P(k), P(v), P(o), None, B, H, L, L, d, d, code, scale, int(causal), None))
            torch.cuda.synchronize()
            for (b, h) in ((0, 0), (B - 1, H - 1)):
                oref, _ = oracle.attention_fwd(q[b, h].cpu(), k[b, h].cpu(), v[b, h].cpu(), scale, causal)
                st = oracle.error_stats(o[b, h].cpu(), oref)
                assert oracle.within(st, dtype_name), (dtype_name, causal, st)
            _lib.check(lib.attn_b200_fa_fwd(P(q), P(k), P(ones), P(o), None, B, H, L, L, d, d, code, scale, int(causal), None))
            torch.cuda.synchronize()
            assert (o.float() - 1).abs().max().item() < (4e-3 if dtype_name == "fp16" else 2e-2)
    assert _lib.device_status() == 0


@pytest.mark.parametrize("dtype_name,causal,nbatch", [("fp16", False, 8), ("fp16", True, 8), ("bf16", False, 1), ("bf16", True, 1)])
def test_config2_every_slice_against_the_oracle(lib, dtype_name, causal, nbatch):
    """B=8 H=16 L=4096 d=128 with the per-slice seeded inputs: fp16 checks all 128 (batch, head) slices, bf16 the 16
    heads of the first batch entry, each slice over all rows against the fp32 oracle. Prints the error figures."""
    c = oracle.CONFIGS["C2"]
    B, H, L, d = c["B"], c["H"], c["Lq"], c["dqk"]
    dt, code = DT[dtype_name]
    scale = d ** -0.5
    q, k, v = (torch.empty(B, H, L, d, dtype=dt) for _ in range(3))
    for b in range(B):
        for h in range(H):
            q[b, h], k[b, h], v[b, h] = oracle.slice_inputs("C2", b, h, H, L, L, d, d, dt)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.full((B, H, L, d), float("nan"), device="cuda", dtype=dt)
    _lib.check(lib.attn_b200_fa_fwd(P(qd), P(kd), P(vd), P(o), None, B, H, L, L, d, d, code, scale, int(causal), None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    oc = o.cpu()
    worst = dict(max_abs=0.0, mean_abs=0.0, max_rel_to_peak=0.0, ref_peak=0.0)
    for b in range(nbatch):
        oref, _ = oracle.attention_fwd(q[b], k[b], v[b], scale, causal)     # the 16 heads of one batch entry at once
        for h in range(H):
            st = oracle.error_stats(oc[b, h], oref[h])
            assert oracle.within(st, dtype_name), (b, h, st)
            worst = {key: max(worst[key], st[key]) for key in worst}
    assert oracle.report(f"C2 {dtype_name}{' causal' if causal else ''} worst of {nbatch * H} slices", worst, dtype_name)
    assert not torch.isnan(oc).any()


def test_python_operator_matches_capi(lib):
    from attention_autotuner_b200.ops.attention_interface import flash_attn_func
    q, k, v = rand_qkv(19, 2, 2, 512, 768, 128, 128, torch.float16)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = flash_attn_func(qd, kd, vd, B200())                      # reference defaults: scale 0.125, non-causal
    oc, _ = run_capi(lib, q, k, v, 0.125, False)
    assert torch.equal(o.cpu(), oc)
    o2, lse = flash_attn_func(qd, kd, vd, B200(), True, 0.07, True)
    check(o2.cpu(), lse.cpu(), q, k, v, 0.07, True, "fp16")
    with pytest.raises(ValueError):
        flash_attn_func(qd[..., :96], kd[..., :96], vd, B200())   # key_dim % 64 != 0 (the reference asserts the same)
    with pytest.raises(ValueError, match="batch/heads"):
        flash_attn_func(qd, kd[:, :1], vd[:, :1], B200())          # fewer k/v heads: rejected, not read out of bounds


def test_legacy_kernel_entry_symbol():
    """kernel_entry(q,k,v,o,B,H,Seq_k,Seq_q) and profile(q,k,v,o,B,H,Seq_q,Seq_k) of a per-config library keep
    the reference's argument orders (csrc/kernels/attention/regfuse/profile_code.py:30,68)."""
    from attention_autotuner_b200.autotuner.configs import AttnConfig
    from attention_autotuner_b200.autotuner.runtime import Runtime
    q, k, v = rand_qkv(23, 1, 2, 256, 640, 64, 64, torch.float16)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.zeros(1, 2, 256, 64, device="cuda", dtype=torch.float16)
    rt = Runtime(B200(), AttnConfig(256, 128, 64, 64, q_tiles=2, kv_stages=4))
    rt.apply([qd, kd, vd, o])
    torch.cuda.synchronize()
    oref, _ = oracle.attention_fwd(q, k, v, 0.125, False)
    assert oracle.within(oracle.error_stats(o.cpu(), oref), "fp16")
    so = ctypes.CDLL(rt.lib_path)
    so.profile.restype = ctypes.c_float
    ms = so.profile(P(qd), P(kd), P(vd), P(o), 1, 2, 256, 640)
    assert 0 < ms < 10


@pytest.mark.parametrize("split,emu,mw", [(2, 0, 1), (2, 3, 1), (1, 3, 1), (1, 0, 2), (2, 0, 2)])
@pytest.mark.parametrize("causal", [False, True])
def test_softmax_split_and_exp_emulation_knobs(split, emu, mw, causal):
    """Tuner knobs that change the softmax code path: two warpgroups per query tile (two threads per score row
    exchanging the row maximum), the FMA-pipe exp2 polynomial for part of the exponentials, two MMA warps taking turns."""
    from attention_autotuner_b200.autotuner.configs import AttnConfig
    from attention_autotuner_b200.autotuner.runtime import Runtime
    q, k, v = rand_qkv(29, 1, 3, 700, 900, 128, 128, torch.float16)
    k = (k.float() * torch.linspace(0.5, 2.0, 900)[None, None, :, None]).half()   # growing scores: rescales happen
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.zeros(1, 3, 700, 128, device="cuda", dtype=torch.float16)
    lse = torch.zeros(1, 3, 700, device="cuda")
    rt = Runtime(B200(), AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=4, softmax_split=split, exp_emu=emu, mma_warps=mw))
    rt.apply([qd, kd, vd, o], scale=0.11, causal=causal, extra_ptrs=(lse.data_ptr(),))
    torch.cuda.synchronize()
    assert rt.device_status() == 0
    check(o.cpu(), lse.cpu(), q, k, v, 0.11, causal, "fp16")


@pytest.mark.parametrize("persistent", [0, 1])
@pytest.mark.parametrize("causal", [False, True])
def test_grid_form_knob_of_the_tuner(persistent, causal):
    """`persistent` in a tile configuration forces one form of the grid (the default, -1, lets the launcher choose by
    the length of the work items)."""
    from attention_autotuner_b200.autotuner.configs import AttnConfig
    from attention_autotuner_b200.autotuner.runtime import Runtime
    q, k, v = rand_qkv(31, 2, 3, 700, 900, 128, 128, torch.float16)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.zeros(2, 3, 700, 128, device="cuda", dtype=torch.float16)
    lse = torch.zeros(2, 3, 700, device="cuda")
    rt = Runtime(B200(), AttnConfig(256, 128, 128, 128, q_tiles=2, kv_stages=4, persistent=persistent))
    rt.apply([qd, kd, vd, o], scale=0.11, causal=causal, extra_ptrs=(lse.data_ptr(),))
    torch.cuda.synchronize()
    assert rt.device_status() == 0
    check(o.cpu(), lse.cpu(), q, k, v, 0.11, causal, "fp16")


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("Lq,Lkv", [(512, 512), (640, 384), (200, 328), (1100, 1100)])
def test_cta_pair_configuration(causal, Lq, Lkv, tmp_path):
    """Clusters of two CTAs with cta_group::2 MMAs (512 query rows per pair): ragged lengths leave the second CTA of
    the last pair partly or wholly outside the tensor, causal makes the two CTAs need different block counts."""
    from attention_autotuner_b200.arch import B200
    from attention_autotuner_b200.autotuner.configs import AttnConfig
    from attention_autotuner_b200.autotuner.runtime import Runtime
    g = torch.Generator().manual_seed(Lq + 3 * Lkv + int(causal))
    q = torch.randn(1, 3, Lq, 128, generator=g).half()
    k = torch.randn(1, 3, Lkv, 128, generator=g).half()
    v = torch.randn(1, 3, Lkv, 256, generator=g).half()
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.full((1, 3, Lq, 256), float("nan"), device="cuda", dtype=torch.float16)
    lse = torch.full((1, 3, Lq), float("nan"), device="cuda")
    rt = Runtime(B200(), AttnConfig(256, 128, 128, 256, q_tiles=2, kv_stages=4, dv_chunk=128, cta_pair=1), tmp_dir=str(tmp_path))
    rt.apply([qd, kd, vd, o], scale=0.09, causal=causal, extra_ptrs=(lse.data_ptr(),))
    torch.cuda.synchronize()
    assert rt.device_status() == 0
    oref, lref = oracle.attention_fwd(q, k, v, 0.09, causal)
    ok_rows = torch.isfinite(lref)
    st = oracle.error_stats(o.cpu()[ok_rows], oref[ok_rows])
    assert oracle.within(st, "fp16"), st
    assert (lse.cpu()[ok_rows] - lref[ok_rows]).abs().max().item() < 1e-3
    assert not torch.isnan(o).any()


def test_host_buffer_operator_matches_the_device_operator():
    """flash_attn_host pipelines batch entries through three streams; (batch, head) slices are independent, so the
    result must be bit-identical to one call on the whole batch, for any chunking."""
    from attention_autotuner_b200.arch import B200
    from attention_autotuner_b200.ops.attention_interface import flash_attn_func
    from attention_autotuner_b200.ops.host_interface import flash_attn_host
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(5, 2, 384, 128, generator=g).half().pin_memory() for _ in range(3))
    ref = flash_attn_func(q.cuda(), k.cuda(), v.cuda(), B200(), True, 0.1).cpu()
    for chunks in (None, 2, 1, 7):
        out = flash_attn_host(q, k, v, B200(), True, 0.1, chunks=chunks)
        assert torch.equal(out, ref)          # no device synchronisation here: the call returns complete host results
    # wait=False hands back the event instead; the result is complete once it has been synchronised
    out, done = flash_attn_host(q, k, v, B200(), True, 0.1, wait=False)
    done.synchronize()
    assert torch.equal(out, ref)
    with pytest.raises(ValueError):
        flash_attn_host(q.cuda(), k, v, B200())
