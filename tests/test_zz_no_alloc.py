"""attn_b200_ret_bwd_noalloc: the RetNet backward for callers that cannot allocate device memory and have no workspace
to give (a server whose HBM belongs to its own pool, a plug-in under a host framework's memory budget, a
latency-critical path that must not hit cudaMalloc's synchronisation). Its scratch, the transposed copy of the mask,
lives in an array inside the library image. Checked through the C ABI: two calls in a row (the second on a smaller
problem, so that the array still holds the first call's leftovers) against the ordinary entry point, which must
give the same gradients; no device memory is taken between the calls; a mask beyond the array's 32 MiB is refused
with a message that says so. This file is collected last on purpose: if it fails, every other test has already run."""
import ctypes

import pytest
import torch

from attention_autotuner_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu


def P(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _case(seed, B, H, Lq, Lkv, dqk, dv):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, Lq, dqk, generator=g).half()
    k = torch.randn(B, H, Lkv, dqk, generator=g).half()
    v = torch.randn(B, H, Lkv, dv, generator=g).half()
    do = torch.randn(B, H, Lq, dv, generator=g).half()
    mask = (0.5 * torch.randn(H, Lq, Lkv, generator=g)).half()
    return q, k, v, do, mask


def _forward(lib, q, k, v, mask, scale):
    B, H, Lq, dqk = q.shape
    Lkv, dv = v.shape[2], v.shape[3]
    o = torch.empty(B, H, Lq, dv, device="cuda", dtype=torch.float16)
    r = torch.empty(B, H, Lq, device="cuda")
    _lib.check(lib.attn_b200_ret_fwd(P(q), P(k), P(v), P(mask), P(o), P(r), B, H, Lq, Lkv, dqk, dv, 0, scale, None, 0, None))
    return r


def test_two_calls_in_a_row_match_the_ordinary_entry_point(lib):
    assert lib.attn_b200_ret_bwd_noalloc_max_bytes() == 32 << 20
    scale = 0.2
    for seed, (B, H, Lq, Lkv, dqk, dv) in enumerate([(2, 4, 512, 512, 128, 256), (1, 2, 200, 328, 64, 128)]):
        q, k, v, do, mask = _case(100 + seed, B, H, Lq, Lkv, dqk, dv)
        qd, kd, vd, dod, md = (t.cuda() for t in (q, k, v, do, mask))
        r = _forward(lib, qd, kd, vd, md, scale)
        want = [torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)]
        _lib.check(lib.attn_b200_ret_bwd(P(qd), P(kd), P(vd), P(md), P(dod), P(r), P(want[0]), P(want[1]), P(want[2]), None,
                                         B, H, Lq, Lkv, dqk, dv, 0, scale, None, 0, None))
        got = [torch.full_like(t, float("nan")) for t in want]
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = lib.attn_b200_ret_bwd_noalloc(P(qd), P(kd), P(vd), P(md), P(dod), P(r), P(got[0]), P(got[1]), P(got[2]),
                                           B, H, Lq, Lkv, dqk, dv, 0, scale, None, 0, None)
        assert rc == 0, lib.attn_b200_last_error().decode()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        if seed > 0:   # (the first call on a device may load the kernels' module; from then on nothing may be taken)
            assert free_after == free_before, (free_before, free_after)
        assert _lib.device_status() == 0
        gq, gk, gv = oracle.retnet_bwd(q, k, v, mask.float(), do, scale)
        for name, a, b, ref in zip(("dq", "dk", "dv"), got, want, (gq, gk, gv)):
            # the ordinary entry point (no scratch given) transposes mask columns in registers, this one reads the
            # transposed copy: the same numbers reach the same arithmetic, so the results are identical; the
            # tolerance of the other RetNet tests against the oracle holds as well
            assert torch.equal(a, b), name
            assert oracle.report(f"no-alloc backward call {seed} {name}", oracle.error_stats(a.cpu(), ref), "fp16", scale_by_peak=True)


def test_decay_form_needs_no_scratch_and_large_masks_are_refused(lib):
    B, H, L, dqk, dv = 1, 8, 2048, 64, 64
    z = torch.zeros(B, H, L, dqk, device="cuda", dtype=torch.float16)
    r = torch.ones(B, H, L, device="cuda")
    big_mask = torch.zeros(H, L, L, device="cuda", dtype=torch.float16)      # 64 MiB: twice what the entry point holds
    rc = lib.attn_b200_ret_bwd_noalloc(P(z), P(z), P(z), P(big_mask), P(z), P(r), P(z), P(z), P(z), B, H, L, L, dqk, dv, 0, 1.0,
                                       None, 0, None)
    assert rc == 1
    msg = lib.attn_b200_last_error().decode()
    assert "67108864" in msg and "33554432" in msg and "attn_b200_ret_bwd_ws" in msg, msg
    # per-head decay instead of a mask tensor: no scratch involved, any size goes through
    g = torch.Generator().manual_seed(5)
    q, k, v, do = (torch.randn(1, 2, 384, 64, generator=g).half() for _ in range(4))
    gam = oracle.decay_gammas(2)
    qd, kd, vd, dod, gd = q.cuda(), k.cuda(), v.cuda(), do.cuda(), gam.float().cuda()
    o = torch.empty_like(vd)
    rr = torch.empty(1, 2, 384, device="cuda")
    _lib.check(lib.attn_b200_ret_fwd(P(qd), P(kd), P(vd), None, P(o), P(rr), 1, 2, 384, 384, 64, 64, 0, 0.125, P(gd), 1, None))
    dq, dk, dv_ = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    _lib.check(lib.attn_b200_ret_bwd_noalloc(P(qd), P(kd), P(vd), None, P(dod), P(rr), P(dq), P(dk), P(dv_), 1, 2, 384, 384, 64, 64, 0,
                                             0.125, P(gd), 1, None))
    torch.cuda.synchronize()
    m = oracle.decay_mask(2, 384, 384, gam)
    for a, ref in zip((dq, dk, dv_), oracle.retnet_bwd(q, k, v, m, do, 0.125)):
        assert oracle.within(oracle.error_stats(a.cpu(), ref), "fp16", scale_by_peak=True)
    assert _lib.device_status() == 0
