"""Chunkwise (recurrent-state) RetNet forward on the GPU against the CPU oracle: the position-by-position recurrence
that restates the reference's scan (csrc/kernels/retnet/recurrent/recurrent.h:110-114) for small cases, and the same
function evaluated over all pairs for the larger ones; and against this library's own parallel kernel where the
normaliser r is 1 (tiny scores), where both must agree.

Tolerance: fp16 max-abs <= 2e-3 and mean-abs <= 2e-4 against the fp32 oracle, scaled by max(1, peak |ref|) (the
retention is not normalised, its magnitude grows with the number of keys a row sees); bf16 8x those."""
import ctypes

import pytest
import torch

from attention_autotuner_b200 import _lib
from attention_autotuner_b200.arch import B200
from oracle import oracle

pytestmark = pytest.mark.gpu


def P(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def run_chunk(lib, q, k, v, gam, scale):
    B, H, L, dqk = q.shape
    dv = v.shape[3]
    code = 0 if q.dtype == torch.float16 else 1
    qd, kd, vd, gd = q.cuda(), k.cuda(), v.cuda(), gam.float().cuda()
    o = torch.full((B, H, L, dv), float("nan"), device="cuda", dtype=q.dtype)
    _lib.check(lib.attn_b200_ret_chunk_fwd(P(qd), P(kd), P(vd), P(gd), P(o), B, H, L, dqk, dv, code, scale, None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return o.cpu()


def rand(seed, B, H, L, dqk, dv, dt=torch.float16):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, H, L, dqk, generator=g).to(dt), torch.randn(B, H, L, dqk, generator=g).to(dt),
            torch.randn(B, H, L, dv, generator=g).to(dt))


@pytest.mark.parametrize("dqk,dv", [(128, 128), (256, 128), (128, 64), (256, 512), (256, 192)])
def test_against_the_position_by_position_recurrence(lib, dqk, dv):
    H, L = 3, 320   # two and a half chunks: the state is carried twice, the last chunk is ragged
    q, k, v = rand(dqk + dv, 1, H, L, dqk, dv)
    gam = oracle.decay_gammas(H)
    scale = dqk ** -0.5
    o = run_chunk(lib, q, k, v, gam, scale)
    ref = oracle.retnet_recurrent(q, k, v, gam, scale)
    assert oracle.report(f"chunkwise dqk={dqk} dv={dv} vs recurrence", oracle.error_stats(o, ref), "fp16", scale_by_peak=True)
    ref2 = oracle.retnet_retention(q, k, v, gam, scale)
    assert (ref - ref2).abs().max().item() < 1e-4 * max(1.0, ref2.abs().max().item())


@pytest.mark.parametrize("dqk,dv", [(256, 512), (128, 128)])
def test_many_slices_take_the_wide_tile(lib, dqk, dv):
    """With at least a hundred (slice, 128-column) pairs every CTA owns 128 columns of V (fewer pairs: 64, so that
    more SMs get a CTA); both tiles must give the same function."""
    B, H, L = 4, 32 if dv == 128 else 8, 300
    q, k, v = rand(77, B, H, L, dqk, dv)
    gam = oracle.decay_gammas(H)
    scale = dqk ** -0.5
    o = run_chunk(lib, q, k, v, gam, scale)
    ref = oracle.retnet_retention(q, k, v, gam, scale)
    assert oracle.report(f"chunkwise wide tile dqk={dqk} dv={dv}", oracle.error_stats(o, ref), "fp16", scale_by_peak=True)


@pytest.mark.parametrize("L", [1, 100, 128, 129, 1000, 2048])
def test_lengths(lib, L):
    H = 2
    q, k, v = rand(L, 2, H, L, 128, 128)
    gam = torch.tensor([0.9, 0.99609375], dtype=torch.float64)   # 0.9^127 = 1.5e-6: far below the fp16 normal range
    o = run_chunk(lib, q, k, v, gam, 0.1)
    ref = oracle.retnet_retention(q, k, v, gam, 0.1)
    assert oracle.report(f"chunkwise L={L}", oracle.error_stats(o, ref), "fp16", scale_by_peak=True)


def test_bf16_and_slow_decay(lib):
    """gamma close to one keeps the carried state alive over many chunks."""
    H, L = 2, 1536
    q, k, v = rand(5, 1, H, L, 256, 256, torch.bfloat16)
    gam = torch.tensor([0.999, 1.0], dtype=torch.float64)
    o = run_chunk(lib, q, k, v, gam, 1 / 16)
    ref = oracle.retnet_retention(q, k, v, gam, 1 / 16)
    assert oracle.report("chunkwise bf16 slow decay", oracle.error_stats(o, ref), "bf16", scale_by_peak=True)


def test_agrees_with_the_parallel_kernel_where_r_is_one(lib):
    """With scores small enough that sum_j |S~_ij| < 1 for every row the parallel form's normaliser is r = 1 and
    RetNetAttnFunc computes the same function."""
    from attention_autotuner_b200.ops.retnet_interface import RetNetAttnFunc, retnet_chunkwise
    H, L = 4, 512
    q, k, v = rand(9, 2, H, L, 256, 512)
    gam = oracle.decay_gammas(H)
    scale = 1e-4
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    a = retnet_chunkwise(qd, kd, vd, gam, B200(), scale=scale)
    b = RetNetAttnFunc(qd, kd, vd, None, B200(), True, scale=scale, decay=gam)
    torch.cuda.synchronize()
    ref = oracle.retnet_retention(q, k, v, gam, scale)
    assert oracle.report("chunkwise (operator)", oracle.error_stats(a.cpu(), ref), "fp16", scale_by_peak=True)
    assert oracle.report("parallel kernel, r = 1", oracle.error_stats(b.cpu(), ref), "fp16", scale_by_peak=True)
    with pytest.raises(ValueError):
        retnet_chunkwise(qd[..., :64], kd[..., :64], vd, gam, B200())                 # dqk 64: no state tile
    with pytest.raises(ValueError):
        retnet_chunkwise(qd, kd[:, :, :256], vd[:, :, :256], gam, B200())             # one length for q, k, v


def test_long_sequence_full_slice(lib):
    """L = 16384 (128 chunks), dqk = 256, dv = 512: one slice against the all-pairs evaluation; bit-identical reruns."""
    H, L = 1, 16384
    q, k, v = rand(21, 1, H, L, 256, 512)
    gam = torch.tensor([1.0 - 2.0 ** -7], dtype=torch.float64)
    o1 = run_chunk(lib, q, k, v, gam, 1 / 16)
    o2 = run_chunk(lib, q, k, v, gam, 1 / 16)
    assert torch.equal(o1, o2)
    ref = oracle.retnet_retention(q, k, v, gam, 1 / 16)
    assert oracle.report("chunkwise L=16384", oracle.error_stats(o1, ref), "fp16", scale_by_peak=True)


def run_segments(lib, q, k, v, gam, scale, segments, poison=True):
    """Through the entry point with scratch memory; the scratch starts as NaNs, so a tile read before it is written shows."""
    B, H, L, dqk = q.shape
    dv = v.shape[3]
    code = 0 if q.dtype == torch.float16 else 1
    qd, kd, vd, gd = q.cuda(), k.cuda(), v.cuda(), gam.float().cuda()
    o = torch.full((B, H, L, dv), float("nan"), device="cuda", dtype=q.dtype)
    nbytes = lib.attn_b200_ret_chunk_workspace_bytes(B, H, L, dqk, dv, segments)
    ws = torch.full((max(nbytes, 16) // 4,), float("nan"), device="cuda")
    _lib.check(lib.attn_b200_ret_chunk_fwd_ws(P(qd), P(kd), P(vd), P(gd), P(o), P(ws), nbytes, segments, B, H, L, dqk, dv, code,
                                              scale, None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return o.cpu(), nbytes


@pytest.mark.parametrize("dqk,dv,dt", [(128, 128, torch.float16), (256, 512, torch.float16), (256, 192, torch.bfloat16),
                                        (128, 64, torch.float16)])
def test_segments_run_at_once(lib, dqk, dv, dt):
    """The sequence cut into 2, 3, 4 and 9 segments (nine chunks, the last one ragged; a segment of one chunk included)
    against the oracle, to the tolerance of the walk in order, and close to the walk in order itself; one segment is
    the walk in order bit for bit."""
    H, L = 3, 1100
    q, k, v = rand(dqk + dv + 1, 1, H, L, dqk, dv, dt)
    gam = torch.tensor([0.9, 0.984375, 1.0], dtype=torch.float64)   # fast decay, the usual one, none
    scale = dqk ** -0.5
    name = "fp16" if dt == torch.float16 else "bf16"
    ref = oracle.retnet_retention(q, k, v, gam, scale)
    seq = run_chunk(lib, q, k, v, gam, scale)
    one, nb = run_segments(lib, q, k, v, gam, scale, 1)
    assert nb == 0 and torch.equal(one, seq)
    for segments in (2, 3, 4, 9, 50):
        o, nb = run_segments(lib, q, k, v, gam, scale, segments)
        count = min(segments, 9)
        count = -(-9 // -(-9 // count))
        assert nb == (count - 1) * H * dqk * dv * 4
        assert oracle.report(f"chunkwise {segments} segments dqk={dqk} dv={dv}", oracle.error_stats(o, ref), name, scale_by_peak=True)
        assert oracle.report(f"chunkwise {segments} segments vs in order", oracle.error_stats(o, seq.float()), name, scale_by_peak=True)


def test_segments_chosen_by_the_library(lib):
    """Two slices of 4096 positions: the library asks for scratch and cuts the sequence; with no scratch, or too little
    for two segments, it walks in order; the operator allocates the scratch itself. Reruns are bit-identical."""
    from attention_autotuner_b200.ops.retnet_interface import retnet_chunkwise
    B, H, L, dqk, dv = 1, 2, 4096, 256, 256
    q, k, v = rand(31, B, H, L, dqk, dv)
    gam = torch.tensor([0.96875, 0.998], dtype=torch.float64)
    ref = oracle.retnet_retention(q, k, v, gam, 1 / 16)
    o1, nb = run_segments(lib, q, k, v, gam, 1 / 16, 0)
    assert nb == 7 * B * H * dqk * dv * 4          # 4 tiles of 128 columns, 32 chunks: 8 segments of 4 chunks
    o2, _ = run_segments(lib, q, k, v, gam, 1 / 16, 0)
    assert torch.equal(o1, o2)
    assert oracle.report("chunkwise, library's segments", oracle.error_stats(o1, ref), "fp16", scale_by_peak=True)
    seq = run_chunk(lib, q, k, v, gam, 1 / 16)
    assert not torch.equal(o1, seq)                # another order of rounding: the segments did run
    a = retnet_chunkwise(q.cuda(), k.cuda(), v.cuda(), gam, B200(), scale=1 / 16)
    assert torch.equal(a.cpu(), o1)
    # no scratch, or too little for two segments: the walk in order
    qd, kd, vd, gd = q.cuda(), k.cuda(), v.cuda(), gam.float().cuda()
    for ws, nbytes in ((None, 0), (torch.empty(1024, device="cuda"), 4096)):
        o = torch.empty(B, H, L, dv, device="cuda", dtype=q.dtype)
        _lib.check(lib.attn_b200_ret_chunk_fwd_ws(P(qd), P(kd), P(vd), P(gd), P(o), P(ws), nbytes, 0, B, H, L, dqk, dv, 0, 1 / 16, None))
        torch.cuda.synchronize()
        assert torch.equal(o.cpu(), seq)
    # many slices: no scratch wanted
    assert lib.attn_b200_ret_chunk_workspace_bytes(8, 8, 2048, 256, 512, 0) == 0
    # segments asked for by number and scratch too small: an error, nothing launched
    o = torch.empty(B, H, L, dv, device="cuda", dtype=q.dtype)
    small = torch.empty(1024, device="cuda")
    assert lib.attn_b200_ret_chunk_fwd_ws(P(qd), P(kd), P(vd), P(gd), P(o), P(small), 4096, 4, B, H, L, dqk, dv, 0, 1 / 16, None) == 1
    assert "scratch" in lib.attn_b200_last_error().decode()
    assert lib.attn_b200_ret_chunk_fwd_ws(P(qd), P(kd), P(vd), P(gd), P(o), None, 0, -1, B, H, L, dqk, dv, 0, 1 / 16, None) == 1
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def test_argument_errors(lib):
    x = torch.zeros(1, 1, 128, 128, device="cuda", dtype=torch.float16)
    d = torch.ones(1, device="cuda")
    call = lambda **kw: lib.attn_b200_ret_chunk_fwd(P(x), P(x), P(x), P(kw.get("d", d)), P(x), 1, 1, 128, kw.get("dqk", 128),
                                                    kw.get("dv", 128), kw.get("dtype", 0), kw.get("scale", 1.0), None)
    assert call(dqk=64) == 2
    assert call(dv=96) == 2
    assert call(dtype=5) == 1
    assert call(scale=0.0) == 1
    assert lib.attn_b200_ret_chunk_fwd(P(x), P(x), P(x), None, P(x), 1, 1, 128, 128, 128, 0, 1.0, None) == 1
    assert call() == 0
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
