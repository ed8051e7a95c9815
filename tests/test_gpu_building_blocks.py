"""tcgen05 / TMA building blocks in isolation (single-CTA GEMMs and the CTA-pair chain, through the C ABI)
against torch matmul."""
import ctypes

import pytest
import torch

from attention_autotuner_b200 import _lib

pytestmark = pytest.mark.gpu


def P(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("dt,code", [(torch.float16, 0), (torch.bfloat16, 1)])
@pytest.mark.parametrize("N,K", [(128, 64), (128, 128), (128, 256), (256, 128), (64, 128), (32, 64)])
def test_gemm_ss_kmajor(lib, dt, code, N, K):
    g = torch.Generator(device="cuda").manual_seed(N * 1000 + K)
    a = torch.randn(128, K, device="cuda", generator=g).to(dt)
    b = torch.randn(N, K, device="cuda", generator=g).to(dt)
    d = torch.full((128, N), float("nan"), device="cuda")
    _lib.check(lib.attn_b200_selftest_gemm_ss(P(a), P(b), P(d), N, K, code, None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    ref = a.double() @ b.double().t()
    assert (d.double() - ref).abs().max().item() < 1e-3


@pytest.mark.parametrize("dt,code", [(torch.float16, 0), (torch.bfloat16, 1)])
@pytest.mark.parametrize("N", [64, 128, 192, 256])
def test_gemm_ts_mnmajor(lib, dt, code, N):
    g = torch.Generator(device="cuda").manual_seed(N)
    p = torch.randn(128, 128, device="cuda", generator=g).to(dt)
    v = torch.randn(128, N, device="cuda", generator=g).to(dt)
    d = torch.full((128, N), float("nan"), device="cuda")
    _lib.check(lib.attn_b200_selftest_gemm_ts(P(p), P(v), P(d), N, code, None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    ref = p.double() @ v.double()
    assert (d.double() - ref).abs().max().item() < 1e-3


@pytest.mark.parametrize("dt,code", [(torch.float16, 0), (torch.bfloat16, 1)])
@pytest.mark.parametrize("K,N2", [(64, 128), (128, 256), (192, 128), (256, 256)])
def test_cta_pair_chain(lib, dt, code, K, N2):
    """Two CTAs of one cluster with cta_group::2 MMAs: SS GEMM with B split by rows between the CTAs, 16-bit
    round trip through tensor memory, TS GEMM with the MN-major operand split by columns."""
    g = torch.Generator(device="cuda").manual_seed(K * 7 + N2)
    a = (torch.randn(256, K, device="cuda", generator=g) * 0.5).to(dt)
    b = (torch.randn(128, K, device="cuda", generator=g) * 0.5).to(dt)
    t = (torch.randn(128, N2, device="cuda", generator=g) * 0.5).to(dt)
    z = torch.full((256, 128), float("nan"), device="cuda")
    d = torch.full((256, N2), float("nan"), device="cuda")
    _lib.check(lib.attn_b200_selftest_pair(P(a), P(b), P(t), P(z), P(d), K, N2, code, None))
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    zref = a.double() @ b.double().t()
    assert (z.double() - zref).abs().max().item() < 1e-3
    dref = z.to(dt).double() @ t.double()  # the kernel rounds z to 16 bits before the second GEMM
    assert (d.double() - dref).abs().max().item() < 1e-3 * max(1.0, dref.abs().max().item())


def test_rejects_bad_sizes(lib):
    x = torch.zeros(128, 128, device="cuda", dtype=torch.float16)
    d = torch.zeros(128, 128, device="cuda")
    assert lib.attn_b200_selftest_gemm_ss(P(x), P(x), P(d), 100, 64, 0, None) == 1
    assert lib.attn_b200_selftest_gemm_ts(P(x), P(x), P(d), 96, 0, None) == 1
    assert lib.attn_b200_selftest_pair(P(x), P(x), P(x), P(d), P(d), 64, 192, 0, None) == 1
