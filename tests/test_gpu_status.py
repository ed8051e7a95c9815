"""The bounded-wait machinery end to end, without faulting or hanging anything: a one-warp kernel waits on a barrier
that nobody arrives at, with a limit of a millisecond instead of the kernels' second; the wait runs out, the kernel
sets the status words and returns normally. Checked: the status and its tag reach the host, the launchers refuse to
run while the status is set (they read a host-mapped copy of the word, no synchronisation), clearing works, and the
next ordinary launch is correct and leaves the status at zero."""
import ctypes

import pytest
import torch

from attention_autotuner_b200 import _lib
from oracle import oracle

pytestmark = pytest.mark.gpu


def P(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _attention_launch(lib, q, k, v, o):
    B, H, L, d = q.shape
    return lib.attn_b200_fa_fwd(P(q), P(k), P(v), P(o), None, B, H, L, L, d, d, 0, d ** -0.5, 0, None)


@pytest.mark.parametrize("whole_warp", [1, 0])
def test_wait_that_runs_out_is_reported_and_recoverable(lib, whole_warp):
    g = torch.Generator().manual_seed(31)
    q, k, v = (torch.randn(1, 2, 256, 64, generator=g).half() for _ in range(3))
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.zeros_like(qd)
    assert _lib.device_status() == 0
    # a first ordinary launch sets up the host-mapped copy of the status word on this device
    assert _attention_launch(lib, qd, kd, vd, o) == 0
    torch.cuda.synchronize()

    assert lib.attn_b200_selftest_wait(1000, whole_warp, None) == 0      # 1 ms limit; the launch itself succeeds
    torch.cuda.synchronize()
    # the launchers notice without any synchronisation of their own and do not launch
    o.zero_()
    rc = _attention_launch(lib, qd, kd, vd, o)
    assert rc == 4, rc                                                    # ATTN_B200_ERR_DEVICE
    msg = lib.attn_b200_last_error().decode()
    assert "bounded wait" in msg and "tag 99" in msg, msg
    torch.cuda.synchronize()
    assert (o == 0).all()                                                 # nothing ran
    with pytest.raises(_lib.AttnB200Error):
        _lib.check(rc)
    # reading without clearing keeps it, the text names the tag; reading with clear resets it
    assert lib.attn_b200_device_status(0) == 1
    assert "tag 99" in lib.attn_b200_last_error().decode()
    assert lib.attn_b200_device_status(1) == 1
    assert lib.attn_b200_device_status(0) == 0
    # the next ordinary launch runs, is correct, and leaves the status at zero
    assert _attention_launch(lib, qd, kd, vd, o) == 0
    torch.cuda.synchronize()
    oref, _ = oracle.attention_fwd(q, k, v, 64 ** -0.5, False)
    assert oracle.report("attention after a cleared timeout", oracle.error_stats(o.cpu(), oref), "fp16")
    assert lib.attn_b200_device_status(0) == 0


def test_selftest_wait_rejects_limits_that_could_stall():
    lib = _lib.load()
    assert lib.attn_b200_selftest_wait(0, 1, None) == 1
    assert lib.attn_b200_selftest_wait(10_000_000, 1, None) == 1
