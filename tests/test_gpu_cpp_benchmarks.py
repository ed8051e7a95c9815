"""The standalone C++ micro-benchmarks (benchmarks/attention.cu, benchmarks/retnet.cu; the counterpart of the
reference's benchmarks/attention.cu and benchmarks/retnet/*.cu) build, run on small shapes, print the reference's
"Time: <ms>ms" line per configuration, and the attention program's own host check passes."""
import re
import subprocess

import pytest

from attention_autotuner_b200.build import build_benchmarks

pytestmark = pytest.mark.gpu


def _run(exe, *args):
    res = subprocess.run([exe, *args], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    return res.stdout


def test_attention_program():
    attn, _ = build_benchmarks()
    out = _run(attn, "--B", "1", "--H", "4", "--Seq_q", "1024", "--Seq_k", "1024", "--check")
    assert out.count("Time: ") == 5 and "FAILED" not in out
    assert re.search(r"check: max abs error .* \(ok\)", out), out
    for ms in re.findall(r"median ([0-9.]+) ms", out):
        assert 0 < float(ms) < 5
    out = _run(attn, "--B", "1", "--H", "2", "--Seq_q", "512", "--Seq_k", "768", "--d", "64", "--bf16", "--check")
    assert out.count("Time: ") == 2 and "(ok)" in out
    out = _run(attn, "--B", "1", "--H", "2", "--Seq_q", "1024", "--Seq_k", "1024", "--causal")
    assert "attention fwd causal" in out and "FAILED" not in out


def test_retnet_program():
    _, ret = build_benchmarks()
    for extra in ((), ("--bwd",), ("--mask", "--bwd")):
        out = _run(ret, "--B", "1", "--H", "2", "--Seq_q", "512", "--Seq_k", "512", *extra)
        assert out.count("Time: ") == 2 and "FAILED" not in out, out
        assert "cta_pair" in out and "single CTA" in out
