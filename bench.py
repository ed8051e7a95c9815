#!/usr/bin/env python
"""Headline benchmark: flash-attention forward TFLOPS on B200, with every other target workload in the same line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--no-extras]
    python bench.py --impl reference ...          # the reference's CPU formula on the host cores
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline (`value`): one "step" = one launch of the fused forward kernel over the whole workload batch (B=8 H=16
L=4096 d=128 fp16, non-causal); K steps between one pair of CUDA events on the launching stream, inputs resident in
HBM. With N > 1 every rank owns its own batch of the same shape (weak scaling, no data-path collective); the time is
the max over ranks. `e2e` times the public host-buffer operator with pinned host inputs and a host copy of the
output inside the timed region.

The same JSON line carries, under `workloads`, every other configuration the targets are quoted on (causal, bf16,
RetNet forward and forward+backward with the decay mask and with a mask tensor, attention forward+backward), each
timed the way the reference times kernels (python/benchmarks/do_bench.py: 256 MB L2 flush before every launch, one
event pair per launch, median with p20/p80), once through the bare C-ABI launch and once through the
device-resident Python operator (`op_ms`, which adds the operator's allocation, tuner lookup and FFI cost);
`sustained` legs that run the headline kernel and the RetNet forward+backward back to back for at least two seconds
with the clocks sampled over that window; and the long-sequence bf16 cases (L=16384, B*H = 512 slices) split over
the ranks by (batch, head) slices, total problem fixed (`"scaling": "strong"`), with a checksum of the outputs that
must not depend on the number of ranks. Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ.setdefault("ATTN_B200_AUTOTUNE", "0")  # never search for tile configs inside the benchmark

WORKLOADS = {
    # name: (B, H, Lq, Lkv, dqk, dv, dtype, causal)
    # C3 / C4: RetNet parallel forward / forward+backward with the per-head decay mask (FLOPs count the i >= j pairs)
    "C3": (8, 8, 2048, 2048, 256, 512, "fp16", True),
    "C4": (8, 8, 2048, 2048, 256, 512, "fp16", True),
    # the same decay mask handed over as the reference's [H, Lq, Lkv] mask tensor
    "C3mask": (8, 8, 2048, 2048, 256, 512, "fp16", True),
    "C4mask": (8, 8, 2048, 2048, 256, 512, "fp16", True),
    "C1": (2, 4, 512, 512, 64, 64, "fp16", False),
    "C2": (8, 16, 4096, 4096, 128, 128, "fp16", False),
    "C2causal": (8, 16, 4096, 4096, 128, 128, "fp16", True),
    "C2bf16": (8, 16, 4096, 4096, 128, 128, "bf16", False),
    # flash-attention forward + backward (1 + 3 launches per step; 2 + 5 GEMMs counted)
    "C2bwd": (8, 16, 4096, 4096, 128, 128, "fp16", False),
    "C2bwdcausal": (8, 16, 4096, 4096, 128, 128, "fp16", True),
    "C2bf16causal": (8, 16, 4096, 4096, 128, 128, "bf16", True),
    # reduced batches of the same shapes for profiler captures (inputs still larger than the L2)
    "C2small": (2, 16, 4096, 4096, 128, 128, "fp16", False),
    "C2bwdsmall": (2, 16, 4096, 4096, 128, 128, "fp16", False),
    "C4small": (2, 8, 2048, 2048, 256, 512, "fp16", True),
    # chunkwise (recurrent-state) RetNet forward: the unnormalised retention, cost linear in L
    "R3chunk": (8, 8, 2048, 2048, 256, 512, "fp16", True),
    "R16kchunk": (1, 8, 16384, 16384, 256, 512, "fp16", True),
    # long sequences, bf16, 512 (batch, head) slices split over the ranks
    "C5sq": (16, 32, 16384, 16384, 128, 128, "bf16", False),
    "C5sqcausal": (16, 32, 16384, 16384, 128, 128, "bf16", True),
    "C5dec": (16, 32, 1024, 16384, 128, 128, "bf16", False),
}
METRIC = "attn fwd TFLOPS at B=8,H=16,L=4096,d=128 fp16"
UNIT = "TFLOP/s"
ATTN_BWD = ("C2bwd", "C2bwdcausal", "C2bwdsmall")
RETNET = {"C3": "fwd", "C4": "fwd+bwd", "C3mask": "fwd", "C4mask": "fwd+bwd", "C4small": "fwd+bwd"}
CHUNKWISE = ("R3chunk", "R16kchunk")
STRONG = ("C5sq", "C5sqcausal", "C5dec")
EXTRA_SHORT = ("C4", "C3", "C2causal", "C2bf16", "C2bf16causal", "C3mask", "C4mask", "C2bwd", "R3chunk", "R16kchunk")
SUSTAINED = ("C2", "C4")
SEED = 20240229
# dram__bytes_read.sum + dram__bytes_write.sum per step from the ncu captures summarised under profiles/
# (one file per kernel and workload); None where no capture was taken
NCU_TRAFFIC_BYTES = {"C2": 516.2e6, "C3": 383.6e6, "C4": 1725.3e6}


def metric_name(workload):
    if workload in CHUNKWISE:
        B, H, Lq = WORKLOADS[workload][:3]
        return "RetNet chunkwise fwd TFLOPS at B=%d,H=%d,L=%d,dqk=256,dv=512 fp16 (FLOPs of the chunkwise algorithm)" % (B, H, Lq)
    if workload in RETNET:
        return "RetNet %s TFLOPS at B=%d,H=8,L=2048,dqk=256,dv=512 fp16 (decay mask%s, unmasked pairs counted)" % (
            RETNET[workload], WORKLOADS[workload][0], " as a mask tensor" if workload.endswith("mask") else "")
    if workload == "C2":
        return METRIC
    B, H, Lq, Lkv, dqk, dv, dtype, causal = WORKLOADS[workload]
    if workload in ATTN_BWD:
        return "attn fwd+bwd TFLOPS at B=%d,H=%d,L=%d,d=%d %s%s" % (B, H, Lq, dqk, dtype, " causal" if causal else "")
    return "attn fwd TFLOPS at B=%d,H=%d,Lq=%d,Lkv=%d,d=%d %s%s" % (B, H, Lq, Lkv, dqk, dtype, " causal" if causal else "")


def kernel_of(workload):
    if workload in CHUNKWISE:
        return "ret_chunk_sm100_kernel"
    if workload in RETNET:
        return "chain_pair_sm100_kernel"
    if workload in ATTN_BWD:
        return "fa_bwd_kv_sm100_kernel"
    # the forward runs as the persistent kernel where a CTA's work items are short (csrc/fa_fwd_launch.cuh)
    B, H, Lq, Lkv, dqk, dv, dtype, causal = WORKLOADS[workload]
    nblk = (Lkv + 127) // 128
    return "fa_fwd_persist_sm100_kernel" if ((nblk + 1) // 2 if causal else nblk) <= 40 else "fa_fwd_sm100_kernel"


def flops_fwd(B, H, Lq, Lkv, dqk, dv, causal):
    if causal:
        shift = Lkv - Lq
        pairs = sum(max(0, min(Lkv, i + shift + 1)) for i in range(Lq))
    else:
        pairs = Lq * Lkv
    return 2.0 * B * H * pairs * (dqk + dv)


def flops_of(workload, n_slices=None):
    """Algorithmic FLOPs of one step over `n_slices` (batch, head) slices (default: the whole batch)."""
    B, H, Lq, Lkv, dqk, dv, dtype, causal = WORKLOADS[workload]
    if workload in CHUNKWISE:  # per 128-position chunk: Q K^T, W V, Q S, K^T V
        per_chunk = 2.0 * 128 * 128 * dqk + 2.0 * 128 * 128 * dv + 4.0 * 128 * dqk * dv
        return (B * H if n_slices is None else n_slices) * ((Lq + 127) // 128) * per_chunk
    f = flops_fwd(1, 1, Lq, Lkv, dqk, dv, causal) * (B * H if n_slices is None else n_slices)
    if RETNET.get(workload) == "fwd+bwd":
        f += f / (dqk + dv) * (3 * dqk + 2 * dv)
    if workload in ATTN_BWD:
        f += f / 2 * 5  # S, dP, dV, dQ, dK
    return f


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured", float(d.get("bf16_tflops_sustained", 0.0))
    return 1590.0, 6650.0, "fallback", 1400.0


class ClockSampler:
    """Samples nvidia-smi clocks, power and throttle reasons of one GPU while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
            if len(parts) > 6:
                try:
                    pw.append(float(parts[6]))
                except ValueError:
                    pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons),
                "power_w_median": statistics.median(pw) if pw else None, "power_w_max": max(pw) if pw else None}


def cpu_reference_run(workload, steps, warmup, budget_s=20.0):
    """Times the CPU fp32 formula of the reference (python/utils/ref_op.py:2-6, restated in oracle/) on a
    bounded sample of (batch, head) slices of the workload, with all host threads."""
    from oracle import oracle
    B, H, Lq, Lkv, dqk, dv, dtype, causal = WORKLOADS[workload]
    torch.set_num_threads(os.cpu_count() or 1)
    dt = oracle.torch_dtype(dtype)
    scale = dqk ** -0.5
    ret = RETNET.get(workload)
    masks = oracle.decay_mask(H, Lq, Lkv) if ret else None

    gam = oracle.decay_gammas(H)

    def run_slice(i, sl):
        if workload in CHUNKWISE:  # the same function over all pairs (the reference's recurrent kernel is CUDA only)
            oracle.retnet_retention(sl[0][None, None], sl[1][None, None], sl[2][None, None], gam[i % H: i % H + 1], scale)
        elif workload in ATTN_BWD:
            oracle.attention_bwd_autograd(sl[0], sl[1], sl[2], sl[3], scale, causal)
        elif not ret:
            oracle.attention_fwd(sl[0], sl[1], sl[2], scale, causal)
        elif ret == "fwd":
            oracle.retnet_fwd(sl[0], sl[1], sl[2], masks[i % H], scale)
        else:  # the reference's own way: autograd through the formula with r detached (ref_op.py:8-13)
            oracle.retnet_bwd_autograd(sl[0], sl[1], sl[2], masks[i % H], sl[3], scale)

    first = oracle.slice_inputs(workload, 0, 0, H, Lq, Lkv, dqk, dv, dt, with_do=bool(ret) or workload in ATTN_BWD)
    t0 = time.perf_counter()
    run_slice(0, first)
    per_slice = time.perf_counter() - t0
    n_slices = max(1, min(B * H, int(budget_s / max(per_slice, 1e-6) / max(1, steps + warmup))))
    slices = [oracle.slice_inputs(workload, (i // H) % B, i % H, H, Lq, Lkv, dqk, dv, dt, with_do=bool(ret) or workload in ATTN_BWD)
              for i in range(n_slices)]
    fl = flops_of(workload, n_slices)

    def one_step():
        for i, sl in enumerate(slices):
            run_slice(i, sl)
    for _ in range(warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    dt_s = (time.perf_counter() - t0) / steps
    return {"value": fl / dt_s / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_slices} of {B * H} (batch, head) slices of {workload} per step, fp32, torch CPU",
            "ms_per_step": dt_s * 1e3}


def P(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


class Runner:
    """One workload resident on one GPU: `step()` launches it through the C ABI, `op_step()` through the
    device-resident Python operator. `n_slices` (batch, head) slices starting at global slice `lo`; every slice
    is generated from its own seed, so a shard holds the same numbers whichever rank owns it."""

    def __init__(self, name, dev, lib, stream, lo=0, n_slices=None, per_slice_seed=False, rank=0):
        from attention_autotuner_b200 import _lib
        self.name, self.dev, self.lib, self._lib = name, dev, lib, _lib
        B, H, Lq, Lkv, dqk, dv, dtype, causal = WORKLOADS[name]
        if n_slices is not None:  # a shard of the flattened (batch, head) grid: a batch of n_slices single heads
            B, H = n_slices, 1
        self.shape = (B, H, Lq, Lkv, dqk, dv)
        self.causal = causal
        self.n_slices = B * H
        self.tdt = torch.float16 if dtype == "fp16" else torch.bfloat16
        self.code = _lib.F16 if dtype == "fp16" else _lib.BF16
        self.scale = dqk ** -0.5
        self.sp = ctypes.c_void_p(stream.cuda_stream)
        self.ret = RETNET.get(name)
        self.chunk = name in CHUNKWISE
        self.bwd = name in ATTN_BWD
        g = torch.Generator(device=dev)

        def gen(L, d, salt):
            if not per_slice_seed:
                return torch.randn(B, H, L, d, device=dev, generator=g).to(self.tdt)
            out = torch.empty(B, H, L, d, device=dev, dtype=self.tdt)
            for s in range(B):
                g.manual_seed(SEED + 7919 * (lo + s) + salt)
                out[s, 0] = torch.randn(L, d, device=dev, generator=g).to(self.tdt)
            return out
        g.manual_seed(SEED + rank)
        self.q, self.k, self.v = gen(Lq, dqk, 1), gen(Lkv, dqk, 2), gen(Lkv, dv, 3)
        self.o = torch.empty(B, H, Lq, dv, device=dev, dtype=self.tdt)
        self.launches = 1
        self.mask = self.decay = self.do = None
        if self.chunk:
            self.gam = (1.0 - torch.pow(2.0, -5.0 - torch.arange(H, dtype=torch.float64))).float().to(dev)
            # few slices and a long sequence: scratch for the segment states, so that the sequence is cut into segments
            # that run at once (one more launch: the kernel that computes the segment states)
            self.ws_bytes = int(self.lib.attn_b200_ret_chunk_workspace_bytes(B, H, Lq, dqk, dv, 0))
            self.ws = torch.empty(max(self.ws_bytes, 16), device=dev, dtype=torch.uint8)
            self.launches = 2 if self.ws_bytes else 1
        elif self.ret:
            WH = WORKLOADS[name][1]
            self.gam = (1.0 - torch.pow(2.0, -5.0 - torch.arange(WH, dtype=torch.float64))).float().to(dev)
            self.r = torch.empty(B, H, Lq, device=dev, dtype=torch.float32)
            self.do = gen(Lq, dv, 4)
            self.dq, self.dk, self.dvo = torch.empty_like(self.q), torch.empty_like(self.k), torch.empty_like(self.v)
            self.launches = 1 if self.ret == "fwd" else 4
            self.dq_accum = None
            if name.endswith("mask"):
                # the reference's call form passes a pre-zeroed fp32 dq_accum of this shape; here it is scratch
                self.dq_accum = torch.zeros(B, H, Lq, dqk, device=dev, dtype=torch.float32)
                idx = torch.arange(Lq, device=dev, dtype=torch.float64)
                diff = idx[:, None] - torch.arange(Lkv, device=dev, dtype=torch.float64)[None, :]
                self.mask = torch.where(diff >= 0, self.gam.double()[:, None, None] ** diff.clamp(min=0),
                                        torch.zeros((), device=dev, dtype=torch.float64)).to(self.tdt)
            else:
                self.decay = self.gam
        elif self.bwd:
            self.lse = torch.empty(B, H, Lq, device=dev, dtype=torch.float32)
            self.do = gen(Lq, dv, 4)
            self.dq, self.dk, self.dvo = torch.empty_like(self.q), torch.empty_like(self.k), torch.empty_like(self.v)
            self.launches = 4
        self.flops = flops_of(name, self.n_slices)
        self.input_bytes = sum(t.numel() * t.element_size() for t in (self.q, self.k, self.v, self.o))

    def step(self):
        B, H, Lq, Lkv, dqk, dv = self.shape
        lib, chk = self.lib, self._lib.check
        if self.chunk:
            chk(lib.attn_b200_ret_chunk_fwd_ws(P(self.q), P(self.k), P(self.v), P(self.gam), P(self.o), P(self.ws), self.ws_bytes, 0,
                                               B, H, Lq, dqk, dv, self.code, self.scale, self.sp))
        elif self.ret:
            chk(lib.attn_b200_ret_fwd(P(self.q), P(self.k), P(self.v), P(self.mask), P(self.o), P(self.r), B, H, Lq, Lkv, dqk,
                                      dv, self.code, self.scale, P(self.decay), 1, self.sp))
            if self.ret != "fwd":
                chk(lib.attn_b200_ret_bwd(P(self.q), P(self.k), P(self.v), P(self.mask), P(self.do), P(self.r), P(self.dq),
                                          P(self.dk), P(self.dvo), P(self.dq_accum), B, H, Lq, Lkv, dqk, dv, self.code, self.scale,
                                          P(self.decay), 1, self.sp))
        elif self.bwd:
            chk(lib.attn_b200_fa_fwd(P(self.q), P(self.k), P(self.v), P(self.o), P(self.lse), B, H, Lq, Lkv, dqk, dv, self.code,
                                     self.scale, int(self.causal), self.sp))
            chk(lib.attn_b200_fa_bwd(P(self.q), P(self.k), P(self.v), P(self.o), P(self.do), P(self.lse), P(self.dq), P(self.dk),
                                     P(self.dvo), B, H, Lq, Lkv, dqk, self.code, self.scale, int(self.causal), self.sp))
        else:
            chk(lib.attn_b200_fa_fwd(P(self.q), P(self.k), P(self.v), P(self.o), None, B, H, Lq, Lkv, dqk, dv, self.code,
                                     self.scale, int(self.causal), self.sp))

    def op_step(self):
        """The same work through the public device-resident operators (allocation of the outputs, tuner cache lookup,
        per-config library, ctypes call; autograd for the backward)."""
        from attention_autotuner_b200.arch import B200
        from attention_autotuner_b200.ops.attention_interface import flash_attn_func
        from attention_autotuner_b200.ops.retnet_interface import RetNetAttnFunc
        arch = B200()
        if self.chunk:
            from attention_autotuner_b200.ops.retnet_interface import retnet_chunkwise
            retnet_chunkwise(self.q, self.k, self.v, self.gam, arch, scale=self.scale)
        elif self.ret:
            if self.ret == "fwd":
                with torch.no_grad():
                    RetNetAttnFunc(self.q, self.k, self.v, self.mask, arch, True, scale=self.scale, decay=self.decay)
                return
            q, k, v = (t.detach().requires_grad_(True) for t in (self.q, self.k, self.v))
            RetNetAttnFunc(q, k, v, self.mask, arch, True, scale=self.scale, decay=self.decay).backward(self.do)
        elif self.bwd:
            q, k, v = (t.detach().requires_grad_(True) for t in (self.q, self.k, self.v))
            flash_attn_func(q, k, v, arch, self.causal, self.scale).backward(self.do)
        else:
            with torch.no_grad():
                flash_attn_func(self.q, self.k, self.v, arch, self.causal, self.scale)

    def checksums(self):
        """One integer per slice: the sum of the output's 16-bit patterns. Exact and independent of summation order,
        so equal inputs must give equal checksums whatever rank, batch position or launch computed the slice."""
        B, H, Lq, Lkv, dqk, dv = self.shape
        return self.o.view(torch.int16).reshape(B * H, -1).to(torch.int64).sum(dim=1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="C2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline only: skip the `workloads` dict (other configurations, sustained and strong-scaled legs)")
    ap.add_argument("--sustained-seconds", type=float, default=2.5)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    B, H, Lq, Lkv, dqk, dv, dtype, causal = WORKLOADS[args.workload]
    opname = "RetNet parallel " + RETNET[args.workload] + " (decay mask)" if args.workload in RETNET else (
        "flash-attention forward + backward" if args.workload in ATTN_BWD else
        "RetNet chunkwise forward (per-head decay)" if args.workload in CHUNKWISE else "flash-attention forward")
    config = {"workload": f"{args.workload}: {opname} B={B} H={H} Lq={Lq} Lkv={Lkv} dqk={dqk} dv={dv} "
                          f"{dtype} causal={causal} scale=1/sqrt(dqk), per GPU",
              "slices_per_gpu": B * H, "sharding": "(batch, head) slices, no collective",
              "l2": "inputs (4 tensors, %d MB) exceed the 126 MB L2" % (2 * B * H * (Lq * (dqk + dv) + Lkv * (dqk + dv)) // 2**20)}

    if args.impl == "reference":
        if rank != 0:
            return
        r = cpu_reference_run(args.workload, max(1, args.steps), args.warmup)
        line = {"impl": "reference", "metric": metric_name(args.workload), "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "note": "the reference's CUDA kernels do not build offline (CUTLASS submodule absent); this arm times "
                        "its PyTorch CPU formula restated in oracle/"}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from attention_autotuner_b200 import _lib, sharding
    from attention_autotuner_b200.arch import B200
    from attention_autotuner_b200.utils.timing import L2Flusher, time_launches
    lib = _lib.load()
    stream = torch.cuda.current_stream(dev)
    peak_tf, peak_hbm, peak_src, peak_sus = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(*vals):
        if world == 1:
            return list(vals)
        t = torch.tensor(list(vals), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def check_status(where):
        if _lib.device_status() != 0:
            raise SystemExit(f"device status non-zero after {where}: " + lib.attn_b200_last_error().decode())

    # ------------------------------------------------------------------ headline: K steps between one event pair
    run = Runner(args.workload, dev, lib, stream, rank=rank)
    ret = run.ret
    for _ in range(args.warmup):
        run.step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        run.step()
    e1.record(stream)
    torch.cuda.synchronize()
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    check_status("the headline region")
    launches_per_step = run.launches
    gpu_launches = run.launches * args.steps

    # ------------------------------------------------------------------ end to end through the public operator
    e2e_ms, e2e_steps = None, 0
    can_e2e = not args.no_e2e and not run.bwd and not run.chunk and run.mask is None
    if can_e2e:
        arch = B200()
        qh, kh, vh = (t.cpu().pin_memory() for t in (run.q, run.k, run.v))
        oh = torch.empty(run.o.shape, dtype=run.tdt).pin_memory()
        e2e_steps = max(3, min(args.steps, 10))
        if ret == "fwd+bwd":
            doh = run.do.cpu().pin_memory()
            gh = [torch.empty(t.shape, dtype=run.tdt).pin_memory() for t in (run.q, run.k, run.v)]
        from attention_autotuner_b200.ops.host_interface import flash_attn_host, retnet_host

        def e2e_step():
            # host buffers in, host buffers out: the host-buffer operators pipeline the copies of the batch entries
            # with the kernels (three streams) and return when the results are complete on the host
            if not ret:
                flash_attn_host(qh, kh, vh, arch, run.causal, run.scale, out=oh, device=dev)
            elif ret == "fwd":
                retnet_host(qh, kh, vh, arch, decay=run.gam, causal=True, scale=run.scale, outs=[oh], device=dev)
            else:
                retnet_host(qh, kh, vh, arch, decay=run.gam, causal=True, scale=run.scale, dout=doh, outs=[oh] + gh, device=dev)
        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        f1.record(stream)
        torch.cuda.synchronize()
        barrier()
        e2e_ms = f0.elapsed_time(f1) / e2e_steps
        gpu_launches += run.launches * e2e_steps * B  # one launch set per batch entry
        del qh, kh, vh, oh

    ms_step = ms_total / args.steps
    ms_step, e2e_max = max_over_ranks(ms_step, e2e_ms or 0.0)
    e2e_ms = e2e_max if e2e_ms is not None else None

    # ------------------------------------------------------------------ the other target workloads, same JSON line
    workloads = {}
    extras = (not args.no_extras) and args.workload == "C2"
    if extras:
        flusher = L2Flusher(dev)

        def short_leg(r: Runner, reps=20):
            """Reference timing method: flush, one event pair per launch, median and p20/p80; C ABI and operator."""
            # every leg is a burst timed alone, like the peak it is compared with: the SM clock follows the power drawn over
            # the last tens of milliseconds, so a light kernel timed right after a heavy leg would run at that leg's clock
            # (measured: 0.160 ms against 0.136 ms for the same launch); a short idle gap lets the clock come back
            torch.cuda.synchronize()
            time.sleep(0.15)
            smp = ClockSampler(local_rank)
            if rank == 0:
                smp.start()
            st = time_launches(r.step, reps=reps, warmup=3, flusher=flusher, stream=stream, budget_ms=400.0)
            ck = smp.stop() if rank == 0 else None
            op = time_launches(r.op_step, reps=reps, warmup=2, flusher=flusher, stream=stream, budget_ms=400.0)
            ms, op_ms = max_over_ranks(st["median_ms"], op["median_ms"])
            tf = r.flops / (ms * 1e-3) / 1e12
            return {"metric": metric_name(r.name), "ms_per_step": ms, "p20_ms": st["p20_ms"], "p80_ms": st["p80_ms"],
                    "reps": st["reps"], "tflops_per_gpu": tf, "tflops": tf * world, "frac": tf / peak_tf,
                    "op_ms": op_ms, "op_tflops_per_gpu": r.flops / (op_ms * 1e-3) / 1e12,
                    "launches_per_step": r.launches, "kernel": kernel_of(r.name), "scaling": "weak", "clocks": ck,
                    "timing": "0.15 s idle, 3 warm-up launches, then 256 MB L2 flush before every launch, one CUDA event pair per "
                              "launch, median"}, \
                r.launches * (st["reps"] + op["reps"] + 6)

        def sustained_leg(r: Runner, seconds: float):
            """Back-to-back launches for at least `seconds`, clocks and power sampled over that window only."""
            smp = ClockSampler(local_rank)
            for _ in range(3):
                r.step()
            torch.cuda.synchronize()
            barrier()
            if rank == 0:
                smp.start()
                time.sleep(0.1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n = 0
            t0 = time.perf_counter()
            a.record(stream)
            while True:
                for _ in range(25):
                    r.step()
                n += 25
                chk = torch.cuda.Event()
                chk.record(stream)
                chk.synchronize()
                if time.perf_counter() - t0 >= seconds or n >= 200000:
                    break
            b.record(stream)
            b.synchronize()
            ck = smp.stop() if rank == 0 else None
            ms = a.elapsed_time(b) / n
            (ms,) = max_over_ranks(ms)
            tf = r.flops / (ms * 1e-3) / 1e12
            return {"seconds": a.elapsed_time(b) / 1e3, "steps": n, "ms_per_step": ms, "tflops_per_gpu": tf,
                    "frac_of_sustained": tf / peak_sus if peak_sus else None, "frac_of_burst": tf / peak_tf,
                    "peak_sustained": peak_sus, "clocks": ck}, r.launches * (n + 3)

        # the headline workload with the reference's timing method and through the operator, then its sustained leg
        # Order: every short leg first (each a fraction of a second, the GPU at its boost clock), the long-sequence legs
        # next, the two sustained legs last: a 2.5 s run at the power cap leaves the GPU warm and its clock low for a
        # while, which would otherwise leak into whatever short leg follows it.
        workloads["C2"], nl = short_leg(run)
        gpu_launches += nl
        check_status("C2 leg")
    del run
    torch.cuda.empty_cache()
    if extras:
        for name in EXTRA_SHORT:
            r = Runner(name, dev, lib, stream, rank=rank)
            workloads[name], nl = short_leg(r)
            gpu_launches += nl
            check_status(name)
            del r
            torch.cuda.empty_cache()
        # long sequences: 512 slices split over the ranks, total problem fixed
        for name in STRONG:
            WB, WH = WORKLOADS[name][0], WORKLOADS[name][1]
            lo, hi = sharding.slice_range(rank, world, WB * WH)
            r = Runner(name, dev, lib, stream, lo=lo, n_slices=hi - lo, per_slice_seed=True, rank=rank)
            st = time_launches(r.step, reps=5, warmup=2, flusher=flusher, stream=stream)
            (ms,) = max_over_ranks(st["median_ms"])
            total_flops = flops_of(name)
            torch.cuda.synchronize()
            sums = r.checksums()
            if world > 1:
                sums = sharding.gather_slices(sums.view(-1, 1), WB * WH)
            entry = {"metric": metric_name(name), "ms_per_step": ms, "reps": st["reps"],
                     "tflops": total_flops / (ms * 1e-3) / 1e12, "tflops_per_gpu": total_flops / world / (ms * 1e-3) / 1e12,
                     "frac": total_flops / world / (ms * 1e-3) / 1e12 / peak_tf, "scaling": "strong",
                     "slices_total": WB * WH, "slices_per_gpu": hi - lo, "kernel": kernel_of(name),
                     "bytes_per_tensor_total": WB * WH * WORKLOADS[name][3] * WORKLOADS[name][4] * 2}
            if rank == 0:
                entry["o_checksum"] = hashlib.sha256(sums.cpu().numpy().tobytes()).hexdigest()[:16]
            workloads[name] = entry
            gpu_launches += r.launches * (st["reps"] + 2)
            check_status(name)
            del r
            torch.cuda.empty_cache()
        for name in SUSTAINED:
            r = Runner(name, dev, lib, stream, rank=rank)
            workloads[name]["sustained"], nl = sustained_leg(r, args.sustained_seconds)
            gpu_launches += nl
            check_status(name + " sustained")
            del r
            torch.cuda.empty_cache()
        # validation collectives (outside every timed region): scatter a small tensor from rank 0, regenerate the shard
        # locally from the per-slice seeds and compare; gather it back and compare on rank 0
        if world > 1:
            n_val, L_val, d_val = 4 * world + 1, 64, 128

            def val_slice(s):
                gg = torch.Generator(device=dev).manual_seed(SEED + 31 * s)
                return torch.randn(L_val, d_val, device=dev, generator=gg)
            full = torch.stack([val_slice(s) for s in range(n_val)]) if rank == 0 else None
            shard = sharding.scatter_slices(full, n_val, (L_val, d_val), torch.float32, dev)
            lo, hi = sharding.slice_range(rank, world, n_val)
            local = torch.stack([val_slice(s) for s in range(lo, hi)]) if hi > lo else shard
            same = torch.tensor([1.0 if torch.equal(shard, local) else 0.0], device=dev, dtype=torch.float64)
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            back = sharding.gather_slices(shard, n_val)
            workloads["validation"] = {"scatter_matches_local_regeneration": bool(same.item() == 1.0),
                                       "gather_round_trip": bool(torch.equal(back, full)) if rank == 0 else None,
                                       "slices": n_val, "collectives": "NCCL send/recv (scatter_slices, gather_slices), all_reduce"}

    fl_gpu = flops_of(args.workload)
    if rank == 0:
        achieved = fl_gpu / (ms_step * 1e-3) / 1e12
        line = {
            "metric": metric_name(args.workload), "value": world * achieved, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": config,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": achieved / peak_tf, "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                         "peak_source": f"{peak_src} (cuBLAS bf16 burst; the timed region is a burst of a few tens of ms; "
                                        "for the fraction of the sustained peak see workloads.*.sustained)",
                         "flops_per_step": fl_gpu, "launches_per_step": launches_per_step,
                         "kernel": kernel_of(args.workload)},
            "clocks": clocks,
            "gpu_launches": gpu_launches,
        }
        if e2e_ms is not None:
            es = 2
            nq, nk, nv, no = B * H * Lq * dqk, B * H * Lkv * dqk, B * H * Lkv * dv, B * H * Lq * dv
            h2d = (nq + nk + nv) * es + (no * es if ret == "fwd+bwd" else 0)
            d2h = no * es + ((nq + nk + nv) * es if ret == "fwd+bwd" else 0)
            line["e2e"] = {"value": world * fl_gpu / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
                           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                           "pcie_gbs_per_rank": (h2d + d2h) / (e2e_ms * 1e-3) / 1e9,
                           "api": "attention_autotuner_b200.ops.host_interface." + ("retnet_host" if ret else "flash_attn_host")
                                  + " (per batch entry: " + ("ops.retnet_interface.RetNetAttnFunc" if ret else
                                                             "ops.attention_interface.flash_attn_func")
                                  + "); returns when the results are complete in host memory"}
        if workloads:
            line["workloads"] = workloads
        if not args.no_cpu_baseline and world == 1:
            r = cpu_reference_run(args.workload, 2, 1, budget_s=15.0)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
