#!/usr/bin/env python
"""Headline benchmark: flash-attention forward TFLOPS on B200 (and the CPU reference beside it).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C2|C2causal|C2bf16|C2bwd|C1|C3|C4|C5sq|C5dec]
    python bench.py --impl reference ...          # the reference's CPU formula on the host cores
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" = one launch of the fused forward kernel over the whole workload batch. `value` times K
steps on the device with CUDA events, inputs resident in HBM; `e2e` times the public Python operator
with host (pinned) inputs and a host copy of the output inside the timed region. With N > 1 every rank
owns its own (batch, head) slices of the same shape (weak scaling, no data-path collective); the time is
the max over ranks. Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
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
    # the same decay mask handed over as the reference's [H, Lq, Lkv] mask tensor (device timing only)
    "C3mask": (8, 8, 2048, 2048, 256, 512, "fp16", True),
    "C4mask": (8, 8, 2048, 2048, 256, 512, "fp16", True),
    "C1": (2, 4, 512, 512, 64, 64, "fp16", False),
    "C2": (8, 16, 4096, 4096, 128, 128, "fp16", False),
    "C2causal": (8, 16, 4096, 4096, 128, 128, "fp16", True),
    "C2bf16": (8, 16, 4096, 4096, 128, 128, "bf16", False),
    # flash-attention forward + backward (device timing only: 1 + 3 launches per step; 2 + 5 GEMMs counted)
    "C2bwd": (8, 16, 4096, 4096, 128, 128, "fp16", False),
    "C2bwdcausal": (8, 16, 4096, 4096, 128, 128, "fp16", True),
    "C2bf16causal": (8, 16, 4096, 4096, 128, 128, "bf16", True),
    "C5sq": (16, 32, 16384, 16384, 128, 128, "bf16", False),
    "C5sqcausal": (16, 32, 16384, 16384, 128, 128, "bf16", True),
    "C5dec": (16, 32, 1024, 16384, 128, 128, "bf16", False),
}
METRIC = "attn fwd TFLOPS at B=8,H=16,L=4096,d=128 fp16"
UNIT = "TFLOP/s"
ATTN_BWD = ("C2bwd", "C2bwdcausal")
RETNET = {"C3": "fwd", "C4": "fwd+bwd", "C3mask": "fwd", "C4mask": "fwd+bwd"}
# dram__bytes_read.sum + dram__bytes_write.sum per step from the ncu captures summarised under profiles/
# (fa_fwd_sm100_kernel_C2_fp16.md, chain_pair_sm100_kernel_C4_retnet_fp16.md); None where no capture was taken
NCU_TRAFFIC_BYTES = {"C2": 515.2e6, "C3": 383.6e6, "C4": 1725.3e6}


def metric_name(workload):
    if workload in RETNET:
        return "RetNet %s TFLOPS at B=8,H=8,L=2048,dqk=256,dv=512 fp16 (decay mask%s, unmasked pairs counted)" % (
            RETNET[workload], " as a mask tensor" if workload.endswith("mask") else "")
    if workload == "C2":
        return METRIC
    B, H, Lq, Lkv, dqk, dv, dtype, causal = WORKLOADS[workload]
    if workload in ATTN_BWD:
        return "attn fwd+bwd TFLOPS at B=%d,H=%d,L=%d,d=%d %s%s" % (B, H, Lq, dqk, dtype, " causal" if causal else "")
    return "attn fwd TFLOPS at B=%d,H=%d,Lq=%d,Lkv=%d,d=%d %s%s" % (B, H, Lq, Lkv, dqk, dtype, " causal" if causal else "")


def flops_of(workload):
    B, H, Lq, Lkv, dqk, dv, dtype, causal = WORKLOADS[workload]
    f = flops_fwd(B, H, Lq, Lkv, dqk, dv, causal)
    if RETNET.get(workload) == "fwd+bwd":
        f += f / (dqk + dv) * (3 * dqk + 2 * dv)
    if workload in ATTN_BWD:
        f += f / 2 * 5  # S, dP, dV, dQ, dK
    return f


def flops_fwd(B, H, Lq, Lkv, dqk, dv, causal):
    if causal:
        shift = Lkv - Lq
        pairs = sum(max(0, min(Lkv, i + shift + 1)) for i in range(Lq))
    else:
        pairs = Lq * Lkv
    return 2.0 * B * H * pairs * (dqk + dv)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured", float(d.get("bf16_tflops_sustained", 0.0))
    return 1590.0, 6650.0, "fallback", 1400.0


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

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
        sm, mx, reasons = [], [], set()
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
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


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

    def run_slice(i, sl):
        if workload in ATTN_BWD:
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
    fl = flops_of(workload) * n_slices / (B * H)

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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="C2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    B, H, Lq, Lkv, dqk, dv, dtype, causal = WORKLOADS[args.workload]
    opname = "RetNet parallel " + RETNET[args.workload] + " (decay mask)" if args.workload in RETNET else (
        "flash-attention forward + backward" if args.workload in ATTN_BWD else "flash-attention forward")
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
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from attention_autotuner_b200 import _lib
    from attention_autotuner_b200.arch import B200
    from attention_autotuner_b200.ops.attention_interface import flash_attn_func
    lib = _lib.load()
    tdt = torch.float16 if dtype == "fp16" else torch.bfloat16
    code = _lib.F16 if dtype == "fp16" else _lib.BF16
    scale = dqk ** -0.5

    g = torch.Generator(device=dev).manual_seed(20240229 + rank)
    q = torch.randn(B, H, Lq, dqk, device=dev, generator=g).to(tdt)
    k = torch.randn(B, H, Lkv, dqk, device=dev, generator=g).to(tdt)
    v = torch.randn(B, H, Lkv, dv, device=dev, generator=g).to(tdt)
    o = torch.empty(B, H, Lq, dv, device=dev, dtype=tdt)
    stream = torch.cuda.current_stream(dev)
    P = lambda t: ctypes.c_void_p(t.data_ptr() if t is not None else 0)
    ret = RETNET.get(args.workload)
    launches_per_step = 1
    if ret:
        from attention_autotuner_b200.ops.retnet_interface import RetNetAttnFunc
        gam = (1.0 - torch.pow(2.0, -5.0 - torch.arange(H, dtype=torch.float64))).float().to(dev)
        r = torch.empty(B, H, Lq, device=dev, dtype=torch.float32)
        do = torch.randn(B, H, Lq, dv, device=dev, generator=g).to(tdt)
        dq, dk, dvo = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        launches_per_step = 1 if ret == "fwd" else 4
        sp = ctypes.c_void_p(stream.cuda_stream)

        maskd = None
        if args.workload.endswith("mask"):
            idx = torch.arange(Lq, device=dev, dtype=torch.float64)
            diff = idx[:, None] - torch.arange(Lkv, device=dev, dtype=torch.float64)[None, :]
            maskd = torch.where(diff >= 0, gam.double()[:, None, None] ** diff.clamp(min=0), torch.zeros((), device=dev,
                                                                                                  dtype=torch.float64)).to(tdt)
            args.no_e2e = True
        dec = None if maskd is not None else gam

        def step():
            _lib.check(lib.attn_b200_ret_fwd(P(q), P(k), P(v), P(maskd), P(o), P(r), B, H, Lq, Lkv, dqk, dv, code, scale,
                                             P(dec), 1, sp))
            if ret != "fwd":
                _lib.check(lib.attn_b200_ret_bwd(P(q), P(k), P(v), P(maskd), P(do), P(r), P(dq), P(dk), P(dvo), None, B, H,
                                                 Lq, Lkv, dqk, dv, code, scale, P(dec), 1, sp))
    elif args.workload in ATTN_BWD:
        lse = torch.empty(B, H, Lq, device=dev, dtype=torch.float32)
        do = torch.randn(B, H, Lq, dv, device=dev, generator=g).to(tdt)
        dq, dk, dvo = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        launches_per_step = 4
        sp = ctypes.c_void_p(stream.cuda_stream)
        args.no_e2e = True

        def step():
            _lib.check(lib.attn_b200_fa_fwd(P(q), P(k), P(v), P(o), P(lse), B, H, Lq, Lkv, dqk, dv, code, scale, int(causal), sp))
            _lib.check(lib.attn_b200_fa_bwd(P(q), P(k), P(v), P(o), P(do), P(lse), P(dq), P(dk), P(dvo), B, H, Lq, Lkv, dqk,
                                            code, scale, int(causal), sp))
    else:
        def step():
            _lib.check(lib.attn_b200_fa_fwd(P(q), P(k), P(v), P(o), None, B, H, Lq, Lkv, dqk, dv, code, scale,
                                            int(causal), ctypes.c_void_p(stream.cuda_stream)))

    def barrier():
        if world > 1:
            dist.barrier()

    for _ in range(args.warmup):
        step()
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
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    if _lib.device_status() != 0:
        raise SystemExit("device status non-zero: " + lib.attn_b200_last_error().decode())

    # ---- end to end through the public operator, host buffers in, host result out
    e2e = None
    if not args.no_e2e:
        arch = B200()
        qh, kh, vh = (t.cpu().pin_memory() for t in (q, k, v))
        oh = torch.empty(o.shape, dtype=tdt).pin_memory()
        e2e_steps = max(3, min(args.steps, 10))

        if ret == "fwd+bwd":
            doh = do.cpu().pin_memory()
            gh = [torch.empty(t.shape, dtype=tdt).pin_memory() for t in (q, k, v)]

        from attention_autotuner_b200.ops.host_interface import flash_attn_host, retnet_host

        def e2e_step():
            # host buffers in, host buffers out: the package's host-buffer operators pipeline the copies of the
            # batch entries with the kernels (three streams); every byte of the step crosses PCIe inside the region
            if not ret:
                flash_attn_host(qh, kh, vh, arch, causal, scale, out=oh, device=dev)
            elif ret == "fwd":
                retnet_host(qh, kh, vh, arch, decay=gam, causal=True, scale=scale, outs=[oh], device=dev)
            else:
                retnet_host(qh, kh, vh, arch, decay=gam, causal=True, scale=scale, dout=doh, outs=[oh] + gh, device=dev)
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
    else:
        e2e_ms, e2e_steps = None, 0

    ms_step = ms_total / args.steps
    if world > 1:
        t = torch.tensor([ms_step, e2e_ms or 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, e2e_ms = t[0].item(), (t[1].item() if e2e_ms is not None else None)

    fl_gpu = flops_of(args.workload)
    if rank == 0:
        peak_tf, peak_hbm, peak_src, peak_sus = measured_peaks()
        achieved = fl_gpu / (ms_step * 1e-3) / 1e12
        line = {
            "metric": metric_name(args.workload), "value": world * achieved, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": config,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": achieved / peak_tf, "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                         "peak_source": f"{peak_src} (cuBLAS bf16 burst; the timed region is a burst of a few tens of ms)",
                         "peak_sustained": peak_sus, "frac_of_sustained": (achieved / peak_sus if peak_sus else None),
                         "flops_per_step": fl_gpu, "launches_per_step": launches_per_step,
                         "kernel": ("chain_pair_sm100_kernel" if ret else
                                    "fa_bwd_sm100_kernel" if args.workload in ATTN_BWD else "fa_fwd_sm100_kernel")},
            "clocks": clocks,
            # launches inside the two timed regions; the end-to-end leg launches once per batch entry (the host-buffer
            # operators cut the batch into B pieces)
            "gpu_launches": launches_per_step * (args.steps + (e2e_steps * B if e2e_ms is not None else 0)),
        }
        if e2e_ms is not None:
            es = q.element_size()
            h2d = (q.numel() + k.numel() + v.numel()) * es + (o.numel() * es if ret == "fwd+bwd" else 0)
            d2h = o.numel() * es + ((q.numel() + k.numel() + v.numel()) * es if ret == "fwd+bwd" else 0)
            line["e2e"] = {"value": world * fl_gpu / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
                           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                           "api": "attention_autotuner_b200.ops.host_interface." + ("retnet_host" if ret else "flash_attn_host")
                                  + " (per batch entry: " + ("ops.retnet_interface.RetNetAttnFunc" if ret else
                                                             "ops.attention_interface.flash_attn_func") + ")"}
        if not args.no_cpu_baseline and world == 1:
            r = cpu_reference_run(args.workload, 2, 1, budget_s=15.0)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
