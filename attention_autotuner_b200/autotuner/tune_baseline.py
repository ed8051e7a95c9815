"""Runs the tile search of every operator on the benchmark shapes and writes logs + cache entries.

    python -m attention_autotuner_b200.autotuner.tune_baseline [--log-dir DIR] [--cache-dir DIR] [--quick]

Needs a B200 and nvcc. The logs (reference text format + JSON with TFLOP/s and fraction of peak) and the
cache files it writes are the ones committed under attention_autotuner_b200/{logs,cache}/.
"""
import argparse
import os

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--log-dir", default=None)
    ap.add_argument("--cache-dir", default=None)
    ap.add_argument("--quick", action="store_true", help="small batch (same head dims and sequence lengths)")
    ap.add_argument("--force", action="store_true", help="search even where a cache entry exists, and overwrite it")
    ap.add_argument("--top-k", type=int, default=None, help="prune every search to the cost model's k best candidates")
    args = ap.parse_args()
    if args.cache_dir:
        os.environ["ATTN_B200_CACHE_DIR"] = args.cache_dir
    os.environ["ATTN_B200_AUTOTUNE"] = "1"
    from ..arch import B200
    from .tunner import AttnTunner, RetBwdTunner, RetTunner

    arch = B200()
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)

    def rnd(*shape, dt=torch.float16):
        return torch.randn(*shape, device=dev, generator=g).to(dt)

    # attention: config 2 (d = 128) fp16 / bf16, causal or not; config 1 head dim (d = 64)
    for (B, H, L, d, dt, causal) in ((8, 16, 4096, 128, torch.float16, False), (8, 16, 4096, 128, torch.float16, True),
                                     (8, 16, 4096, 128, torch.bfloat16, False), (8, 16, 4096, 128, torch.bfloat16, True),
                                     (8, 16, 4096, 64, torch.float16, False)):
        if args.quick:
            B = 2
        q, k, v = rnd(B, H, L, d, dt=dt), rnd(B, H, L, d, dt=dt), rnd(B, H, L, d, dt=dt)
        o = torch.empty_like(q)
        cfg = AttnTunner(arch, [q, k, v, o], scale=d ** -0.5, causal=causal).tune(args.log_dir, force=args.force, top_k=args.top_k)
        print("attention", d, dt, causal, "->", repr(cfg), flush=True)
        del q, k, v, o

    # RetNet: config 3 / 4 with the decay mask
    B, H, L, dqk, dv = (2 if args.quick else 8), 8, 2048, 256, 512
    q, k, v, do = rnd(B, H, L, dqk), rnd(B, H, L, dqk), rnd(B, H, L, dv), rnd(B, H, L, dv)
    o, r = torch.empty_like(v), torch.empty(B, H, L, device=dev)
    gam = (1.0 - torch.pow(2.0, -5.0 - torch.arange(H, dtype=torch.float64))).float().to(dev)
    cfg = RetTunner(arch, [q, k, v, None, o, r], scale=dqk ** -0.5, decay=gam).tune(args.log_dir, force=args.force, top_k=args.top_k)
    print("retnet fwd ->", repr(cfg), flush=True)
    from .runtime import Runtime
    Runtime(arch, cfg).apply([q, k, v, None, o, r], scale=dqk ** -0.5, decay=gam)   # a valid r for the backward
    dq, dk, dvo = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    cfg = RetBwdTunner(arch, [q, k, v, None, do, r, dq, dk, dvo, None], scale=dqk ** -0.5, decay=gam).tune(args.log_dir, force=args.force, top_k=args.top_k)
    print("retnet bwd ->", repr(cfg), flush=True)


if __name__ == "__main__":
    main()
