"""Generates tests/golden/*.npz by running the REFERENCE's own formulas (python/utils/ref_op.py of
smallscientist1/attention_autotuner, imported unmodified) on seeded inputs, on CPU in fp32.

    python tests/golden/make_golden.py /path/to/attention_autotuner

The reference checkout is only needed to (re)generate the fixtures; the tests read the .npz files.
Inputs are stored in fp16 exactly as a kernel would receive them; outputs are the reference formulas
evaluated on those inputs upcast to fp32. Gradients come from torch.autograd through retnet_ref (which
detaches r, ref_op.py:11).
"""
import os
import sys

import numpy as np
import torch

if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py /path/to/attention_autotuner (a checkout of the reference project)")
ref_root = sys.argv[1]
sys.path.insert(0, os.path.join(ref_root, "python"))
from utils.ref_op import attention_ref, retnet_ref  # noqa: E402  (the reference's module)

out_dir = os.path.dirname(os.path.abspath(__file__))


def attn_case(name, seed, B, H, Lq, Lkv, dqk, dv, kscale=1.0, vscale=1.0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, Lq, dqk, generator=g).half()
    k = (kscale * torch.randn(B, H, Lkv, dqk, generator=g)).half()
    v = (vscale * torch.randn(B, H, Lkv, dv, generator=g)).half()
    o = attention_ref(q.float(), k.float(), v.float())
    np.savez_compressed(os.path.join(out_dir, name + ".npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(),
                        o=o.numpy())


def attn_bwd_case(name, seed, B, H, Lq, Lkv, d):
    """Gradients of the reference's attention formula by torch.autograd (the reference's own backward is empty,
    python/ops/attention_interface.py:38-39)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, Lq, d, generator=g).half()
    k = torch.randn(B, H, Lkv, d, generator=g).half()
    v = torch.randn(B, H, Lkv, d, generator=g).half()
    do = torch.randn(B, H, Lq, d, generator=g).half()
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    o = attention_ref(qf, kf, vf)
    o.backward(do.float())
    np.savez_compressed(os.path.join(out_dir, name + ".npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(), do=do.numpy(),
                        o=o.detach().numpy(), dq=qf.grad.numpy(), dk=kf.grad.numpy(), dv=vf.grad.numpy())


def ret_case(name, seed, B, H, Lq, Lkv, dqk, dv, qscale=1.0, kscale=1.0, vscale=1.0, mscale=1.0, decay=False):
    g = torch.Generator().manual_seed(seed)
    q = (qscale * torch.randn(B, H, Lq, dqk, generator=g)).half()
    k = (kscale * torch.randn(B, H, Lkv, dqk, generator=g)).half()
    v = (vscale * torch.randn(B, H, Lkv, dv, generator=g)).half()
    if decay:
        gam = 1.0 - torch.pow(2.0, -5.0 - torch.arange(H, dtype=torch.float64))
        i = torch.arange(Lq, dtype=torch.float64)[:, None]
        j = torch.arange(Lkv, dtype=torch.float64)[None, :]
        m = torch.where(i >= j, torch.pow(gam[:, None, None], (i - j).clamp(min=0)[None]), torch.zeros(1, dtype=torch.float64))
        mask = m.half()
    else:
        mask = (mscale * torch.randn(H, Lq, Lkv, generator=g)).half()
    do = torch.randn(B, H, Lq, dv, generator=g).half()
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    o = retnet_ref(qf, kf, vf, mask.float())
    o.backward(do.float())
    np.savez_compressed(os.path.join(out_dir, name + ".npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(),
                        mask=mask.numpy(), do=do.numpy(), o=o.detach().numpy(), dq=qf.grad.numpy(),
                        dk=kf.grad.numpy(), dv=vf.grad.numpy())


if __name__ == "__main__":
    torch.set_num_threads(os.cpu_count() or 1)
    # attention: the reference's fixed 0.125 scale
    attn_case("attn_d64", 11, 1, 2, 256, 256, 64, 64)
    attn_case("attn_d128_ragged", 12, 1, 2, 200, 333, 128, 128)
    attn_case("attn_d256_128_demo_scaling", 13, 1, 1, 256, 256, 256, 128, kscale=3.0, vscale=3.0)
    attn_bwd_case("attn_bwd_d128_ragged", 14, 1, 2, 200, 333, 128)
    attn_bwd_case("attn_bwd_d64", 15, 1, 2, 256, 256, 64)
    # retnet: general randn mask (as python/tests/test_runtime.py:103), demo scalings
    # (python/tests/attntuner_demo.py:45-48), and the decay mask of the benchmark configs
    ret_case("ret_randmask", 21, 1, 2, 256, 256, 64, 64)
    ret_case("ret_demo_scaling", 22, 1, 2, 256, 256, 128, 128, kscale=3.0, vscale=3.0, mscale=0.5)
    ret_case("ret_decay", 23, 1, 4, 384, 384, 64, 128, qscale=0.125, decay=True)
    print("wrote", sorted(f for f in os.listdir(out_dir) if f.endswith(".npz")))
