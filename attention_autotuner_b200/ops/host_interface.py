"""Host-buffer forms of the two operators: inputs and results live in (pinned) host memory.

    o = flash_attn_host(q, k, v, device_type, causal=False, softmax_scale=None, out=None, device=None)
    o, dq, dk, dv = retnet_host(q, k, v, device_type, mask=None, decay=None, causal=False, scale=None,
                                dout=None, outs=None, device=None)      # dout=None: forward only, returns o

The reference has no such entry point: its callers move tensors with ``.cuda()`` / ``.cpu()`` around
``flash_attn_func`` / ``RetNetAttnFunc`` (python/tests/attntuner_demo.py:50-60). For tensors of benchmark size
those copies, not the kernels, are the time: at config 2 the kernel takes 1 ms and the copies over PCIe 10 ms.
Here the [batch, heads] grid is cut into pieces that flow through three streams (host -> device copies, the
operator, device -> host copies), so the two copy directions run at the same time and the kernels disappear
under them; the device holds a few pieces instead of the whole batch. Per piece the launch path of the
public operators runs (same tuner lookup, same kernels and tile configurations), without the autograd wrapper.

(batch, head) slices are independent, which is what makes the chunking exact; results are bit-identical to one
call on the whole batch.
"""
import torch

from .attention_interface import flash_attn_func
from .retnet_interface import retnet_backward, retnet_forward

_STREAMS: dict = {}


def _streams(dev: torch.device):
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    if key not in _STREAMS:
        _STREAMS[key] = tuple(torch.cuda.Stream(device=dev) for _ in range(3))
    return _STREAMS[key]


def _bounds(n: int, parts: int):
    parts = max(1, min(int(parts), n))
    base, extra = divmod(n, parts)
    out, b0 = [], 0
    for i in range(parts):
        b1 = b0 + base + (1 if i < extra else 0)
        out.append((b0, b1))
        b0 = b1
    return out


def _pieces(batch: int, heads: int, chunks):
    """Pieces of the [batch, heads] grid that are contiguous in memory: ranges of batch entries, or ranges of heads
    inside one batch entry. Returns (b0, b1, h0, h1). Default: one piece per batch entry, or the heads of a single
    entry one by one (measured at the benchmark shapes: 8, 16 and 32 pieces finish within 3 % of each other, at the
    rate PCIe sustains in both directions at once; 64 pieces cost launch overhead)."""
    if chunks is None:
        chunks = batch if batch > 1 else heads
    chunks = max(1, int(chunks))
    if chunks <= batch:
        return [(b0, b1, 0, heads) for b0, b1 in _bounds(batch, chunks)]
    per_entry = min(heads, -(-chunks // batch))
    return [(b, b + 1, h0, h1) for b in range(batch) for h0, h1 in _bounds(heads, per_entry)]


def _check_host(*tensors):
    for t in tensors:
        if t is None:
            continue
        if t.device.type != "cpu":
            raise ValueError("host-buffer operators take CPU tensors (pinned memory for asynchronous copies)")
        if not t.is_contiguous():
            raise ValueError("host tensors must be contiguous")


def _device(device):
    if not torch.cuda.is_available():
        raise RuntimeError("a CUDA device is required; there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)


def _host_like(shape, dtype):
    return torch.empty(shape, dtype=dtype).pin_memory()


def _finish(s_out, cur, wait):
    """The results are written by asynchronous device -> host copies on s_out. With wait=True (the default) the
    calling thread blocks until the last of them has landed, so the returned host tensors can be read at once.
    With wait=False the event that marks the last copy is returned instead and the caller must synchronise on
    it (or on the device) before touching the results."""
    done = s_out.record_event()
    cur.wait_stream(s_out)
    if wait:
        done.synchronize()
        return None
    return done


def _check_host_shapes(op, q, k, v):
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError(f"{op}: q, k, v must be 4-d [batch, heads, length, head_dim]")
    if tuple(k.shape[:2]) != tuple(q.shape[:2]) or tuple(v.shape[:2]) != tuple(q.shape[:2]):
        raise ValueError(f"{op}: k / v batch and heads {tuple(k.shape[:2])} / {tuple(v.shape[:2])} differ from q's "
                         f"{tuple(q.shape[:2])}")
    if k.shape[3] != q.shape[3] or v.shape[2] != k.shape[2] or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError(f"{op}: inconsistent shapes or dtypes: q {tuple(q.shape)} {q.dtype}, k {tuple(k.shape)} {k.dtype}, "
                         f"v {tuple(v.shape)} {v.dtype}")


def flash_attn_host(q, k, v, device_type, causal=False, softmax_scale=None, *, out=None, device=None, chunks=None,
                    wait=True):
    """q [B,H,Lq,dqk], k [B,H,Lkv,dqk], v [B,H,Lkv,dv] on the host; returns o [B,H,Lq,dv] on the host (``out`` if
    given). ``softmax_scale=None`` keeps the reference's 0.125. ``chunks``: number of pieces the [batch, heads]
    grid is cut into (default: one per batch entry). The call returns once ``o`` is complete; with ``wait=False``
    it returns ``(o, event)`` without blocking and ``o`` may only be read after ``event.synchronize()``."""
    _check_host_shapes("flash_attn_host", q, k, v)
    _check_host(q, k, v, out)
    dev = _device(device)
    B = q.shape[0]
    if out is None:
        out = _host_like((B, q.shape[1], q.shape[2], v.shape[3]), q.dtype)
    s_in, s_op, s_out = _streams(dev)
    cur = torch.cuda.current_stream(dev)
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    for b0, b1, h0, h1 in _pieces(B, q.shape[1], chunks):
        with torch.cuda.stream(s_in):
            qd, kd, vd = (t[b0:b1, h0:h1].to(dev, non_blocking=True) for t in (q, k, v))
            ev_in = s_in.record_event()
        with torch.cuda.stream(s_op):
            s_op.wait_event(ev_in)
            od = flash_attn_func(qd, kd, vd, device_type, causal, softmax_scale)
            ev_op = s_op.record_event()
            for t in (qd, kd, vd):
                t.record_stream(s_op)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_op)
            out[b0:b1, h0:h1].copy_(od, non_blocking=True)
            od.record_stream(s_out)
    done = _finish(s_out, cur, wait)
    return out if wait else (out, done)


def retnet_host(q, k, v, device_type, *, mask=None, decay=None, causal=False, scale=None, dout=None, outs=None,
                device=None, chunks=None, wait=True):
    """RetNet parallel forward (``dout=None``; returns o) or forward + backward (returns o, dq, dk, dv) on host
    tensors. ``mask`` [H,Lq,Lkv] (host or device; uploaded once) or ``decay`` (H gammas), as RetNetAttnFunc.
    ``outs``: optional host tensors to receive the results, in the order they are returned. The call returns once
    the results are complete; with ``wait=False`` it returns ``(results, event)`` without blocking and the results
    may only be read after ``event.synchronize()``."""
    _check_host_shapes("retnet_host", q, k, v)
    _check_host(q, k, v, dout)
    dev = _device(device)
    B = q.shape[0]
    backward = dout is not None
    if outs is None:
        outs = [_host_like((B, q.shape[1], q.shape[2], v.shape[3]), q.dtype)]
        if backward:
            outs += [_host_like(t.shape, t.dtype) for t in (q, k, v)]
    _check_host(*outs)
    s_in, s_op, s_out = _streams(dev)
    cur = torch.cuda.current_stream(dev)
    for s in (s_in, s_op, s_out):
        s.wait_stream(cur)
    with torch.cuda.stream(s_op):
        maskd = mask.to(dev, non_blocking=True) if mask is not None else None
        decayd = decay.to(device=dev, dtype=torch.float32) if decay is not None else None
    for b0, b1, h0, h1 in _pieces(B, q.shape[1], chunks):
        with torch.cuda.stream(s_in):
            ins = [t[b0:b1, h0:h1].to(dev, non_blocking=True) for t in ((q, k, v, dout) if backward else (q, k, v))]
            ev_in = s_in.record_event()
        with torch.cuda.stream(s_op):
            s_op.wait_event(ev_in)
            qd, kd, vd = ins[:3]
            od, rd, mk, dc = retnet_forward(qd, kd, vd, maskd[h0:h1] if maskd is not None else None, device_type, causal,
                                            scale, decayd[h0:h1] if decayd is not None else None)
            res = [od]
            if backward:
                res += list(retnet_backward(qd, kd, vd, mk, ins[3], rd, device_type, causal, scale, dc))
            ev_op = s_op.record_event()
            for t in ins:
                t.record_stream(s_op)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_op)
            for dst, src in zip(outs, res):
                dst[b0:b1, h0:h1].copy_(src, non_blocking=True)
                src.record_stream(s_out)
    done = _finish(s_out, cur, wait)
    res_host = tuple(outs) if backward else outs[0]
    return res_host if wait else (res_host, done)
