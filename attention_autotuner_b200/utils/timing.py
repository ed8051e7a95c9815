"""Per-launch device timing with a cold L2, the method of the reference's python/benchmarks/do_bench.py:1-74:
before every timed call a buffer larger than the L2 is overwritten, every call gets its own pair of CUDA events,
and the median is reported with the 20th / 80th percentiles. Differences: the repeat count is given (or derived
from a time budget) instead of estimated from five probe runs, events are recorded on the stream the caller
launches on, and the result carries every statistic at once.
"""
from __future__ import annotations

import statistics

import torch

FLUSH_BYTES = 256 * 1000 * 1000  # twice the 126 MB L2 of a B200; the reference flushes the same 256 MB


class L2Flusher:
    """Owns the flush buffer of one device; ``flusher()`` rewrites it on the current stream."""

    def __init__(self, device, nbytes: int = FLUSH_BYTES):
        self.buf = torch.empty(nbytes // 4, dtype=torch.int32, device=device)

    def __call__(self):
        self.buf.zero_()


def percentile(sorted_vals, q: float) -> float:
    """Linear-interpolated percentile (q in [0, 1]) of an ascending list."""
    if not sorted_vals:
        raise ValueError("no samples")
    pos = q * (len(sorted_vals) - 1)
    lo = int(pos)
    hi = min(lo + 1, len(sorted_vals) - 1)
    return sorted_vals[lo] + (sorted_vals[hi] - sorted_vals[lo]) * (pos - lo)


def summarize(times_ms) -> dict:
    s = sorted(float(t) for t in times_ms)
    return {"median_ms": statistics.median(s), "p20_ms": percentile(s, 0.2), "p80_ms": percentile(s, 0.8),
            "min_ms": s[0], "mean_ms": sum(s) / len(s), "reps": len(s)}


def time_launches(fn, *, reps: int = 20, warmup: int = 3, flusher: L2Flusher | None = None, stream=None,
                  budget_ms: float | None = None) -> dict:
    """Times ``fn()`` ``reps`` times, one event pair per call, the L2 flushed before each timed call.
    With ``budget_ms`` the repeat count is cut so that the timed calls take about that long (at least 3)."""
    stream = stream if stream is not None else torch.cuda.current_stream()
    for _ in range(max(1, warmup)):
        fn()
    if budget_ms is not None:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        fn()
        b.record(stream)
        b.synchronize()
        reps = max(3, min(reps, int(budget_ms / max(a.elapsed_time(b), 1e-3))))
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
    for i in range(reps):
        if flusher is not None:
            flusher()
        starts[i].record(stream)
        fn()
        stops[i].record(stream)
    stops[-1].synchronize()
    torch.cuda.synchronize()
    return summarize(a.elapsed_time(b) for a, b in zip(starts, stops))
