"""CUDA-event micro-benchmark helper in the spirit of linghe/tools/benchmark.py:
warm up, time each call with an event pair on the current stream, trim the tails."""

from __future__ import annotations

import torch


def benchmark_func(fn, *args, n_warmup=10, n_repeat=100, ref_bytes=None, ref_time=None, name="", **kwargs):
    """Returns the trimmed mean time per call in microseconds (linghe/tools/benchmark.py:12)."""
    for _ in range(n_warmup):
        fn(*args, **kwargs)
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    for i in range(n_repeat):
        starts[i].record()
        fn(*args, **kwargs)
        stops[i].record()
    torch.cuda.synchronize()
    times = sorted(s.elapsed_time(e) * 1e3 for s, e in zip(starts, stops))
    k = max(1, n_repeat // 100)
    core = times[k:-k] if n_repeat > 2 * k else times
    us = sum(core) / len(core)
    line = f"{name or getattr(fn, '__name__', 'fn'):<48} {us:9.1f} us"
    if ref_bytes is not None:
        line += f"  {ref_bytes / us / 1e3:8.1f} GB/s"
    if ref_time is not None:
        line += f"  x{ref_time / us:.2f}"
    print(line)
    return us
