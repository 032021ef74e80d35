"""Latency statistics and CUDA-event timing loops for kernel and step benchmarks.

Reference parity: pegainfer-bench/src/lib.rs:22-273 (measure_loop, LatencyStats).
"""
from __future__ import annotations

import math
from dataclasses import dataclass


def percentile(sorted_vals, p: float) -> float:
    """Linear interpolation on sorted values (the HTTP bench's definition)."""
    if not sorted_vals:
        return float("nan")
    if len(sorted_vals) == 1:
        return float(sorted_vals[0])
    k = (len(sorted_vals) - 1) * p / 100.0
    lo, hi = math.floor(k), math.ceil(k)
    return float(sorted_vals[lo] + (sorted_vals[hi] - sorted_vals[lo]) * (k - lo))


@dataclass
class LatencyStats:
    mean: float
    stddev: float
    min: float
    p50: float
    p95: float
    p99: float
    max: float
    samples: int

    @staticmethod
    def of(values) -> "LatencyStats":
        v = sorted(float(x) for x in values)
        n = len(v)
        if n == 0:
            nan = float("nan")
            return LatencyStats(nan, nan, nan, nan, nan, nan, nan, 0)
        mean = sum(v) / n
        var = sum((x - mean) ** 2 for x in v) / n
        return LatencyStats(mean, math.sqrt(var), v[0], percentile(v, 50), percentile(v, 95), percentile(v, 99), v[-1], n)


def measure_loop(fn, warmup: int = 3, iters: int = 20) -> LatencyStats:
    """Time ``fn()`` with CUDA events on the current stream (ms per call)."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return LatencyStats.of(times)
