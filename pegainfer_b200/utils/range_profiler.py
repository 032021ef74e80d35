"""Range profiler: the GPU kernels of one user range, by name, from CUPTI activity records.

``RangeProfiler`` wraps a block of host code.  While the block runs, CUPTI's activity API (through the
Kineto tracer that ships inside PyTorch) records every kernel launch with its device-side start and end;
afterwards ``kernels()`` gives one row per kernel name (launches, total / mean / min / max microseconds,
grid and block of the last launch) and ``sol()`` turns the algorithmic bytes or FLOPs of the range into
achieved GB/s and TFLOP/s against given peaks.  No hardware counters are collected and nothing is
replayed, so the range runs once, at its own speed, and the clocks are left alone.  A kernel launched with programmatic
dependent launch starts while its predecessor still runs and waits inside: its record covers that wait, so per-kernel times
of such chains overlap and add up to more than the span (the span itself is exact).

On a machine without a GPU (or when the tracer cannot start) the range still runs; ``kernels()`` is then
empty and ``available`` is False.

    with RangeProfiler("decode step") as rp:
        engine_step()
    print(rp.report())

Reference parity: pegainfer-cupti/csrc/range_profiler.cpp + src/lib.rs:90-145 (profile one user range and
return metric values for the kernel reports).  The reference's wrapper drives CUPTI's counter-based range
profiler; the per-kernel durations here come from CUPTI's activity records, and the counter-based
figures of this repository are the ncu summaries under ``profiles/``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch


@dataclass
class KernelRow:
    name: str
    launches: int = 0
    total_us: float = 0.0
    min_us: float = float("inf")
    max_us: float = 0.0
    grid: tuple = ()
    block: tuple = ()

    @property
    def mean_us(self) -> float:
        return self.total_us / self.launches if self.launches else 0.0


class RangeProfiler:
    def __init__(self, name: str = "range", device: Optional[str] = None):
        self.name = name
        self.device = device
        self.available = False
        self.wall_ms = 0.0
        self._prof = None
        self._rows: Dict[str, KernelRow] = {}
        self._span_us = 0.0

    def __enter__(self) -> "RangeProfiler":
        if torch.cuda.is_available():
            try:
                from torch.profiler import ProfilerActivity, profile

                torch.cuda.synchronize(self.device)
                self._prof = profile(activities=[ProfilerActivity.CUDA], record_shapes=False, with_stack=False)
                self._prof.__enter__()
                self.available = True
            except Exception:  # the tracer is optional: the range itself must still run
                self._prof = None
                self.available = False
        import time

        self._t0 = time.perf_counter()
        return self

    def __exit__(self, et, ev, tb) -> bool:
        import time

        if torch.cuda.is_available():
            torch.cuda.synchronize(self.device)
        self.wall_ms = (time.perf_counter() - self._t0) * 1e3
        if self._prof is not None:
            try:
                self._prof.__exit__(et, ev, tb)
                self._collect()
            except Exception:
                self.available = False
        return False

    def _collect(self) -> None:
        first, last = None, None
        for ev in self._prof.events():
            # device-side records only: kernels (memcpy / memset records carry their own names)
            if getattr(ev, "device_type", None) is None or "cuda" not in str(ev.device_type).lower():
                continue
            dur = float(getattr(ev, "device_time", 0.0) or getattr(ev, "cuda_time", 0.0) or 0.0)
            if dur <= 0.0 and hasattr(ev, "time_range"):
                dur = float(ev.time_range.end - ev.time_range.start)
            row = self._rows.setdefault(ev.name, KernelRow(ev.name))
            row.launches += 1
            row.total_us += dur
            row.min_us = min(row.min_us, dur)
            row.max_us = max(row.max_us, dur)
            if hasattr(ev, "time_range"):
                first = ev.time_range.start if first is None else min(first, ev.time_range.start)
                last = ev.time_range.end if last is None else max(last, ev.time_range.end)
        if first is not None:
            self._span_us = float(last - first)

    def kernels(self) -> List[KernelRow]:
        """One row per kernel name, longest total first."""
        return sorted(self._rows.values(), key=lambda r: -r.total_us)

    @property
    def device_us(self) -> float:
        """Sum of the kernels' device time (kernels that overlap on several streams count twice)."""
        return sum(r.total_us for r in self._rows.values())

    @property
    def span_us(self) -> float:
        """First kernel start to last kernel end on the device."""
        return self._span_us

    def sol(self, bytes_moved: float = 0.0, flops: float = 0.0, peak_gbs: float = 0.0, peak_tflops: float = 0.0) -> dict:
        """Achieved rates of the range from its algorithmic bytes / FLOPs over the device span, and the
        fractions of the given peaks (pass the measured copy bandwidth and GEMM throughput)."""
        t = self.span_us * 1e-6
        out = {"span_us": self.span_us, "kernel_us": self.device_us}
        if t > 0 and bytes_moved:
            out["gbs"] = bytes_moved / t / 1e9
            if peak_gbs:
                out["frac_of_copy_peak"] = out["gbs"] / peak_gbs
        if t > 0 and flops:
            out["tflops"] = flops / t / 1e12
            if peak_tflops:
                out["frac_of_gemm_peak"] = out["tflops"] / peak_tflops
        return out

    def report(self, top: int = 30) -> str:
        if not self.available:
            return f"# {self.name}: kernel tracer not available on this machine (host wall time {self.wall_ms:.3f} ms)"
        rows = self.kernels()
        total = self.device_us or 1.0
        lines = [f"# {self.name}: {sum(r.launches for r in rows)} launches of {len(rows)} kernels, {self.device_us:.1f} us in kernels, {self.span_us:.1f} us first start to last end",
                 f"{'kernel':<72} {'launches':>8} {'total us':>10} {'mean us':>9} {'min':>8} {'max':>8} {'share':>6}"]
        for r in rows[:top]:
            lines.append(f"{r.name[:72]:<72} {r.launches:>8} {r.total_us:>10.1f} {r.mean_us:>9.2f} {r.min_us:>8.2f} {r.max_us:>8.2f} {100 * r.total_us / total:>5.1f}%")
        return "\n".join(lines)
