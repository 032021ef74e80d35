"""Kernel-call trace: which ops a forward pass issues, on which shapes, how often, how long.

``trace_calls()`` wraps the public functions of the active op implementation
(``ops.cuda`` on a GPU, ``ops.reference`` on CPU) for the duration of a ``with`` block and
records one ``KernelCall`` per invocation: op name, the shapes / dtypes of its tensor
arguments, the number of kernel launches it made (GPU) and its duration (CUDA events on
a GPU, wall clock on CPU).  ``rollup`` groups calls by (op, shapes) and ``report`` renders
the per-model kernel table that the reference produces with its kernel-report binaries.

    python -m pegainfer_b200.ops.call_trace --preset qwen3-0.6b --batch 8 --context 256

Reference parity: pegainfer-core/src/ops/call_trace.rs:1-126 (KernelCall records),
pegainfer-bench/src/lib.rs:22-273 (rollups, latency statistics),
pegainfer-qwen3/src/bin/qwen3_kernel_report.rs (per-model report).
"""
from __future__ import annotations

import contextlib
import inspect
import time
from dataclasses import dataclass, field
from typing import List, Optional

import torch


@dataclass
class KernelCall:
    op: str
    shapes: tuple
    launches: int = 0
    ms: float = 0.0
    _events: Optional[tuple] = field(default=None, repr=False)


def _describe(a):
    if isinstance(a, torch.Tensor):
        return f"{str(a.dtype).replace('torch.', '')}{list(a.shape)}"
    if hasattr(a, "xw") and hasattr(a, "ssp"):  # rows whose RMSNorm scale is still owed
        return f"deferred{list(a.xw.shape)}"
    if isinstance(a, (list, tuple)) and a and all(isinstance(x, tuple) and x and isinstance(x[0], torch.Tensor) for x in a):
        return "phases[" + ", ".join(f"{list(x[0].shape)}:{x[1]}" for x in a) + "]"
    return None


class CallTrace:
    def __init__(self):
        self.calls: List[KernelCall] = []

    def finalize(self) -> None:
        if any(c._events for c in self.calls):
            torch.cuda.synchronize()
        for c in self.calls:
            if c._events is not None:
                c.ms = c._events[0].elapsed_time(c._events[1])
                c._events = None

    def rollup(self) -> list:
        """[(op, shapes, count, launches, total_ms, mean_ms)] sorted by total time."""
        self.finalize()
        groups: dict = {}
        for c in self.calls:
            g = groups.setdefault((c.op, c.shapes), [0, 0, 0.0])
            g[0] += 1
            g[1] += c.launches
            g[2] += c.ms
        rows = [(op, shapes, n, launches, ms, ms / n) for (op, shapes), (n, launches, ms) in groups.items()]
        return sorted(rows, key=lambda r: -r[4])

    def report(self, title: str = "kernel calls") -> str:
        rows = self.rollup()
        total = sum(r[4] for r in rows) or 1.0
        lines = [f"# {title}: {len(self.calls)} calls, {sum(r[3] for r in rows)} launches, {total:.3f} ms in ops", f"{'op':24s} {'calls':>6s} {'launch':>7s} {'total ms':>9s} {'mean us':>9s} {'share':>6s}  shapes"]
        for op, shapes, n, launches, ms, mean in rows:
            lines.append(f"{op:24s} {n:6d} {launches:7d} {ms:9.3f} {mean * 1e3:9.1f} {100 * ms / total:5.1f}%  {' '.join(s for s in shapes if s)}")
        return "\n".join(lines)


@contextlib.contextmanager
def trace_calls(module=None):
    """Record every call into the op implementation ``module`` (default: ``ops.cuda`` when a GPU is
    present and the library loads, else ``ops.reference``) made inside the block."""
    if module is None:
        if torch.cuda.is_available():
            from . import cuda as module
        else:
            from . import reference as module
    trace = CallTrace()
    gpu = module.__name__.endswith(".cuda") and torch.cuda.is_available()
    saved = {}
    skip = {"ctx", "lib", "launch_count", "read_status", "clear_status", "gemm_plan", "fused_plan_ok", "plan_decode_splits", "set_batch_invariant", "batch_invariant", "prefetch_weights", "quant_code", "paired_int4",
            "rope_tables"}
    for name, fn in list(vars(module).items()):
        if name.startswith("_") or name in skip or not inspect.isfunction(fn) or fn.__module__ != module.__name__:
            continue

        def make(name, fn):
            def wrapped(*args, **kwargs):
                shapes = tuple(d for d in (_describe(a) for a in list(args) + list(kwargs.values())) if d)
                call = KernelCall(name, shapes)
                before = module.launch_count() if gpu else 0
                if gpu:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    out = fn(*args, **kwargs)
                    e1.record()
                    call._events = (e0, e1)
                    call.launches = module.launch_count() - before
                else:
                    t0 = time.perf_counter()
                    out = fn(*args, **kwargs)
                    call.ms = (time.perf_counter() - t0) * 1e3
                trace.calls.append(call)
                return out

            return wrapped

        saved[name] = fn
        setattr(module, name, make(name, fn))
    try:
        yield trace
    finally:
        for name, fn in saved.items():
            setattr(module, name, fn)
        trace.finalize()


def model_report(preset_name: str, batch: int = 8, context: int = 256, device: Optional[str] = None, kernels: bool = False, **overrides) -> str:
    """Kernel table of one prefill step (``batch`` prompts of ``context`` tokens) and one decode step; with ``kernels`` also
    the GPU kernels of each step by name (CUPTI activity records, ``utils.range_profiler``)."""
    from ..config import EngineConfig, preset
    from ..engine.build import build_engine
    from ..kv.request_kv import KvView
    from ..sched.executor import SeqStep, build_meta

    device = device or ("cuda:0" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if device.startswith("cuda") else torch.float32
    mcfg = preset(preset_name, **overrides)
    page = 16
    per = (context + 1 + page - 1) // page
    ecfg = EngineConfig(preset=preset_name, num_kv_blocks=batch * per + 8, kv_page_size=page, cuda_graph=False, max_decode_batch=max(batch, 8), max_model_len=context + 2 * page)
    eng = build_engine(ecfg, mcfg, device=device, dtype=dtype, start=False)
    try:
        g = torch.Generator().manual_seed(0)
        pages = [list(range(1 + i * per, 1 + (i + 1) * per)) for i in range(batch)]
        prompts = [torch.randint(0, mcfg.vocab_size, (context,), generator=g).tolist() for _ in range(batch)]
        prefill = [SeqStep(rid=i, input_tokens=p, start_pos=0, view=KvView(pages[i][: (context + page - 1) // page], context, page)) for i, p in enumerate(prompts)]
        decode = [SeqStep(rid=i, input_tokens=[1 + i], start_pos=context, view=KvView(pages[i], context + 1, page)) for i in range(batch)]
        out = []
        for title, seqs in ((f"{preset_name}: prefill {batch} x {context}", prefill), (f"{preset_name}: decode step, batch {batch}, context {context}", decode)):
            tok, meta = build_meta(seqs, page, device)
            eng.executor.prepare_meta(seqs, meta)
            eng.model.forward(tok, meta, eng.kv)  # warm-up: module loads, workspace allocation
            with trace_calls() as tr:
                eng.model.forward(tok, meta, eng.kv)
            out.append(tr.report(title))
            if kernels:
                from ..utils.range_profiler import RangeProfiler

                with RangeProfiler(title + " (GPU kernels by name)") as rp:
                    eng.model.forward(tok, meta, eng.kv)
                out.append(rp.report())
        return "\n\n".join(out)
    finally:
        eng.shutdown()


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="per-model kernel report: ops, shapes, launches and time of a prefill and a decode step")
    ap.add_argument("--preset", default="qwen3-0.6b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=256)
    ap.add_argument("--layers", type=int, default=0, help="truncate the model (0 = as configured)")
    ap.add_argument("--kernels", action="store_true", help="also list the GPU kernels of each step by name (range profiler)")
    a = ap.parse_args(argv)
    kw = {"num_layers": a.layers} if a.layers else {}
    print(model_report(a.preset, a.batch, a.context, kernels=a.kernels, **kw))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
