"""Interpreter settings of a serving process.

The scheduler thread creates a few thousand short-lived objects per step.  With CPython's
default thresholds that means a young-generation collection every few steps and, every few
hundred of those, a full collection that walks every object of the process: model, tensors,
tokenizer tables.  A full collection takes tens of milliseconds, longer than the one decode
step that run-ahead keeps queued on the GPU, so the GPU idles (measured: one 36 ms gap per
~64 decode steps at concurrency 64, 9 % of the throughput).  ``tune_gc`` moves everything
that exists after start-up out of the collector's sight (``gc.freeze``) and raises the
thresholds; garbage that is really cyclic is still collected, just less often.

The reference is a Rust process (jemalloc, no tracing collector: pegainfer-server
src/main.rs); this is the Python counterpart of not having one on the step path.
"""
from __future__ import annotations

import gc

_done = False


def tune_gc(gen0: int = 50_000, gen1: int = 50, gen2: int = 100) -> None:
    """Idempotent.  Call once the model, KV pool and graphs exist."""
    global _done
    gc.collect()
    gc.freeze()
    if not _done:
        gc.set_threshold(gen0, gen1, gen2)
        _done = True
