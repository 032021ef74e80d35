"""Request phase tracing: queue -> prefill -> decode spans per request.

Off unless ``PEGAINFER_TRACE_FILE`` (JSON lines) or ``PEGAINFER_TRACE_OTLP_ENDPOINT``
is set: with tracing off the scheduler holds no tracer object and builds no spans.
Spans carry the caller's trace parent when the request has one.  Both exporters need
nothing but the standard library: the OTLP exporter posts OTLP/HTTP JSON
(``ExportTraceServiceRequest``) to ``<endpoint>/v1/traces`` from a background thread in
batches, so a slow or absent collector never blocks the scheduler (batches that cannot
be delivered are dropped and counted).

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


class OtlpHttpExporter:
    """Batches spans and posts them as OTLP/HTTP JSON.  ``endpoint``: collector base URL
    (``http://host:4318``) or the full ``.../v1/traces`` URL."""

    def __init__(self, endpoint: str, service_name: str = "pegainfer_b200", flush_interval_s: float = 1.0, max_batch: int = 256):
        import queue

        self.url = endpoint if endpoint.rstrip("/").endswith("/v1/traces") else endpoint.rstrip("/") + "/v1/traces"
        self.service_name = service_name
        self.flush_interval_s = flush_interval_s
        self.max_batch = max_batch
        self._q: "queue.Queue" = queue.Queue(maxsize=8192)
        self.sent = self.dropped = self.posts = 0
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="otlp-exporter", daemon=True)
        self._thread.start()

    def submit(self, span: dict) -> None:
        try:
            self._q.put_nowait(span)
        except Exception:
            self.dropped += 1

    @staticmethod
    def _attr(key, value):
        if isinstance(value, bool):
            return {"key": key, "value": {"boolValue": value}}
        if isinstance(value, int):
            return {"key": key, "value": {"intValue": str(value)}}
        if isinstance(value, float):
            return {"key": key, "value": {"doubleValue": value}}
        return {"key": key, "value": {"stringValue": str(value)}}

    def encode(self, spans: list) -> dict:
        """``ExportTraceServiceRequest`` as JSON: ids are hex strings, times are nanoseconds as strings."""
        out = []
        for sp in spans:
            parent = sp.get("parent") or ""
            parent_span = ""
            if parent.count("-") >= 3:  # W3C traceparent: version-traceid-spanid-flags
                parent_span = parent.split("-")[2]
            out.append({
                "traceId": sp["trace_id"],
                "spanId": uuid.uuid4().hex[:16],
                "parentSpanId": parent_span,
                "name": sp["span"],
                "kind": 1,
                "startTimeUnixNano": str(int(sp["start"] * 1e9)),
                "endTimeUnixNano": str(int(sp["end"] * 1e9)),
                "attributes": [self._attr("request.id", sp["request"]), self._attr("duration_ms", float(sp["duration_ms"]))],
            })
        return {"resourceSpans": [{"resource": {"attributes": [self._attr("service.name", self.service_name)]},
                                   "scopeSpans": [{"scope": {"name": "pegainfer_b200.scheduler"}, "spans": out}]}]}

    def _post(self, spans: list) -> None:
        import urllib.request

        body = json.dumps(self.encode(spans)).encode()
        req = urllib.request.Request(self.url, data=body, headers={"Content-Type": "application/json"}, method="POST")
        try:
            with urllib.request.urlopen(req, timeout=2.0) as resp:
                resp.read()
            self.sent += len(spans)
            self.posts += 1
        except Exception:
            self.dropped += len(spans)

    def _drain(self) -> list:
        import queue

        batch = []
        while len(batch) < self.max_batch:
            try:
                batch.append(self._q.get_nowait())
            except queue.Empty:
                break
        return batch

    def _run(self) -> None:
        while not self._stop.is_set():
            self._stop.wait(self.flush_interval_s)
            while True:
                batch = self._drain()
                if not batch:
                    break
                self._post(batch)

    def flush(self) -> None:
        while True:
            batch = self._drain()
            if not batch:
                return
            self._post(batch)

    def close(self) -> None:
        """Stop the sender, wait for the post it may be in the middle of, then send what is left."""
        self._stop.set()
        if self._thread.is_alive() and threading.current_thread() is not self._thread:
            self._thread.join(timeout=5.0)
        self.flush()


class PhaseTracer:
    def __init__(self, path: Optional[str] = None, exporter: Optional[OtlpHttpExporter] = None):
        self.path = path
        self.exporter = exporter
        self._lock = threading.Lock()
        self._open: dict = {}  # rid -> (phase, t_start, trace_id, parent)
        self.finished: list = []
        self._fh = open(path, "a") if path else None

    def _enter(self, q, phase: str) -> None:
        now = time.time()
        with self._lock:
            prev = self._open.get(q.id)
            parent = getattr(q.request, "trace_parent", None)
            inherited = parent.split("-")[1] if parent and parent.count("-") >= 3 else None  # join the caller's trace
            trace_id = prev[2] if prev else (inherited or uuid.uuid4().hex)
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
        if self.exporter is not None:
            self.exporter.submit(span)


def tracer_from_env() -> Optional[PhaseTracer]:
    path = os.environ.get("PEGAINFER_TRACE_FILE")
    if path:
        return PhaseTracer(path)
    endpoint = os.environ.get("PEGAINFER_TRACE_OTLP_ENDPOINT")
    if endpoint:
        return PhaseTracer(None, OtlpHttpExporter(endpoint, os.environ.get("PEGAINFER_TRACE_SERVICE", "pegainfer_b200")))
    return None
