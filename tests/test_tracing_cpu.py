"""Tracing aids on CPU: OTLP/HTTP export against a local collector stand-in, request phase
spans through the scheduler, and the kernel-call trace / per-model kernel report."""
import json
import threading
import time
from http.server import BaseHTTPRequestHandler, HTTPServer

import torch

from pegainfer_b200.config import EngineConfig, preset
from pegainfer_b200.engine.build import build_engine
from pegainfer_b200.engine.contract import Request, SamplingParams
from pegainfer_b200.ops.call_trace import model_report, trace_calls
from pegainfer_b200.utils.tracing import OtlpHttpExporter, PhaseTracer


class _Collector(BaseHTTPRequestHandler):
    received = []

    def do_POST(self):
        body = self.rfile.read(int(self.headers.get("Content-Length", "0")))
        _Collector.received.append((self.path, self.headers.get("Content-Type"), json.loads(body)))
        self.send_response(200)
        self.end_headers()
        self.wfile.write(b"{}")

    def log_message(self, *a):
        pass


def test_otlp_http_export_of_request_phase_spans():
    _Collector.received.clear()
    srv = HTTPServer(("127.0.0.1", 0), _Collector)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        exp = OtlpHttpExporter(f"http://127.0.0.1:{srv.server_port}", service_name="unit", flush_interval_s=0.05)
        tracer = PhaseTracer(None, exp)
        eng = build_engine(EngineConfig(preset="tiny-qwen3", kv_page_size=16, num_kv_blocks=64, cuda_graph=False), preset("tiny-qwen3"), device="cpu", dtype=torch.float32, start=False)
        eng.scheduler.tracer = tracer
        eng.start()
        try:
            tp = "00-0af7651916cd43dd8448eb211c80319c-b7ad6b7169203331-01"
            req = Request(prompt_tokens=list(range(20)), params=SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=4)
            req.trace_parent = tp
            toks, term, _ = eng.submit(req).collect(60)
            assert term.kind == "finished" and len(toks) == 4
        finally:
            eng.shutdown()
        exp.close()
        assert exp.sent >= 2 and exp.dropped == 0
        path, ctype, body = _Collector.received[0]
        assert path == "/v1/traces" and ctype == "application/json"
        rs = body["resourceSpans"][0]
        assert {"key": "service.name", "value": {"stringValue": "unit"}} in rs["resource"]["attributes"]
        spans = [s for _, _, b in _Collector.received for s in b["resourceSpans"][0]["scopeSpans"][0]["spans"]]
        names = [s["name"] for s in spans]
        assert "prefill" in names and "decode" in names
        for s in spans:
            assert s["traceId"] == "0af7651916cd43dd8448eb211c80319c" and s["parentSpanId"] == "b7ad6b7169203331"  # joined the caller's trace
            assert len(s["spanId"]) == 16 and int(s["endTimeUnixNano"]) >= int(s["startTimeUnixNano"])
    finally:
        srv.shutdown()


def test_exporter_drops_instead_of_blocking_when_no_collector_listens():
    exp = OtlpHttpExporter("http://127.0.0.1:9", flush_interval_s=0.05)  # port 9: nothing listens
    t0 = time.monotonic()
    for i in range(10):
        exp.submit({"request": i, "span": "decode", "start": 1.0, "end": 2.0, "duration_ms": 1000.0, "trace_id": "ab" * 16, "parent": None})
    assert time.monotonic() - t0 < 0.5  # submit never waits for the network
    exp.close()
    assert exp.sent == 0 and exp.dropped == 10


def test_kernel_call_trace_and_model_report_on_cpu():
    from pegainfer_b200.ops import reference as R

    x = torch.randn(6, 64)
    w = torch.ones(64)
    with trace_calls(R) as tr:
        R.rms_norm(x, w, 1e-6)
        R.rms_norm(x, w, 1e-6)
        R.swiglu(torch.randn(6, 128))
    assert R.rms_norm.__name__ == "rms_norm"  # unwrapped again
    rows = tr.rollup()
    by_op = {r[0]: r for r in rows}
    assert by_op["rms_norm"][2] == 2 and by_op["swiglu"][2] == 1 and "float32[6, 64]" in by_op["rms_norm"][1][0]
    rep = model_report("tiny-qwen3", batch=2, context=24, device="cpu")
    assert "prefill 2 x 24" in rep and "decode step, batch 2" in rep and "paged_attention" in rep and "linear" in rep
