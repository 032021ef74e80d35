"""Prometheus text exposition for the serving frontend.

Two sources: per-request facts observed by the HTTP layer (TTFT, inter-token latency,
queue time, token counters, finish reasons) and per-partition scheduler gauges
published once per driver iteration (running / waiting requests, KV usage,
speculative-decoding counters).  Metric names follow vLLM's so existing dashboards work.

Reference parity: docs/subsystems/frontend/prometheus-metrics.md,
pegainfer-frontend/src/engine/metrics.rs:20-94, src/vllm/bridge.rs:486-512,608-625,
pegainfer-sim/tests/frontend_e2e.rs:206-344 (gauge names and labels).
"""
from __future__ import annotations

import threading
from bisect import bisect_left

_TIME_BUCKETS = (0.001, 0.005, 0.01, 0.02, 0.04, 0.06, 0.08, 0.1, 0.25, 0.5, 0.75, 1.0, 2.5, 5.0, 7.5, 10.0, 20.0, 40.0, 80.0)


class _Histogram:
    def __init__(self, buckets=_TIME_BUCKETS):
        self.buckets = buckets
        self.counts = [0] * (len(buckets) + 1)
        self.sum = 0.0
        self.n = 0

    def observe(self, v: float) -> None:
        self.counts[bisect_left(self.buckets, v)] += 1
        self.sum += v
        self.n += 1

    def render(self, name: str, labels: str) -> list:
        out, acc = [], 0
        sep = "," if labels else ""
        for b, c in zip(self.buckets, self.counts):
            acc += c
            out.append(f'{name}_bucket{{{labels}{sep}le="{b}"}} {acc}')
        out.append(f'{name}_bucket{{{labels}{sep}le="+Inf"}} {self.n}')
        out.append(f"{name}_sum{{{labels}}} {self.sum}")
        out.append(f"{name}_count{{{labels}}} {self.n}")
        return out


class ServerMetrics:
    def __init__(self, model_name: str):
        self.model_name = model_name
        self._lock = threading.Lock()
        self.prompt_tokens = 0
        self.generation_tokens = 0
        self.cached_tokens = 0
        self.success = {}  # finish reason -> count
        self.ttft = _Histogram()
        self.itl = _Histogram()
        self.queue = _Histogram()
        self.e2e = _Histogram()
        self._last_spec = {}

    def observe_first_token(self, ttft_s: float, queue_s: float, prompt_tokens: int, cached: int) -> None:
        with self._lock:
            self.ttft.observe(ttft_s)
            self.queue.observe(max(queue_s, 0.0))
            self.prompt_tokens += prompt_tokens
            self.cached_tokens += cached

    def observe_tokens(self, n: int, gap_s: float) -> None:
        with self._lock:
            self.generation_tokens += n
            if gap_s is not None and n > 0:
                for _ in range(n):
                    self.itl.observe(gap_s / n)

    def observe_finish(self, reason: str, e2e_s: float) -> None:
        with self._lock:
            self.success[reason] = self.success.get(reason, 0) + 1
            self.e2e.observe(e2e_s)

    def render(self, engine_metrics: list) -> str:
        """``engine_metrics``: one ``SchedulerMetrics`` per partition."""
        m = f'model_name="{self.model_name}"'
        L = []
        with self._lock:
            for kind, name, help_ in (
                ("gauge", "vllm:num_requests_running", "Requests currently in a model batch."),
                ("gauge", "vllm:num_requests_waiting", "Requests waiting for admission."),
                ("gauge", "vllm:kv_cache_usage_perc", "Fraction of KV blocks in use (1 = full)."),
            ):
                L.append(f"# HELP {name} {help_}")
                L.append(f"# TYPE {name} {kind}")
                for i, em in enumerate(engine_metrics):
                    val = {"vllm:num_requests_running": em.num_running_reqs, "vllm:num_requests_waiting": em.num_waiting_reqs, "vllm:kv_cache_usage_perc": em.kv_usage()}[name]
                    L.append(f'{name}{{engine="{i}",{m}}} {val}')
            for name, attr in (("vllm:prefix_cache_queries", "prefix_query_tokens"), ("vllm:prefix_cache_hits", "prefix_hit_tokens")):
                L.append(f"# TYPE {name} counter")
                for i, em in enumerate(engine_metrics):
                    L.append(f'{name}_total{{engine="{i}",{m}}} {getattr(em, attr)}')
            for name, attr in (
                ("vllm:spec_decode_num_drafts", "num_drafts"),
                ("vllm:spec_decode_num_draft_tokens", "num_draft_tokens"),
                ("vllm:spec_decode_num_accepted_tokens", "num_accepted_tokens"),
            ):
                L.append(f"# TYPE {name} counter")
                for i, em in enumerate(engine_metrics):
                    L.append(f'{name}_total{{engine="{i}",{m}}} {getattr(em.spec_decode, attr)}')
            L.append("# TYPE vllm:prompt_tokens counter")
            L.append(f"vllm:prompt_tokens_total{{{m}}} {self.prompt_tokens}")
            L.append("# TYPE vllm:generation_tokens counter")
            L.append(f"vllm:generation_tokens_total{{{m}}} {self.generation_tokens}")
            L.append("# TYPE vllm:prompt_tokens_cached counter")
            L.append(f"vllm:prompt_tokens_cached_total{{{m}}} {self.cached_tokens}")
            L.append("# TYPE vllm:request_success counter")
            for reason, c in sorted(self.success.items()):
                L.append(f'vllm:request_success_total{{finished_reason="{reason}",{m}}} {c}')
            for name, h in (
                ("vllm:time_to_first_token_seconds", self.ttft),
                ("vllm:inter_token_latency_seconds", self.itl),
                ("vllm:request_queue_time_seconds", self.queue),
                ("vllm:e2e_request_latency_seconds", self.e2e),
            ):
                L.append(f"# TYPE {name} histogram")
                L.extend(h.render(name, m))
        return "\n".join(L) + "\n"
