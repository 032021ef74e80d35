"""CPU-only simulated engine on the step contract.

``SimScheduler`` answers requests without a model: time to first token is
``base_ttft + prompt_tokens / prefill_tok_s``, then one token every ``tpot`` seconds,
tokens taken from a script (cycled) or echoing the prompt.  It exercises the whole
frontend (HTTP, streaming, metrics, abort) in CI with no GPU, and can inject a fatal
step or per-request failures.

Reference parity: pegainfer-sim/src/lib.rs:24-403, src/main.rs:12-65,
pegainfer-frontend/examples/echo-server.rs, engine/driver.rs:119-130 (EchoScheduler
with fatal_next_step).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional

from ..engine.contract import EngineInfo, FinishReason, KvCapacity, QueuedRequest, RejectReason, SchedulerMetrics
from ..engine.driver import Engine


@dataclass
class SimConfig:
    base_ttft_s: float = 0.0
    prefill_tok_s: float = 1e9
    tpot_s: float = 0.0
    script: Optional[list] = None  # token ids to emit (cycled); None = echo the prompt
    max_running: int = 256
    kv_blocks: int = 1024
    block_size: int = 16
    max_model_len: int = 8192
    eos_token_ids: tuple = ()
    known_loras: tuple = ()


class _Sim:
    __slots__ = ("q", "next_at", "emitted", "scheduled")

    def __init__(self, q, next_at):
        self.q = q
        self.next_at = next_at
        self.emitted = 0
        self.scheduled = False


class SimScheduler:
    def __init__(self, cfg: SimConfig = None):
        self.cfg = cfg or SimConfig()
        self.waiting: list = []
        self.running: dict = {}
        self.fatal_next_step = False
        self.fail_request_ids: set = set()

    def submit(self, q: QueuedRequest) -> None:
        self.waiting.append(q)

    def metrics(self) -> SchedulerMetrics:
        used = sum((len(s.q.request.prompt_tokens) + s.emitted + self.cfg.block_size - 1) // self.cfg.block_size for s in self.running.values())
        return SchedulerMetrics(kv_used_blocks=min(used, self.cfg.kv_blocks), kv_total_blocks=self.cfg.kv_blocks, num_running_reqs=len(self.running), num_waiting_reqs=len(self.waiting))

    def _token(self, s: _Sim) -> int:
        script = self.cfg.script
        if script:
            return script[s.emitted % len(script)]
        p = s.q.request.prompt_tokens
        return p[s.emitted % len(p)]

    def step(self, ledger) -> bool:
        if self.fatal_next_step:
            self.fatal_next_step = False
            raise RuntimeError("injected fatal step")
        now = time.monotonic()
        busy = False
        while self.waiting and len(self.running) < self.cfg.max_running:
            q = self.waiting.pop(0)
            req = q.request
            if not req.prompt_tokens:
                ledger.reject(q.id, RejectReason.EMPTY_PROMPT, "prompt has no tokens")
                continue
            if len(req.prompt_tokens) >= self.cfg.max_model_len:
                ledger.reject(q.id, RejectReason.PROMPT_TOO_LONG, "prompt exceeds the context window")
                continue
            if req.lora_adapter is not None and req.lora_adapter not in self.cfg.known_loras:
                ledger.reject(q.id, RejectReason.UNKNOWN_LORA, f"LoRA adapter {req.lora_adapter!r} is not loaded")
                continue
            ttft = self.cfg.base_ttft_s + len(req.prompt_tokens) / self.cfg.prefill_tok_s
            self.running[q.id] = _Sim(q, now + ttft)
            ledger.mark_scheduled(q.id, len(req.prompt_tokens))
            ledger.report_cached_tokens(q.id, 0)
            busy = True
        for rid in list(self.running):
            s = self.running[rid]
            if s.q.is_aborted():
                ledger.finish(rid, FinishReason.ABORT)
                del self.running[rid]
                busy = True
                continue
            if rid in self.fail_request_ids:
                ledger.fail(rid, "injected request failure")
                del self.running[rid]
                continue
            if now < s.next_at:
                continue
            busy = True
            tok = self._token(s)
            req = s.q.request
            stop = tok in req.params.stop_token_ids or (not req.params.ignore_eos and tok in self.cfg.eos_token_ids)
            if stop:
                ledger.finish(rid, FinishReason.STOP)
                del self.running[rid]
                continue
            ledger.push_tokens(rid, [tok])
            s.emitted += 1
            s.next_at = now + self.cfg.tpot_s
            if s.emitted >= req.max_tokens:
                ledger.finish(rid, FinishReason.LENGTH)
                del self.running[rid]
        return busy or bool(self.running)


def make_sim_engine(cfg: SimConfig = None, partitions: int = 1, model_name: str = "sim") -> Engine:
    cfg = cfg or SimConfig()
    scheds = [SimScheduler(cfg) for _ in range(partitions)]
    info = EngineInfo(model_name=model_name, max_model_len=cfg.max_model_len, kv_capacity=KvCapacity(cfg.kv_blocks, cfg.block_size), dp_size=partitions, eos_token_ids=cfg.eos_token_ids)
    eng = Engine(scheds, info)
    eng.sim_schedulers = scheds
    return eng
