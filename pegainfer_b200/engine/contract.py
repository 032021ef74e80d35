"""Step-batched contract between a model scheduler and a frontend.

One scheduler step yields one :class:`StepOutputs`; each request appears in it at
most once, as a flat :class:`RequestUpdate` (admission facts, then new tokens, then
the terminal).  A request's lifetime ends with exactly one :class:`Terminal`.

Reference parity: pegainfer-frontend/src/engine/step.rs:22-247 (Request,
StepOutputs, RequestUpdate, Terminal, RejectReason), engine/event.rs:17-52
(FinishReason, TokenLogprob), sampler.rs:2-39 (SamplingParams),
parallel.rs:6-50 (ParallelConfig).
"""
from __future__ import annotations

import enum
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Optional, Protocol


@dataclass
class SamplingParams:
    """Per-request sampling controls.

    ``temperature <= 0`` means greedy.  ``top_k <= 0`` disables top-k,
    ``top_p >= 1`` disables nucleus filtering, ``min_p == 0`` disables min-p.
    ``seed`` selects the deterministic per-request Philox stream.
    """

    temperature: float = 0.0
    top_k: int = -1
    top_p: float = 1.0
    min_p: float = 0.0
    seed: Optional[int] = None
    ignore_eos: bool = False
    stop_token_ids: tuple = ()

    def effectively_greedy(self, vocab_size: int) -> bool:
        """True when sampling collapses to argmax (pegainfer-sample/src/lib.rs:56-116)."""
        if self.temperature < 1e-5:
            return True
        if self.top_k == 1:
            return True
        if self.top_p <= 1.0 / max(vocab_size, 1):
            return True
        return False


@dataclass
class ParallelConfig:
    tp_size: int = 1
    dp_size: int = 1
    ep_size: int = 1

    def world_size(self) -> int:
        return max(self.tp_size * self.dp_size, self.ep_size)

    def validate(self) -> None:
        for name in ("tp_size", "dp_size", "ep_size"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1")


class FinishReason(enum.Enum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"


class RejectReason(enum.Enum):
    """Typed reasons a scheduler refuses a request before running it."""

    PROMPT_TOO_LONG = "prompt_too_long"
    EMPTY_PROMPT = "empty_prompt"
    KV_CAPACITY = "kv_capacity"
    UNKNOWN_LORA = "unknown_lora"
    UNSUPPORTED_PARAMS = "unsupported_params"
    SHUTTING_DOWN = "shutting_down"
    INVALID_TOKEN = "invalid_token"


@dataclass
class Terminal:
    """End of a request's lifetime: finished, rejected or failed."""

    kind: str  # "finished" | "rejected" | "failed"
    finish_reason: Optional[FinishReason] = None
    reject_reason: Optional[RejectReason] = None
    message: str = ""

    @staticmethod
    def finished(reason: FinishReason) -> "Terminal":
        return Terminal("finished", finish_reason=reason)

    @staticmethod
    def rejected(reason: RejectReason, message: str = "") -> "Terminal":
        return Terminal("rejected", reject_reason=reason, message=message)

    @staticmethod
    def failed(message: str) -> "Terminal":
        return Terminal("failed", message=message)


@dataclass
class TokenLogprob:
    token: int
    logprob: float
    top: list = field(default_factory=list)  # [(token, logprob)] alternatives


@dataclass
class PromptEcho:
    tokens: list
    logprobs: list  # Optional[TokenLogprob] per prompt token


@dataclass
class ScheduledInfo:
    """Admission facts, reported once in the step that admitted the request."""

    queued_at: float
    scheduled_at: float
    prompt_tokens: int


@dataclass
class Request:
    prompt_tokens: list
    params: SamplingParams = field(default_factory=SamplingParams)
    max_tokens: int = 16
    lora_adapter: Optional[str] = None
    kv_transfer_params: Optional[Any] = None
    logprobs: int = 0
    echo: bool = False
    trace_parent: Optional[Any] = None
    client_label: Optional[str] = None
    cache_salt: Optional[str] = None
    data_parallel_rank: Optional[int] = None


@dataclass
class QueuedRequest:
    id: int
    request: Request
    queued_at: float = field(default_factory=time.monotonic)
    abort_flag: threading.Event = field(default_factory=threading.Event)

    def is_aborted(self) -> bool:
        return self.abort_flag.is_set()


@dataclass
class RequestUpdate:
    id: int
    scheduled: Optional[ScheduledInfo] = None
    tokens: list = field(default_factory=list)
    logprobs: list = field(default_factory=list)
    cached_tokens: Optional[int] = None
    prompt_echo: Optional[PromptEcho] = None
    kv_transfer: Optional[Any] = None
    terminal: Optional[Terminal] = None

    def is_empty(self) -> bool:
        return (
            self.scheduled is None
            and not self.tokens
            and self.cached_tokens is None
            and self.prompt_echo is None
            and self.kv_transfer is None
            and self.terminal is None
        )


@dataclass
class StepOutputs:
    updates: list = field(default_factory=list)
    metrics: Optional["SchedulerMetrics"] = None


@dataclass
class SpecDecodeCounters:
    """Cumulative speculative-decoding counters (engine/metrics.rs:59-94)."""

    num_drafts: int = 0
    num_draft_tokens: int = 0
    num_accepted_tokens: int = 0
    accepted_per_pos: list = field(default_factory=list)

    def record(self, proposed: int, accepted: int) -> None:
        self.num_drafts += 1
        self.num_draft_tokens += proposed
        self.num_accepted_tokens += accepted
        while len(self.accepted_per_pos) < proposed:
            self.accepted_per_pos.append(0)
        for i in range(accepted):
            self.accepted_per_pos[i] += 1


@dataclass
class SchedulerMetrics:
    kv_used_blocks: int = 0
    kv_total_blocks: int = 0
    num_running_reqs: int = 0
    num_waiting_reqs: int = 0
    spec_decode: SpecDecodeCounters = field(default_factory=SpecDecodeCounters)
    prefix_hit_tokens: int = 0
    prefix_query_tokens: int = 0
    host_tier_hit_blocks: int = 0

    def kv_usage(self) -> float:
        return self.kv_used_blocks / self.kv_total_blocks if self.kv_total_blocks else 0.0


@dataclass
class KvCapacity:
    """KV facts a frontend advertises (engine/kv.rs:22-119)."""

    num_blocks: int
    block_size: int

    def tokens(self) -> int:
        return self.num_blocks * self.block_size


@dataclass
class EngineInfo:
    model_name: str
    max_model_len: int
    kv_capacity: KvCapacity
    dtype: str = "bfloat16"
    dp_size: int = 1
    vocab_size: int = 0
    eos_token_ids: tuple = ()


class Scheduler(Protocol):
    """What a model line implements (engine/driver.rs:20-41)."""

    def submit(self, req: QueuedRequest) -> None: ...

    def step(self, ledger: "Any") -> bool:
        """Run one iteration.  Returns False when there was nothing to do."""

    def metrics(self) -> SchedulerMetrics: ...
