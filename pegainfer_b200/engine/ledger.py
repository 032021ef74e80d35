"""Scheduler-side request ledger: terminal-exactly-once accounting.

Every submitted request opens an account.  A scheduler writes tokens and at most
one terminal against it per lifetime; a write against a closed or unknown account
raises :class:`LedgerMisuse` (the reference panics).  ``commit_step`` folds all
writes of the iteration into one :class:`StepOutputs`.

Reference parity: pegainfer-frontend/src/engine/ledger.rs:103-330,
engine/request_lifecycle.rs:44-198 (envelope / deferred-finish drop guards).
"""
from __future__ import annotations

import time
from typing import Callable, Optional

from .contract import (
    FinishReason,
    PromptEcho,
    QueuedRequest,
    RejectReason,
    RequestUpdate,
    ScheduledInfo,
    StepOutputs,
    Terminal,
)


class LedgerMisuse(RuntimeError):
    """A scheduler broke the contract (double terminal, unknown id, ...)."""


class _Account:
    __slots__ = ("queued", "scheduled_reported", "closed", "tokens_out", "deferred")

    def __init__(self, queued: QueuedRequest):
        self.queued = queued
        self.scheduled_reported = False
        self.closed = False
        self.tokens_out = 0
        self.deferred = False


class RequestLedger:
    def __init__(self, sink: Optional[Callable[[StepOutputs], None]] = None):
        self._accounts: dict[int, _Account] = {}
        self._pending: dict[int, RequestUpdate] = {}
        self._sink = sink
        self.steps_committed = 0

    # -- account lifecycle -------------------------------------------------
    def register(self, queued: QueuedRequest) -> None:
        if queued.id in self._accounts:
            raise LedgerMisuse(f"request {queued.id} registered twice")
        self._accounts[queued.id] = _Account(queued)

    def is_open(self, rid: int) -> bool:
        acc = self._accounts.get(rid)
        return acc is not None and not acc.closed

    def open_ids(self) -> list:
        return [rid for rid, a in self._accounts.items() if not a.closed]

    def is_aborted(self, rid: int) -> bool:
        acc = self._accounts.get(rid)
        return acc is not None and acc.queued.is_aborted()

    def _open(self, rid: int) -> _Account:
        acc = self._accounts.get(rid)
        if acc is None:
            raise LedgerMisuse(f"request {rid} has no account")
        if acc.closed:
            raise LedgerMisuse(f"request {rid} already received its terminal")
        return acc

    def _update(self, rid: int) -> RequestUpdate:
        upd = self._pending.get(rid)
        if upd is None:
            upd = RequestUpdate(id=rid)
            self._pending[rid] = upd
        return upd

    # -- writes --------------------------------------------------------------
    def mark_scheduled(self, rid: int, prompt_tokens: int) -> None:
        acc = self._open(rid)
        if acc.scheduled_reported:
            raise LedgerMisuse(f"request {rid} scheduled twice")
        acc.scheduled_reported = True
        self._update(rid).scheduled = ScheduledInfo(
            queued_at=acc.queued.queued_at, scheduled_at=time.monotonic(), prompt_tokens=prompt_tokens
        )

    def push_tokens(self, rid: int, tokens, logprobs=None) -> None:
        acc = self._open(rid)
        upd = self._update(rid)
        tokens = list(tokens)
        upd.tokens.extend(tokens)
        if logprobs is None:
            upd.logprobs.extend([None] * len(tokens))
        else:
            if len(logprobs) != len(tokens):
                raise LedgerMisuse("logprobs must be parallel to tokens")
            upd.logprobs.extend(logprobs)
        acc.tokens_out += len(tokens)

    def report_cached_tokens(self, rid: int, n: int) -> None:
        self._open(rid)
        self._update(rid).cached_tokens = n

    def push_prompt_echo(self, rid: int, echo: PromptEcho) -> None:
        self._open(rid)
        self._update(rid).prompt_echo = echo

    def set_kv_transfer(self, rid: int, payload) -> None:
        self._open(rid)
        self._update(rid).kv_transfer = payload

    def _close(self, rid: int, terminal: Terminal) -> None:
        acc = self._open(rid)
        acc.closed = True
        self._update(rid).terminal = terminal

    def finish(self, rid: int, reason: FinishReason) -> None:
        self._close(rid, Terminal.finished(reason))

    def reject(self, rid: int, reason: RejectReason, message: str = "") -> None:
        self._close(rid, Terminal.rejected(reason, message))

    def fail(self, rid: int, message: str) -> None:
        self._close(rid, Terminal.failed(message))

    def defer_finish(self, rid: int) -> "DeferredFinish":
        """Withhold a terminal until some later event (e.g. a KV flush barrier)."""
        acc = self._open(rid)
        acc.deferred = True
        return DeferredFinish(self, rid)

    def fail_all(self, message: str) -> None:
        for rid in self.open_ids():
            self.fail(rid, message)

    # -- commit ----------------------------------------------------------------
    def commit_step(self) -> Optional[StepOutputs]:
        updates = [u for u in self._pending.values() if not u.is_empty()]
        self._pending = {}
        # Closed accounts are retired after their terminal went out.
        for u in updates:
            if u.terminal is not None:
                self._accounts.pop(u.id, None)
        if not updates:
            return None
        out = StepOutputs(updates=updates)
        self.steps_committed += 1
        if self._sink is not None:
            self._sink(out)
        return out


class DeferredFinish:
    """Handle that must be resolved exactly once; dropping it unresolved turns into
    a ``Failed`` terminal so the client never waits forever."""

    def __init__(self, ledger: RequestLedger, rid: int):
        self._ledger = ledger
        self._rid = rid
        self._done = False

    def resolve(self, reason: FinishReason) -> None:
        if self._done:
            raise LedgerMisuse("deferred finish resolved twice")
        self._done = True
        self._ledger.finish(self._rid, reason)

    def abandon(self) -> None:
        if not self._done and self._ledger.is_open(self._rid):
            self._done = True
            self._ledger.fail(self._rid, "deferred finish abandoned")

    def __del__(self):  # drop guard
        try:
            self.abandon()
        except Exception:
            pass
