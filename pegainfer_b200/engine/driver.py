"""Scheduler driver thread, submit handles and multi-partition engine wiring.

``spawn_scheduler`` runs a scheduler on its own OS thread: drain the submit queue,
``scheduler.step(ledger)``, publish metrics, ``ledger.commit_step()``.  A fatal
exception in ``step`` fails every open request and winds the driver down; the
frontend observes ``Failed`` terminals rather than hanging.

``Engine`` fronts N scheduler partitions (data-parallel ranks).  A request names a
partition (``data_parallel_rank``) or is routed to the least loaded one by
``running + 4 * waiting``.

Reference parity: pegainfer-frontend/src/engine/driver.rs:20-104 (drive loop),
engine/wiring.rs:29-175 (scheduler_pair, Engine, metrics cell),
engine/handle.rs:71-261 (partition routing), engine/sink.rs:37-118 (per-request
sinks with abort on disconnect).
"""
from __future__ import annotations

import itertools
import queue
import threading
import time
from typing import Callable, Optional

from .contract import (
    EngineInfo,
    QueuedRequest,
    Request,
    RequestUpdate,
    SchedulerMetrics,
    StepOutputs,
    Terminal,
)
from .ledger import RequestLedger


class RequestStream:
    """Consumer side of one request: a thread-safe queue of RequestUpdate."""

    def __init__(self, rid: int, queued: QueuedRequest, partition: int):
        self.id = rid
        self.partition = partition
        self._queued = queued
        self._q: "queue.Queue[RequestUpdate]" = queue.Queue()
        self._listeners: list = []
        self.closed = False

    def add_listener(self, fn: Callable[[RequestUpdate], None]) -> None:
        """Register a callback (e.g. asyncio loop.call_soon_threadsafe bridge)."""
        self._listeners.append(fn)

    def _deliver(self, upd: RequestUpdate) -> None:
        if upd.terminal is not None:
            self.closed = True
        self._q.put(upd)
        for fn in self._listeners:
            fn(upd)

    def abort(self) -> None:
        """Client went away: flag the request; the scheduler retires it reactively."""
        self._queued.abort_flag.set()

    def get(self, timeout: Optional[float] = None) -> RequestUpdate:
        return self._q.get(timeout=timeout)

    def __iter__(self):
        while True:
            upd = self._q.get()
            yield upd
            if upd.terminal is not None:
                return

    def collect(self, timeout: float = 600.0):
        """Block until the terminal; returns (tokens, terminal, updates)."""
        deadline = time.monotonic() + timeout
        toks, updates = [], []
        while True:
            remaining = deadline - time.monotonic()
            if remaining <= 0:
                raise TimeoutError(f"request {self.id} did not finish in {timeout}s")
            upd = self._q.get(timeout=remaining)
            updates.append(upd)
            toks.extend(upd.tokens)
            if upd.terminal is not None:
                return toks, upd.terminal, updates


class _MetricsCell:
    def __init__(self):
        self._lock = threading.Lock()
        self._value = SchedulerMetrics()

    def publish(self, m: SchedulerMetrics) -> None:
        with self._lock:
            self._value = m

    def read(self) -> SchedulerMetrics:
        with self._lock:
            return self._value


class SchedulerHandle:
    """Submit side of one scheduler partition."""

    def __init__(self, partition: int):
        self.partition = partition
        self._submit_q: "queue.Queue[QueuedRequest]" = queue.Queue()
        self._ids = itertools.count(1)
        self._streams: dict[int, RequestStream] = {}
        self._lock = threading.Lock()
        self.metrics_cell = _MetricsCell()
        self._wake = threading.Event()
        self.alive = True
        self.waiting_hint = 0

    def submit(self, request: Request, listener=None) -> RequestStream:
        rid = next(self._ids)
        queued = QueuedRequest(id=rid, request=request)
        stream = RequestStream(rid, queued, self.partition)
        if listener is not None:
            stream.add_listener(listener)
        with self._lock:
            self._streams[rid] = stream
            self.waiting_hint += 1
        if not self.alive:
            stream._deliver(RequestUpdate(id=rid, terminal=Terminal.failed("engine is down")))
            return stream
        self._submit_q.put(queued)
        self._wake.set()
        return stream

    def dispatch(self, outputs: StepOutputs) -> None:
        for upd in outputs.updates:
            with self._lock:
                stream = self._streams.get(upd.id)
                if upd.scheduled is not None:
                    self.waiting_hint = max(0, self.waiting_hint - 1)
                if upd.terminal is not None:
                    self._streams.pop(upd.id, None)
            if stream is not None:
                stream._deliver(upd)

    def load(self) -> int:
        m = self.metrics_cell.read()
        return m.num_running_reqs + 4 * max(m.num_waiting_reqs, self.waiting_hint)


def _bind_thread_to_device(scheduler) -> None:
    """Make the executor's GPU the current CUDA device of the calling thread.  The current device
    is per host thread and starts at device 0: on any other GPU a thread that does not do this
    records events and picks "current" streams on the wrong device, and kernels launched through
    the C API (which follow the thread's current device) land on GPU 0."""
    dev = getattr(getattr(scheduler, "ex", None), "device", None)
    if dev is not None and getattr(dev, "type", None) == "cuda":
        import torch

        torch.cuda.set_device(dev)


def drive(scheduler, handle: SchedulerHandle, stop: threading.Event, idle_sleep: float = 0.0005) -> None:
    """Busy-poll drive loop for one scheduler partition."""
    ledger = RequestLedger(sink=handle.dispatch)
    _bind_thread_to_device(scheduler)
    try:
        while not stop.is_set():
            drained = 0
            while True:
                try:
                    q = handle._submit_q.get_nowait()
                except queue.Empty:
                    break
                ledger.register(q)
                scheduler.submit(q)
                drained += 1
            try:
                busy = scheduler.step(ledger)
            except Exception as exc:  # fatal step: fail-stop, never hang clients
                ledger.fail_all(f"scheduler step failed: {exc!r}")
                ledger.commit_step()
                handle.alive = False
                raise
            handle.metrics_cell.publish(scheduler.metrics())
            ledger.commit_step()
            if not busy and drained == 0:
                handle._wake.wait(idle_sleep)
                handle._wake.clear()
    finally:
        handle.alive = False
        ledger.fail_all("engine shut down")
        ledger.commit_step()
        # requests submitted after the loop stopped must not hang either
        while True:
            try:
                q = handle._submit_q.get_nowait()
            except queue.Empty:
                break
            handle.dispatch(StepOutputs(updates=[RequestUpdate(id=q.id, terminal=Terminal.failed("engine shut down"))]))


class Engine:
    """One engine identity fronting ``len(schedulers)`` partitions."""

    def __init__(self, schedulers: list, info: EngineInfo, lora_client=None, start: bool = True):
        if not schedulers:
            raise ValueError("an engine needs at least one scheduler")
        self.info = info
        self.lora = lora_client
        self._schedulers = schedulers
        self._handles = [SchedulerHandle(i) for i in range(len(schedulers))]
        self._stop = threading.Event()
        self._threads = []
        self._errors: list = []
        if start:
            self.start()

    def start(self) -> None:
        """Spawn the scheduler threads.  An engine built with ``start=False`` queues
        submissions until then, which gives replicated (SPMD) ranks an identical,
        timing-independent admission order."""
        if self._threads:
            return
        for i, (s, h) in enumerate(zip(self._schedulers, self._handles)):
            t = threading.Thread(target=self._run, args=(s, h), name=f"scheduler-{i}", daemon=True)
            t.start()
            self._threads.append(t)

    def _run(self, scheduler, handle):
        try:
            drive(scheduler, handle, self._stop)
        except Exception as exc:  # already surfaced to clients as Failed terminals
            self._errors.append(exc)

    @property
    def num_partitions(self) -> int:
        return len(self._handles)

    def submit(self, request: Request, listener=None) -> RequestStream:
        """Route and enqueue a request.  ``listener`` (called from the scheduler thread
        for every update) is attached before the request becomes visible to the
        scheduler, so no update can be missed."""
        rank = request.data_parallel_rank
        if rank is not None:
            if not (0 <= rank < len(self._handles)):
                raise ValueError(f"data_parallel_rank {rank} out of range for {len(self._handles)} partitions")
            return self._handles[rank].submit(request, listener)
        handle = min(self._handles, key=lambda h: (h.load(), h.partition))
        return handle.submit(request, listener)

    def metrics(self) -> list:
        return [h.metrics_cell.read() for h in self._handles]

    def healthy(self) -> bool:
        return all(h.alive for h in self._handles)

    def shutdown(self, timeout: float = 10.0) -> None:
        self._stop.set()
        for h in self._handles:
            h._wake.set()
        for t in self._threads:
            t.join(timeout)

    def generate(self, prompts, params=None, max_tokens: int = 16, timeout: float = 600.0):
        """Blocking convenience API: run a batch of token-id prompts to completion."""
        from .contract import SamplingParams

        streams = [
            self.submit(Request(prompt_tokens=list(p), params=params or SamplingParams(), max_tokens=max_tokens))
            for p in prompts
        ]
        return [s.collect(timeout) for s in streams]
