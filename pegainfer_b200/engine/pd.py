"""Prefill / decode disaggregation inside one process: two engines, one KV store between them.

A prefill engine (its own GPU, scheduler thread and KV pool) runs the prompt and publishes every
block it seals into a shared ``TierStore``; its finish is withheld until those copies have landed.
The decode engine then admits the same request: its admission probe finds the prompt's blocks in
the store by content hash, restores them into its own KV pool while the request is parked, and
starts from a prefix hit that covers all full blocks of the prompt, so it only recomputes the
last partial block before it decodes.  With the store's slab placed on the decode engine's GPU a
block crosses NVLink once, as a peer copy issued by the prefill engine, and the restore is a
local copy; with the slab in pinned host memory the same code is the two-hop PCIe path.

``PdEngine`` has the surface the HTTP frontend uses from an engine (``submit`` with a listener,
``info``, ``metrics``, ``healthy``, ``shutdown``, ``generate``).

Reference parity: docs/models/qwen3/pd-disaggregation-m2.md and pegainfer-qwen3/src/executor.rs:1006-1009
(``flush_on_finish``: a finish is reported only after the saves are visible), src/frontend_adapter.rs:558-569,
src/model_line.rs:157-174 (``--kv-p2p-*``); the reference moves blocks by content hash between two
server processes over RDMA, here the two engines share a process and the blocks move over NVLink.
"""
from __future__ import annotations

import dataclasses
import queue
import threading
import time
from typing import Optional

from .contract import FinishReason, Request


class PdStream:
    """Consumer side of a disaggregated request: the decode stage's updates, or the prefill stage's
    terminal if that stage did not finish normally."""

    def __init__(self, rid: int):
        self.id = rid
        self._q: "queue.Queue" = queue.Queue()
        self._listeners: list = []
        self._lock = threading.Lock()
        self._stage = None  # the stream of the stage that is running
        self._aborted = False
        self.closed = False
        self.prefill_s: Optional[float] = None

    def add_listener(self, fn) -> None:
        self._listeners.append(fn)

    def _deliver(self, upd) -> None:
        if upd.terminal is not None:
            self.closed = True
        self._q.put(upd)
        for fn in self._listeners:
            fn(upd)

    def _enter(self, stream) -> bool:
        with self._lock:
            self._stage = stream
            if self._aborted:
                stream.abort()
            return not self._aborted

    def abort(self) -> None:
        with self._lock:
            self._aborted = True
            if self._stage is not None:
                self._stage.abort()

    def get(self, timeout: Optional[float] = None):
        return self._q.get(timeout=timeout)

    def collect(self, timeout: float = 600.0):
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


class PdEngine:
    def __init__(self, prefill, decode, store):
        self.prefill, self.decode, self.store = prefill, decode, store
        self.info = decode.info
        self._ids = 0
        self._lock = threading.Lock()
        self.handoffs = 0

    def submit(self, request: Request, listener=None) -> PdStream:
        with self._lock:
            self._ids += 1
            out = PdStream(self._ids)
        if listener is not None:
            out.add_listener(listener)
        t0 = time.monotonic()
        first = dataclasses.replace(request, max_tokens=1, logprobs=0)

        def on_prefill(upd):
            if upd.terminal is None:
                return
            term = upd.terminal
            normal = getattr(term, "finish_reason", None) in (FinishReason.LENGTH, FinishReason.STOP)
            if not normal or out._aborted:
                out._deliver(dataclasses.replace(upd, tokens=[]) if dataclasses.is_dataclass(upd) else upd)
                return
            out.prefill_s = time.monotonic() - t0
            self.handoffs += 1
            out._enter(self.decode.submit(request, listener=out._deliver))

        out._enter(self.prefill.submit(first, listener=on_prefill))
        return out

    def generate(self, prompts, params=None, max_tokens: int = 16, timeout: float = 600.0):
        from .contract import SamplingParams

        streams = [self.submit(Request(prompt_tokens=list(p), params=params or SamplingParams(), max_tokens=max_tokens)) for p in prompts]
        return [s.collect(timeout) for s in streams]

    def metrics(self) -> list:
        return self.decode.metrics()

    def healthy(self) -> bool:
        return self.prefill.healthy() and self.decode.healthy()

    def shutdown(self, timeout: float = 10.0) -> None:
        self.prefill.shutdown(timeout)
        self.decode.shutdown(timeout)


def build_pd_engine(ecfg, mcfg=None, prefill_device=None, decode_device=None, dtype=None, store_bytes: int = 0, store_device=None, prefill_model=None, decode_model=None):
    """Two engines of the same model joined by one KV store.  ``store_device`` defaults to the decode
    engine's device (blocks cross NVLink once); ``"cpu"`` keeps the store in pinned host memory."""
    import copy

    import torch

    from ..kv.host_tier import TierStore
    from .build import build_engine

    if ecfg.spec_method:
        raise ValueError("speculative decoding switches the prefix cache off, which prefill / decode disaggregation relies on")
    cuda = torch.cuda.is_available()
    prefill_device = prefill_device or ("cuda:0" if cuda else "cpu")
    decode_device = decode_device or (f"cuda:{1 if torch.cuda.device_count() > 1 else 0}" if cuda else "cpu")
    pcfg, dcfg = copy.copy(ecfg), copy.copy(ecfg)
    for c in (pcfg, dcfg):
        c.kv_offload = False  # the tiers are attached below, around the shared store
        c.no_prefix_cache = False
    if torch.device(prefill_device) == torch.device(decode_device) and cuda:
        pcfg.gpu_memory_utilization = dcfg.gpu_memory_utilization = ecfg.gpu_memory_utilization / 2
    decode = build_engine(dcfg, mcfg, device=decode_device, dtype=dtype, model=decode_model, start=False)
    prefill = build_engine(pcfg, mcfg, device=prefill_device, dtype=dtype, model=prefill_model, start=False)
    nbytes = store_bytes or int(ecfg.kv_offload_host_gib * (1 << 30))
    store = TierStore.for_kv(decode.kv, nbytes, store_device or decode_device)
    for eng, producer in ((prefill, True), (decode, False)):
        from ..kv.host_tier import HostTier

        tier = HostTier(eng.kv, eng.pool, 0, store=store, flush_on_finish=producer)
        eng.scheduler.host_tier = tier
        eng.host_tier = tier
        eng.scheduler._ahead = False  # run-ahead and parking do not mix (same rule as --kv-offload)
        eng.start()
    return PdEngine(prefill, decode, store)
