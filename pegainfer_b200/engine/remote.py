"""The engine in a process of its own, behind the surface the HTTP frontend uses.

A Python frontend that streams a few thousand SSE events per second holds the interpreter lock for most of the time;
a scheduler thread in the same interpreter then waits for that lock between the launches of every decode step, and a
6 ms GPU step turns into 8 ms between tokens.  ``RemoteEngine`` starts the engine in a child process (``spawn``) and
talks to it over one pipe: requests and aborts go down, and every step's updates come back as ONE message (a list of
``RequestUpdate``), which a receiver thread hands to the per-request listeners.  The frontend's interpreter lock and the
engine's are then two different locks.

``RemoteEngine`` offers ``submit(request, listener)`` (returning a stream with ``abort`` / ``collect``), ``info``,
``metrics()``, ``healthy()``, ``generate`` and ``shutdown``.

Reference parity: the reference's frontend and engines are native threads without a shared interpreter lock
(pegainfer-frontend/src/engine/driver.rs, handle.rs); this is what that separation looks like for a Python frontend.
"""
from __future__ import annotations

import queue
import threading
import time
from typing import Optional

from .contract import Request, RequestUpdate, Terminal


def _engine_main(conn, ecfg, mcfg, device, dtype_name) -> None:
    """Child process: build the engine, then shuttle commands and updates."""
    import torch

    from .build import build_engine

    try:
        dtype = getattr(torch, dtype_name) if dtype_name else None
        eng = build_engine(ecfg, mcfg, device=device, dtype=dtype)
    except Exception as e:  # the parent learns why there is no engine
        conn.send(("failed", repr(e)))
        return
    conn.send(("ready", eng.info))
    out: "queue.Queue" = queue.Queue()
    streams: dict = {}
    stop = threading.Event()

    def sender():
        # everything that is waiting goes out as one message: a decode step's updates arrive back to back
        while not stop.is_set():
            try:
                first = out.get(timeout=0.05)
            except queue.Empty:
                continue
            batch = [first]
            try:
                while True:
                    batch.append(out.get_nowait())
            except queue.Empty:
                pass
            try:
                conn.send(("updates", batch))
            except (BrokenPipeError, OSError):
                stop.set()
                return

    threading.Thread(target=sender, daemon=True).start()
    last_metrics = 0.0
    while not stop.is_set():
        if conn.poll(0.05):
            try:
                msg = conn.recv()
            except (EOFError, OSError):
                break
            kind = msg[0]
            if kind == "submit":
                _, rid, request = msg

                def listener(upd, rid=rid):
                    upd.id = rid
                    out.put(upd)
                    if upd.terminal is not None:
                        streams.pop(rid, None)

                try:
                    streams[rid] = eng.submit(request, listener=listener)
                except Exception as e:
                    out.put(RequestUpdate(id=rid, terminal=Terminal.failed(f"submit failed: {e!r}")))
            elif kind == "abort":
                s = streams.get(msg[1])
                if s is not None:
                    s.abort()
            elif kind == "shutdown":
                break
        now = time.monotonic()
        if now - last_metrics > 0.5:
            last_metrics = now
            try:
                conn.send(("metrics", eng.metrics(), eng.healthy()))
            except (BrokenPipeError, OSError):
                break
    stop.set()
    eng.shutdown()
    try:
        conn.send(("bye",))
    except Exception:
        pass


class RemoteStream:
    def __init__(self, rid: int, owner: "RemoteEngine"):
        self.id = rid
        self._owner = owner
        self._q: "queue.Queue" = queue.Queue()
        self._listeners: list = []
        self.closed = False

    def add_listener(self, fn) -> None:
        self._listeners.append(fn)

    def _deliver(self, upd: RequestUpdate) -> None:
        if upd.terminal is not None:
            self.closed = True
        self._q.put(upd)
        for fn in self._listeners:
            fn(upd)

    def abort(self) -> None:
        self._owner._send(("abort", self.id))

    def get(self, timeout: Optional[float] = None) -> RequestUpdate:
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


class RemoteEngine:
    def __init__(self, ecfg, mcfg=None, device=None, dtype=None, start_timeout: float = 900.0):
        import multiprocessing as mp

        ctx = mp.get_context("spawn")
        self._conn, child = ctx.Pipe()
        name = str(dtype).replace("torch.", "") if dtype is not None else ""
        self._proc = ctx.Process(target=_engine_main, args=(child, ecfg, mcfg, device, name), daemon=True)
        self._proc.start()
        child.close()
        if not self._conn.poll(start_timeout):
            self._proc.terminate()
            raise RuntimeError("the engine process did not come up in time")
        msg = self._conn.recv()
        if msg[0] != "ready":
            raise RuntimeError(f"the engine process failed to start: {msg[1] if len(msg) > 1 else msg}")
        self.info = msg[1]
        self._streams: dict = {}
        self._lock = threading.Lock()
        self._send_lock = threading.Lock()
        self._ids = 0
        self._metrics: list = []
        self._healthy = True
        self._closing = False
        self._rx = threading.Thread(target=self._receive, daemon=True)
        self._rx.start()

    def _send(self, msg) -> None:
        with self._send_lock:
            try:
                self._conn.send(msg)
            except (BrokenPipeError, OSError):
                self._healthy = False

    def _receive(self) -> None:
        while True:
            try:
                msg = self._conn.recv()
            except (EOFError, OSError):
                break
            kind = msg[0]
            if kind == "updates":
                for upd in msg[1]:
                    with self._lock:
                        s = self._streams.get(upd.id)
                        if s is not None and upd.terminal is not None:
                            del self._streams[upd.id]
                    if s is not None:
                        s._deliver(upd)
            elif kind == "metrics":
                self._metrics, self._healthy = msg[1], msg[2]
            elif kind == "bye":
                break
        self._healthy = False
        # whoever still waits learns that the engine is gone
        with self._lock:
            left, self._streams = list(self._streams.values()), {}
        if not self._closing:
            for s in left:
                s._deliver(RequestUpdate(id=s.id, terminal=Terminal.failed("the engine process went away")))

    def submit(self, request: Request, listener=None) -> RemoteStream:
        with self._lock:
            self._ids += 1
            s = RemoteStream(self._ids, self)
            self._streams[s.id] = s
        if listener is not None:
            s.add_listener(listener)
        self._send(("submit", s.id, request))
        return s

    def generate(self, prompts, params=None, max_tokens: int = 16, timeout: float = 600.0):
        from .contract import SamplingParams

        streams = [self.submit(Request(prompt_tokens=list(p), params=params or SamplingParams(), max_tokens=max_tokens)) for p in prompts]
        return [s.collect(timeout) for s in streams]

    def metrics(self) -> list:
        return self._metrics

    def healthy(self) -> bool:
        return self._healthy and self._proc.is_alive()

    def shutdown(self, timeout: float = 20.0) -> None:
        self._closing = True
        self._send(("shutdown",))
        self._proc.join(timeout)
        if self._proc.is_alive():
            self._proc.terminate()
