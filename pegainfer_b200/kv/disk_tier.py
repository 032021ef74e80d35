"""Disk (SSD) tier below the host tier: blocks evicted from pinned host memory are written to
files named by their content hash and read back when a later request's prefix asks for them.

Writes happen on a background thread (the scheduler thread only copies the block out of the
slab and queues it); reads are synchronous and happen at admission, while the request is
parked anyway.  The tier is bounded in bytes and evicts the least recently used files.  Every
failure (disk full, unreadable file, short read) degrades to "not cached": the request
prefills from scratch.

Reference parity: pegainfer-kv-store/src/tier.rs (SSD tier below the host pool),
src/policy.rs (bounded, LRU), src/store.rs:90-730 (resolve_prefix consults every tier).
"""
from __future__ import annotations

import os
import queue
import threading
from collections import OrderedDict
from typing import Optional

import torch


class DiskTier:
    def __init__(self, directory: str, max_bytes: int, block_bytes: int):
        self.dir = directory
        os.makedirs(directory, exist_ok=True)
        self.block_bytes = block_bytes
        self.max_blocks = max(1, max_bytes // max(block_bytes, 1))
        self.index: "OrderedDict[bytes, str]" = OrderedDict()  # hash -> path, least recently used first
        self._lock = threading.Lock()
        self._q: "queue.Queue" = queue.Queue(maxsize=64)
        self.writes = self.write_drops = self.hits = self.evictions = self.read_failures = 0
        self._stop = False
        self._thread = threading.Thread(target=self._writer, name="kv-disk-writer", daemon=True)
        self._thread.start()
        for fn in os.listdir(directory):  # blocks left by an earlier run are usable again (content addressed)
            if fn.endswith(".kv") and os.path.getsize(os.path.join(directory, fn)) == block_bytes:
                try:
                    self.index[bytes.fromhex(fn[:-3])] = os.path.join(directory, fn)
                except ValueError:
                    pass

    def _path(self, h: bytes) -> str:
        return os.path.join(self.dir, h.hex() + ".kv")

    def offer(self, h: bytes, block: torch.Tensor) -> None:
        """Queue a copy of ``block`` (a host tensor) for writing; dropped when the queue is full."""
        with self._lock:
            if h in self.index:
                self.index.move_to_end(h)
                return
        try:
            self._q.put_nowait((h, block.contiguous().view(torch.uint8).reshape(-1).clone()))
        except queue.Full:
            self.write_drops += 1

    def _writer(self) -> None:
        while not self._stop:
            try:
                h, data = self._q.get(timeout=0.2)
            except queue.Empty:
                continue
            path = self._path(h)
            try:
                tmp = path + ".tmp"
                with open(tmp, "wb") as f:
                    f.write(data.numpy().tobytes())
                os.replace(tmp, path)  # a reader never sees a half-written block
            except OSError:
                self.write_drops += 1
                continue
            finally:
                self._q.task_done()
            with self._lock:
                self.index[h] = path
                self.index.move_to_end(h)
                self.writes += 1
                while len(self.index) > self.max_blocks:
                    _, old = self.index.popitem(last=False)
                    self.evictions += 1
                    try:
                        os.unlink(old)
                    except OSError:
                        pass

    def contains(self, h: bytes) -> bool:
        with self._lock:
            return h in self.index

    def read_into(self, h: bytes, dst: torch.Tensor) -> bool:
        """Read block ``h`` into the host tensor ``dst`` (same shape / dtype as when it was offered)."""
        with self._lock:
            path = self.index.get(h)
            if path is not None:
                self.index.move_to_end(h)
        if path is None:
            return False
        try:
            with open(path, "rb") as f:
                raw = f.read()
            if len(raw) != self.block_bytes:
                raise OSError("short block file")
            dst.view(torch.uint8).reshape(-1).copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
        except OSError:
            self.read_failures += 1
            with self._lock:
                self.index.pop(h, None)
            return False
        self.hits += 1
        return True

    def flush(self, timeout_s: float = 10.0) -> None:
        """Wait until every queued write has reached the disk (tests, orderly shutdown)."""
        import time

        t0 = time.monotonic()
        while self._q.unfinished_tasks and time.monotonic() - t0 < timeout_s:
            time.sleep(0.005)

    def close(self) -> None:
        self.flush()
        self._stop = True
