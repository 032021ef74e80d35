"""Host-memory tier of the KV cache (offload + restore by content hash).

* SAVE: when a running request seals (fills and registers) a block, and after the step
  that wrote it has synchronised, the block's data (all layers: a strided view of the
  KV buffer) is copied to a pinned host slab on a dedicated copy stream.  The source
  block is pinned (one extra pool reference) until the copy has landed, so an evicted
  and rewritten block can never be stored under an old hash.  A failed or skipped save
  only forfeits a future hit.
* QUERY / LOAD: at admission the request's prefix hashes are probed: blocks already on
  the GPU are left to the normal prefix match; the following run of blocks present in
  the host tier is loaded into freshly reserved GPU blocks (never dipping below the
  scheduler's reserve floor) while the request is *parked*; when the copy has landed the
  blocks are committed into the prefix cache under their hashes, so the ordinary
  ``match_and_add_prefix`` simply sees a longer hit.
* Any error or lack of space degrades to "prefill from scratch", never to a client error.
* ``flush_saves_then`` is the barrier used when a finish must not be reported before
  the KV is visible to a peer (prefill/decode disaggregation).

Reference parity: pegainfer-kv-offload/src/engine.rs:67-505 (register / save / query /
load / flush), pegainfer-qwen3/src/executor.rs:1037-1091,1706-1845,1986-2030 (prefetch
state machine, save of sealed blocks, settle), src/scheduler.rs:146-197 (parking),
pegainfer-kv-store/src/store.rs:90-730 (resolve_prefix orchestration).
"""
from __future__ import annotations

import time
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from .request_kv import RequestKv, chain_hash


@dataclass
class _Save:
    bid: int
    slot: int
    h: bytes
    event: Optional[object]


@dataclass
class _Load:
    rid: int
    blocks: list
    hashes: list
    parent: Optional[bytes]
    event: Optional[object]
    started: float


@dataclass
class TierStats:
    saves: int = 0
    save_skips: int = 0
    host_hits: int = 0
    loads: int = 0
    load_failures: int = 0
    evictions: int = 0


class TierStore:
    """The slab of a KV tier and its hash index, as an object of its own so that two engines can share it:
    a prefill engine publishes the blocks it seals, a decode engine finds them by hash (prefill / decode
    disaggregation inside one process).  ``device`` is where the slab lives: pinned host memory (``cpu``), or
    the decode engine's GPU, in which case a published block crosses NVLink once, as a peer copy from the
    prefill GPU, and the decode engine's restore is a local copy.  ``busy`` counts the loads reading a slot:
    such an entry is never chosen for eviction."""

    def __init__(self, block_shape, dtype, num_slots: int, device="cpu", pin: bool = False):
        import threading

        self.lock = threading.RLock()
        self.slab = torch.empty((num_slots,) + tuple(block_shape), dtype=dtype, device=device)
        if pin and torch.device(device).type == "cpu":
            self.slab = self.slab.pin_memory()
        self.by_hash: "OrderedDict[bytes, int]" = OrderedDict()  # LRU: oldest first
        self.free_slots = list(range(num_slots - 1, -1, -1))
        self.busy: dict = {}
        self.num_slots = num_slots

    @classmethod
    def for_kv(cls, kv, nbytes: int, device="cpu") -> "TierStore":
        one = kv.data[:, 0]
        slots = max(1, nbytes // (one.numel() * one.element_size()))
        return cls(tuple(one.shape), kv.data.dtype, slots, device, pin=kv.data.device.type == "cuda")


class HostTier:
    def __init__(self, kv, pool, host_bytes: int, reserve_floor: int = 2, l1_retention_disabled: bool = False, load_deadline_s: float = 15.0,
                 disk_dir: Optional[str] = None, disk_bytes: int = 0, store: Optional[TierStore] = None, flush_on_finish: bool = False):
        self.kv, self.pool = kv, pool
        self.data = kv.data
        self.device = self.data.device
        one = self.data[:, 0]
        self.block_shape = tuple(one.shape)
        self.block_bytes = one.numel() * one.element_size()
        self.cuda = self.device.type == "cuda"
        if store is None:
            store = TierStore(self.block_shape, self.data.dtype, max(1, host_bytes // self.block_bytes), "cpu", pin=self.cuda)
        elif tuple(store.slab.shape[1:]) != self.block_shape or store.slab.dtype != self.data.dtype:
            raise ValueError("the shared KV store holds blocks of another shape: both engines must run the same model and page size")
        self.store = store
        self.lock = store.lock
        self.num_slots = store.num_slots
        self.slab = store.slab
        if self.cuda:
            self.stream = torch.cuda.Stream(self.device)
        self.by_hash = store.by_hash
        self.free_slots = store.free_slots
        self.flush_on_finish = flush_on_finish  # a finish is reported only after the request's sealed blocks are in the store
        self.saving: list = []
        self.loading: dict = {}
        self.ready: list = []
        self.saved_upto: dict = {}  # rid -> number of this request's blocks already offered
        self.reserve_floor = reserve_floor
        self.l1_retention_disabled = l1_retention_disabled
        self.load_deadline_s = load_deadline_s
        self.stats = TierStats()
        self._probed: set = set()
        # optional third tier: blocks evicted from the pinned slab go to files, see kv/disk_tier.py
        self.disk = None
        if disk_dir and disk_bytes > 0:
            from .disk_tier import DiskTier

            self.disk = DiskTier(disk_dir, disk_bytes, self.block_bytes)

    # -- save path ---------------------------------------------------------------------
    def _take_slot(self, protect=()) -> Optional[int]:
        """A free slot, else the least recently used entry that is not in ``protect``."""
        if self.free_slots:
            return self.free_slots.pop()
        if self.saving:
            self.poll()  # saves that have landed become evictable entries
        victim = next((h for h in self.by_hash if h not in protect and not self.store.busy.get(h)), None)
        if victim is not None:
            h, slot = victim, self.by_hash.pop(victim)
            self.stats.evictions += 1
            if self.disk is not None:
                self.disk.offer(h, self.slab[slot])  # copied out before the slot is reused
            return slot
        return None

    def _promote_from_disk(self, h: bytes, protect=()) -> bool:
        """Bring a block that only the disk tier holds back into a host slot (never at the cost of a
        block in ``protect``: the run being assembled must stay resident until it is copied)."""
        if self.disk is None or not self.disk.contains(h):
            return False
        slot = self._take_slot(protect)
        if slot is None:
            return False
        if not self.disk.read_into(h, self.slab[slot]):
            self.free_slots.append(slot)
            return False
        self.by_hash[h] = slot
        return True

    def on_blocks_sealed(self, r, sched) -> None:
        """Offer every newly registered block of request ``r`` to the host tier."""
        kv: RequestKv = r.kv
        done = self.saved_upto.get(r.q.id, kv.cached_tokens // kv.bs)
        upto = kv._registered_blocks
        if upto <= done:
            return
        # recompute the chain hashes of the new blocks
        parent = None
        hashes = []
        for i in range(upto):
            parent = chain_hash(parent, kv.tokens[i * kv.bs : (i + 1) * kv.bs], kv.salt)
            hashes.append(parent)
        for i in range(done, upto):
            self._save_block(kv.blocks[i], hashes[i])
        self.saved_upto[r.q.id] = upto

    def _save_block(self, bid: int, h: bytes) -> None:
        with self.lock:
            self._save_block_locked(bid, h)

    def _save_block_locked(self, bid: int, h: bytes) -> None:
        if h in self.by_hash or any(s.h == h for s in self.saving):
            self.stats.save_skips += 1
            return
        if self.pool.block_hash(bid) != h:  # block is a private duplicate: nothing to publish
            self.stats.save_skips += 1
            return
        slot = self._take_slot()
        if slot is None:
            self.stats.save_skips += 1
            return
        self.pool.acquire(bid)  # keep-alive until the copy landed
        ev = None
        try:
            if self.cuda:
                self.stream.wait_stream(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(self.stream):
                    self.slab[slot].copy_(self.data[:, bid], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
            else:
                self.slab[slot].copy_(self.data[:, bid])
        except Exception:
            self.pool.release([bid])
            self.free_slots.append(slot)
            self.stats.save_skips += 1
            return
        self.saving.append(_Save(bid, slot, h, ev))

    # -- query / load path -----------------------------------------------------------------
    def host_hit_run(self, hashes: list, start: int) -> int:
        with self.lock:
            return self._host_hit_run_locked(hashes, start)

    def _host_hit_run_locked(self, hashes: list, start: int) -> int:
        n = 0
        run = set()
        for h in hashes[start:]:
            if h not in self.by_hash and not self._promote_from_disk(h, run):
                break
            run.add(h)
            n += 1
        return n

    def should_park(self, q, sched) -> bool:
        """Called at admission.  Starts a host->GPU load when it would extend the prefix
        hit; the request then waits in ``sched.parked`` until ``drain_ready``."""
        if q.id in self._probed:
            return False
        self._probed.add(q.id)
        if not self.pool.enable_prefix_cache:
            return False
        self.poll(sched)
        if self.l1_retention_disabled:
            self.pool.evict_inactive()
        req = q.request
        salt = b""
        if req.lora_adapter:
            salt += b"lora:" + req.lora_adapter.encode()
        if req.cache_salt:
            salt += b"salt:" + req.cache_salt.encode()
        bs = self.pool.block_size
        max_blocks = (len(req.prompt_tokens) - 1) // bs
        hashes, parent = [], None
        for i in range(max_blocks):
            parent = chain_hash(parent, req.prompt_tokens[i * bs : (i + 1) * bs], salt)
            hashes.append(parent)
        gpu_hit = self.pool.probe(hashes)
        with self.lock:
            n = self._host_hit_run_locked(hashes, gpu_hit)
            if n == 0:
                return False
            blocks = self.pool.reserve(n, floor=self.reserve_floor + sched._future_blocks())
            if blocks is None:
                return False  # no room: recompute instead
            self.stats.host_hits += n
            want = hashes[gpu_hit : gpu_hit + n]
            slots = []
            for h in want:
                self.by_hash.move_to_end(h)
                slots.append(self.by_hash[h])
                self.store.busy[h] = self.store.busy.get(h, 0) + 1  # not evictable while the copy reads it
        ev = None
        try:
            if self.cuda:
                with torch.cuda.stream(self.stream):
                    for bid, slot in zip(blocks, slots):
                        self.data[:, bid].copy_(self.slab[slot], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
            else:
                for bid, slot in zip(blocks, slots):
                    self.data[:, bid].copy_(self.slab[slot])
        except Exception:
            self._unbusy(want)
            self.pool.free_unregistered_tail(blocks)
            self.stats.load_failures += 1
            return False
        self.loading[q.id] = _Load(q.id, blocks, want, hashes[gpu_hit - 1] if gpu_hit else None, ev, time.monotonic())
        self.stats.loads += 1
        return True

    def _unbusy(self, hashes) -> None:
        with self.lock:
            for h in hashes:
                n = self.store.busy.get(h, 0) - 1
                if n > 0:
                    self.store.busy[h] = n
                else:
                    self.store.busy.pop(h, None)

    def poll(self, sched=None) -> None:
        # completed saves: publish hash -> slot, drop the keep-alive
        still = []
        with self.lock:
            for s in self.saving:
                if s.event is None or s.event.query():
                    self.by_hash[s.h] = s.slot
                    self.by_hash.move_to_end(s.h)
                    self.pool.release([s.bid])
                    self.stats.saves += 1
                else:
                    still.append(s)
        self.saving = still
        # completed loads: the blocks join the prefix cache, the request may be admitted
        for rid in list(self.loading):
            ld = self.loading[rid]
            if ld.event is None or ld.event.query():
                if self.cuda:
                    torch.cuda.current_stream(self.device).wait_event(ld.event)
                self.pool.commit_reserved(ld.blocks, ld.hashes, ld.parent)
                self._unbusy(ld.hashes)
                del self.loading[rid]
                self.ready.append(rid)
            elif time.monotonic() - ld.started > self.load_deadline_s:
                # give up: the reservation is returned once the copy can no longer write
                ld.event.synchronize()
                self.pool.free_unregistered_tail(ld.blocks)
                self._unbusy(ld.hashes)
                del self.loading[rid]
                self.stats.load_failures += 1
                self.ready.append(rid)

    def drain_ready(self, sched) -> list:
        out, self.ready = self.ready, []
        return out

    def cancel(self, rid: int) -> None:
        ld = self.loading.pop(rid, None)
        if ld is not None:
            if ld.event is not None:
                ld.event.synchronize()
            self.pool.free_unregistered_tail(ld.blocks)
            self._unbusy(ld.hashes)

    def on_retire(self, r, sched) -> None:
        self.saved_upto.pop(r.q.id, None)
        self._probed.discard(r.q.id)

    def flush_saves_then(self, cb: Callable[[], None], deadline_s: float = 5.0) -> None:
        """Run ``cb`` once every in-flight save has landed (or the deadline passed)."""
        t0 = time.monotonic()
        while self.saving and time.monotonic() - t0 < deadline_s:
            self.poll()
            if self.saving:
                time.sleep(0.0005)
        cb()

    def contains(self, h: bytes) -> bool:
        with self.lock:
            return h in self.by_hash
