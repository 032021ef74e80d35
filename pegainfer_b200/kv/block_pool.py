"""Logical paged-KV block pool with a hash-chained prefix cache.

Blocks move between three sets: *free* (never registered / reset), *active*
(refcount > 0) and *inactive* (refcount 0 but still registered under a content
hash, kept in LRU order so a later request with the same prefix can revive them).
Block 0 is never handed out: CUDA-graph padding rows point their page tables at it.

A block's identity is the chained hash of (parent hash, its tokens, salt), so equal
hashes imply equal full prefixes.  Only full blocks are registered.

Reference parity: pegainfer-kv-cache/src/pool.rs:30-330 (BlockPool, padding page,
probe/reserve/commit), kvbm/kvbm-logical/src/manager/mod.rs:38-225 (reset / active
/ inactive pools, registry dedup, LRU eviction), kvbm-logical/src/events/* (KV
events for cache-aware routers).
"""
from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict, deque
from dataclasses import dataclass, field
from typing import Callable, Iterable, Optional, Sequence

PADDING_BLOCK = 0


def chain_hash(parent: Optional[bytes], tokens: Sequence[int], salt: bytes = b"") -> bytes:
    """Content hash of one full block given its parent's hash."""
    h = hashlib.blake2b(digest_size=16)
    h.update(parent if parent is not None else b"\x00" * 16)
    h.update(salt)
    h.update(struct.pack(f"<{len(tokens)}I", *tokens))
    return h.digest()


def block_hashes(tokens: Sequence[int], block_size: int, salt: bytes = b"", parent: Optional[bytes] = None) -> list:
    """Hashes of every *full* block of ``tokens``."""
    out = []
    for i in range(0, len(tokens) - block_size + 1, block_size):
        parent = chain_hash(parent, tokens[i : i + block_size], salt)
        out.append(parent)
    return out


@dataclass
class KvEvent:
    kind: str  # "stored" | "removed"
    block_hashes: list
    parent_hash: Optional[bytes] = None


@dataclass
class PoolStats:
    allocations: int = 0
    evictions: int = 0
    prefix_hits: int = 0
    prefix_queries: int = 0
    registered: int = 0
    dedup_drops: int = 0


class OutOfBlocks(RuntimeError):
    pass


class BlockPool:
    def __init__(
        self,
        num_blocks: int,
        block_size: int,
        enable_prefix_cache: bool = True,
        event_sink: Optional[Callable[[KvEvent], None]] = None,
    ):
        if num_blocks < 2:
            raise ValueError("need at least 2 blocks (block 0 is the padding page)")
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.enable_prefix_cache = enable_prefix_cache
        self._free = deque(range(1, num_blocks))
        self._inactive: "OrderedDict[int, None]" = OrderedDict()  # bid -> None, LRU first
        self._ref = [0] * num_blocks
        self._hash: list = [None] * num_blocks
        self._parent: list = [None] * num_blocks
        self._by_hash: dict = {}
        self._event_sink = event_sink
        self.stats = PoolStats()

    # -- capacity ------------------------------------------------------------
    @property
    def usable_blocks(self) -> int:
        return self.num_blocks - 1

    def available(self) -> int:
        """Blocks that an allocation could obtain right now (free + evictable)."""
        return len(self._free) + len(self._inactive)

    def used(self) -> int:
        return self.usable_blocks - self.available()

    def num_inactive(self) -> int:
        return len(self._inactive)

    # -- allocation ----------------------------------------------------------
    def allocate(self, n: int) -> list:
        if n > self.available():
            raise OutOfBlocks(f"need {n} blocks, {self.available()} available")
        out = []
        removed = []
        for _ in range(n):
            if self._free:
                bid = self._free.popleft()
            else:
                bid, _ = self._inactive.popitem(last=False)  # evict LRU
                h = self._hash[bid]
                if h is not None and self._by_hash.get(h) == bid:
                    del self._by_hash[h]
                    removed.append(h)
                self._hash[bid] = None
                self._parent[bid] = None
                self.stats.evictions += 1
            self._ref[bid] = 1
            out.append(bid)
        self.stats.allocations += n
        if removed and self._event_sink:
            self._event_sink(KvEvent("removed", removed))
        return out

    def acquire(self, bid: int) -> None:
        if self._ref[bid] == 0:
            self._inactive.pop(bid, None)
        self._ref[bid] += 1

    def release(self, bids: Iterable[int]) -> None:
        # Release in reverse so the deepest (least shareable) blocks become LRU first.
        for bid in reversed(list(bids)):
            if bid == PADDING_BLOCK:
                continue
            assert self._ref[bid] > 0, f"block {bid} released more often than acquired"
            self._ref[bid] -= 1
            if self._ref[bid] == 0:
                if self._hash[bid] is not None and self.enable_prefix_cache:
                    self._inactive[bid] = None
                    self._inactive.move_to_end(bid)
                else:
                    self._hash[bid] = None
                    self._free.append(bid)

    def free_unregistered_tail(self, bids: Sequence[int]) -> None:
        """LIFO-free blocks that were scheduled but never filled (spec rollback)."""
        for bid in reversed(list(bids)):
            assert self._ref[bid] == 1 and self._hash[bid] is None
            self._ref[bid] = 0
            self._free.appendleft(bid)

    # -- prefix cache ----------------------------------------------------------
    def match_prefix(self, hashes: Sequence[bytes], acquire: bool = True) -> list:
        """Longest run of registered blocks matching ``hashes`` from the start."""
        self.stats.prefix_queries += len(hashes)
        out = []
        if not self.enable_prefix_cache:
            return out
        for h in hashes:
            bid = self._by_hash.get(h)
            if bid is None:
                break
            out.append(bid)
        if acquire:
            for bid in out:
                self.acquire(bid)
        self.stats.prefix_hits += len(out)
        return out

    def probe(self, hashes: Sequence[bytes]) -> int:
        """How many leading blocks are resident, without taking references."""
        n = 0
        for h in hashes:
            if h not in self._by_hash:
                break
            n += 1
        return n

    def register(self, bid: int, h: bytes, parent: Optional[bytes] = None) -> int:
        """Publish a filled block under its hash.  Returns the canonical block id:
        if another block already owns the hash, the caller keeps its own private
        (unregistered) copy and that other id is returned for information."""
        if not self.enable_prefix_cache:
            return bid
        other = self._by_hash.get(h)
        if other is not None and other != bid:
            self.stats.dedup_drops += 1
            return other
        if self._hash[bid] == h:
            return bid
        self._hash[bid] = h
        self._parent[bid] = parent
        self._by_hash[h] = bid
        self.stats.registered += 1
        if self._event_sink:
            self._event_sink(KvEvent("stored", [h], parent))
        return bid

    def block_hash(self, bid: int) -> Optional[bytes]:
        return self._hash[bid]

    def refcount(self, bid: int) -> int:
        return self._ref[bid]

    def evict_inactive(self) -> int:
        """Drop every inactive block (test mode: force host-tier hits)."""
        n = 0
        removed = []
        while self._inactive:
            bid, _ = self._inactive.popitem(last=False)
            h = self._hash[bid]
            if h is not None and self._by_hash.get(h) == bid:
                del self._by_hash[h]
                removed.append(h)
            self._hash[bid] = None
            self._free.append(bid)
            n += 1
        if removed and self._event_sink:
            self._event_sink(KvEvent("removed", removed))
        return n

    # -- reservation for host-tier loads ---------------------------------------
    def reserve(self, n: int, floor: int = 0) -> Optional[list]:
        """Take ``n`` blocks for an incoming host->GPU load, never dipping below
        ``floor`` available blocks (protects in-flight prefills from starvation)."""
        if self.available() - n < floor:
            return None
        return self.allocate(n)

    def commit_reserved(self, bids: Sequence[int], hashes: Sequence[bytes], parent: Optional[bytes]) -> None:
        """Loaded blocks become ordinary prefix-cache entries, then go inactive."""
        for bid, h in zip(bids, hashes):
            self.register(bid, h, parent)
            parent = h
        self.release(bids)

    def check_invariants(self) -> None:
        seen = set(self._free) | set(self._inactive)
        assert len(seen) == len(self._free) + len(self._inactive)
        for bid in range(1, self.num_blocks):
            if self._ref[bid] == 0:
                assert bid in seen, f"block {bid} leaked"
            else:
                assert bid not in seen
        for h, bid in self._by_hash.items():
            assert self._hash[bid] == h
