"""Per-request KV bookkeeping over a :class:`BlockPool`.

Lifecycle (all positions are token counts):

``match_and_add_prefix`` -> ``schedule_prefill(n)`` -> ``prefill_view`` ->
``apply_prefill_chunk`` ... -> ``schedule_decode`` -> ``decode_view`` ->
``apply_decode(token)`` ..., or the speculative triple ``schedule_speculative(k)``
/ ``apply_speculative(accepted)`` / ``revert_schedule``; finally ``release``.

``schedule_*`` makes pages exist for tokens about to be written; ``apply_*``
commits the tokens, registering every block that became full so later requests
can share it.  A prefix match always leaves at least one prompt token to compute,
because the forward pass must produce logits for the last prompt position.

Reference parity: pegainfer-kv-cache/src/pool.rs:330-620 (RequestKv),
src/view.rs:12-101 (KvView), kvbm/kvbm-logical/src/integrations/scheduled.rs:380-839.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

from .block_pool import BlockPool, chain_hash


@dataclass
class KvView:
    page_indices: list
    seq_len: int
    page_size: int

    @property
    def last_page_len(self) -> int:
        if self.seq_len == 0:
            return 0
        r = self.seq_len % self.page_size
        return r if r else self.page_size

    def slot_of(self, pos: int) -> int:
        return self.page_indices[pos // self.page_size] * self.page_size + pos % self.page_size


def blocks_for(tokens: int, block_size: int) -> int:
    return (tokens + block_size - 1) // block_size


class RequestKv:
    def __init__(self, pool: BlockPool, prompt: Sequence[int], salt: bytes = b""):
        self.pool = pool
        self.bs = pool.block_size
        self.tokens = list(prompt)  # committed tokens (prompt prefix being filled + outputs)
        self.prompt_len = len(prompt)
        self.salt = salt
        self.blocks: list = []
        self.committed = 0  # tokens whose KV is written
        self.scheduled = 0  # tokens with pages reserved (>= committed)
        self.cached_tokens = 0
        self._registered_blocks = 0
        self._last_hash: Optional[bytes] = None
        self._sched_new_blocks: list = []
        self.released = False

    # -- prefix ----------------------------------------------------------------
    def match_and_add_prefix(self) -> int:
        """Attach the longest cached prefix; returns cached token count."""
        assert self.committed == 0 and not self.blocks
        max_blocks = (self.prompt_len - 1) // self.bs  # leave >= 1 token uncached
        if max_blocks <= 0:
            return 0
        hashes = []
        parent = None
        for i in range(max_blocks):
            parent = chain_hash(parent, self.tokens[i * self.bs : (i + 1) * self.bs], self.salt)
            hashes.append(parent)
        hit = self.pool.match_prefix(hashes)
        self.blocks = list(hit)
        n = len(hit)
        self.committed = self.scheduled = n * self.bs
        self.cached_tokens = self.committed
        self._registered_blocks = n
        self._last_hash = hashes[n - 1] if n else None
        return self.cached_tokens

    def prefix_hashes(self) -> list:
        """Hashes of all cacheable prompt blocks (for host-tier probes)."""
        max_blocks = (self.prompt_len - 1) // self.bs
        out, parent = [], None
        for i in range(max_blocks):
            parent = chain_hash(parent, self.tokens[i * self.bs : (i + 1) * self.bs], self.salt)
            out.append(parent)
        return out

    # -- scheduling --------------------------------------------------------------
    def blocks_needed(self, new_tokens: int) -> int:
        return max(0, blocks_for(self.committed + new_tokens, self.bs) - len(self.blocks))

    def _schedule(self, n: int, lookahead: int = 0) -> None:
        assert self.scheduled == self.committed, "previous schedule not applied or reverted"
        need = self.blocks_needed(n + lookahead)
        new = self.pool.allocate(need) if need else []
        self.blocks.extend(new)
        self._sched_new_blocks = new
        self.scheduled = self.committed + n

    def schedule_prefill(self, n: int) -> None:
        assert self.committed + n <= self.prompt_len
        self._schedule(n)

    def schedule_decode(self, lookahead: int = 0) -> None:
        """Pages for the token fed this step; with ``lookahead`` also for that many positions
        after it, so that the following step can be launched before this one is applied."""
        self._schedule(1, lookahead)

    def schedule_speculative(self, k: int) -> None:
        self._schedule(k)

    def revert_schedule(self) -> None:
        if self._sched_new_blocks:
            self.pool.free_unregistered_tail(self._sched_new_blocks)
            del self.blocks[len(self.blocks) - len(self._sched_new_blocks) :]
        self._sched_new_blocks = []
        self.scheduled = self.committed

    # -- views -------------------------------------------------------------------
    def view(self) -> KvView:
        """Pages covering every scheduled token (exactly, no spare pages)."""
        n = blocks_for(self.scheduled, self.bs)
        # the common case (every block is scheduled) hands out the list itself: views are
        # transient, consumed within the step that asked for them
        return KvView(self.blocks if n == len(self.blocks) else self.blocks[:n], self.scheduled, self.bs)

    prefill_view = view
    decode_view = view

    def step_page_indices(self) -> list:
        return self.blocks[: blocks_for(self.scheduled, self.bs)]

    # -- apply -------------------------------------------------------------------
    def _register_full_blocks(self) -> None:
        full = self.committed // self.bs
        while self._registered_blocks < full:
            i = self._registered_blocks
            h = chain_hash(self._last_hash, self.tokens[i * self.bs : (i + 1) * self.bs], self.salt)
            self.pool.register(self.blocks[i], h, self._last_hash)
            self._last_hash = h
            self._registered_blocks += 1

    def apply_prefill_chunk(self, n: Optional[int] = None) -> None:
        n = self.scheduled - self.committed if n is None else n
        assert self.committed + n == self.scheduled
        self.committed = self.scheduled
        self._sched_new_blocks = []
        self._register_full_blocks()

    def push_token(self, token: int) -> None:
        """Record a sampled token whose KV is not written yet (end of prefill)."""
        self.tokens.append(token)

    def apply_decode(self, token: int) -> None:
        """KV of the token fed this step is written; ``token`` is the new sample."""
        assert self.scheduled == self.committed + 1
        self.committed = self.scheduled
        self._sched_new_blocks = []
        self.tokens.append(token)
        self._register_full_blocks()

    def apply_speculative(self, accepted_inputs: int, new_tokens: Sequence[int]) -> None:
        """Keep the KV of the first ``accepted_inputs`` scheduled positions, free the
        rest (LIFO), and append ``new_tokens`` to the token history."""
        assert self.committed + accepted_inputs <= self.scheduled
        keep_tokens = self.committed + accepted_inputs
        keep_blocks = blocks_for(keep_tokens, self.bs)
        extra = self.blocks[keep_blocks:]
        if extra:
            self.pool.free_unregistered_tail(extra)
            del self.blocks[keep_blocks:]
        self.committed = self.scheduled = keep_tokens
        self._sched_new_blocks = []
        self.tokens.extend(new_tokens)
        self._register_full_blocks()

    # -- teardown ----------------------------------------------------------------
    def release(self) -> None:
        if self.released:
            return
        self.released = True
        self.pool.release(self.blocks)
        self.blocks = []

    @property
    def seq_len(self) -> int:
        return self.committed
