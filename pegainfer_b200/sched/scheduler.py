"""Continuous-batching scheduler over the paged KV pool.

One ``step``: retire aborted requests, admit waiting requests whose *whole lifetime*
of KV blocks fits (so a running request can never be starved mid-flight), carve up
to ``max_prefill_tokens`` of prompt chunks (FIFO), choose a plan and run it:

========  ==========================================================
Prefill   prompt chunks only
Decode    one token for every running request (CUDA-graph path)
Unified   prompt chunks and decode rows in one ragged forward
Spec      draft + verify round when every running request is draft-ready
========  ==========================================================

then resolve the sampled tokens into ledger writes (stop tokens, ``max_tokens``).
A failing executor call fails only the requests in that batch; the engine keeps
serving.

Reference parity: pegainfer-qwen3/src/scheduler.rs:99-133 (take_prefill_chunks),
:300-353,407-493 (admission, full-lifetime reservation), :499-535 (plan + failure
containment), src/scheduler/plan.rs:22-243, src/scheduler/resolve.rs:46-150
(finish rules), src/frontend_adapter.rs:594-784 (step order).
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from ..engine.contract import (
    FinishReason,
    PromptEcho,
    QueuedRequest,
    RejectReason,
    SchedulerMetrics,
)
from ..kv.block_pool import BlockPool, OutOfBlocks
from ..kv.request_kv import RequestKv, blocks_for
from .executor import ModelExecutor, SeqStep, StepBatch


@dataclass
class SchedulerConfig:
    max_prefill_tokens: int = 1024
    max_decode_batch: int = 256
    max_model_len: int = 4096
    max_blocks_per_request: Optional[int] = None
    eos_token_ids: tuple = ()
    batch_invariant: bool = False
    vocab_size: int = 0
    decode_overlap: bool = False  # prompt chunks run on a second stream while decode steps continue
    run_ahead: bool = False  # a decode step launches the following one before its tokens are read


class _Running:
    __slots__ = ("q", "kv", "prefill_pos", "out_tokens", "step_index", "phase", "echo_done", "t_first", "spec_ready", "lora_slot", "state_slot", "report_cached", "spec_state", "inflight")

    def __init__(self, q: QueuedRequest, kv: RequestKv):
        self.q = q
        self.kv = kv
        self.prefill_pos = 0
        self.out_tokens = 0
        self.step_index = 0
        self.phase = "prefill"  # prefill | decode
        self.echo_done = False
        self.t_first = None
        self.spec_ready = False
        self.lora_slot = -1
        self.state_slot = -1
        self.report_cached = None
        self.spec_state = None
        self.inflight = False  # a prompt chunk of this request is executing on the prefill lane


def plan_kind(has_prefill: bool, has_decode: bool, spec_ready: bool) -> Optional[str]:
    """Plan truth table (pegainfer-qwen3/src/scheduler/plan.rs:51-82)."""
    if has_prefill and has_decode:
        return "unified"
    if has_prefill:
        return "prefill"
    if has_decode:
        return "spec" if spec_ready else "decode"
    return None


class ContinuousScheduler:
    def __init__(self, executor: ModelExecutor, pool: BlockPool, cfg: SchedulerConfig, spec=None, host_tier=None, lora_registry=None, tracer=None):
        self.ex = executor
        self.pool = pool
        self.cfg = cfg
        self.spec = spec
        self._lane = None  # (chunks, pending) of the prompt chunks running on the executor's second stream
        self._ahead = bool(cfg.run_ahead) and spec is None and bool(getattr(executor, "supports_run_ahead", False))
        self.overlapped_chunks = 0
        self.host_tier = host_tier
        self.lora = lora_registry
        self.tracer = tracer
        self.waiting: deque = deque()
        self.parked: dict = {}  # rid -> (QueuedRequest, prefetch state)
        self.running: dict = {}  # rid -> _Running (insertion order = admission order)
        self._metrics = SchedulerMetrics(kv_total_blocks=pool.usable_blocks)
        self.steps = 0
        self.failed_batches = 0

    # -- contract ----------------------------------------------------------------
    def submit(self, q: QueuedRequest) -> None:
        self.waiting.append(q)
        if self.tracer:
            self.tracer.enter_queue(q)

    def metrics(self) -> SchedulerMetrics:
        m = self._metrics
        m.kv_used_blocks = self.pool.used()
        m.kv_total_blocks = self.pool.usable_blocks
        m.num_running_reqs = len(self.running)
        m.num_waiting_reqs = len(self.waiting) + len(self.parked)
        m.prefix_hit_tokens = self.pool.stats.prefix_hits * self.pool.block_size
        m.prefix_query_tokens = self.pool.stats.prefix_queries * self.pool.block_size
        return m

    # -- admission ---------------------------------------------------------------
    def _lifetime_blocks(self, prompt_len: int, max_tokens: int) -> int:
        total = min(prompt_len + max_tokens, self.cfg.max_model_len)
        if self.spec is not None:  # a verify step schedules the current token plus the drafts past the last output
            total += 1 + int(getattr(self.spec, "draft_len", 1))
        return blocks_for(total, self.pool.block_size)

    def _future_blocks(self) -> int:
        n = 0
        for r in self.running.values():
            need = self._lifetime_blocks(r.kv.prompt_len, r.q.request.max_tokens)
            n += max(0, need - len(r.kv.blocks))
        return n

    def _validate(self, q: QueuedRequest, ledger) -> bool:
        req = q.request
        n = len(req.prompt_tokens)
        if n == 0:
            ledger.reject(q.id, RejectReason.EMPTY_PROMPT, "prompt has no tokens")
            return False
        if n >= self.cfg.max_model_len:
            ledger.reject(q.id, RejectReason.PROMPT_TOO_LONG, f"prompt of {n} tokens does not fit the {self.cfg.max_model_len}-token context")
            return False
        if self.cfg.vocab_size and any((t < 0 or t >= self.cfg.vocab_size) for t in req.prompt_tokens):
            ledger.reject(q.id, RejectReason.INVALID_TOKEN, "prompt token id outside the vocabulary")
            return False
        need = self._lifetime_blocks(n, req.max_tokens)
        cap = self.cfg.max_blocks_per_request or self.pool.usable_blocks
        if need > min(cap, self.pool.usable_blocks):
            ledger.reject(q.id, RejectReason.KV_CAPACITY, f"request needs {need} KV blocks, limit is {min(cap, self.pool.usable_blocks)}")
            return False
        if req.lora_adapter is not None and (self.lora is None or not self.lora.has(req.lora_adapter)):
            ledger.reject(q.id, RejectReason.UNKNOWN_LORA, f"LoRA adapter {req.lora_adapter!r} is not loaded")
            return False
        return True

    def _admit(self, ledger) -> None:
        budget = self.pool.available() - self._future_blocks()
        while self.waiting and len(self.running) < self.cfg.max_decode_batch:
            q = self.waiting[0]
            if q.is_aborted():
                self.waiting.popleft()
                ledger.finish(q.id, FinishReason.ABORT)
                continue
            if not self._validate(q, ledger):
                self.waiting.popleft()
                continue
            if self.host_tier is not None and self.host_tier.should_park(q, self):
                self.waiting.popleft()
                self.parked[q.id] = q
                continue
            need = self._lifetime_blocks(len(q.request.prompt_tokens), q.request.max_tokens)
            if need > budget:
                break  # FIFO: do not let small requests starve a big one
            self.waiting.popleft()
            budget -= need
            salt = b""
            if q.request.lora_adapter:
                salt += b"lora:" + q.request.lora_adapter.encode()
            if q.request.cache_salt:
                salt += b"salt:" + q.request.cache_salt.encode()
            r = _Running(q, RequestKv(self.pool, q.request.prompt_tokens, salt))
            if self.lora is not None and q.request.lora_adapter:
                r.lora_slot = self.lora.slot_of(q.request.lora_adapter)
            self.running[q.id] = r
            ledger.mark_scheduled(q.id, len(q.request.prompt_tokens))
            if self.tracer:
                self.tracer.enter_prefill(q)

    def _unpark_ready(self) -> None:
        if self.host_tier is None or not self.parked:
            return
        for rid in self.host_tier.drain_ready(self):
            q = self.parked.pop(rid, None)
            if q is not None:
                self.waiting.appendleft(q)

    # -- retirement --------------------------------------------------------------
    def _retire(self, rid: int) -> None:
        r = self.running.pop(rid, None)
        if r is not None:
            if self.host_tier is not None:
                self.host_tier.on_retire(r, self)
            r.kv.release()
            self.ex.release_request(rid)
            if self.spec is not None and hasattr(self.spec, "release"):
                self.spec.release(rid)
            if self.tracer:
                self.tracer.finish(r.q)

    def _reap_aborted(self, ledger) -> None:
        for rid in [rid for rid, r in self.running.items() if r.q.is_aborted() and not r.inflight]:  # pages of an in-flight chunk are still being written
            ledger.finish(rid, FinishReason.ABORT)
            self._retire(rid)
        for rid in [rid for rid, q in self.parked.items() if q.is_aborted()]:
            ledger.finish(rid, FinishReason.ABORT)
            self.parked.pop(rid)
            if self.host_tier is not None:
                self.host_tier.cancel(rid)

    # -- chunking ----------------------------------------------------------------
    def take_prefill_chunks(self) -> list:
        """FIFO prompt chunks within the per-step token budget: ``[(running, n)]``."""
        budget = self.cfg.max_prefill_tokens
        out = []
        for r in self.running.values():
            if r.phase != "prefill" or budget <= 0 or r.inflight:
                continue
            if r.prefill_pos == 0 and r.kv.committed == 0 and not r.kv.blocks:
                cached = r.kv.match_and_add_prefix() if (self.spec is None or self.spec.allows_prefix_cache) else 0
                r.prefill_pos = cached
                r.report_cached = cached
            remaining = r.kv.prompt_len - r.prefill_pos
            n = min(remaining, budget)
            if n <= 0:
                continue
            out.append((r, n))
            budget -= n
            if self.cfg.batch_invariant:
                break  # request-local prefill keeps reduction shapes fixed
        return out

    # -- step ----------------------------------------------------------------------
    def _chunk_steps(self, chunks) -> list:
        """Schedule the KV of every chunk and describe it as executor input."""
        seqs = []
        for r, n in chunks:
            r.kv.schedule_prefill(n)
            last = r.prefill_pos + n == r.kv.prompt_len
            seqs.append(
                SeqStep(
                    rid=r.q.id,
                    input_tokens=r.kv.tokens[r.prefill_pos : r.prefill_pos + n],
                    start_pos=r.prefill_pos,
                    view=r.kv.view(),
                    sample=last,
                    params=r.q.request.params,
                    step_index=0,
                    logprobs=r.q.request.logprobs if last else 0,
                    lora_slot=r.lora_slot,
                    fresh_state=r.prefill_pos == 0,
                    next_token=-1 if last else r.kv.tokens[r.prefill_pos + n],
                )
            )
        return seqs

    def _resolve_chunks(self, chunks, result, ledger) -> None:
        for r, n in chunks:
            rid = r.q.id
            if rid not in self.running:
                continue
            r.kv.apply_prefill_chunk()
            if r.report_cached is not None:  # once, with the first chunk
                ledger.report_cached_tokens(rid, r.report_cached)
                r.report_cached = None
            r.prefill_pos += n
            if r.prefill_pos == r.kv.prompt_len:
                r.phase = "decode"
                if self.tracer:
                    self.tracer.enter_decode(r.q)
                if r.q.request.echo and not r.echo_done:
                    ledger.push_prompt_echo(rid, PromptEcho(tokens=list(r.q.request.prompt_tokens), logprobs=[None] * r.kv.prompt_len))
                    r.echo_done = True
                tok = result.tokens[rid][0]
                lp = result.logprobs.get(rid)
                r.spec_state = result.drafts.get(rid)
                self._resolve_token(r, tok, lp[0] if lp else None, ledger, first=True)
            if self.host_tier is not None and rid in self.running:
                self.host_tier.on_blocks_sealed(r, self)

    # -- prefill lane (decode overlap) ---------------------------------------------
    def _poll_lane(self, ledger, wait: bool = False) -> None:
        """Collect the prompt chunks that were running beside the decode steps, if they are done."""
        if self._lane is None:
            return
        chunks, pending = self._lane
        try:
            result = self.ex.finish_async(pending, wait=wait)
        except Exception as exc:
            self._lane = None
            self.failed_batches += 1
            for r, _ in chunks:
                r.inflight = False
            self._fail_batch([r for r, _ in chunks], ledger, f"step failed: {exc!r}")
            return
        if result is None:
            return
        self._lane = None
        for r, _ in chunks:
            r.inflight = False
        self._resolve_chunks(chunks, result, ledger)

    def _lane_accepts(self, chunks) -> bool:
        # the lane samples greedily on the device and returns tokens only
        for r, n in chunks:
            req = r.q.request
            if r.lora_slot >= 0 or req.logprobs or not req.params.effectively_greedy(self.cfg.vocab_size or (1 << 30)):
                return False
        return hasattr(self.ex, "launch_async")

    # -- step ----------------------------------------------------------------------
    def step(self, ledger) -> bool:
        self.steps += 1
        self._poll_lane(ledger)
        self._reap_aborted(ledger)
        if self.host_tier is not None:
            self.host_tier.poll(self)
            self._unpark_ready()
        self._admit(ledger)
        chunks = self.take_prefill_chunks() if self._lane is None else []  # one set of chunks on the lane at a time
        decoders = [r for r in self.running.values() if r.phase == "decode"]
        if self._lane is not None and not decoders:
            self._poll_lane(ledger, wait=True)  # nothing to overlap with: wait for the lane
            return True
        if self.cfg.decode_overlap and chunks and decoders and self.spec is None and self._lane_accepts(chunks):
            # Decode overlap: the prompt chunks go to the executor's second stream and this step
            # continues as a pure decode step, so running requests keep their token cadence while
            # a long prompt is being processed.
            try:
                pending = self.ex.launch_async(StepBatch(seqs=self._chunk_steps(chunks), kind="prefill"))
            except OutOfBlocks as exc:
                self._fail_batch([r for r, _ in chunks], ledger, f"KV pool exhausted: {exc}")
                return True
            except Exception as exc:
                self.failed_batches += 1
                self._fail_batch([r for r, _ in chunks], ledger, f"step failed: {exc!r}")
                return True
            for r, _ in chunks:
                r.inflight = True
            self._lane = (chunks, pending)
            self.overlapped_chunks += len(chunks)
            chunks = []
        spec_ready = self.spec is not None and bool(decoders) and not chunks and all(self.spec.ready(r) for r in decoders)
        kind = plan_kind(bool(chunks), bool(decoders), spec_ready)
        if kind is None:
            return self._lane is not None
        if kind == "spec":
            self._run_spec(decoders, ledger)
            return True
        seqs, touched = [], []
        try:
            seqs.extend(self._chunk_steps(chunks))
            touched.extend(r for r, _ in chunks)
            ahead = self._ahead
            for r in decoders:
                # run-ahead: the page of the next position exists before this step is applied, and a
                # request whose length limit this step reaches is marked so nothing runs ahead for it
                final = ahead and (r.out_tokens + 1 >= r.q.request.max_tokens or r.kv.committed + 2 >= self.cfg.max_model_len)
                r.kv.schedule_decode(1 if ahead and not final else 0)
                seqs.append(
                    SeqStep(
                        rid=r.q.id,
                        input_tokens=[r.kv.tokens[-1]],
                        start_pos=r.kv.committed,
                        view=r.kv.view(),
                        sample=True,
                        params=r.q.request.params,
                        step_index=r.step_index,
                        logprobs=r.q.request.logprobs,
                        lora_slot=r.lora_slot,
                        table_pages=r.kv.blocks if ahead else None,
                        final=final,
                    )
                )
                touched.append(r)
        except OutOfBlocks as exc:  # cannot happen with lifetime reservation; fail safe
            self._fail_batch(touched, ledger, f"KV pool exhausted: {exc}")
            return True
        try:
            result = self.ex.execute(StepBatch(seqs=seqs, kind=kind, run_ahead=self._ahead and kind == "decode"))
        except Exception as exc:
            self.failed_batches += 1
            self._fail_batch(touched, ledger, f"step failed: {exc!r}")
            return True
        # resolve
        self._resolve_chunks(chunks, result, ledger)
        for r in decoders:
            rid = r.q.id
            if rid not in self.running:
                continue
            tok = result.tokens[rid][0]
            lp = result.logprobs.get(rid)
            r.kv.apply_decode(tok)
            r.step_index += 1
            r.spec_state = result.drafts.get(rid)
            self._resolve_token(r, tok, lp[0] if lp else None, ledger, first=False, appended=True)
            if self.host_tier is not None and rid in self.running:
                self.host_tier.on_blocks_sealed(r, self)
        return True

    def _fail_batch(self, touched, ledger, message: str) -> None:
        for r in touched:
            rid = r.q.id
            if rid in self.running:
                try:
                    r.kv.revert_schedule()
                except AssertionError:
                    pass
                ledger.fail(rid, message)
                self._retire(rid)

    def _is_stop(self, r: _Running, tok: int) -> bool:
        p = r.q.request.params
        if tok in p.stop_token_ids:
            return True
        return (not p.ignore_eos) and tok in self.cfg.eos_token_ids

    def _resolve_token(self, r: _Running, tok: int, lp, ledger, first: bool, appended: bool = False) -> None:
        """Finish rules: a stop token is never emitted; ``max_tokens`` ends with Length."""
        rid = r.q.id
        req = r.q.request
        if first:
            # the token sampled at the end of the prompt used request-local step 0: the first decode
            # step must draw with step 1, or a seeded request would reuse one random number
            r.step_index += 1
        if self._is_stop(r, tok):
            ledger.finish(rid, FinishReason.STOP)
            self._retire(rid)
            return
        if not appended:
            r.kv.push_token(tok)
        ledger.push_tokens(rid, [tok], [lp] if lp is not None else None)
        r.out_tokens += 1
        if r.t_first is None:
            r.t_first = time.monotonic()
        if r.out_tokens >= req.max_tokens or r.kv.committed + 1 >= self.cfg.max_model_len:
            if self.host_tier is not None and self.host_tier.flush_on_finish:
                # prefill side of a disaggregated pair: the finish is the peer's cue to look the blocks up,
                # so it goes out only once they have landed in the shared store
                self.host_tier.on_blocks_sealed(r, self)
                self.host_tier.flush_saves_then(lambda: None)
            ledger.finish(rid, FinishReason.LENGTH)
            self._retire(rid)

    # -- speculative round -----------------------------------------------------------
    def _run_spec(self, decoders, ledger) -> None:
        """One verify round: feed ``[current, drafts...]``, keep the matching prefix."""
        from ..spec.speculative import accept_prefix_match

        seqs = []
        propose = getattr(self.spec, "propose", None)
        on_accept = getattr(self.spec, "on_accept", None)
        all_drafts = {}
        try:
            if propose is not None:
                # a separate draft model: schedule the verify pages first, the drafts are written at the same positions
                for r in decoders:
                    r.kv.schedule_speculative(1 + self.spec.draft_len)
                all_drafts = propose(decoders)
            for r in decoders:
                if propose is None:
                    all_drafts[r.q.id] = list(r.spec_state)
                    r.kv.schedule_speculative(1 + len(all_drafts[r.q.id]))
                drafts = all_drafts[r.q.id]
                seqs.append(
                    SeqStep(rid=r.q.id, input_tokens=[r.kv.tokens[-1]] + drafts, start_pos=r.kv.committed, view=r.kv.view(), sample=True, params=r.q.request.params, step_index=r.step_index, all_rows=True)
                )
            result = self.ex.execute(StepBatch(seqs=seqs, kind="verify"))
        except Exception as exc:
            self.failed_batches += 1
            self._fail_batch(decoders, ledger, f"speculative step failed: {exc!r}")
            return
        for r in decoders:
            rid = r.q.id
            drafts = all_drafts[rid]
            accepted = accept_prefix_match(drafts, result.tokens[rid])
            self._metrics.spec_decode.record(len(drafts), len(accepted) - 1)
            r.kv.apply_speculative(len(accepted), accepted)
            if on_accept is not None:
                on_accept(rid, len(accepted))
            nd = result.drafts.get(rid)
            r.spec_state = [nd[len(accepted) - 1]] if nd else None
            emitted, finished = [], None
            for tok in accepted:
                if self._is_stop(r, tok):
                    finished = FinishReason.STOP
                    break
                emitted.append(tok)
                if r.out_tokens + len(emitted) >= r.q.request.max_tokens or r.kv.committed + 1 >= self.cfg.max_model_len:
                    finished = FinishReason.LENGTH
                    break
            if emitted:
                ledger.push_tokens(rid, emitted)
                r.out_tokens += len(emitted)
                r.step_index += len(emitted)
            if finished is not None:
                ledger.finish(rid, finished)
                self._retire(rid)
