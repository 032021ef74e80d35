"""Data-parallel attention with expert-parallel MoE: ranks in lock-step.

Each rank owns its own requests, KV pool and scheduler (attention weights are
replicated), while routed experts are spread over the ranks.  Every MoE layer is a
collective, so every rank must run every forward pass with the same token bucket:

* ``LockstepExecutor`` wraps a rank's executor.  Before each forward pass the ranks
  agree (one small host all-reduce, MAX) on the number of token rows; a rank with fewer
  rows pads with inert rows (padding sequences on page 0), a rank with nothing to do
  runs a pure padding step.  Padding rows route to no expert.
* ``DpScheduler`` makes sure a rank whose scheduler had no work this iteration still
  joins the agreement (``idle_step``), so iterations stay aligned across ranks.
* ``pick_rank`` routes a new request to the rank with the most free decode slots.

A rank that fails between steps is noticed on the host: the agreement all-reduce uses
a short process-group timeout and raises on the surviving ranks, which fail their
running requests instead of hanging inside a device-side collective.

Reference parity: pegainfer-kimi-k2/src/runner/scheduler/dp.rs:33-53,229-287,764-795
(coordinator, synchronized step, padding commands), runner/load_balancer.rs:13-21,
dp.rs:1014-1037 (fail-stop on a lost rank).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kv.request_kv import KvView
from ..sched.executor import ModelExecutor, SeqStep, StepBatch, StepResult, TorchExecutor, build_meta
from ..sched.scheduler import ContinuousScheduler


def pick_rank(free_slots: list) -> int:
    """Rank with the most free decode slots (ties: lowest rank)."""
    best = 0
    for i, f in enumerate(free_slots):
        if f > free_slots[best]:
            best = i
    return best


class LockstepExecutor(ModelExecutor):
    def __init__(self, inner: TorchExecutor, group=None, world: int = 1):
        self.inner = inner
        self.group = group
        self.world = world
        self.vocab_size = inner.vocab_size
        self.calls = 0
        self.padding_steps = 0
        self.device = inner.device
        self.mtp = None

    def _agree(self, rows: int) -> int:
        if self.world <= 1:
            return rows
        import torch.distributed as dist

        t = torch.tensor([rows], dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return int(t.item())

    def _bucket(self, rows: int) -> int:
        b = 16
        while b < rows:
            b *= 2
        return b

    def execute(self, batch: StepBatch) -> StepResult:
        self.calls += 1
        rows = batch.num_tokens
        target = self._bucket(self._agree(rows))
        return self._run(batch.seqs, target)

    def idle_step(self) -> bool:
        """Join the agreement with no work; runs a padding forward if any rank has work."""
        self.calls += 1
        target = self._agree(0)
        if target == 0:
            return False
        self.padding_steps += 1
        self._run([], self._bucket(target))
        return True

    def _run(self, seqs, target_rows: int) -> StepResult:
        ex = self.inner
        n_rows = sum(len(s.input_tokens) for s in seqs)
        pad_seqs = target_rows - n_rows
        token_ids, meta = build_meta(seqs, ex.page_size, ex.device, pad_to=len(seqs) + pad_seqs) if seqs else self._padding_meta(target_rows)
        ep = getattr(ex.model, "ep", None)
        if ep is not None and hasattr(ep, "valid_tokens"):
            ep.valid_tokens = torch.tensor([n_rows], dtype=torch.int32, device=ex.device)
        ex.prepare_meta(seqs, meta)
        hidden = ex.model.forward_hidden(token_ids, meta, ex.kv)
        res = StepResult()
        rows, per, owners = [], [], []
        for i, s in enumerate(seqs):
            if not s.sample:
                continue
            q0, q1 = meta.h_q_indptr[i], meta.h_q_indptr[i + 1]
            r = list(range(q0, q1)) if s.all_rows else [q1 - 1]
            rows.extend(r)
            per.append(len(r))
            owners.append(s)
        if rows:
            idx = torch.tensor(rows, dtype=torch.int32, device=ex.device)
            logits = ex.model.logits(hidden, idx)
            toks, lps = ex._sample(logits, owners, per)
            toks = toks.tolist()
            k = 0
            for s, n in zip(owners, per):
                res.tokens[s.rid] = toks[k : k + n]
                if lps is not None and s.logprobs > 0:
                    res.logprobs[s.rid] = lps[k : k + n]
                k += n
        return res

    def _padding_meta(self, rows: int):
        pad = [SeqStep(rid=-1, input_tokens=[0], start_pos=0, view=KvView([0], 1, self.inner.page_size), sample=False)]
        tok, meta = build_meta(pad, self.inner.page_size, self.inner.device, pad_to=rows)
        # the single "real" row is padding too: it writes into page 0 and is never read
        return tok, meta

    def release_request(self, rid: int) -> None:
        self.inner.release_request(rid)


class DpScheduler(ContinuousScheduler):
    """A scheduler partition that keeps its rank in lock-step with the others."""

    def step(self, ledger) -> bool:
        before = self.ex.calls
        busy = super().step(ledger)
        if self.ex.calls == before:
            busy = self.ex.idle_step() or busy
        return busy
