"""Speculative decoding with a separate, smaller draft model of the same vocabulary.

The draft model keeps its own paged KV buffer with the *same* block ids as the target:
a request's block table addresses both buffers, so the draft needs no allocator of its
own and its cache is rolled back for free (rejected positions are simply overwritten).
Per request the spec tracks how many leading positions of the draft cache are valid.

A round, driven by the scheduler once the verify pages are scheduled:

1. catch-up: every token the target has committed but the draft has not seen yet
   (the whole prompt on the first round, the accepted tokens afterwards) goes through
   the draft as one ragged chunk; its last row yields draft 1;
2. ``k - 1`` single-token draft steps yield drafts 2..k;
3. the target verifies ``[current, d1..dk]`` in one forward and keeps the matching prefix.

Reference parity: pegainfer-qwen3/src/speculative.rs:18-131 (draft config, proposer
contract), src/executor.rs execute_speculative_draft, docs: "k draft steps, one verify".
"""
from __future__ import annotations

import torch

from .. import ops
from ..sched.executor import SeqStep, build_meta


def load_draft_model(ecfg, model):
    """The draft model of ``--draft-model-path``: a checkpoint directory, or ``preset:NAME``
    for a random-init model of a named shape (benchmarks, tests).  Same device, dtype and
    tensor-parallel context as the target; the vocabularies must agree."""
    from ..config import EngineConfig, load_model_config, preset
    from ..engine.build import build_model

    path = ecfg.draft_model_path
    if not path:
        raise ValueError("--spec-method draft needs --draft-model-path")
    if path.startswith("preset:"):
        # preset:NAME[:seed=K]: random weights of a named shape; the default seed differs from the target's
        parts = path.split(":")
        seed = next((int(p[5:]) for p in parts[2:] if p.startswith("seed=")), ecfg.seed + 1)
        dcfg = preset(parts[1])
        decfg = EngineConfig(preset=parts[1], seed=seed)
    else:
        dcfg = load_model_config(path)
        decfg = EngineConfig(model_path=path, seed=ecfg.seed)
    if dcfg.vocab_size != model.cfg.vocab_size:
        raise ValueError(f"draft vocabulary ({dcfg.vocab_size}) differs from the target's ({model.cfg.vocab_size})")
    return build_model(dcfg, decfg, model.device, model.dtype, getattr(model, "tp", None) or _single())


def _single():
    from ..parallel.tp import TPContext

    return TPContext()


def _num_pages(kv) -> int:
    for holder in (kv, getattr(kv, "layout", None)):
        n = getattr(holder, "num_pages", None)
        if n is not None:
            return int(n)
    raise ValueError("cannot size the draft KV buffer: the target KV buffer does not expose num_pages")


def _make_kv(model, num_pages: int, page_size: int):
    if hasattr(model, "make_kv"):
        return model.make_kv(num_pages, page_size)
    from ..kv.buffer import KvBuffer, KvLayout

    return KvBuffer(KvLayout(page_size=page_size, num_pages=num_pages, dtype=model.dtype, **model.kv_geometry()), model.device)


class DraftModelSpec:
    allows_prefix_cache = False
    kind = "draft"

    def __init__(self, ecfg, model, executor, draft_model=None):
        self.draft_len = max(1, int(ecfg.spec_draft_len))
        if draft_model is None:
            draft_model = getattr(model, "draft_model", None) or load_draft_model(ecfg, model)
        self.draft = draft_model
        self.page_size = executor.page_size
        self.device = model.device
        self.kv = _make_kv(draft_model, _num_pages(executor.kv), executor.page_size)
        self.chunk = max(16, int(getattr(ecfg, "max_prefill_tokens", 1024)))
        self.valid: dict = {}  # rid -> leading positions of the draft cache that hold committed tokens
        self.draft_forwards = 0

    def ready(self, r) -> bool:
        req = r.q.request
        return r.phase == "decode" and req.logprobs == 0 and req.params.temperature < 1e-5 and r.lora_slot < 0

    def release(self, rid: int) -> None:
        self.valid.pop(rid, None)

    def _forward_last(self, seqs) -> list:
        """One draft forward over ragged ``seqs``; greedy token after each sequence's last row."""
        token_ids, meta = build_meta(seqs, self.page_size, self.device)
        hidden = self.draft.forward_hidden(token_ids, meta, self.kv)
        rows = [meta.h_q_indptr[i + 1] - 1 for i in range(len(seqs))]
        idx = torch.tensor(rows, dtype=torch.int32, device=self.device)
        self.draft_forwards += 1
        return ops.argmax(self.draft.logits(hidden, idx)).tolist()

    def propose(self, decoders) -> dict:
        """``rid -> [d1..dk]``.  Every request's view must already cover ``committed + 1 + k`` positions."""
        k = self.draft_len
        drafts = {r.q.id: [] for r in decoders}
        # 1. catch-up, in slices no longer than the prefill chunk budget
        pending = []
        for r in decoders:
            rid = r.q.id
            have = min(self.valid.get(rid, 0), r.kv.committed)
            pending.append([r, have])
        last_tok = {}
        while pending:
            seqs, budget, nxt = [], self.chunk, []
            for ent in pending:
                r, have = ent
                todo = r.kv.committed + 1 - have
                n = min(todo, budget) if seqs else min(todo, max(budget, 1))
                if n <= 0:
                    nxt.append(ent)
                    continue
                seqs.append(SeqStep(rid=r.q.id, input_tokens=r.kv.tokens[have : have + n], start_pos=have, view=r.kv.view()))
                budget -= n
                ent[1] = have + n
                if ent[1] < r.kv.committed + 1:
                    nxt.append(ent)
            toks = self._forward_last(seqs)
            for s, t in zip(seqs, toks):
                last_tok[s.rid] = t
            pending = nxt
        for r in decoders:
            drafts[r.q.id].append(last_tok[r.q.id])
        # 2. k - 1 single-token steps
        for j in range(1, k):
            seqs = [SeqStep(rid=r.q.id, input_tokens=[drafts[r.q.id][-1]], start_pos=r.kv.committed + j, view=r.kv.view()) for r in decoders]
            toks = self._forward_last(seqs)
            for r, t in zip(decoders, toks):
                drafts[r.q.id].append(t)
        for r in decoders:
            # positions committed+1 .. committed+k-1 now hold d1..d(k-1); they stay valid as far as the target accepts them
            self.valid[r.q.id] = r.kv.committed + k
        return drafts
