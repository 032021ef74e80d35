"""EAGLE-3 drafter: one decoder layer over (next token, target feature) pairs, drafting a chain.

The target's residual stream is tapped after three layers (low, middle, high), concatenated and
fused by ``fc`` into one feature per position.  The drafter's single decoder layer reads, for
position ``i``, the pair (embedding of token ``i + 1``, feature of position ``i``): both halves are
normalised separately, concatenated (so the q/k/v projections have ``2 * hidden`` input columns,
and there is no per-head QK norm), and the residual path starts from the feature.  Its output
before the final norm is the feature of the NEXT position, so after the first step (all newly
committed pairs at once, causal) the chain continues on its own: pair (draft ``j``, own output of
step ``j``) gives draft ``j + 1``.  The head predicts over a reduced draft vocabulary; ``d2t`` maps a
draft id to the target id (``target = draft + d2t[draft]``).

The drafter's K/V live in a one-layer paged buffer that shares the target's block ids; pair ``i``
sits at position ``i``.  Features of prompt chunks and decode steps are kept per request until the
next round (the pair of a step's last row needs the token sampled from it); the rows of a verify
step count once the scheduler reports how many were accepted.

Reference parity: pegainfer-qwen3/src/eagle3.rs:17-95 (chain length 3, tapped layers
``(1, N/2 - 1, N - 4)`` counted after the layer, weight layout), src/eagle3/loading.rs:60-160
(tensor names and shapes, ``d2t`` / ``t2d``).  The reference ships the loader and the memory
reservation of this drafter; the forward pass below follows the published EAGLE-3 inference recipe.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..ops.reference import rope_tables
from ..sched.executor import SeqStep, build_meta

EAGLE3_CHAIN_LENGTH = 3


def aux_hidden_state_layers(target_num_layers: int) -> tuple:
    """Tapped target layers, 0-based, counted after the layer has run."""
    low, mid, high = 1, max(target_num_layers // 2 - 1, 0), max(target_num_layers - 4, 0)
    if not (low < mid < high < target_num_layers):
        raise ValueError(f"EAGLE-3 layers ({low}, {mid}, {high}) are not strictly increasing within {target_num_layers} target layers")
    return (low, mid, high)


@dataclass
class Eagle3Config:
    hidden_size: int
    intermediate_size: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    vocab_size: int
    draft_vocab_size: int
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position: int = 40960

    @classmethod
    def from_hf(cls, raw: dict) -> "Eagle3Config":
        heads = raw["num_attention_heads"]
        return cls(hidden_size=raw["hidden_size"], intermediate_size=raw["intermediate_size"], num_q_heads=heads, num_kv_heads=raw.get("num_key_value_heads", heads),
                   head_dim=raw.get("head_dim", raw["hidden_size"] // heads), vocab_size=raw["vocab_size"], draft_vocab_size=raw.get("draft_vocab_size", raw["vocab_size"]),
                   rms_eps=raw.get("rms_norm_eps", 1e-6), rope_theta=float(raw.get("rope_theta", 1e6)), max_position=raw.get("max_position_embeddings", 40960))

    @classmethod
    def for_target(cls, mcfg, draft_vocab: int = 0) -> "Eagle3Config":
        return cls(hidden_size=mcfg.hidden_size, intermediate_size=mcfg.intermediate_size, num_q_heads=mcfg.num_q_heads, num_kv_heads=mcfg.num_kv_heads, head_dim=mcfg.head_dim,
                   vocab_size=mcfg.vocab_size, draft_vocab_size=draft_vocab or mcfg.vocab_size, rms_eps=mcfg.rms_eps, rope_theta=mcfg.rope_theta, max_position=mcfg.max_position)


def eagle3_shapes(c: Eagle3Config) -> dict:
    h, d, m = c.hidden_size, c.head_dim, "midlayer."
    return {
        "fc.weight": (h, 3 * h), "norm.weight": (h,), "lm_head.weight": (c.draft_vocab_size, h),
        m + "input_layernorm.weight": (h,), m + "hidden_norm.weight": (h,), m + "post_attention_layernorm.weight": (h,),
        m + "self_attn.q_proj.weight": (c.num_q_heads * d, 2 * h), m + "self_attn.k_proj.weight": (c.num_kv_heads * d, 2 * h), m + "self_attn.v_proj.weight": (c.num_kv_heads * d, 2 * h),
        m + "self_attn.o_proj.weight": (h, c.num_q_heads * d),
        m + "mlp.gate_proj.weight": (c.intermediate_size, h), m + "mlp.up_proj.weight": (c.intermediate_size, h), m + "mlp.down_proj.weight": (h, c.intermediate_size),
    }


class Eagle3DraftModel:
    def __init__(self, cfg: Eagle3Config, target, source=None, seed: int = 0, d2t: Optional[torch.Tensor] = None):
        from ..loader.sources import RandomSource

        if cfg.vocab_size != target.cfg.vocab_size or cfg.hidden_size != target.cfg.hidden_size:
            raise ValueError(f"drafter (vocab {cfg.vocab_size}, hidden {cfg.hidden_size}) does not fit the target (vocab {target.cfg.vocab_size}, hidden {target.cfg.hidden_size})")
        self.cfg, self.target = cfg, target
        self.device, self.dtype = target.device, target.dtype
        self.aux_layers = aux_hidden_state_layers(target.cfg.num_layers)
        src = source or RandomSource(eagle3_shapes(cfg), seed=seed, dtype=self.dtype)
        dev, dt, m = self.device, self.dtype, "midlayer."
        g = lambda n: src.get(n, dev, dt)  # noqa: E731
        self.fc, self.norm, self.lm_head = g("fc.weight"), g("norm.weight"), g("lm_head.weight")
        self.input_norm, self.hidden_norm, self.post_norm = g(m + "input_layernorm.weight"), g(m + "hidden_norm.weight"), g(m + "post_attention_layernorm.weight")
        self.qkv = torch.cat([g(m + "self_attn.q_proj.weight"), g(m + "self_attn.k_proj.weight"), g(m + "self_attn.v_proj.weight")], 0)
        self.o = g(m + "self_attn.o_proj.weight")
        self.gate_up = torch.cat([g(m + "mlp.gate_proj.weight"), g(m + "mlp.up_proj.weight")], 0)
        self.down = g(m + "mlp.down_proj.weight")
        if d2t is None and source is not None and source.has("d2t"):
            d2t = source.get("d2t", "cpu", torch.int64)
        # draft id -> target id; a checkpoint without the table drafts over the leading ids of the target vocabulary
        ids = torch.arange(cfg.draft_vocab_size, dtype=torch.int64)
        self.d2t = (ids + (d2t.to(torch.int64) if d2t is not None else 0)).to(torch.int32).to(dev)
        if int(self.d2t.max()) >= cfg.vocab_size or int(self.d2t.min()) < 0:
            raise ValueError("EAGLE-3 d2t maps outside the target vocabulary")
        self.t2d = torch.zeros(cfg.vocab_size, dtype=torch.bool)
        self.t2d[self.d2t.cpu().long()] = True
        self.cos, self.sin = rope_tables(min(cfg.max_position, target.cfg.max_position), cfg.head_dim, cfg.rope_theta, dt, dev)

    @classmethod
    def load(cls, path: str, target, seed: int = 0) -> "Eagle3DraftModel":
        """``path``: a checkpoint directory, or ``random[:draft_vocab=N]`` for a random drafter of the target's width."""
        if path.startswith("random"):
            kw = dict(kv.split("=") for kv in path.split(":", 1)[1].split(",")) if ":" in path else {}
            return cls(Eagle3Config.for_target(target.cfg, int(kw.get("draft_vocab", 0))), target, seed=seed)
        from ..loader.sources import SafetensorsSource

        with open(os.path.join(path, "config.json")) as f:
            cfg = Eagle3Config.from_hf(json.load(f))
        return cls(cfg, target, SafetensorsSource(path))

    def kv_geometry(self) -> dict:
        return dict(num_layers=1, kv_heads=self.cfg.num_kv_heads, head_dim=self.cfg.head_dim)

    def weight_bytes(self) -> int:
        return sum(t.numel() for t in (self.fc, self.qkv, self.o, self.gate_up, self.down, self.lm_head)) * self.fc.element_size()

    def fuse(self, aux: list) -> torch.Tensor:
        """Tapped target hidden states -> one feature per row."""
        return ops.linear(torch.cat(aux, dim=-1), self.fc)

    def step(self, tokens: torch.Tensor, feature: torch.Tensor, meta, kv, rows: torch.Tensor):
        """One pass of the decoder layer over (token, feature) pairs laid out by ``meta``.  Returns the
        target-vocabulary drafts after the rows ``rows`` and those rows' output features."""
        c, eps = self.cfg, self.cfg.rms_eps
        residual = feature.clone()
        x = torch.cat([ops.rms_norm(ops.embedding(tokens, self.target.embed), self.input_norm, eps), ops.rms_norm(feature, self.hidden_norm, eps)], dim=-1)
        q = ops.qk_norm_rope_append(ops.linear(x, self.qkv), None, None, self.cos, self.sin, meta, kv.layer(0), c.num_q_heads, c.num_kv_heads, c.head_dim, eps)
        a = ops.paged_attention(q.reshape(x.shape[0], c.num_q_heads, c.head_dim), kv.layer(0), meta)
        x = ops.add_rms_norm(ops.linear(a, self.o), residual, self.post_norm, eps)
        x = ops.add_rms_norm(ops.linear(ops.swiglu(ops.linear(x, self.gate_up)), self.down), residual, self.norm, eps)
        draft = ops.argmax(ops.linear(ops.gather_rows(x, rows), self.lm_head))
        return self.d2t[draft.long()], ops.gather_rows(residual, rows)


class _ChainGraphs:
    """The chain steps of a draft round (every step after the first) as one CUDA graph per request-count bucket.

    The first step of a round takes a ragged number of (token, feature) pairs per request and stays kernel by kernel; the
    ``steps`` steps behind it are decode-shaped (one row per request, positions one further each time), so their
    positions, slots, KV lengths and block tables live in pointer-stable buffers that are refreshed from pinned mirrors
    before a replay, the first step's drafts and features are copied in, and the drafts of all steps come back through
    one small copy."""

    def __init__(self, draft: "Eagle3DraftModel", kv, page_size: int, steps: int, max_batch: int, width: int):
        from ..sched.executor import DECODE_BUCKETS, bucket_for

        self.draft, self.kv, self.page_size, self.steps = draft, kv, page_size, steps
        dev = draft.device
        self.buckets = [b for b in DECODE_BUCKETS if b <= max(bucket_for(max_batch), 1)]
        n, W = self.buckets[-1], max(width, 1)
        self.nmax, self.W = n, W
        self.h_small = torch.zeros(3 * steps * n, dtype=torch.int32).pin_memory()  # positions | slots | kv lengths, [steps, n] each
        self.d_small = torch.zeros(3 * steps * n, dtype=torch.int32, device=dev)
        self.h_table = torch.zeros((n, W), dtype=torch.int32).pin_memory()
        self.d_table = torch.zeros((n, W), dtype=torch.int32, device=dev)
        self.tok = torch.zeros(n, dtype=torch.int32, device=dev)
        self.feat = torch.zeros((n, draft.cfg.hidden_size), dtype=draft.dtype, device=dev)
        self.out = torch.zeros((steps, n), dtype=torch.int32, device=dev)
        self.h_out = torch.zeros((steps, n), dtype=torch.int32).pin_memory()
        self.q_indptr = torch.arange(n + 1, dtype=torch.int32, device=dev)
        self.rows = torch.arange(n, dtype=torch.int32, device=dev)
        self.graphs: dict = {}
        self.pool = None
        self.replays = 0

    def _views(self, j: int, n: int):
        N, S = self.nmax, self.steps
        s = self.d_small
        return s[j * N : j * N + n], s[(S + j) * N : (S + j) * N + n], s[(2 * S + j) * N : (2 * S + j) * N + n]

    def _body(self, n: int) -> None:
        from ..ops import cuda as K
        from ..ops.reference import AttnMeta

        d = self.draft
        geo = d.kv_geometry()
        plan = K.plan_decode_splits(n, geo["kv_heads"], min(self.W * self.page_size, 2048), d.device)
        tok, feat = self.tok[:n], self.feat[:n]
        for j in range(self.steps):
            pos, slot, kvl = self._views(j, n)
            meta = AttnMeta(q_indptr=self.q_indptr[: n + 1], kv_lens=kvl, block_table=self.d_table[:n], slot_mapping=slot, positions=pos, page_size=self.page_size, num_seqs=n,
                            num_tokens=n, max_q_len=1, max_kv_len=self.W * self.page_size, decode_only=True, plan=plan)
            draft, feat = d.step(tok, feat, meta, self.kv, self.rows[:n])
            tok = draft.to(torch.int32)
            self.out[j, :n].copy_(tok)

    def capture(self, n: int):
        dev = self.draft.device
        self.d_small.zero_()
        self.d_table.zero_()
        s = torch.cuda.Stream(dev)
        s.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(s):
            self._body(n)  # warm-up on padding inputs (page 0, KV length 0)
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            if self.pool is None:
                self.pool = torch.cuda.graph_pool_handle()
            g.capture_begin(pool=self.pool)
            try:
                self._body(n)
            finally:
                g.capture_end()
            g.replay()
        torch.cuda.current_stream(dev).wait_stream(s)
        self.graphs[n] = g
        return g

    def run(self, decoders, first_draft: torch.Tensor, first_feat: torch.Tensor) -> list:
        """Drafts of the chain steps, ``[steps][requests]``.  ``decoders``: the scheduler's request states;
        ``first_draft`` / ``first_feat``: what the round's first step produced for them."""
        from ..sched.executor import bucket_for

        n, N, S, ps = len(decoders), self.nmax, self.steps, self.page_size
        b = bucket_for(n, self.buckets)
        if b not in self.graphs:
            self.capture(b)
        sm, tb = self.h_small.numpy(), self.h_table.numpy()
        sm[:] = 0
        tb[:] = 0
        for i, r in enumerate(decoders):
            pages = r.kv.view().page_indices
            tb[i, : len(pages)] = pages
            c = r.kv.committed
            for j in range(S):
                pos = c + j  # chain step j + 1 appends at position committed + j
                sm[j * N + i] = pos
                sm[(S + j) * N + i] = pages[pos // ps] * ps + pos % ps
                sm[(2 * S + j) * N + i] = pos + 1
        self.d_small.copy_(self.h_small, non_blocking=True)
        self.d_table.copy_(self.h_table, non_blocking=True)
        self.tok[:n].copy_(first_draft.to(torch.int32))
        self.feat[:n].copy_(first_feat)
        self.graphs[b].replay()
        self.replays += 1
        self.h_out.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream(self.draft.device).synchronize()
        return [self.h_out[j, :n].tolist() for j in range(S)]

    def release(self) -> None:
        self.graphs.clear()
        self.pool = None


class Eagle3Spec:
    allows_prefix_cache = False
    kind = "eagle3"

    def __init__(self, ecfg, model, executor, draft_model: Optional[Eagle3DraftModel] = None):
        from .draft_model import _make_kv, _num_pages

        if draft_model is None:
            draft_model = getattr(model, "draft_model", None) or Eagle3DraftModel.load(ecfg.draft_model_path or "random", model, seed=ecfg.seed + 1)
        self.draft = draft_model
        self.draft_len = int(ecfg.spec_draft_len) if int(ecfg.spec_draft_len) > 1 else EAGLE3_CHAIN_LENGTH
        self.page_size = executor.page_size
        self.device = model.device
        self.kv = _make_kv(draft_model, _num_pages(executor.kv), executor.page_size)
        self.aux_layers = draft_model.aux_layers
        self.valid: dict = {}  # rid -> pairs already in the draft cache
        self.pending: dict = {}  # rid -> [feature rows] of committed positions valid .. committed - 1
        self.staged: dict = {}
        self.rounds = 0
        import os

        # the chain steps of a round as one CUDA graph per bucket (PEGAINFER_DRAFT_GRAPH=0: kernel by kernel)
        self._use_graph = self.device.type == "cuda" and os.environ.get("PEGAINFER_DRAFT_GRAPH", "1") != "0"
        self._chain = None
        self._max_batch = int(getattr(executor, "max_decode_batch", 64))
        self._width = int(getattr(executor, "max_blocks_per_seq", 0) or 1)
        executor.aux_sink = self

    def observe(self, kind: str, seqs, meta, aux: list) -> None:
        if not seqs:
            return
        feat = self.draft.fuse([a[: meta.num_tokens] for a in aux])
        for i, s in enumerate(seqs):
            rows = feat[meta.h_q_indptr[i] : meta.h_q_indptr[i + 1]]
            if kind == "verify":
                self.staged[s.rid] = (s.start_pos, rows)
                continue
            if s.start_pos == 0:
                self.valid[s.rid], self.pending[s.rid] = 0, []
            have = self.valid.get(s.rid, -1) + sum(p.shape[0] for p in self.pending.get(s.rid, ()))
            if have == s.start_pos:
                self.pending[s.rid].append(rows)
            else:
                self.valid[s.rid] = -1  # features are missing for some position: decode this request without drafts

    def on_accept(self, rid: int, rows: int) -> None:
        st = self.staged.pop(rid, None)
        if st is not None and self.valid.get(rid, -1) == st[0]:
            self.pending[rid] = [st[1][:rows]]

    def ready(self, r) -> bool:
        req, rid = r.q.request, r.q.id
        if self.valid.get(rid, -1) < 0 or r.phase != "decode" or req.logprobs != 0 or req.params.temperature >= 1e-5 or r.lora_slot >= 0:
            return False
        have = self.valid[rid] + sum(p.shape[0] for p in self.pending[rid])
        return have == r.kv.committed and bool(self.pending[rid]) and r.kv.committed + self.draft_len + 1 < self.draft.cos.shape[0]

    def release(self, rid: int) -> None:
        for d in (self.valid, self.pending, self.staged):
            d.pop(rid, None)

    def propose(self, decoders) -> dict:
        dev = self.device
        seqs, toks, feats, last = [], [], [], []
        for r in decoders:
            rid, v, c = r.q.id, self.valid[r.q.id], r.kv.committed
            seqs.append(SeqStep(rid=rid, input_tokens=r.kv.tokens[v + 1 : c + 1], start_pos=v, view=r.kv.view()))
            feats.extend(self.pending[rid])
        tok, meta = build_meta(seqs, self.page_size, dev)
        rows = torch.tensor([meta.h_q_indptr[i + 1] - 1 for i in range(len(seqs))], dtype=torch.int32, device=dev)
        draft, feat = self.draft.step(tok, torch.cat(feats) if len(feats) > 1 else feats[0], meta, self.kv, rows)
        if self._use_graph and self.draft_len > 1 and len(decoders) <= self._max_batch:
            if self._chain is None:
                self._chain = _ChainGraphs(self.draft, self.kv, self.page_size, self.draft_len - 1, self._max_batch, self._width)
            chain = self._chain.run(decoders, draft, feat)
            first = draft.tolist()
            for r in decoders:
                self.valid[r.q.id], self.pending[r.q.id] = r.kv.committed, []
            self.rounds += 1
            return {r.q.id: [int(first[i])] + [int(step[i]) for step in chain] for i, r in enumerate(decoders)}
        out = [draft]
        one = torch.arange(len(seqs), dtype=torch.int32, device=dev)
        for j in range(1, self.draft_len):
            seqs = [SeqStep(rid=r.q.id, input_tokens=[0], start_pos=r.kv.committed + j - 1, view=r.kv.view()) for r in decoders]
            _, meta = build_meta(seqs, self.page_size, dev)
            draft, feat = self.draft.step(draft.to(torch.int32), feat, meta, self.kv, one)
            out.append(draft)
        picked = torch.stack(out, 1).tolist()
        for r in decoders:
            self.valid[r.q.id], self.pending[r.q.id] = r.kv.committed, []
        self.rounds += 1
        return {r.q.id: [int(t) for t in picked[i]] for i, r in enumerate(decoders)}
