"""Block drafters that read the target's hidden states: DFlash and DSpark.

A DFlash drafter is a small stack of decoder layers that drafts a whole block of tokens in ONE
forward pass.  The block is ``[current token, mask, mask, ...]`` embedded with the target's
embedding; its attention is bidirectional over the block and over a *context* made of the target's
own hidden states: the residual stream of a few target layers, concatenated, projected by ``fc``
and normalised by ``hidden_norm``.  The context rows enter every draft layer's K/V projections as
they are (no layer norm, no update from layer to layer); the block rows go through the usual
pre-norm decoder layer.  Logits come from the target's output projection.  DSpark adds a low-rank
Markov head: the block's logits are corrected left to right by ``w2 . w1[previous token]``, so each
draft depends on the one before it at the cost of one rank-``r`` GEMM and one arg-max per position.

How this maps to the engine:

* the draft K/V live in a paged buffer that shares the target's block ids and positions, so a
  request's block table addresses both caches and rejected positions are simply overwritten;
* context rows of prompt chunks and plain decode steps are written into the draft cache as soon as
  the target has produced them (``observe``); the rows of a verify step wait until the scheduler
  says how many were accepted (``on_accept``) and join the next round's tail;
* the bidirectional block attention runs on the decode attention kernel: every block row is a
  one-row sequence whose KV length is the whole tail, so no mask is needed;
* the Markov loop stays on the device: embedding gather, ``w2`` GEMM and a fused add + arg-max
  kernel per position, one host read for the finished block.

Reference parity: pegainfer-qwen3/src/dflash.rs:318-790 (draft forward, request state, context
projection), src/dspark.rs:44-110 (Markov head), src/config.rs:54-330 (drafter config: nested
``dflash_config`` or flat schema, anchor-first versus anchor-drop blocks).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from types import SimpleNamespace
from typing import Optional

import torch

from .. import ops
from ..ops.reference import rope_tables
from ..sched.executor import SeqStep, build_meta


@dataclass
class DFlashConfig:
    hidden_size: int
    intermediate_size: int
    num_layers: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    vocab_size: int
    block_size: int
    mask_token_id: int
    target_layer_ids: tuple
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position: int = 40960
    markov_rank: int = 0
    anchor_first: bool = False  # block position 0 already predicts the first draft (DeepSpec checkpoints)
    confidence_head: bool = False  # present in some checkpoints; not used (every block is verified in full)

    @property
    def num_drafts(self) -> int:
        return self.block_size if self.anchor_first else self.block_size - 1

    @property
    def context_dim(self) -> int:
        return self.hidden_size * len(self.target_layer_ids)

    @classmethod
    def from_hf(cls, raw: dict) -> "DFlashConfig":
        inner = raw.get("dflash_config") or {}
        theta = raw.get("rope_theta") or (raw.get("rope_parameters") or {}).get("rope_theta")
        mask = inner.get("mask_token_id", raw.get("mask_token_id"))
        layers = inner.get("target_layer_ids", raw.get("target_layer_ids"))
        if theta is None or mask is None or layers is None:
            raise ValueError("drafter config needs rope_theta, mask_token_id and target_layer_ids")
        rank = int(raw.get("markov_rank", 0))
        return cls(
            hidden_size=raw["hidden_size"], intermediate_size=raw["intermediate_size"], num_layers=raw["num_hidden_layers"], num_q_heads=raw["num_attention_heads"],
            num_kv_heads=raw["num_key_value_heads"], head_dim=raw["head_dim"], vocab_size=raw["vocab_size"], block_size=raw["block_size"], mask_token_id=int(mask),
            target_layer_ids=tuple(layers), rms_eps=raw.get("rms_norm_eps", 1e-6), rope_theta=float(theta), max_position=raw.get("max_position_embeddings", 40960),
            markov_rank=rank, anchor_first=raw.get("num_anchors") is not None or rank > 0, confidence_head=bool(raw.get("enable_confidence_head", False)),
        )

    def to_hf(self) -> dict:
        out = dict(hidden_size=self.hidden_size, intermediate_size=self.intermediate_size, num_hidden_layers=self.num_layers, num_attention_heads=self.num_q_heads,
                   num_key_value_heads=self.num_kv_heads, head_dim=self.head_dim, vocab_size=self.vocab_size, block_size=self.block_size, rms_norm_eps=self.rms_eps,
                   rope_theta=self.rope_theta, max_position_embeddings=self.max_position, num_target_layers=0, markov_rank=self.markov_rank)
        if self.anchor_first:
            out.update(mask_token_id=self.mask_token_id, target_layer_ids=list(self.target_layer_ids), num_anchors=1)
        else:
            out["dflash_config"] = dict(mask_token_id=self.mask_token_id, target_layer_ids=list(self.target_layer_ids))
        return out

    @classmethod
    def for_target(cls, mcfg, num_layers: int = 2, block_size: int = 4, markov_rank: int = 0, anchor_first: Optional[bool] = None, aux: int = 3) -> "DFlashConfig":
        """A drafter of the target's width (random weights: benchmarks and tests)."""
        n = mcfg.num_layers
        ids = sorted({max(0, min(n - 1, round((i + 1) * n / (aux + 1)) - 1)) for i in range(aux)})
        return cls(hidden_size=mcfg.hidden_size, intermediate_size=mcfg.intermediate_size, num_layers=num_layers, num_q_heads=mcfg.num_q_heads, num_kv_heads=mcfg.num_kv_heads,
                   head_dim=mcfg.head_dim, vocab_size=mcfg.vocab_size, block_size=block_size, mask_token_id=mcfg.vocab_size - 1, target_layer_ids=tuple(ids), rms_eps=mcfg.rms_eps,
                   rope_theta=mcfg.rope_theta, max_position=mcfg.max_position, markov_rank=markov_rank, anchor_first=(markov_rank > 0) if anchor_first is None else anchor_first)


def dflash_shapes(c: DFlashConfig) -> dict:
    h, d = c.hidden_size, c.head_dim
    s = {"fc.weight": (h, c.context_dim), "hidden_norm.weight": (h,), "norm.weight": (h,)}
    for i in range(c.num_layers):
        p = f"layers.{i}."
        s.update({
            p + "input_layernorm.weight": (h,), p + "post_attention_layernorm.weight": (h,),
            p + "self_attn.q_proj.weight": (c.num_q_heads * d, h), p + "self_attn.k_proj.weight": (c.num_kv_heads * d, h), p + "self_attn.v_proj.weight": (c.num_kv_heads * d, h),
            p + "self_attn.o_proj.weight": (h, c.num_q_heads * d), p + "self_attn.q_norm.weight": (d,), p + "self_attn.k_norm.weight": (d,),
            p + "mlp.gate_proj.weight": (c.intermediate_size, h), p + "mlp.up_proj.weight": (c.intermediate_size, h), p + "mlp.down_proj.weight": (h, c.intermediate_size),
        })
    if c.markov_rank:
        s["markov_head.markov_w1.weight"] = (c.vocab_size, c.markov_rank)
        s["markov_head.markov_w2.weight"] = (c.vocab_size, c.markov_rank)
    return s


class DFlashDraftModel:
    """Weights and forward pass of a DFlash / DSpark drafter bound to one target model."""

    def __init__(self, cfg: DFlashConfig, target, source=None, seed: int = 0):
        from ..loader.sources import RandomSource

        if cfg.vocab_size != target.cfg.vocab_size or cfg.hidden_size != target.cfg.hidden_size:
            raise ValueError(f"drafter (vocab {cfg.vocab_size}, hidden {cfg.hidden_size}) does not fit the target (vocab {target.cfg.vocab_size}, hidden {target.cfg.hidden_size})")
        if max(cfg.target_layer_ids) >= target.cfg.num_layers:
            raise ValueError(f"drafter reads target layers {cfg.target_layer_ids}; the target has {target.cfg.num_layers}")
        if cfg.max_position < target.cfg.max_position and cfg.max_position < 1 << 15:
            raise ValueError("drafter max_position_embeddings is shorter than the target's")
        self.cfg, self.target = cfg, target
        self.device, self.dtype = target.device, target.dtype
        src = source or RandomSource(dflash_shapes(cfg), seed=seed, dtype=self.dtype)
        dev, dt = self.device, self.dtype
        g = lambda n: src.get(n, dev, dt)  # noqa: E731
        self.fc, self.hidden_norm, self.norm = g("fc.weight"), g("hidden_norm.weight"), g("norm.weight")
        self.layers = []
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            self.layers.append(SimpleNamespace(
                input_norm=g(p + "input_layernorm.weight"), post_norm=g(p + "post_attention_layernorm.weight"),
                qkv=torch.cat([g(p + "self_attn.q_proj.weight"), g(p + "self_attn.k_proj.weight"), g(p + "self_attn.v_proj.weight")], 0),
                q_norm=g(p + "self_attn.q_norm.weight"), k_norm=g(p + "self_attn.k_norm.weight"), o=g(p + "self_attn.o_proj.weight"),
                gate_up=torch.cat([g(p + "mlp.gate_proj.weight"), g(p + "mlp.up_proj.weight")], 0), down=g(p + "mlp.down_proj.weight"),
            ))
        self.markov = None
        if cfg.markov_rank:
            self.markov = (g("markov_head.markov_w1.weight"), g("markov_head.markov_w2.weight"))
        self.cos, self.sin = rope_tables(min(cfg.max_position, target.cfg.max_position), cfg.head_dim, cfg.rope_theta, dt, dev)

    @classmethod
    def load(cls, path: str, target, seed: int = 0) -> "DFlashDraftModel":
        """``path``: a checkpoint directory, or ``random:layers=2,block=4,markov=16,anchor_first=1`` for a
        random drafter of the target's width."""
        if path.startswith("random"):
            kw = dict(kv.split("=") for kv in path.split(":", 1)[1].split(",")) if ":" in path else {}
            af = kw.get("anchor_first")
            cfg = DFlashConfig.for_target(target.cfg, int(kw.get("layers", 2)), int(kw.get("block", 4)), int(kw.get("markov", 0)), None if af is None else bool(int(af)))
            return cls(cfg, target, seed=seed)
        from ..loader.sources import SafetensorsSource

        with open(os.path.join(path, "config.json")) as f:
            cfg = DFlashConfig.from_hf(json.load(f))
        return cls(cfg, target, SafetensorsSource(path))

    def kv_geometry(self) -> dict:
        return dict(num_layers=self.cfg.num_layers, kv_heads=self.cfg.num_kv_heads, head_dim=self.cfg.head_dim)

    def weight_bytes(self) -> int:
        n = self.fc.numel() + sum(t.numel() for l in self.layers for t in (l.qkv, l.o, l.gate_up, l.down))
        if self.markov:
            n += 2 * self.markov[0].numel()
        return n * self.fc.element_size()

    # -- context ---------------------------------------------------------------------
    def project_context(self, aux: list) -> torch.Tensor:
        """Target hidden states of the tapped layers ``[T, hidden]`` each -> context rows ``[T, hidden]``."""
        x = aux[0] if len(aux) == 1 else torch.cat(aux, dim=-1)
        return ops.rms_norm(ops.linear(x, self.fc), self.hidden_norm, self.cfg.rms_eps)

    def ingest(self, ctx: torch.Tensor, meta, kv) -> None:
        """Write the draft K/V of context rows at the positions and slots of ``meta`` (the target step's own)."""
        c = self.cfg
        for i, l in enumerate(self.layers):
            qkv = ops.linear(ctx, l.qkv)
            ops.qk_norm_rope_append(qkv, l.q_norm, l.k_norm, self.cos, self.sin, meta, kv.layer(i), c.num_q_heads, c.num_kv_heads, c.head_dim, c.rms_eps)

    # -- one round ---------------------------------------------------------------------
    def block_logits(self, kv, page_size: int, reqs: list) -> torch.Tensor:
        """``reqs``: ``(view, base, ctx_rows or None, current_token)`` per request, where ``base`` counts the
        positions already in the draft cache and ``ctx_rows [c, hidden]`` are context rows not yet written.
        Returns the block's logits ``[len(reqs) * block, vocab]`` (request-major)."""
        c, dev = self.cfg, self.device
        B, n = c.block_size, len(reqs)
        tail, blocks, ctx_idx, blk_idx, ctx_rows, toks, off = [], [], [], [], [], [], 0
        for view, base, ctx, cur in reqs:
            nc = 0 if ctx is None else ctx.shape[0]
            tail.append(SeqStep(rid=0, input_tokens=[0] * (nc + B), start_pos=base, view=view))
            for _ in range(B):  # every block row attends to the whole tail: a one-row sequence ending at the tail's end
                blocks.append(SeqStep(rid=0, input_tokens=[0], start_pos=base + nc + B - 1, view=view))
            ctx_idx.extend(range(off, off + nc))
            blk_idx.extend(range(off + nc, off + nc + B))
            if nc:
                ctx_rows.append(ctx)
            toks.extend([cur] + [c.mask_token_id] * (B - 1))
            off += nc + B
        _, meta_tail = build_meta(tail, page_size, dev)
        _, meta_blk = build_meta(blocks, page_size, dev)
        blk_t = torch.tensor(blk_idx, dtype=torch.long, device=dev)
        ctx_t = torch.tensor(ctx_idx, dtype=torch.long, device=dev) if ctx_idx else None
        ctx_all = torch.cat(ctx_rows) if ctx_rows else None
        residual = ops.embedding(torch.tensor(toks, dtype=torch.int32, device=dev), self.target.embed)
        x = ops.rms_norm(residual, self.layers[0].input_norm, c.rms_eps)
        eps = c.rms_eps
        for i, l in enumerate(self.layers):
            if ctx_t is None:
                tail_in = x
            else:
                tail_in = torch.empty((off, c.hidden_size), dtype=x.dtype, device=dev)
                tail_in.index_copy_(0, ctx_t, ctx_all)
                tail_in.index_copy_(0, blk_t, x)
            qkv = ops.linear(tail_in, l.qkv)
            q = ops.qk_norm_rope_append(qkv, l.q_norm, l.k_norm, self.cos, self.sin, meta_tail, kv.layer(i), c.num_q_heads, c.num_kv_heads, c.head_dim, eps)
            q = q.reshape(off, c.num_q_heads, c.head_dim)
            if ctx_t is not None:
                q = q.index_select(0, blk_t)
            a = ops.paged_attention(q, kv.layer(i), meta_blk)
            x = ops.add_rms_norm(ops.linear(a, l.o), residual, l.post_norm, eps)
            act = ops.swiglu(ops.linear(x, l.gate_up))
            nxt = self.layers[i + 1].input_norm if i + 1 < len(self.layers) else self.norm
            x = ops.add_rms_norm(ops.linear(act, l.down), residual, nxt, eps)
        logits = self.target.logits(x)
        return self.target.full_logits(logits) if hasattr(self.target, "full_logits") else logits

    def pick(self, logits: torch.Tensor, current: list) -> list:
        """Draft tokens of every request (``num_drafts`` each) from the block's logits."""
        c = self.cfg
        B, n = c.block_size, len(current)
        if self.markov is None:
            toks = ops.argmax(logits).view(n, B).tolist()
            return [t if c.anchor_first else t[1:] for t in toks]
        w1, w2 = self.markov
        prev = torch.tensor(current, dtype=torch.int32, device=self.device)
        nxt = torch.empty_like(prev)
        drafts = torch.zeros(n * B, dtype=torch.int32, device=self.device)
        for step in range(B):
            bias = ops.linear(ops.embedding(prev, w1), w2)
            if bias.dtype != logits.dtype:
                bias = bias.to(logits.dtype)
            ops.markov_step_argmax(logits, bias, B, step, nxt, drafts)
            prev, nxt = nxt, prev
        return drafts.view(n, B).tolist()


class _DraftGraphs:
    """The draft round as one CUDA graph per request-count bucket.

    A round's shapes vary only through the number of context rows each request brings (the rows its last verify step
    committed, at most ``span``), so every request gets ``span`` context slots: unused slots carry zero rows whose
    K/V land in the padding page, and the block rows' KV lengths simply do not cover them.  Positions, slots, KV
    lengths, block tables, current tokens and context rows live in pointer-stable buffers that are refreshed from
    pinned mirrors before each replay; the picked drafts come back through one small copy."""

    def __init__(self, draft: "DFlashDraftModel", kv, page_size: int, span: int, max_batch: int, width: int):
        from ..sched.executor import DECODE_BUCKETS, bucket_for

        self.draft, self.kv, self.page_size, self.span = draft, kv, page_size, span
        c, dev = draft.cfg, draft.device
        self.B, self.R = c.block_size, span + c.block_size
        self.buckets = [b for b in DECODE_BUCKETS if b <= max(bucket_for(max_batch), 1)]
        n, B, R, W = self.buckets[-1], self.B, self.R, max(width, 1)
        self.nmax, self.W = n, W
        self.ctx = torch.zeros((n * span, c.hidden_size), dtype=draft.dtype, device=dev)
        words = n + 2 * n * R + n * B  # current tokens | tail positions | tail slots | block-row KV lengths
        self.h_small = torch.zeros(words, dtype=torch.int32).pin_memory()
        self.d_small = torch.zeros(words, dtype=torch.int32, device=dev)
        self.h_table = torch.zeros((n, W), dtype=torch.int32).pin_memory()
        self.d_table = torch.zeros((n, W), dtype=torch.int32, device=dev)
        self.d_table_blk = torch.zeros((n * B, W), dtype=torch.int32, device=dev)
        self.toks = torch.full((n * B,), c.mask_token_id, dtype=torch.int32, device=dev)
        self.out = torch.zeros(n * B, dtype=torch.int32, device=dev)
        self.h_out = torch.zeros(n * B, dtype=torch.int32).pin_memory()
        self.prev = torch.zeros(n, dtype=torch.int32, device=dev)
        self.nxt = torch.zeros(n, dtype=torch.int32, device=dev)
        self.tail_ptr = torch.arange(n + 1, dtype=torch.int32, device=dev) * R
        self.blk_ptr = torch.arange(n * B + 1, dtype=torch.int32, device=dev)
        ar = torch.arange(n, device=dev).view(n, 1) * R
        self.ctx_idx = (ar + torch.arange(span, device=dev).view(1, span)).reshape(-1)
        self.blk_idx = (ar + span + torch.arange(B, device=dev).view(1, B)).reshape(-1)
        self.graphs: dict = {}
        self.pool = None
        self.replays = 0

    def _views(self, n: int):
        N, R, B = self.nmax, self.R, self.B
        s = self.d_small
        return s[:n], s[N : N + n * R], s[N + N * R : N + N * R + n * R], s[N + 2 * N * R : N + 2 * N * R + n * B]

    def _body(self, n: int) -> None:
        from ..ops import cuda as K
        from ..ops.reference import AttnMeta

        d, c = self.draft, self.draft.cfg
        B, R, S, eps = self.B, self.R, self.span, c.rms_eps
        cur, pos, slot, kvl = self._views(n)
        geo = d.kv_geometry()
        plan = K.plan_decode_splits(n * B, geo["kv_heads"], min(self.W * self.page_size, 2048), d.device)
        meta_tail = AttnMeta(q_indptr=self.tail_ptr[: n + 1], kv_lens=kvl, block_table=self.d_table[:n], slot_mapping=slot, positions=pos, page_size=self.page_size, num_seqs=n,
                             num_tokens=n * R, max_q_len=R, max_kv_len=self.W * self.page_size)
        self.d_table_blk[: n * B].copy_(self.d_table[:n].repeat_interleave(B, 0))
        meta_blk = AttnMeta(q_indptr=self.blk_ptr[: n * B + 1], kv_lens=kvl, block_table=self.d_table_blk[: n * B], slot_mapping=slot, positions=pos, page_size=self.page_size,
                            num_seqs=n * B, num_tokens=n * B, max_q_len=1, max_kv_len=self.W * self.page_size, decode_only=True, plan=plan)
        self.toks.view(self.nmax, B)[:n, 0].copy_(cur)
        ctx_idx, blk_idx = self.ctx_idx[: n * S], self.blk_idx[: n * B]
        residual = ops.embedding(self.toks[: n * B], d.target.embed)
        x = ops.rms_norm(residual, d.layers[0].input_norm, eps)
        for i, l in enumerate(d.layers):
            tail_in = torch.empty((n * R, c.hidden_size), dtype=x.dtype, device=x.device)
            tail_in.index_copy_(0, ctx_idx, self.ctx[: n * S])
            tail_in.index_copy_(0, blk_idx, x)
            qkv = ops.linear(tail_in, l.qkv)
            q = ops.qk_norm_rope_append(qkv, l.q_norm, l.k_norm, d.cos, d.sin, meta_tail, self.kv.layer(i), c.num_q_heads, c.num_kv_heads, c.head_dim, eps)
            q = q.reshape(n * R, c.num_q_heads, c.head_dim).index_select(0, blk_idx)
            a = ops.paged_attention(q, self.kv.layer(i), meta_blk)
            x = ops.add_rms_norm(ops.linear(a, l.o), residual, l.post_norm, eps)
            act = ops.swiglu(ops.linear(x, l.gate_up))
            nxt_norm = d.layers[i + 1].input_norm if i + 1 < len(d.layers) else d.norm
            x = ops.add_rms_norm(ops.linear(act, l.down), residual, nxt_norm, eps)
        logits = d.target.logits(x)
        if d.markov is None:
            K.argmax(logits, out=self.out[: n * B])
            return
        w1, w2 = d.markov
        self.prev[:n].copy_(cur)
        a_, b_ = self.prev[:n], self.nxt[:n]
        for step in range(B):
            bias = ops.linear(ops.embedding(a_, w1), w2)
            K.markov_step_argmax(logits, bias if bias.dtype == logits.dtype else bias.to(logits.dtype), B, step, b_, self.out[: n * B])
            a_, b_ = b_, a_

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

    def run(self, reqs: list) -> list:
        """``reqs`` as for ``DFlashDraftModel.block_logits``.  Returns the block's picks, ``block_size`` per request."""
        from ..sched.executor import bucket_for

        n, N, B, R, S, ps = len(reqs), self.nmax, self.B, self.R, self.span, self.page_size
        b = bucket_for(n, self.buckets)
        if b not in self.graphs:
            self.capture(b)
        sm = self.h_small.numpy()
        tb = self.h_table.numpy()
        sm[:] = 0
        ctx_rows, ctx_at = [], []
        for i, (view, base, ctx, cur) in enumerate(reqs):
            nc = 0 if ctx is None else ctx.shape[0]
            pages = view.page_indices
            tb[i, : len(pages)] = pages
            sm[i] = cur
            p0, s0 = N + i * R, N + N * R + i * R
            for j in range(nc):  # real context rows first; the unused context slots keep position 0 and slot 0 (padding page)
                pos = base + j
                sm[p0 + j] = pos
                sm[s0 + j] = pages[pos // ps] * ps + pos % ps
            for j in range(B):
                pos = base + nc + j
                sm[p0 + S + j] = pos
                sm[s0 + S + j] = pages[pos // ps] * ps + pos % ps
            sm[N + 2 * N * R + i * B : N + 2 * N * R + (i + 1) * B] = base + nc + B
            if nc:
                ctx_rows.append(ctx)
                ctx_at.append((i * S, nc))
        self.d_small.copy_(self.h_small, non_blocking=True)
        self.d_table[:b].copy_(self.h_table[:b], non_blocking=True)
        self.ctx[: b * S].zero_()
        for (at, nc), rows in zip(ctx_at, ctx_rows):
            self.ctx[at : at + nc].copy_(rows, non_blocking=True)
        self.graphs[b].replay()
        self.replays += 1
        self.h_out[: n * B].copy_(self.out[: n * B], non_blocking=True)
        torch.cuda.current_stream(self.draft.device).synchronize()
        return self.h_out[: n * B].view(n, B).tolist()

    def release(self) -> None:
        self.graphs.clear()
        self.pool = None


@dataclass
class _ReqState:
    valid: int = 0  # leading positions of the draft cache that hold committed context
    pending: Optional[torch.Tensor] = None  # context rows accepted by the last verify step, not yet in the cache
    staged: Optional[torch.Tensor] = None  # context rows of a verify step whose outcome is not known yet
    staged_pos: int = 0
    extra: dict = field(default_factory=dict)


class DFlashSpec:
    """Scheduler-side driver: keeps the draft cache in step with the target and proposes blocks."""

    allows_prefix_cache = False

    def __init__(self, ecfg, model, executor, draft_model: Optional[DFlashDraftModel] = None):
        from .draft_model import _make_kv, _num_pages

        if draft_model is None:
            draft_model = getattr(model, "draft_model", None) or DFlashDraftModel.load(ecfg.draft_model_path or "random", model, seed=ecfg.seed + 1)
        self.draft = draft_model
        self.kind = "dspark" if draft_model.markov is not None else "dflash"
        self.draft_len = draft_model.cfg.num_drafts
        self.page_size = executor.page_size
        self.device = model.device
        self.kv = _make_kv(draft_model, _num_pages(executor.kv), executor.page_size)
        self.state: dict = {}
        self.rounds = 0
        executor.aux_sink = self
        self.aux_layers = tuple(draft_model.cfg.target_layer_ids)
        # the draft round as a CUDA graph (one GPU; with tensor parallelism the target's sharded output projection
        # would put a collective into the graph)
        self.graphs = None
        tp = getattr(model, "tp", None)
        if self.device.type == "cuda" and getattr(executor, "use_graph", False) and (tp is None or tp.world == 1) and os.environ.get("PEGAINFER_DRAFT_GRAPH", "1") != "0":
            self.graphs = _DraftGraphs(draft_model, self.kv, self.page_size, 1 + self.draft_len, executor.max_decode_batch, executor.max_blocks_per_seq)

    # -- called by the executor after every target forward ---------------------------------
    def observe(self, kind: str, seqs, meta, aux: list) -> None:
        if not seqs:
            return
        ctx = self.draft.project_context([a[: meta.num_tokens] for a in aux])
        if kind != "verify":
            # every row of a prompt chunk or a plain decode step is committed: straight into the draft cache
            flush, rows = [], []
            for s in seqs:
                st = self.state.setdefault(s.rid, _ReqState())
                if st.pending is not None and st.valid + st.pending.shape[0] == s.start_pos:
                    # rows a verify step accepted, followed by a step without a draft round: they go in first
                    flush.append(SeqStep(rid=s.rid, input_tokens=[0] * st.pending.shape[0], start_pos=st.valid, view=s.view))
                    rows.append(st.pending)
                    st.valid = s.start_pos
                st.pending = None
                if s.start_pos <= st.valid:
                    st.valid = s.start_pos + len(s.input_tokens)
                else:
                    st.valid = -1  # a gap in the draft cache: this request decodes without drafts
            if flush:
                self.draft.ingest(torch.cat(rows), build_meta(flush, self.page_size, self.device)[1], self.kv)
            self.draft.ingest(ctx, meta, self.kv)
            return
        for i, s in enumerate(seqs):
            st = self.state.setdefault(s.rid, _ReqState())
            st.staged = ctx[meta.h_q_indptr[i] : meta.h_q_indptr[i + 1]]
            st.staged_pos = s.start_pos

    def on_accept(self, rid: int, rows: int) -> None:
        """The verify step of ``rid`` committed its first ``rows`` input rows."""
        st = self.state.get(rid)
        if st is None or st.staged is None:
            return
        if st.staged_pos == st.valid:
            st.pending = st.staged[:rows]
        st.staged = None

    def ready(self, r) -> bool:
        req = r.q.request
        st = self.state.get(r.q.id)
        if st is None or st.valid < 0 or r.phase != "decode" or req.logprobs != 0 or req.params.temperature >= 1e-5 or r.lora_slot >= 0:
            return False
        have = st.valid + (0 if st.pending is None else st.pending.shape[0])
        return have == r.kv.committed and r.kv.committed + self.draft.cfg.block_size + 1 < self.draft.cos.shape[0]

    def release(self, rid: int) -> None:
        self.state.pop(rid, None)

    def propose(self, decoders) -> dict:
        """``rid -> drafts``.  Every request's view already covers the verify span."""
        reqs, cur = [], []
        for r in decoders:
            st = self.state[r.q.id]
            reqs.append((r.kv.view(), st.valid, st.pending, r.kv.tokens[-1]))
            cur.append(r.kv.tokens[-1])
        g = self.graphs
        if g is not None and len(reqs) <= g.nmax and all(q[2] is None or q[2].shape[0] <= g.span for q in reqs):
            blocks = g.run(reqs)
            picked = blocks if (self.draft.markov is not None or self.draft.cfg.anchor_first) else [t[1:] for t in blocks]
        else:
            logits = self.draft.block_logits(self.kv, self.page_size, reqs)
            picked = self.draft.pick(logits, cur)
        for r in decoders:
            st = self.state[r.q.id]
            if st.pending is not None:
                st.valid += st.pending.shape[0]
                st.pending = None
        self.rounds += 1
        return {r.q.id: picked[i] for i, r in enumerate(decoders)}
