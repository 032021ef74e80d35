"""Qwen3 dense decoder (GQA, per-head QK-RMSNorm, half-split RoPE, SwiGLU).

Weights are held per tensor-parallel rank: ``qkv`` is the row-concatenation
``[q_rows; k_rows; v_rows]`` of this rank's head shards, ``gate_up`` is
``[gate_rows; up_rows]`` of its FFN shard, ``o``/``down`` are column shards;
embedding, lm_head and norms are replicated.  The forward pass consumes one ragged
step (prefill chunks and decode rows mixed) described by an ``AttnMeta``.

Reference parity: pegainfer-qwen3/src/weights/load.rs:61-286 (tensor names, fused
qkv / gate_up, TP shard ranges, tied embeddings), src/batch_decode.rs:184-399 and
src/prefill.rs:206-490 (layer op order), src/unified_forward.rs:138-613 (mixed step).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..loader.sources import RandomSource, WeightSource, shard_range
from ..ops.reference import AttnMeta, rope_tables
from ..parallel.tp import SINGLE, TPContext


def qwen3_shapes(cfg: ModelConfig) -> dict:
    """HF tensor names -> full (unsharded) shapes."""
    h, d = cfg.hidden_size, cfg.head_dim
    s = {"model.embed_tokens.weight": (cfg.vocab_size, h), "model.norm.weight": (h,)}
    if not cfg.tie_word_embeddings:
        s["lm_head.weight"] = (cfg.vocab_size, h)
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        s[p + "input_layernorm.weight"] = (h,)
        s[p + "post_attention_layernorm.weight"] = (h,)
        s[p + "self_attn.q_proj.weight"] = (cfg.num_q_heads * d, h)
        s[p + "self_attn.k_proj.weight"] = (cfg.num_kv_heads * d, h)
        s[p + "self_attn.v_proj.weight"] = (cfg.num_kv_heads * d, h)
        s[p + "self_attn.o_proj.weight"] = (h, cfg.num_q_heads * d)
        s[p + "self_attn.q_norm.weight"] = (d,)
        s[p + "self_attn.k_norm.weight"] = (d,)
        s[p + "mlp.gate_proj.weight"] = (cfg.intermediate_size, h)
        s[p + "mlp.up_proj.weight"] = (cfg.intermediate_size, h)
        s[p + "mlp.down_proj.weight"] = (h, cfg.intermediate_size)
    return s


@dataclass
class Qwen3Layer:
    input_norm: torch.Tensor
    qkv: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    o: torch.Tensor
    post_norm: torch.Tensor
    gate_up: torch.Tensor
    down: torch.Tensor


class Qwen3Model:
    family = "qwen3"

    def __init__(self, cfg: ModelConfig, source: Optional[WeightSource] = None, device="cpu", dtype=torch.bfloat16, tp: TPContext = SINGLE, seed: int = 0):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self.tp = tp
        if cfg.num_q_heads % tp.world or cfg.num_kv_heads % tp.world or cfg.intermediate_size % tp.world:
            raise ValueError(f"heads {cfg.num_q_heads}/{cfg.num_kv_heads} and FFN {cfg.intermediate_size} must divide tp={tp.world}")
        self.lora = None  # set by lora.manager.LoraManager
        self.q_heads = cfg.num_q_heads // tp.world
        self.kv_heads = cfg.num_kv_heads // tp.world
        source = source or RandomSource(qwen3_shapes(cfg), seed=seed, dtype=dtype)
        self.gate_up_interleaved = False
        self._load(source)
        self.cos, self.sin = rope_tables(cfg.max_position, cfg.rotary_dim, cfg.rope_theta, dtype, self.device)
        # Decode steps on one GPU run a fused chain: SwiGLU inside the gate_up GEMM (its weight rows
        # interleaved as gate_0, up_0, gate_1, ...) and the residual add + RMSNorm folded into the
        # row-parallel GEMMs and their consumers.  PEGAINFER_FUSED_DECODE=0 keeps the separate kernels.
        import os

        chain_tp = tp.world > 1 and tp.comm == "chain"
        self.fused_decode = self.device.type == "cuda" and (tp.world == 1 or chain_tp) and dtype == torch.bfloat16 and os.environ.get("PEGAINFER_FUSED_DECODE", "1") != "0"
        if self.fused_decode:
            self.set_gate_up_layout(True)
        # With the chain collective the output projection is sharded by vocabulary as well: each rank
        # streams 1 / world of lm_head and the ranks exchange (best value, index) pairs or logits.
        self.vocab_sharded = chain_tp and cfg.vocab_size % tp.world == 0
        if self.vocab_sharded:
            v0, v1 = shard_range(cfg.vocab_size, tp.rank, tp.world)
            self.vocab_range = (v0, v1)
            self.lm_head = self.lm_head[v0:v1] if self.lm_head is self.embed else self.lm_head[v0:v1].contiguous()

    def set_gate_up_layout(self, interleaved: bool) -> None:
        """Reorder the rows of every fused gate_up weight in place: ``[gate; up]`` halves
        (``interleaved=False``; what adapter deltas address) or alternating (gate_i, up_i) rows
        (what the fused SwiGLU epilogue reads)."""
        if interleaved == self.gate_up_interleaved:
            return
        for l in self.layers:
            w = l.gate_up
            i = w.shape[0] // 2
            if interleaved:
                l.gate_up = torch.stack((w[:i], w[i:]), 1).reshape(w.shape).contiguous()
            else:
                l.gate_up = torch.cat((w[0::2], w[1::2]), 0).contiguous()
            del w
        self.gate_up_interleaved = interleaved

    # -- loading ---------------------------------------------------------------
    def _load(self, src: WeightSource) -> None:
        cfg, dev, dt, tp = self.cfg, self.device, self.dtype, self.tp
        d = cfg.head_dim
        self.embed = src.get("model.embed_tokens.weight", dev, dt)
        self.lm_head = self.embed if cfg.tie_word_embeddings else src.get("lm_head.weight", dev, dt)
        self.final_norm = src.get("model.norm.weight", dev, dt)
        qr = shard_range(cfg.num_q_heads, tp.rank, tp.world)
        kr = shard_range(cfg.num_kv_heads, tp.rank, tp.world)
        fr = shard_range(cfg.intermediate_size, tp.rank, tp.world)
        self.layers = []
        for i in range(cfg.num_layers):
            p = f"model.layers.{i}."
            q = src.get(p + "self_attn.q_proj.weight", dev, dt, rows=(qr[0] * d, qr[1] * d))
            k = src.get(p + "self_attn.k_proj.weight", dev, dt, rows=(kr[0] * d, kr[1] * d))
            v = src.get(p + "self_attn.v_proj.weight", dev, dt, rows=(kr[0] * d, kr[1] * d))
            g = src.get(p + "mlp.gate_proj.weight", dev, dt, rows=fr)
            u = src.get(p + "mlp.up_proj.weight", dev, dt, rows=fr)
            self.layers.append(
                Qwen3Layer(
                    input_norm=src.get(p + "input_layernorm.weight", dev, dt),
                    qkv=torch.cat([q, k, v], 0),
                    q_norm=src.get(p + "self_attn.q_norm.weight", dev, dt),
                    k_norm=src.get(p + "self_attn.k_norm.weight", dev, dt),
                    o=src.get(p + "self_attn.o_proj.weight", dev, dt, cols=(qr[0] * d, qr[1] * d)),
                    post_norm=src.get(p + "post_attention_layernorm.weight", dev, dt),
                    gate_up=torch.cat([g, u], 0),
                    down=src.get(p + "mlp.down_proj.weight", dev, dt, cols=fr),
                )
            )
            del q, k, v, g, u

    def weight_bytes(self) -> int:
        n = self.embed.numel() + self.final_norm.numel()
        if self.lm_head is not self.embed:
            n += self.lm_head.numel()
        for l in self.layers:
            n += sum(t.numel() for t in (l.input_norm, l.qkv, l.q_norm, l.k_norm, l.o, l.post_norm, l.gate_up, l.down))
        return n * self.embed.element_size()

    # -- KV geometry -----------------------------------------------------------
    def kv_geometry(self) -> dict:
        return dict(num_layers=self.cfg.num_layers, kv_heads=self.kv_heads, head_dim=self.cfg.head_dim)

    # -- forward -----------------------------------------------------------------
    def forward_hidden(self, token_ids: torch.Tensor, meta: AttnMeta, kv, aux_layers=()) -> torch.Tensor:
        """Returns final-normed hidden states ``[T, hidden]`` for every input row.
        ``aux_layers``: layer indices whose residual-stream output is captured into
        ``self.last_aux`` (speculative drafters consume target hidden states)."""
        cfg, tp = self.cfg, self.tp
        eps = cfg.rms_eps
        tp.begin_step()
        residual = ops.embedding(token_ids, self.embed)
        x = ops.rms_norm(residual, self.layers[0].input_norm, eps)
        aux = []
        n = len(self.layers)
        il = self.gate_up_interleaved
        fused = self._fused_chain_ok(meta)
        if fused:
            from ..ops import cuda as K

            if self._chain_ok(meta):
                return self._forward_chain(x, residual, meta, kv, aux_layers, K)
        for i, l in enumerate(self.layers):
            ls = meta.lora_slots if self.lora is not None else None
            decode = ls is None and meta.num_tokens <= 256  # weight-streaming regime: chain L2 prefetches GEMM to GEMM
            if decode:
                ops.prefetch_weights(l.o)
            if fused:
                qkv = K.linear_fused(x, l.qkv)  # completes the previous layer's deferred norm, if any
            else:
                qkv = tp.col_linear(x, l.qkv)
            if ls is not None:
                qs, ks = self.q_heads * cfg.head_dim, self.kv_heads * cfg.head_dim
                self.lora.apply_shared(i, ("q_proj", "k_proj", "v_proj"), x, (qkv[:, :qs], qkv[:, qs : qs + ks], qkv[:, qs + ks :]), ls)
            q = ops.qk_norm_rope_append(qkv, l.q_norm, l.k_norm, self.cos, self.sin, meta, kv.layer(i), self.q_heads, self.kv_heads, cfg.head_dim, eps)
            a = ops.paged_attention(q, kv.layer(i), meta)
            next_norm = self.layers[i + 1].input_norm if i + 1 < n else self.final_norm
            if fused:
                # o_proj (+ residual, x post_norm weight) -> gate_up (x inverse RMS, SwiGLU) -> down (+ residual,
                # x next norm weight); the next qkv GEMM (or the final norm kernel) completes the last norm
                ops.prefetch_weights(l.gate_up)
                xd = K.linear_fused(a, l.o, K.EPI_RESID_NORMW, residual=residual, norm_w=l.post_norm, eps=eps)
                ops.prefetch_weights(l.down)
                act = K.linear_fused(xd, l.gate_up, K.EPI_SWIGLU)
                last = i + 1 == n or i in aux_layers
                if last:
                    ops.prefetch_weights(self.layers[i + 1].qkv if i + 1 < n else self.lm_head)
                    x = ops.add_rms_norm(K.linear(act, l.down), residual, next_norm, eps)
                else:
                    ops.prefetch_weights(self.layers[i + 1].qkv)
                    x = K.linear_fused(act, l.down, K.EPI_RESID_NORMW, residual=residual, norm_w=next_norm, eps=eps)
            elif ls is None:
                if decode:
                    ops.prefetch_weights(l.gate_up)
                x = tp.row_linear_add_norm(a, l.o, residual, l.post_norm, eps)
                if decode:
                    ops.prefetch_weights(l.down)
                act = None
                if il and tp.world == 1 and x.is_cuda and ops.get_mode() == "sm100":
                    from ..ops import cuda as Kc

                    act = Kc.linear_swiglu_2sm(x, l.gate_up)  # prefill-sized steps: SwiGLU in the epilogue of the two-SM GEMM
                if act is None:
                    act = ops.swiglu(tp.col_linear(x, l.gate_up), il)
                if decode:
                    ops.prefetch_weights(self.layers[i + 1].qkv if i + 1 < n else self.lm_head)
                x = tp.row_linear_add_norm(act, l.down, residual, next_norm, eps)
            else:  # adapter deltas join the partial sums before the all-reduce
                y = ops.linear(a, l.o)
                self.lora.apply(i, "o_proj", a, y, ls)
                x = ops.add_rms_norm(tp.all_reduce(y), residual, l.post_norm, eps)
                gu = ops.linear(x, l.gate_up)
                ff = gu.shape[1] // 2
                self.lora.apply_shared(i, ("gate_proj", "up_proj"), x, (gu[:, :ff], gu[:, ff:]), ls)
                act = ops.swiglu(gu)
                y = ops.linear(act, l.down)
                self.lora.apply(i, "down_proj", act, y, ls)
                x = ops.add_rms_norm(tp.all_reduce(y), residual, next_norm, eps)
            if i in aux_layers:
                aux.append(residual.clone())
        self.last_aux = aux
        tp.sync()
        return x

    def _chain_ok(self, meta: AttnMeta) -> bool:
        """One persistent kernel per layer for the four projections behind attention (o_proj, gate_up,
        down, the next layer's qkv): steps of up to 64 rows, hidden size a multiple of 128 up to 8192."""
        import os

        from ..ops import cuda as K

        h = self.cfg.hidden_size
        # never on the prefill lane: the chain kernel's grid barriers need all of its CTAs resident at once, which a
        # second chain kernel on the main stream, or a lane confined to part of the SMs, does not allow
        return os.environ.get("PEGAINFER_DECODE_CHAIN", "1") != "0" and h % 128 == 0 and h <= 8192 and self.gate_up_interleaved and K._LANE[0] == 0

    def _forward_chain(self, x, residual, meta, kv, aux_layers, K):
        cfg, eps, n = self.cfg, self.cfg.rms_eps, len(self.layers)
        aux = []
        # 128-wide heads with full rotary: QK-norm, RoPE and the KV append run in the epilogue of the qkv phase
        rope_fused = cfg.head_dim == 128 and cfg.rotary_dim == 128

        def qkv_phase(i):
            l = self.layers[i]
            if not rope_fused:
                return (l.qkv, K.CH_PLAIN, None, False)
            spec = dict(q_norm=l.q_norm, k_norm=l.k_norm, cos=self.cos, sin=self.sin, meta=meta, kv_layer=kv.layer(i), hq=self.q_heads, hkv=self.kv_heads, eps=eps)
            return (l.qkv, K.CH_QKV_ROPE, spec, False)

        tpc = self.tp if self.tp.world > 1 else None
        q = K.decode_chain(x, [qkv_phase(0)])[0]
        for i, l in enumerate(self.layers):
            if not rope_fused:
                q = ops.qk_norm_rope_append(q, l.q_norm, l.k_norm, self.cos, self.sin, meta, kv.layer(i), self.q_heads, self.kv_heads, cfg.head_dim, eps)
            a = ops.paged_attention(q, kv.layer(i), meta)
            phases = [(l.o, K.CH_RESID_NORM, l.post_norm, False), (l.gate_up, K.CH_SWIGLU, None, False)]
            if i + 1 < n:
                phases += [(l.down, K.CH_RESID_NORM, self.layers[i + 1].input_norm, False), qkv_phase(i + 1)]
                outs = K.decode_chain(a, phases, residual=residual, eps=eps, tp=tpc)
                q = outs[3]
            else:
                phases += [(l.down, K.CH_RESID_NORM, self.final_norm, False)]
                outs = K.decode_chain(a, phases, residual=residual, eps=eps, tp=tpc)
            x = outs[2]  # final-norm weight applied, per-token scale still owed: the lm_head GEMM completes it
            if i in aux_layers:
                aux.append(residual.clone())
        self.last_aux = aux
        if tpc is not None:
            tpc.sites_by_rows[int(meta.num_tokens)] = (2 * n, 0)
        return x

    def _fused_chain_ok(self, meta: AttnMeta) -> bool:
        """The fused decode chain serves steps of up to 64 token rows without adapter deltas, when every
        projection plans onto the GEMM's on-chip split-K path (decided once per row count)."""
        if not self.fused_decode or self.lora is not None or meta.num_tokens > 64 or ops.get_mode() != "sm100":
            return False
        if self.tp.world > 1:  # tensor parallel: only the chain kernel carries a collective
            from ..ops import cuda as K

            return self._chain_ok(meta) and not K.batch_invariant()
        from ..ops import cuda as K

        t = int(meta.num_tokens)
        ok = self._fused_ok.get(t) if hasattr(self, "_fused_ok") else None
        if ok is None:
            if not hasattr(self, "_fused_ok"):
                self._fused_ok = {}
            l = self.layers[0]
            ok = all(K.fused_plan_ok(t, w.shape[0], w.shape[1]) for w in (l.qkv, l.o, l.gate_up, l.down)) and self.cfg.hidden_size % 128 == 0
            self._fused_ok[t] = ok
        return ok and not K.batch_invariant()

    def logits(self, hidden, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not isinstance(hidden, torch.Tensor):  # rows from the decode chain whose final RMSNorm scale is still owed
            from ..ops import cuda as K

            if rows is not None:
                hidden = K.DeferredNorm(ops.gather_rows(hidden.xw, rows), hidden.ssp.index_select(0, rows.long()), hidden.parts, hidden.width, hidden.eps)
            return K.linear_fused(hidden, self.lm_head)
        if rows is not None:
            hidden = ops.gather_rows(hidden, rows)
        return ops.linear(hidden, self.lm_head)

    def full_logits(self, logits: torch.Tensor) -> torch.Tensor:
        """All-gather vocabulary-sharded logits ``[T, V / world]`` into ``[T, V]`` (a no-op otherwise)."""
        if not getattr(self, "vocab_sharded", False):
            return logits
        import torch.distributed as dist

        t, vs = logits.shape
        out = torch.empty((self.tp.world, t, vs), dtype=logits.dtype, device=logits.device)
        dist.all_gather_into_tensor(out, logits.contiguous(), group=self.tp.group)
        return out.permute(1, 0, 2).reshape(t, self.tp.world * vs)

    def greedy_tokens(self, logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Row-wise argmax (ties -> lowest index).  With vocabulary-sharded logits every rank finds
        its local best and the ranks exchange (value, index) pairs: 8 bytes per row and rank
        instead of the logits (reference: pegainfer-kernels csrc/shared/argmax.cu sharded argmax)."""
        if not getattr(self, "vocab_sharded", False):
            if out is not None and logits.is_cuda and ops.get_mode() != "library":
                from ..ops import cuda as K

                return K.argmax(logits, out=out)
            res = ops.argmax(logits)
            if out is not None:
                out.copy_(res)
                return out
            return res
        import torch.distributed as dist

        w = self.tp.world
        idx = ops.argmax(logits)  # local index, ties -> lowest
        val = logits.float().gather(1, idx.long().unsqueeze(1)).squeeze(1)
        pair = torch.stack((val, (idx + self.vocab_range[0]).float()), 1)  # indices below 2^24 are exact in f32
        allp = torch.empty((w,) + tuple(pair.shape), dtype=torch.float32, device=logits.device)
        dist.all_gather_into_tensor(allp, pair, group=self.tp.group)
        vals, ids = allp[:, :, 0], allp[:, :, 1]
        best = vals.max(0, keepdim=True).values
        ranks = torch.arange(w, device=logits.device).unsqueeze(1).expand_as(vals)
        first = torch.where(vals == best, ranks, torch.full_like(ranks, w)).min(0).values  # lowest rank = lowest index on ties
        tok = ids.gather(0, first.unsqueeze(0)).squeeze(0).to(torch.int32)
        if out is not None:
            out.copy_(tok)
            return out
        return tok

    def forward(self, token_ids, meta, kv, logits_rows=None):
        return self.full_logits(self.logits(self.forward_hidden(token_ids, meta, kv), logits_rows))
