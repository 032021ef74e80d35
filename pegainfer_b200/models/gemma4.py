"""Gemma 4 dense text decoder: sliding-window layers interleaved with global layers of a wider head.

Per layer (the released pattern is five sliding layers, then one global):

* sliding layer: ``head_dim`` (256) query / key / value heads, ``num_kv_heads`` KV heads, full half-split RoPE with
  ``rope_theta_local``, causal attention over the last ``sliding_window`` keys;
* global layer: ``global_head_dim`` (512) heads, ``num_global_kv_heads`` KV heads, RoPE on a quarter of the head
  ("proportional": the first ``partial_rotary_factor * d / 2`` frequency pairs (i, i + d / 2) rotate with
  ``rope_theta ** (-2 i / d)``, the others are the identity), full causal attention; with ``attention_k_eq_v`` there is no
  value projection and V is the key projection before key norm and RoPE;
* every layer: per-head RMSNorm on Q and K (weights), weightless per-head RMSNorm on V, softmax scale 1, "sandwich"
  norms (input / post-attention / pre-feed-forward / post-feed-forward), GeGLU (tanh) feed-forward, a per-layer output
  scalar; embeddings scaled by sqrt(hidden) (rounded to the activation dtype), tied output projection, optional
  soft-capping of the final logits.

KV cache: one row width for all layers, ``max(kv_heads * head_dim, global_kv_heads * global_head_dim)`` elements per
token and K / V; a layer whose own width is smaller keeps its pages packed at the front of its slab (prefix caching and
KV offload then do not apply: a page of such a layer is not the page-sized slice of the slab).  The small
variants' per-layer input embeddings, cross-layer KV sharing and the mixture-of-experts block are not built.

Reference parity: pegainfer-gemma4/src/layer.rs, src/engine.rs (layer order, the two KV families), pegainfer-kernels
csrc/shared/prefill_attention_hd256_plain.cu:44-540 (plain-weight norms, v_norm, runtime rotary dim),
csrc/shared/prefill_attention_hd512.cu:64-540 and paged_attention_hd512.cu:71-224 (global layers).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..loader.sources import RandomSource, WeightSource
from ..ops.reference import AttnMeta, rope_tables
from ..parallel.tp import SINGLE, TPContext


def _is_global(cfg: ModelConfig, i: int) -> bool:
    return cfg.layer_type(i) == "full_attention"


def _geom(cfg: ModelConfig, i: int) -> tuple:
    """(head dim, KV heads) of layer ``i``."""
    if _is_global(cfg, i):
        return cfg.global_head_dim or cfg.head_dim, cfg.num_global_kv_heads or cfg.num_kv_heads
    return cfg.head_dim, cfg.num_kv_heads


def gemma4_shapes(cfg: ModelConfig) -> dict:
    """HF tensor names -> shapes (``Gemma4ForCausalLM`` over the text model)."""
    h = cfg.hidden_size
    s = {"model.embed_tokens.weight": (cfg.vocab_size, h), "model.norm.weight": (h,)}
    if not cfg.tie_word_embeddings:
        s["lm_head.weight"] = (cfg.vocab_size, h)
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        d, hkv = _geom(cfg, i)
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            s[p + n + ".weight"] = (h,)
        s[p + "layer_scalar"] = (1,)
        s[p + "self_attn.q_proj.weight"] = (cfg.num_q_heads * d, h)
        s[p + "self_attn.k_proj.weight"] = (hkv * d, h)
        if not (cfg.attention_k_eq_v and _is_global(cfg, i)):
            s[p + "self_attn.v_proj.weight"] = (hkv * d, h)
        s[p + "self_attn.o_proj.weight"] = (h, cfg.num_q_heads * d)
        s[p + "self_attn.q_norm.weight"] = (d,)
        s[p + "self_attn.k_norm.weight"] = (d,)
        s[p + "mlp.gate_proj.weight"] = (cfg.intermediate_size, h)
        s[p + "mlp.up_proj.weight"] = (cfg.intermediate_size, h)
        s[p + "mlp.down_proj.weight"] = (h, cfg.intermediate_size)
    return s


def _kind(name: str) -> str:
    """Random-weight distributions.  The softmax scale of this line is 1 and Q / K are RMS-normalised per head, so
    unit norm weights would give scores of standard deviation sqrt(head_dim) and a softmax that is an argmax; the
    released checkpoints carry learned norm weights well below one."""
    if name.endswith("q_norm.weight") or name.endswith("k_norm.weight"):
        return "const:0.25"
    return RandomSource._default_kind(name)


def gemma4_source(cfg: ModelConfig, seed: int = 0, dtype=torch.bfloat16) -> RandomSource:
    return RandomSource(gemma4_shapes(cfg), seed=seed, dtype=dtype, kind=_kind)


def proportional_rope_tables(max_pos: int, head_dim: int, fraction: float, theta: float, dtype, device):
    """cos / sin ``[max_pos, head_dim / 2]`` of the global layers: ``int(fraction * head_dim // 2)`` rotating pairs with
    ``theta ** (-2 i / head_dim)``, angle zero (the identity) for the other pairs."""
    half = head_dim // 2
    angles = int(fraction * head_dim // 2)
    inv = torch.zeros(half, dtype=torch.float64)
    inv[:angles] = 1.0 / (theta ** (torch.arange(0, 2 * angles, 2, dtype=torch.float64) / head_dim))
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), inv)
    return ang.cos().float().to(dtype).to(device), ang.sin().float().to(dtype).to(device)


@dataclass
class Gemma4Layer:
    is_global: bool
    head_dim: int
    kv_heads: int
    input_norm: torch.Tensor
    qkv: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    o: torch.Tensor
    post_attn_norm: torch.Tensor
    pre_ffn_norm: torch.Tensor
    gate_up: torch.Tensor
    down: torch.Tensor
    post_ffn_norm: torch.Tensor
    scalar: float


class Gemma4Model:
    family = "gemma4"
    supports_prefix_cache = True

    def __init__(self, cfg: ModelConfig, source: Optional[WeightSource] = None, device="cpu", dtype=torch.bfloat16, tp: TPContext = SINGLE, seed: int = 0):
        if tp.world != 1:
            raise ValueError("the Gemma 4 line runs on one GPU")
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype
        self.tp = tp
        self.lora = None
        source = source or gemma4_source(cfg, seed=seed, dtype=dtype)
        self._load(source)
        dg = cfg.global_head_dim or cfg.head_dim
        self.cos_l, self.sin_l = rope_tables(cfg.max_position, cfg.head_dim, cfg.rope_theta_local, dtype, self.device)
        self.cos_g, self.sin_g = proportional_rope_tables(cfg.max_position, dg, cfg.partial_rotary_factor, cfg.rope_theta, dtype, self.device)
        widths = {l.kv_heads * l.head_dim for l in self.layers}
        self.kv_width = max(widths)
        # one width for all layers: a layer's slab is exactly its pages; otherwise narrower layers pack their pages at
        # the front of the slab and block-wise copies (prefix cache, KV offload) do not see whole pages
        self.supports_prefix_cache = len(widths) == 1

    def _load(self, src: WeightSource) -> None:
        cfg, dev, dt = self.cfg, self.device, self.dtype
        emb = src.get("model.embed_tokens.weight", dev, dt)
        self.lm_head = emb if cfg.tie_word_embeddings else src.get("lm_head.weight", dev, dt)
        # the embedding lookup is followed by a multiplication with sqrt(hidden) rounded to the activation dtype and the
        # product is rounded again: the same numbers as a table multiplied once
        self.embed = (emb.float() * torch.tensor(cfg.hidden_size ** 0.5, dtype=dt).float()).to(dt)
        self.final_norm = src.get("model.norm.weight", dev, dt)
        self.layers = []
        for i in range(cfg.num_layers):
            p = f"model.layers.{i}."
            d, hkv = _geom(cfg, i)
            q = src.get(p + "self_attn.q_proj.weight", dev, dt)
            k = src.get(p + "self_attn.k_proj.weight", dev, dt)
            v = k if (cfg.attention_k_eq_v and _is_global(cfg, i)) else src.get(p + "self_attn.v_proj.weight", dev, dt)
            g = src.get(p + "mlp.gate_proj.weight", dev, dt)
            u = src.get(p + "mlp.up_proj.weight", dev, dt)
            sc = src.get(p + "layer_scalar", dev, torch.float32) if src.has(p + "layer_scalar") else torch.ones(1)
            self.layers.append(
                Gemma4Layer(
                    is_global=_is_global(cfg, i),
                    head_dim=d,
                    kv_heads=hkv,
                    input_norm=src.get(p + "input_layernorm.weight", dev, dt),
                    qkv=torch.cat([q, k, v], 0),
                    q_norm=src.get(p + "self_attn.q_norm.weight", dev, dt),
                    k_norm=src.get(p + "self_attn.k_norm.weight", dev, dt),
                    o=src.get(p + "self_attn.o_proj.weight", dev, dt),
                    post_attn_norm=src.get(p + "post_attention_layernorm.weight", dev, dt),
                    pre_ffn_norm=src.get(p + "pre_feedforward_layernorm.weight", dev, dt),
                    gate_up=torch.cat([g, u], 0),
                    down=src.get(p + "mlp.down_proj.weight", dev, dt),
                    post_ffn_norm=src.get(p + "post_feedforward_layernorm.weight", dev, dt),
                    scalar=float(sc.float().reshape(-1)[0].item()),
                )
            )
            del q, k, v, g, u

    def weight_bytes(self) -> int:
        n = self.embed.numel() + self.final_norm.numel() + self.lm_head.numel()
        for l in self.layers:
            n += sum(t.numel() for t in (l.input_norm, l.qkv, l.q_norm, l.k_norm, l.o, l.post_attn_norm, l.pre_ffn_norm, l.gate_up, l.down, l.post_ffn_norm))
        return n * self.embed.element_size()

    # -- KV geometry -----------------------------------------------------------
    def kv_geometry(self) -> dict:
        return dict(num_layers=self.cfg.num_layers, kv_heads=1, head_dim=self.kv_width)

    def _kv_layer(self, kv, i: int) -> torch.Tensor:
        """``[pages, 2, page_size, kv_heads, head_dim]`` of layer ``i`` inside its slab of the common row width."""
        l = self.layers[i]
        slab = kv.layer(i)  # [pages, 2, page_size, 1, kv_width]
        pages, _, page = slab.shape[0], slab.shape[1], slab.shape[2]
        n = pages * 2 * page * l.kv_heads * l.head_dim
        return slab.reshape(-1)[:n].view(pages, 2, page, l.kv_heads, l.head_dim)

    # -- forward -----------------------------------------------------------------
    def forward_hidden(self, token_ids: torch.Tensor, meta: AttnMeta, kv, aux_layers=()) -> torch.Tensor:
        cfg = self.cfg
        eps = cfg.rms_eps
        residual = ops.embedding(token_ids, self.embed)
        x = ops.rms_norm(residual, self.layers[0].input_norm, eps)
        n = len(self.layers)
        aux = []
        for i, l in enumerate(self.layers):
            kvl = self._kv_layer(kv, i)
            cos, sin = (self.cos_g, self.sin_g) if l.is_global else (self.cos_l, self.sin_l)
            qkv = ops.linear(x, l.qkv)
            q = ops.qk_norm_rope_append(qkv, l.q_norm, l.k_norm, cos, sin, meta, kvl, cfg.num_q_heads, l.kv_heads, l.head_dim, eps, v_norm=True)
            a = ops.paged_attention(q.reshape(x.shape[0], cfg.num_q_heads, l.head_dim), kvl, meta, 1.0, 0 if l.is_global else cfg.sliding_window)
            t = ops.rms_norm(ops.linear(a, l.o), l.post_attn_norm, eps)
            x = ops.add_rms_norm(t, residual, l.pre_ffn_norm, eps)  # residual += t
            act = ops.geglu(ops.linear(x, l.gate_up))
            t = ops.rms_norm(ops.linear(act, l.down), l.post_ffn_norm, eps)
            next_norm = self.layers[i + 1].input_norm if i + 1 < n else self.final_norm
            if l.scalar == 1.0:
                x = ops.add_rms_norm(t, residual, next_norm, eps)
            else:  # the layer's output, residual included, is multiplied by its scalar
                residual.copy_(((residual.float() + t.float()).to(residual.dtype).float() * l.scalar).to(residual.dtype))
                x = ops.rms_norm(residual, next_norm, eps)
            if i in aux_layers:
                aux.append(residual.clone())
        self.last_aux = aux
        self.last_residual = residual
        return x

    def logits(self, hidden, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if rows is not None:
            hidden = ops.gather_rows(hidden, rows)
        lg = ops.linear(hidden, self.lm_head)
        if self.cfg.final_logit_softcapping > 0:
            lg = ops.softcap(lg, self.cfg.final_logit_softcapping)
        return lg

    def forward(self, token_ids, meta, kv, logits_rows=None):
        return self.logits(self.forward_hidden(token_ids, meta, kv), logits_rows)
