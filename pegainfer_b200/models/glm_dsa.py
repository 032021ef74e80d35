"""GLM-5 line: MLA + MoE decoder with a sparse-attention indexer (DSA) and a native MTP layer.

The decoder is the MLA + MoE model of ``models.mla_moe`` (absorbed latent attention over a paged
latent cache, sigmoid router with correction bias, shared expert, block-scaled FP8 or bf16 experts,
one multi-token-prediction layer) with one addition per layer: an *indexer*.  The indexer projects
the query's low-rank residual to ``index_n_heads`` small heads and the hidden state to ONE small key
per token (LayerNorm, rotary on the leading dims), keeps those keys in a paged cache of their own,
and scores every earlier token as ``sum_h w_h * relu(q_h . k)``.  The main attention then looks only
at the ``index_topk`` best-scoring keys of each query, so its cost stops growing with the context.
While a sequence is no longer than ``index_topk`` every key is kept and the step takes the dense
path; beyond that the selected latent rows are gathered and the dense latent kernel runs over them
(attention does not care about key order, and the rotary phase is already in the cached keys).

The checkpoints rotate q_pe / k_pe in the half-split convention; this package's latent kernels
rotate adjacent pairs.  The rows that produce those dims are reordered once at load (pair
``(i, i + d/2)`` becomes ``(2i, 2i + 1)``), which leaves every score unchanged.

Reference parity: pegainfer-glm52/src/{config.rs, indexer.rs, mla_front.rs, mla_decode.rs, mtp.rs,
model/mod.rs} (indexer: 32 heads x 128, top-2048, own key cache; sparse MLA decode; native MTP),
pegainfer-kernels/csrc/glm52/{glm52_indexer*.cu, glm52_topk.cu, glm52_deepgemm_mqa.cu}.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..kv.buffer import LatentKvBuffer
from ..loader.sources import WeightSource
from ..ops.reference import AttnMeta
from .mla_moe import MlaLayer, MlaMoeModel, load_dense, mla_moe_shapes


def glm_dsa_shapes(cfg: ModelConfig) -> dict:
    s = mla_moe_shapes(cfg)
    hi, di = cfg.index_n_heads, cfg.index_head_dim
    for i in range(cfg.num_layers + cfg.num_mtp_layers):
        p = f"model.layers.{i}.self_attn.indexer."
        s.update({p + "wq_b.weight": (hi * di, cfg.q_lora_rank), p + "wk.weight": (di, cfg.hidden_size), p + "k_norm.weight": (di,), p + "k_norm.bias": (di,),
                  p + "weights_proj.weight": (hi, cfg.hidden_size)})
        if cfg.dense_quant == "fp8_block128" and (hi * di) % 128 == 0 and cfg.q_lora_rank % 128 == 0:
            s[p + "wq_b.weight_scale_inv"] = (hi * di // 128, cfg.q_lora_rank // 128)
    return s


def _pairs_from_halves(w, start: int, width: int) -> None:
    """In place: rows ``start .. start + width`` go from half-split order (i, i + width/2) to adjacent pairs.
    An FP8 matrix is reordered in its e4m3 rows; the rows of one rotary block share one 128-row scale block."""
    if isinstance(w, ops.Fp8Weight):
        if start // 128 != (start + width - 1) // 128:
            raise ValueError("rotary rows straddle two FP8 scale blocks")
        q = w.q.view(torch.uint8)
        _pairs_from_halves(q, start, width)
        return
    blk = w[start : start + width]
    half = width // 2
    w[start : start + width] = torch.stack((blk[:half], blk[half:]), 1).reshape(blk.shape)


class _GlmKv(LatentKvBuffer):
    """Latent cache plus the indexer's key cache; both are addressed by the same page ids."""

    def __init__(self, num_layers, num_pages, page_size, width, index_width, dtype, device):
        super().__init__(num_layers, num_pages, page_size, width, dtype, device)
        self.index = LatentKvBuffer(num_layers, num_pages, page_size, index_width, dtype, device)


class GlmDsaModel(MlaMoeModel):
    def __init__(self, cfg: ModelConfig, source: Optional[WeightSource] = None, device="cpu", dtype=torch.bfloat16, seed: int = 0, **kw):
        if not cfg.q_lora_rank or not cfg.index_n_heads:
            raise ValueError("the GLM-5 line needs q_lora_rank and an indexer (index_n_heads > 0)")
        if source is None:
            from .mla_moe import _QuantRandomSource

            source = _QuantRandomSource(glm_dsa_shapes(cfg), seed=seed, dtype=dtype)
        self._index_kv = None
        super().__init__(cfg, source, device, dtype, seed=seed, **kw)
        self.index_scale = cfg.index_n_heads ** -0.5 * cfg.index_head_dim ** -0.5

    def _load_layer(self, src: WeightSource, i: int) -> MlaLayer:
        cfg, dev, dt = self.cfg, self.device, self.dtype
        L = super()._load_layer(src, i)
        qk, nope, rope = cfg.qk_head_dim, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim
        for h in range(cfg.num_q_heads):
            _pairs_from_halves(L.q_b, h * qk + nope, rope)
        _pairs_from_halves(L.kv_a, cfg.kv_lora_rank, rope)
        p = f"{self.P}layers.{i}.self_attn.indexer."
        L.layer_index = i
        L.idx_wq_b = load_dense(src, p + "wq_b.weight", dev, dt, cfg)
        L.idx_wk = src.get(p + "wk.weight", dev, dt)
        L.idx_k_norm_w = src.get(p + "k_norm.weight", dev, torch.float32)
        L.idx_k_norm_b = src.get(p + "k_norm.bias", dev, torch.float32)
        L.idx_wproj = src.get(p + "weights_proj.weight", dev, dt)
        return L

    # -- KV geometry ---------------------------------------------------------------
    def kv_geometry(self) -> dict:
        g = super().kv_geometry()
        n, w = g["num_layers"], self.latent_width + self.cfg.index_head_dim
        g["bytes_per_block"] = lambda page: n * page * w * 2
        return g

    def make_kv(self, num_pages: int, page_size: int):
        n = self.cfg.num_layers + (1 if self.mtp is not None else 0)
        return _GlmKv(n, num_pages, page_size, self.latent_width, self.cfg.index_head_dim, self.dtype, self.device)

    # -- attention -------------------------------------------------------------------
    def attention(self, L: MlaLayer, x, meta: AttnMeta, latent_layer):
        cfg = self.cfg
        t = x.shape[0]
        qa = ops.rms_norm(ops.linear(x, L.q_a), L.q_a_norm, cfg.rms_eps)
        q = ops.linear(qa, L.q_b).view(t, cfg.num_q_heads, cfg.qk_head_dim)
        kv_a = ops.linear(x, L.kv_a)
        ops.mla_append(kv_a, L.kv_a_norm, self.cos, self.sin, meta, latent_layer, cfg.kv_lora_rank, cfg.rms_eps)
        q = ops.mla_rope_q(q, self.cos, self.sin, meta, cfg.qk_nope_head_dim)
        # the indexer's key of every row joins its cache whether or not this step needs the selection
        index_layer = self._index_kv.layer(L.layer_index)
        ops.dsa_index_append(ops.linear(x, L.idx_wk), L.idx_k_norm_w, L.idx_k_norm_b, self.cos, self.sin, meta, index_layer)
        if meta.max_kv_len > cfg.index_topk:
            iq = ops.dsa_rope_q(ops.linear(qa, L.idx_wq_b).view(t, cfg.index_n_heads, cfg.index_head_dim), self.cos, self.sin, meta)
            w = ops.linear(x, L.idx_wproj, out_dtype=torch.float32) * self.index_scale
            select = ops.dsa_topk(ops.dsa_index_scores(iq, w, index_layer, meta), cfg.index_topk)
            a = ops.mla_attention_sparse(q, L.w_uk, L.w_uv, latent_layer, meta, self.scale, cfg.kv_lora_rank, select)
        else:
            a = ops.mla_attention(q, L.w_uk, L.w_uv, latent_layer, meta, self.scale, cfg.kv_lora_rank)
        return ops.linear(a, L.o)

    def forward_hidden(self, token_ids, meta: AttnMeta, kv, aux_layers=()):
        self._index_kv = kv.index
        return super().forward_hidden(token_ids, meta, kv, aux_layers)
