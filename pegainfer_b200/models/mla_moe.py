"""MLA + MoE decoder: DeepSeek-V2-Lite and Kimi-K2 shaped models.

Attention is multi-head latent attention in absorbed form over a paged latent cache
(one ``kv_lora_rank + rope`` row per token): q_nope is folded through W_UK so scores
are taken against the compressed KV directly, and W_UV is applied after the softmax.
Layers ``>= first_k_dense_replace`` are mixture-of-experts: a router (softmax top-k, or
sigmoid + correction bias + group-limited top-k with renormalisation and scaling),
routed experts owned by expert-parallel ranks, and always-on shared experts.  Routed
expert weights are bf16 or INT4 group-32 (compressed-tensors pack-quantized).

Reference parity: pegainfer-deepseek-v2-lite/src/{config.rs:69-190, weights.rs:160-325,
host_ops.rs:225-386, runtime/moe.rs:405-656}, pegainfer-kimi-k2/src/{config.rs:16-175,
weights/manifest.rs:600-720, runner/worker/forward.rs:129-259, runner/moe_deepep.rs:243-397},
pegainfer-kernels/csrc/kimi_k2/{kimi_mla.cu, kimi_router.cu:20-97}.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..kv.buffer import LatentKvBuffer
from ..loader.sources import RandomSource, WeightSource, shard_range
from ..ops.reference import AttnMeta, rope_tables
from ..parallel.ep import LOCAL_EP, EPContext
from ..parallel.tp import SINGLE, TPContext


def layer_prefix(cfg: ModelConfig) -> str:
    return "language_model.model." if cfg.family == "kimi_k2" else "model."


def mla_moe_shapes(cfg: ModelConfig) -> dict:
    h = cfg.hidden_size
    P = layer_prefix(cfg)
    top = "language_model." if cfg.family == "kimi_k2" else ""
    s = {P + "embed_tokens.weight": (cfg.vocab_size, h), P + "norm.weight": (h,), top + "lm_head.weight": (cfg.vocab_size, h)}
    qk = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
    n_layers = cfg.num_layers + cfg.num_mtp_layers
    for i in range(n_layers):
        p = f"{P}layers.{i}."
        s[p + "input_layernorm.weight"] = (h,)
        s[p + "post_attention_layernorm.weight"] = (h,)
        a = p + "self_attn."
        if cfg.q_lora_rank:
            s[a + "q_a_proj.weight"] = (cfg.q_lora_rank, h)
            s[a + "q_a_layernorm.weight"] = (cfg.q_lora_rank,)
            s[a + "q_b_proj.weight"] = (cfg.num_q_heads * qk, cfg.q_lora_rank)
        else:
            s[a + "q_proj.weight"] = (cfg.num_q_heads * qk, h)
        s[a + "kv_a_proj_with_mqa.weight"] = (cfg.kv_lora_rank + cfg.qk_rope_head_dim, h)
        s[a + "kv_a_layernorm.weight"] = (cfg.kv_lora_rank,)
        s[a + "kv_b_proj.weight"] = (cfg.num_q_heads * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank)
        s[a + "o_proj.weight"] = (h, cfg.num_q_heads * cfg.v_head_dim)
        m = p + "mlp."
        if i >= cfg.num_layers:  # MTP block: projection of [norm(embed) ; norm(hidden)] and its norms
            s[p + "enorm.weight"] = (h,)
            s[p + "hnorm.weight"] = (h,)
            s[p + "eh_proj.weight"] = (h, 2 * h)
            s[p + "shared_head.norm.weight"] = (h,)
        if cfg.layer_is_moe(i):
            s[m + "gate.weight"] = (cfg.n_routed_experts, h)
            if cfg.router_bias:
                s[m + "gate.e_score_correction_bias"] = (cfg.n_routed_experts,)
            si = cfg.moe_intermediate_size * cfg.n_shared_experts
            if si:
                s[m + "shared_experts.gate_proj.weight"] = (si, h)
                s[m + "shared_experts.up_proj.weight"] = (si, h)
                s[m + "shared_experts.down_proj.weight"] = (h, si)
            I = cfg.moe_intermediate_size
            for e in range(cfg.n_routed_experts):
                ep = f"{m}experts.{e}."
                for name, shp in (("gate_proj", (I, h)), ("up_proj", (I, h)), ("down_proj", (h, I))):
                    if cfg.expert_quant == "int4_g32":
                        s[ep + name + ".weight_packed"] = (shp[0], shp[1] // 8)
                        s[ep + name + ".weight_scale"] = (shp[0], shp[1] // cfg.quant_group_size)
                    elif cfg.expert_quant == "fp8_block128":
                        s[ep + name + ".weight"] = shp
                        s[ep + name + ".weight_scale_inv"] = ((shp[0] + 127) // 128, (shp[1] + 127) // 128)
                    else:
                        s[ep + name + ".weight"] = shp
        else:
            s[m + "gate_proj.weight"] = (cfg.intermediate_size, h)
            s[m + "up_proj.weight"] = (cfg.intermediate_size, h)
            s[m + "down_proj.weight"] = (h, cfg.intermediate_size)
    if cfg.dense_quant == "fp8_block128":
        for name, shp in list(s.items()):
            if _fp8_dense_name(name) and len(shp) == 2 and shp[0] % 128 == 0 and shp[1] % 128 == 0:
                s[name + "_scale_inv"] = (shp[0] // 128, shp[1] // 128)
    return s


_FP8_DENSE = ("q_a_proj.weight", "q_b_proj.weight", "q_proj.weight", "o_proj.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight",
              "shared_experts.gate_proj.weight", "shared_experts.up_proj.weight", "shared_experts.down_proj.weight", "indexer.wq_b.weight")


def _fp8_dense_name(name: str) -> bool:
    return name.endswith(_FP8_DENSE) and ".experts." not in name


def load_dense(src, name, dev, dt, cfg):
    """A projection matrix: bf16, or kept as block-scaled FP8 when the checkpoint stores it that way and the
    model runs its dense projections in FP8."""
    if cfg.dense_quant == "fp8_block128" and dev.type == "cuda" or cfg.dense_quant == "fp8_block128" and dt == torch.float32:
        if src.has(name + "_scale_inv"):
            shp = src.shape(name)
            if len(shp) == 2 and shp[0] % 128 == 0 and shp[1] % 128 == 0:
                return ops.Fp8Weight(src.get(name, dev, torch.float8_e4m3fn), src.get(name + "_scale_inv", dev, torch.float32))
    return src.get(name, dev, dt)


def cat_rows(parts):
    return ops.Fp8Weight.cat(parts) if isinstance(parts[0], ops.Fp8Weight) else torch.cat(parts, 0)


class _QuantRandomSource(RandomSource):
    """Random source that also synthesises INT4 packed tensors and their scales."""

    def get(self, name, device, dtype=None, rows=None, cols=None):
        if name.endswith("weight_packed"):
            shape = self.shapes[name]
            g = torch.Generator(device=torch.device(device))
            g.manual_seed(self._seed_for(name))
            return torch.randint(-(2 ** 31), 2 ** 31 - 1, shape, dtype=torch.int32, device=device, generator=g)
        if name.endswith("weight_scale"):
            shape = self.shapes[name]
            g = torch.Generator(device=torch.device(device))
            g.manual_seed(self._seed_for(name))
            t = torch.empty(shape, dtype=torch.float32, device=device).uniform_(0.003, 0.0056, generator=g)
            return t.to(dtype or self.dtype)
        if name.endswith("weight_scale_inv"):
            shape = self.shapes[name]
            g = torch.Generator(device=torch.device(device))
            g.manual_seed(self._seed_for(name))
            # N(0, 0.02) weights have block maxima near 4.5 sigma: scale_inv ~ 0.09 / 448
            return torch.empty(shape, dtype=torch.float32, device=device).uniform_(1.6e-4, 2.4e-4, generator=g)
        if dtype == torch.float8_e4m3fn:
            # synthetic FP8 experts: N(0, 1) * 100 in e4m3 times scale_inv ~ 2e-4 gives N(0, 0.02)
            w = super().get(name, device, torch.float32, rows, cols) * (100.0 / 0.02)
            return w.clamp_(-448.0, 448.0).to(torch.float8_e4m3fn)
        return super().get(name, device, dtype, rows, cols)


@dataclass
class MlaLayer:
    input_norm: torch.Tensor
    post_norm: torch.Tensor
    q_a: Optional[torch.Tensor]
    q_a_norm: Optional[torch.Tensor]
    q_b: torch.Tensor  # q_proj when there is no q_lora
    kv_a: torch.Tensor
    kv_a_norm: torch.Tensor
    w_uk: torch.Tensor  # [H, nope, kv_lora]
    w_uv: torch.Tensor  # [H, v, kv_lora]
    o: torch.Tensor
    dense_gate_up: Optional[torch.Tensor] = None
    dense_down: Optional[torch.Tensor] = None
    router: Optional[torch.Tensor] = None
    router_bias: Optional[torch.Tensor] = None
    shared_gate_up: Optional[torch.Tensor] = None
    shared_down: Optional[torch.Tensor] = None
    experts: Optional[dict] = None  # w13 / w2 (bf16) or w13_packed, w13_scale, w2_packed, w2_scale


class MlaMoeModel:
    supports_prefix_cache = True

    def __init__(self, cfg: ModelConfig, source: Optional[WeightSource] = None, device="cpu", dtype=torch.bfloat16, tp: TPContext = SINGLE, ep: Optional[EPContext] = None, seed: int = 0):
        self.cfg = cfg
        self.family = cfg.family
        self.device = torch.device(device)
        self.dtype = dtype
        self.tp = tp
        self.ep = ep or LOCAL_EP
        if cfg.is_moe and cfg.n_routed_experts % self.ep.world:
            raise ValueError(f"{cfg.n_routed_experts} experts do not divide ep={self.ep.world}")
        self.latent_width = cfg.kv_lora_rank + cfg.qk_rope_head_dim
        source = source or _QuantRandomSource(mla_moe_shapes(cfg), seed=seed, dtype=dtype)
        self.P = layer_prefix(cfg)
        self.layers = [self._load_layer(source, i) for i in range(cfg.num_layers)]
        self.embed = source.get(self.P + "embed_tokens.weight", self.device, dtype)
        top = "language_model." if cfg.family == "kimi_k2" else ""
        self.lm_head = self.embed if cfg.tie_word_embeddings else source.get(top + "lm_head.weight", self.device, dtype)
        self.final_norm = source.get(self.P + "norm.weight", self.device, dtype)
        self.cos, self.sin = rope_tables(cfg.max_position, cfg.qk_rope_head_dim, cfg.rope_theta, dtype, self.device, cfg.rope_scaling)
        self.scale = cfg.mla_softmax_scale()
        self.mtp = None
        if cfg.num_mtp_layers:
            from .mtp import MtpHead

            self.mtp = MtpHead(self, source, cfg.num_layers)

    # -- loading -----------------------------------------------------------------
    def _load_layer(self, src: WeightSource, i: int) -> MlaLayer:
        cfg, dev, dt = self.cfg, self.device, self.dtype
        p = f"{self.P}layers.{i}."
        a = p + "self_attn."
        H, nope, v, c = cfg.num_q_heads, cfg.qk_nope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        kv_b = src.get(a + "kv_b_proj.weight", dev, dt).view(H, nope + v, c)
        L = MlaLayer(
            input_norm=src.get(p + "input_layernorm.weight", dev, dt),
            post_norm=src.get(p + "post_attention_layernorm.weight", dev, dt),
            q_a=load_dense(src, a + "q_a_proj.weight", dev, dt, cfg) if cfg.q_lora_rank else None,
            q_a_norm=src.get(a + "q_a_layernorm.weight", dev, dt) if cfg.q_lora_rank else None,
            q_b=load_dense(src, a + ("q_b_proj.weight" if cfg.q_lora_rank else "q_proj.weight"), dev, dt, cfg),
            kv_a=src.get(a + "kv_a_proj_with_mqa.weight", dev, dt),
            kv_a_norm=src.get(a + "kv_a_layernorm.weight", dev, dt),
            w_uk=kv_b[:, :nope].contiguous(),
            w_uv=kv_b[:, nope:].contiguous(),
            o=load_dense(src, a + "o_proj.weight", dev, dt, cfg),
        )
        m = p + "mlp."
        if not cfg.layer_is_moe(i):
            L.dense_gate_up = cat_rows([load_dense(src, m + "gate_proj.weight", dev, dt, cfg), load_dense(src, m + "up_proj.weight", dev, dt, cfg)])
            L.dense_down = load_dense(src, m + "down_proj.weight", dev, dt, cfg)
            return L
        L.router = src.get(m + "gate.weight", dev, dt)
        if cfg.router_bias:
            L.router_bias = src.get(m + "gate.e_score_correction_bias", dev, torch.float32)
        if cfg.n_shared_experts:
            L.shared_gate_up = cat_rows([load_dense(src, m + "shared_experts.gate_proj.weight", dev, dt, cfg), load_dense(src, m + "shared_experts.up_proj.weight", dev, dt, cfg)])
            L.shared_down = load_dense(src, m + "shared_experts.down_proj.weight", dev, dt, cfg)
        e0, e1 = shard_range(cfg.n_routed_experts, self.ep.rank, self.ep.world)
        ex: dict = {"offset": e0}
        if cfg.expert_quant == "int4_g32":
            for key, names in (("w13", ("gate_proj", "up_proj")), ("w2", ("down_proj",))):
                pk = torch.stack([torch.cat([src.get(f"{m}experts.{e}.{n}.weight_packed", dev, torch.int32) for n in names], 0) for e in range(e0, e1)])
                sc = torch.stack([torch.cat([src.get(f"{m}experts.{e}.{n}.weight_scale", dev, dt) for n in names], 0) for e in range(e0, e1)])
                if dev.type == "cuda":  # nibble order of the sm_100a grouped GEMM (load-time repack kernel)
                    from ..ops.cuda import repack_int4_pairs

                    pk = repack_int4_pairs(pk)
                ex[key + "_packed"], ex[key + "_scale"] = pk, sc
        elif cfg.expert_quant == "fp8_block128":
            if cfg.moe_intermediate_size % 128 or cfg.hidden_size % 128:
                raise ValueError("block-scaled FP8 experts need hidden and expert intermediate sizes that are multiples of 128")
            f8 = torch.float8_e4m3fn
            for key, names in (("w13", ("gate_proj", "up_proj")), ("w2", ("down_proj",))):
                w8 = torch.stack([torch.cat([src.get(f"{m}experts.{e}.{n}.weight", dev, f8) for n in names], 0) for e in range(e0, e1)])
                sc = torch.stack([torch.cat([src.get(f"{m}experts.{e}.{n}.weight_scale_inv", dev, torch.float32) for n in names], 0) for e in range(e0, e1)])
                ex[key + "_fp8"], ex[key + "_scale"] = w8, sc.contiguous()
        else:
            ex["w13"] = torch.stack([torch.cat([src.get(f"{m}experts.{e}.gate_proj.weight", dev, dt), src.get(f"{m}experts.{e}.up_proj.weight", dev, dt)], 0) for e in range(e0, e1)])
            ex["w2"] = torch.stack([src.get(f"{m}experts.{e}.down_proj.weight", dev, dt) for e in range(e0, e1)])
        L.experts = ex
        return L

    # -- KV geometry ---------------------------------------------------------------
    def kv_geometry(self) -> dict:
        w = self.latent_width
        n = self.cfg.num_layers + (1 if self.mtp is not None else 0)
        return dict(num_layers=n, kv_heads=1, head_dim=w, bytes_per_block=lambda page: n * page * w * 2)

    def make_kv(self, num_pages: int, page_size: int):
        n = self.cfg.num_layers + (1 if self.mtp is not None else 0)
        return LatentKvBuffer(n, num_pages, page_size, self.latent_width, self.dtype, self.device)

    # -- blocks ---------------------------------------------------------------------
    def attention(self, L: MlaLayer, x, meta: AttnMeta, latent_layer):
        cfg = self.cfg
        t = x.shape[0]
        if L.q_a is not None:
            qa = ops.rms_norm(ops.linear(x, L.q_a), L.q_a_norm, cfg.rms_eps)
            q = ops.linear(qa, L.q_b)
        else:
            q = ops.linear(x, L.q_b)
        q = q.view(t, cfg.num_q_heads, cfg.qk_nope_head_dim + cfg.qk_rope_head_dim)
        kv_a = ops.linear(x, L.kv_a)
        ops.mla_append(kv_a, L.kv_a_norm, self.cos, self.sin, meta, latent_layer, cfg.kv_lora_rank, cfg.rms_eps)
        q = ops.mla_rope_q(q, self.cos, self.sin, meta, cfg.qk_nope_head_dim)
        a = ops.mla_attention(q, L.w_uk, L.w_uv, latent_layer, meta, self.scale, cfg.kv_lora_rank)
        return ops.linear(a, L.o)

    def ffn(self, L: MlaLayer, x):
        cfg = self.cfg
        if L.router is None:
            return ops.linear(ops.swiglu(ops.linear(x, L.dense_gate_up)), L.dense_down)
        logits = ops.linear(x, L.router, out_dtype=torch.float32)
        ids, wts = ops.router_topk(logits, cfg.num_experts_per_tok, cfg.scoring_func, L.router_bias, cfg.n_group, cfg.topk_group, cfg.norm_topk_prob, cfg.routed_scaling_factor)
        routed = self.ep.moe(x, ids, wts, L.experts, cfg)
        if L.shared_gate_up is not None:
            shared = ops.linear(ops.swiglu(ops.linear(x, L.shared_gate_up)), L.shared_down)
            return (routed.float() + shared.float()).to(x.dtype)
        return routed.to(x.dtype)

    def block(self, L: MlaLayer, x, residual, meta, latent_layer, next_norm):
        eps = self.cfg.rms_eps
        a = self.attention(L, x, meta, latent_layer)
        x = ops.add_rms_norm(a, residual, L.post_norm, eps)
        f = self.ffn(L, x)
        return ops.add_rms_norm(f, residual, next_norm, eps)

    # -- forward ----------------------------------------------------------------------
    def forward_hidden(self, token_ids, meta: AttnMeta, kv, aux_layers=()):
        self.ep.begin_step()
        residual = ops.embedding(token_ids, self.embed)
        x = ops.rms_norm(residual, self.layers[0].input_norm, self.cfg.rms_eps)
        n = len(self.layers)
        for i, L in enumerate(self.layers):
            nxt = self.layers[i + 1].input_norm if i + 1 < n else self.final_norm
            x = self.block(L, x, residual, meta, kv.layer(i), nxt)
        self.last_residual = residual  # pre-norm hidden of the last layer (MTP input)
        return x

    def logits(self, hidden, rows=None):
        if rows is not None:
            hidden = ops.gather_rows(hidden, rows)
        return ops.linear(hidden, self.lm_head)

    def forward(self, token_ids, meta, kv, logits_rows=None):
        return self.logits(self.forward_hidden(token_ids, meta, kv), logits_rows)
