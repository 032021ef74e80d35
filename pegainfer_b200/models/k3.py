"""Kimi-K3 text tower: KDA linear attention and NoPE MLA over an attention-residual stream, latent MoE.

Layers.  Three of four layers are Kimi Delta Attention: q / k / v / output-gate projections, a short causal
depthwise convolution + SiLU on q, k and v, a forget gate ``f_b(f_a(x))`` that gives one decay per key channel,
``beta = sigmoid(b(x))``, the delta rule over an f32 state ``[heads, Dk, Dv]`` per sequence, a per-head RMSNorm
times ``sigmoid(gate)``, and o_proj.  Every fourth layer and the last one are multi-head latent attention without
positions: the cached row is the normalised 512-wide latent plus the shared 64-wide key half, nothing is rotated,
and the attention output is multiplied by ``sigmoid(g_proj(x))`` before o_proj.  Only the MLA layers own paged KV.

Residual stream.  Every ``attn_res_block`` layers the residual row of a token is stored as a snapshot and the
running residual restarts from that layer's attention output.  What a sub-layer reads is a mix: the softmax over
``dot(x / rms(x), norm_w * proj_w)`` of the live snapshots and the current residual, applied to the un-normalised
rows.  The model output mixes all snapshots and the final residual the same way.

MoE.  Router (sigmoid scores + selection bias, top-k, renormalised, scaled) reads the normalised hidden; the routed
experts run in a latent: ``hidden -> latent`` projection, experts ``latent -> moe_inter -> latent`` with the
saturating activation ``4 tanh(g / 4) sigmoid(g) * 25 tanh(u / 25)``, RMSNorm, ``latent -> hidden``; two shared
experts (stored fused) read the hidden directly.  Released checkpoints store the routed experts as MXFP4 (e2m1
values, one e8m0 scale per 32); this loader dequantises them to bf16 for the bf16 grouped GEMM.

Reference parity: pegainfer-k3/src/config.rs:26-140, src/weights.rs:486-580 (tensor names),
src/model/plan.rs:207-220,465-497 (scoring vector, snapshot geometry), src/executor/forward/step.rs:194-470
(layer order), forward/decode.rs:53-190 (KDA), step.rs:504-650 (MLA), step.rs:654-770 (latent MoE),
kernels/tilelang_defs.py (kernel arithmetic).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..kv.buffer import LatentKvBuffer
from ..loader.sources import RandomSource, WeightSource, shard_range
from ..ops.reference import AttnMeta
from ..parallel.ep import LOCAL_EP, EPContext
from ..parallel.tp import SINGLE, TPContext
from .qwen35 import HybridExecutor, RecurrentState

TEXT = "language_model."


def layer_geometry(num_layers: int, block: int):
    """Per layer ``(snapshot, nb_in, nb_mlp)`` and the number of snapshot blocks: layer ``i`` stores a snapshot when
    ``i % block == 0``; its entry mix sees the snapshots taken before it, its exit mix also its own."""
    out, blocks = [], 0
    for i in range(num_layers):
        snap = i % block == 0
        nb_in = blocks
        blocks += int(snap)
        out.append((snap, nb_in, blocks))
    return out, blocks


def k3_shapes(cfg: ModelConfig) -> dict:
    h, heads, D = cfg.hidden_size, cfg.num_q_heads, cfg.gdn_head_dim
    inner = heads * D
    nope, rope, v, c, qr = cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank, cfg.q_lora_rank
    lat, mi = cfg.latent_moe_dim, cfg.moe_intermediate_size
    m = TEXT + "model."
    s = {m + "embed_tokens.weight": (cfg.vocab_size, h), m + "norm.weight": (h,), TEXT + "lm_head.weight": (cfg.vocab_size, h),
         m + "output_attn_res_norm.weight": (h,), m + "output_attn_res_proj.weight": (1, h)}
    for i in range(cfg.num_layers):
        p = f"{m}layers.{i}."
        a = p + "self_attn."
        for n in ("input_layernorm", "post_attention_layernorm", "self_attention_res_norm", "mlp_res_norm"):
            s[p + n + ".weight"] = (h,)
        s[p + "self_attention_res_proj.weight"] = (1, h)
        s[p + "mlp_res_proj.weight"] = (1, h)
        if cfg.layer_type(i) == "linear_attention":
            s[a + "g_proj.weight"] = (inner, h)
            s[a + "o_proj.weight"] = (h, inner)
            s[a + "A_log"] = (heads,)
            s[a + "dt_bias"] = (inner,)
            s[a + "b_proj.weight"] = (heads, h)
            s[a + "f_a_proj.weight"] = (cfg.kda_gate_rank, h)
            s[a + "f_b_proj.weight"] = (inner, cfg.kda_gate_rank)
            s[a + "o_norm.weight"] = (D,)
            for n in ("q", "k", "v"):
                s[a + n + "_proj.weight"] = (inner, h)
                s[a + n + "_conv1d.weight"] = (inner, 1, cfg.gdn_conv_kernel)
        else:
            s[a + "g_proj.weight"] = (heads * v, h)
            s[a + "o_proj.weight"] = (h, heads * v)
            s[a + "q_a_proj.weight"] = (qr, h)
            s[a + "q_a_layernorm.weight"] = (qr,)
            s[a + "q_b_proj.weight"] = (heads * (nope + rope), qr)
            s[a + "kv_a_proj_with_mqa.weight"] = (c + rope, h)
            s[a + "kv_a_layernorm.weight"] = (c,)
            s[a + "kv_b_proj.weight"] = (heads * (nope + v), c)
        if not cfg.layer_is_moe(i):
            s[p + "mlp.gate_proj.weight"] = (cfg.intermediate_size, h)
            s[p + "mlp.up_proj.weight"] = (cfg.intermediate_size, h)
            s[p + "mlp.down_proj.weight"] = (h, cfg.intermediate_size)
            continue
        e = p + "block_sparse_moe."
        sh = cfg.n_shared_experts * mi
        s[e + "gate.weight"] = (cfg.n_routed_experts, h)
        s[e + "gate.e_score_correction_bias"] = (cfg.n_routed_experts,)
        s[e + "routed_expert_down_proj.weight"] = (lat, h)
        s[e + "routed_expert_norm.weight"] = (lat,)
        s[e + "routed_expert_up_proj.weight"] = (h, lat)
        s[e + "shared_experts.gate_proj.weight"] = (sh, h)
        s[e + "shared_experts.up_proj.weight"] = (sh, h)
        s[e + "shared_experts.down_proj.weight"] = (h, sh)
        for x in range(cfg.n_routed_experts):
            s[f"{e}experts.{x}.w1.weight"] = (mi, lat)
            s[f"{e}experts.{x}.w3.weight"] = (mi, lat)
            s[f"{e}experts.{x}.w2.weight"] = (lat, mi)
    return s


def _kind(name: str) -> str:
    """Random-weight distributions: the scoring projections get a spread that makes the mixes non-uniform."""
    if name.endswith("res_proj.weight"):
        return "normal"
    return RandomSource._default_kind(name)


def k3_source(cfg: ModelConfig, seed: int = 0, dtype=torch.bfloat16) -> RandomSource:
    return RandomSource(k3_shapes(cfg), seed=seed, dtype=dtype, kind=_kind)


@dataclass
class KdaPart:
    wbig: torch.Tensor  # [4 * inner, hidden]: q | k | v | output gate
    wsm: torch.Tensor  # [heads + rank (padded), hidden]: beta | low-rank forget gate
    f_b: torch.Tensor  # [inner, rank]
    conv_w: torch.Tensor  # [3 * inner, K]
    a_log: torch.Tensor
    dt_bias: torch.Tensor
    o_norm: torch.Tensor
    state_index: int


@dataclass
class MlaPart:
    wfu: torch.Tensor  # [q_lora + (kv_lora + rope) + heads * v, hidden]: q_a | kv_a | output gate
    q_a_norm: torch.Tensor
    q_b: torch.Tensor
    kv_a_norm: torch.Tensor
    w_uk: torch.Tensor
    w_uv: torch.Tensor
    kv_index: int


@dataclass
class K3Layer:
    input_norm: torch.Tensor
    post_norm: torch.Tensor
    sw_attn: torch.Tensor  # f32 [hidden]: norm weight * scoring projection of the entry mix
    sw_mlp: torch.Tensor
    o: torch.Tensor
    snapshot: bool
    nb_in: int
    nb_mlp: int
    kda: Optional[KdaPart] = None
    mla: Optional[MlaPart] = None
    dense_gate_up: Optional[torch.Tensor] = None
    dense_down: Optional[torch.Tensor] = None
    router: Optional[torch.Tensor] = None
    router_bias: Optional[torch.Tensor] = None
    lat_down: Optional[torch.Tensor] = None
    lat_norm: Optional[torch.Tensor] = None
    lat_up: Optional[torch.Tensor] = None
    shared_gate_up: Optional[torch.Tensor] = None
    shared_down: Optional[torch.Tensor] = None
    experts: Optional[dict] = None


def _pad_rows(w: torch.Tensor, multiple: int) -> torch.Tensor:
    extra = (-w.shape[0]) % multiple
    return w if not extra else torch.cat([w, torch.zeros((extra, w.shape[1]), dtype=w.dtype, device=w.device)], 0).contiguous()


class K3Model:
    family = "kimi_k3"
    supports_prefix_cache = False  # the KDA state is per request and not cached

    def __init__(self, cfg: ModelConfig, source: Optional[WeightSource] = None, device="cpu", dtype=torch.bfloat16, tp: TPContext = SINGLE, ep: Optional[EPContext] = None, seed: int = 0):
        if tp.world != 1:
            raise ValueError("the Kimi-K3 line scales by expert parallelism (--ep-size); tensor parallelism is not part of it")
        self.cfg, self.device, self.dtype, self.tp = cfg, torch.device(device), dtype, tp
        self.ep = ep or LOCAL_EP
        if cfg.n_routed_experts % self.ep.world:
            raise ValueError(f"{cfg.n_routed_experts} experts do not divide ep={self.ep.world}")
        if getattr(self.ep, "comm", "none") == "fused":
            raise ValueError("the fused expert-parallel kernels apply SwiGLU; run the Kimi-K3 line with --comm nccl")
        self.heads, self.D = cfg.num_q_heads, cfg.gdn_head_dim
        self.inner = self.heads * self.D
        self.latent_width = cfg.kv_lora_rank + cfg.qk_rope_head_dim
        self.geometry, self.blocks = layer_geometry(cfg.num_layers, cfg.attn_res_block)
        if self.blocks + 1 > 16:
            raise ValueError(f"{self.blocks} residual snapshots: the mix kernel handles at most 15")
        src = source or k3_source(cfg, seed=seed, dtype=dtype)
        m = TEXT + "model."
        self.n_lin = self.n_mla = 0
        self.layers = [self._load_layer(src, i) for i in range(cfg.num_layers)]
        self.embed = src.get(m + "embed_tokens.weight", self.device, dtype)
        self.lm_head = self.embed if cfg.tie_word_embeddings else src.get(TEXT + "lm_head.weight", self.device, dtype)
        self.final_norm = src.get(m + "norm.weight", self.device, dtype)
        self.sw_out = self._score_vector(src, m + "output_attn_res_")
        # no positions: the rotation tables are the identity, so the shared MLA kernels append and read the key half unrotated
        n_pos, half = min(cfg.max_position, 1 << 17), cfg.qk_rope_head_dim // 2
        self.cos = torch.ones((n_pos, half), dtype=dtype, device=self.device)
        self.sin = torch.zeros((n_pos, half), dtype=dtype, device=self.device)
        self.scale = (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim) ** -0.5
        self.rec: Optional[RecurrentState] = None
        self.mtp = None

    # -- loading -----------------------------------------------------------------------
    def _score_vector(self, src, prefix: str) -> torch.Tensor:
        g = src.get(prefix + "norm.weight", self.device, torch.float32)
        p = src.get(prefix + "proj.weight", self.device, torch.float32).reshape(-1)
        return (g * p).contiguous()

    def _expert(self, src, name: str) -> torch.Tensor:
        """One routed-expert matrix as bf16: a dense ``.weight``, or MXFP4 ``.weight_packed`` + ``.weight_scale``."""
        if src.has(name + ".weight_packed"):
            pk = src.get(name + ".weight_packed", self.device, torch.uint8)
            sc = src.get(name + ".weight_scale", self.device, torch.uint8)
            return ops.dequant_mxfp4(pk, sc, self.dtype)
        return src.get(name + ".weight", self.device, self.dtype)

    def _load_layer(self, src: WeightSource, i: int) -> K3Layer:
        cfg, dev, dt = self.cfg, self.device, self.dtype
        p = f"{TEXT}model.layers.{i}."
        a = p + "self_attn."
        snap, nb_in, nb_mlp = self.geometry[i]
        L = K3Layer(input_norm=src.get(p + "input_layernorm.weight", dev, dt), post_norm=src.get(p + "post_attention_layernorm.weight", dev, dt),
                    sw_attn=self._score_vector(src, p + "self_attention_res_"), sw_mlp=self._score_vector(src, p + "mlp_res_"), o=src.get(a + "o_proj.weight", dev, dt),
                    snapshot=snap, nb_in=nb_in, nb_mlp=nb_mlp)
        gate = src.get(a + "g_proj.weight", dev, dt)
        if cfg.layer_type(i) == "linear_attention":
            K = cfg.gdn_conv_kernel
            L.kda = KdaPart(
                wbig=torch.cat([src.get(a + n + "_proj.weight", dev, dt) for n in ("q", "k", "v")] + [gate], 0),
                wsm=_pad_rows(torch.cat([src.get(a + "b_proj.weight", dev, dt), src.get(a + "f_a_proj.weight", dev, dt)], 0), 16),
                f_b=src.get(a + "f_b_proj.weight", dev, dt),
                conv_w=torch.cat([src.get(a + n + "_conv1d.weight", dev, dt).reshape(-1, K) for n in ("q", "k", "v")], 0).contiguous(),
                a_log=src.get(a + "A_log", dev, torch.float32).reshape(-1).contiguous(), dt_bias=src.get(a + "dt_bias", dev, torch.float32).reshape(-1).contiguous(),
                o_norm=src.get(a + "o_norm.weight", dev, torch.float32), state_index=self.n_lin)
            self.n_lin += 1
        else:
            H, nope, v, c = cfg.num_q_heads, cfg.qk_nope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
            kv_b = src.get(a + "kv_b_proj.weight", dev, dt).view(H, nope + v, c)
            L.mla = MlaPart(wfu=torch.cat([src.get(a + "q_a_proj.weight", dev, dt), src.get(a + "kv_a_proj_with_mqa.weight", dev, dt), gate], 0),
                            q_a_norm=src.get(a + "q_a_layernorm.weight", dev, dt), q_b=src.get(a + "q_b_proj.weight", dev, dt),
                            kv_a_norm=src.get(a + "kv_a_layernorm.weight", dev, dt), w_uk=kv_b[:, :nope].contiguous(), w_uv=kv_b[:, nope:].contiguous(), kv_index=self.n_mla)
            self.n_mla += 1
        if not cfg.layer_is_moe(i):
            L.dense_gate_up = torch.cat([src.get(p + "mlp.gate_proj.weight", dev, dt), src.get(p + "mlp.up_proj.weight", dev, dt)], 0)
            L.dense_down = src.get(p + "mlp.down_proj.weight", dev, dt)
            return L
        e = p + "block_sparse_moe."
        L.router = src.get(e + "gate.weight", dev, dt)
        L.router_bias = src.get(e + "gate.e_score_correction_bias", dev, torch.float32)
        L.lat_down = src.get(e + "routed_expert_down_proj.weight", dev, dt)
        L.lat_norm = src.get(e + "routed_expert_norm.weight", dev, dt)
        L.lat_up = src.get(e + "routed_expert_up_proj.weight", dev, dt)
        L.shared_gate_up = torch.cat([src.get(e + "shared_experts.gate_proj.weight", dev, dt), src.get(e + "shared_experts.up_proj.weight", dev, dt)], 0)
        L.shared_down = src.get(e + "shared_experts.down_proj.weight", dev, dt)
        e0, e1 = shard_range(cfg.n_routed_experts, self.ep.rank, self.ep.world)
        L.experts = {"offset": e0,
                     "w13": torch.stack([torch.cat([self._expert(src, f"{e}experts.{x}.w1"), self._expert(src, f"{e}experts.{x}.w3")], 0) for x in range(e0, e1)]),
                     "w2": torch.stack([self._expert(src, f"{e}experts.{x}.w2") for x in range(e0, e1)])}
        return L

    # -- geometry / executor -------------------------------------------------------------
    def kv_geometry(self) -> dict:
        w, n = self.latent_width, max(self.n_mla, 1)
        return dict(num_layers=n, kv_heads=1, head_dim=w, bytes_per_block=lambda page: n * page * w * 2)

    def make_kv(self, num_pages: int, page_size: int):
        return LatentKvBuffer(max(self.n_mla, 1), num_pages, page_size, self.latent_width, self.dtype, self.device)

    def make_state(self, num_slots: int) -> RecurrentState:
        self.rec = RecurrentState(num_slots + 1, max(self.n_lin, 1), 3 * self.inner, self.cfg.gdn_conv_kernel, self.heads, self.D, self.D, self.dtype, self.device)
        return self.rec

    @staticmethod
    def make_executor(model, kv, page_size, cuda_graph=False, max_decode_batch=256, max_blocks_per_seq=0, seed=0):
        return HybridExecutor(model, kv, page_size, cuda_graph=cuda_graph, max_decode_batch=min(max_decode_batch, 64), max_blocks_per_seq=max_blocks_per_seq, seed=seed)

    # -- blocks ------------------------------------------------------------------------------
    def kda(self, L: K3Layer, x, meta: AttnMeta):
        K, t, heads, D, inner = L.kda, x.shape[0], self.heads, self.D, self.inner
        big = ops.linear(x, K.wbig)  # q | k | v | output gate
        small = ops.linear(x, K.wsm)  # beta | low-rank forget gate
        f = ops.linear(small[:, heads : heads + self.cfg.kda_gate_rank].contiguous(), K.f_b)
        conv = ops.gdn_conv1d(big[:, : 3 * inner], K.conv_w, self.rec.conv[K.state_index], meta)
        q, k, v = (conv[:, j * inner : (j + 1) * inner].view(t, heads, D) for j in range(3))
        o = ops.kda_recurrent(q, k, v, f, small[:, :heads], K.a_log, K.dt_bias, self.cfg.kda_gate_lower_bound, self.rec.ssm[K.state_index], meta)
        gate = big[:, 3 * inner :].contiguous().view(t, heads, D)
        return ops.gated_rms_norm(o, gate, K.o_norm, self.cfg.rms_eps, act="sigmoid").view(t, inner)

    def mla(self, L: K3Layer, x, meta: AttnMeta, latent_layer):
        cfg, M, t = self.cfg, L.mla, x.shape[0]
        qr, lw = cfg.q_lora_rank, self.latent_width
        fused = ops.linear(x, M.wfu)  # q_a | kv_a | output gate
        qa = ops.rms_norm(fused[:, :qr].contiguous(), M.q_a_norm, cfg.rms_eps)
        q = ops.linear(qa, M.q_b).view(t, cfg.num_q_heads, cfg.qk_nope_head_dim + cfg.qk_rope_head_dim)
        ops.mla_append(fused[:, qr : qr + lw].contiguous(), M.kv_a_norm, self.cos, self.sin, meta, latent_layer, cfg.kv_lora_rank, cfg.rms_eps)
        q = ops.mla_rope_q(q, self.cos, self.sin, meta, cfg.qk_nope_head_dim)
        a = ops.mla_attention(q, M.w_uk, M.w_uv, latent_layer, meta, self.scale, cfg.kv_lora_rank)
        return ops.sigmoid_gate_mul(a.reshape(t, -1), fused[:, qr + lw :].contiguous())

    def ffn(self, L: K3Layer, x):
        cfg = self.cfg
        if L.router is None:
            return ops.linear(ops.situ(ops.linear(x, L.dense_gate_up)), L.dense_down)
        logits = ops.linear(x, L.router, out_dtype=torch.float32)
        ids, wts = ops.router_topk(logits, cfg.num_experts_per_tok, "sigmoid", L.router_bias, 1, 1, cfg.norm_topk_prob, cfg.routed_scaling_factor)
        lat = ops.linear(x, L.lat_down)
        routed = self.ep.moe(lat, ids, wts, L.experts, cfg).to(x.dtype)
        routed = ops.linear(ops.rms_norm(routed, L.lat_norm, cfg.rms_eps), L.lat_up)
        shared = ops.linear(ops.situ(ops.linear(x, L.shared_gate_up)), L.shared_down)
        return routed + shared

    # -- forward -----------------------------------------------------------------------------
    def forward_hidden(self, token_ids, meta: AttnMeta, kv, aux_layers=()):
        eps = self.cfg.rms_eps
        self.ep.begin_step()
        hidden = ops.embedding(token_ids, self.embed)
        snaps = torch.empty((hidden.shape[0], max(self.blocks, 1), hidden.shape[1]), dtype=hidden.dtype, device=hidden.device)
        for L in self.layers:
            mixed = ops.attnres_mix(hidden, snaps, L.nb_in, L.sw_attn, eps) if L.nb_in else hidden
            if L.snapshot:
                snaps[:, L.nb_in].copy_(hidden)
            x = ops.rms_norm(mixed, L.input_norm, eps)
            a = self.kda(L, x, meta) if L.kda is not None else self.mla(L, x, meta, kv.layer(L.mla.kv_index))
            a = ops.linear(a, L.o)
            hidden = a if L.snapshot else hidden + a  # a snapshot layer restarts the running residual
            mixed = ops.attnres_mix(hidden, snaps, L.nb_mlp, L.sw_mlp, eps)
            hidden = hidden + self.ffn(L, ops.rms_norm(mixed, L.post_norm, eps))
        mixed = ops.attnres_mix(hidden, snaps, self.blocks, self.sw_out, eps)
        return ops.rms_norm(mixed, self.final_norm, eps)

    def logits(self, hidden, rows=None):
        if rows is not None:
            hidden = ops.gather_rows(hidden, rows)
        return ops.linear(hidden, self.lm_head)

    def forward(self, token_ids, meta, kv, logits_rows=None):
        return self.logits(self.forward_hidden(token_ids, meta, kv), logits_rows)
