"""Qwen3.5 hybrid decoder: 3 Gated-DeltaNet linear-attention layers to 1 full-attention layer.

Full-attention layers: GQA with head_dim 256, (1+w) QK-norm, partial RoPE (first
``rotary_dim`` dims), q_proj rows per head are ``[q, gate]`` and the attention output
is multiplied by ``sigmoid(gate)`` before o_proj.  Linear layers: in_proj_{qkv,z,b,a}
-> causal depthwise conv(k=4)+SiLU -> gated delta rule over an f32 recurrent state
``[Hv, Dk, Dv]`` per sequence -> per-head RMSNorm * silu(z) -> out_proj.  All hidden
norms use (1+w).  Recurrent and conv state live in a per-request slot pool (not paged);
paged KV exists only for the full-attention layers.  Under tensor parallelism value
heads (and the K heads they share) are sharded, so the recurrent state is sharded too.

Reference parity: pegainfer-qwen35/src/{config.rs:26-215, weights.rs:253-790,
batch_decode.rs:498-775, recurrent.rs:17-560, recurrent_state.rs:16-170},
pegainfer-kernels/csrc/qwen35/{conv1d.cu, gated_delta_rule.cu, prefill_attention_hd256.cu}.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..config import ModelConfig
from ..kv.buffer import KvBuffer, KvLayout
from ..loader.sources import RandomSource, WeightSource, shard_range
from ..ops.reference import AttnMeta, rope_tables
from ..parallel.tp import SINGLE, TPContext
from ..sched.executor import TorchExecutor


def qwen35_shapes(cfg: ModelConfig, wp: str = "model.language_model") -> dict:
    h, d = cfg.hidden_size, cfg.head_dim
    dk = dv = cfg.gdn_head_dim
    s = {f"{wp}.embed_tokens.weight": (cfg.vocab_size, h), f"{wp}.norm.weight": (h,), "lm_head.weight": (cfg.vocab_size, h)}
    for i in range(cfg.num_layers):
        p = f"{wp}.layers.{i}."
        s[p + "input_layernorm.weight"] = (h,)
        s[p + "post_attention_layernorm.weight"] = (h,)
        s[p + "mlp.gate_proj.weight"] = (cfg.intermediate_size, h)
        s[p + "mlp.up_proj.weight"] = (cfg.intermediate_size, h)
        s[p + "mlp.down_proj.weight"] = (h, cfg.intermediate_size)
        if cfg.layer_type(i) == "full_attention":
            a = p + "self_attn."
            s[a + "q_proj.weight"] = (cfg.num_q_heads * d * 2, h)
            s[a + "k_proj.weight"] = (cfg.num_kv_heads * d, h)
            s[a + "v_proj.weight"] = (cfg.num_kv_heads * d, h)
            s[a + "o_proj.weight"] = (h, cfg.num_q_heads * d)
            s[a + "q_norm.weight"] = (d,)
            s[a + "k_norm.weight"] = (d,)
        else:
            a = p + "linear_attn."
            c = 2 * cfg.gdn_num_k_heads * dk + cfg.gdn_num_v_heads * dv
            s[a + "in_proj_qkv.weight"] = (c, h)
            s[a + "in_proj_z.weight"] = (cfg.gdn_num_v_heads * dv, h)
            s[a + "in_proj_b.weight"] = (cfg.gdn_num_v_heads, h)
            s[a + "in_proj_a.weight"] = (cfg.gdn_num_v_heads, h)
            s[a + "conv1d.weight"] = (c, 1, cfg.gdn_conv_kernel)
            s[a + "dt_bias"] = (cfg.gdn_num_v_heads,)
            s[a + "A_log"] = (cfg.gdn_num_v_heads,)
            s[a + "norm.weight"] = (dv,)
            s[a + "out_proj.weight"] = (h, cfg.gdn_num_v_heads * dv)
    return s


def _kind(name: str) -> str:
    # (1+w) norms are stored as offsets around zero; the gated norm weight is a plain scale
    if name.endswith("linear_attn.norm.weight"):
        return "ones"
    if name.endswith("norm.weight") or "layernorm" in name:
        return "zeros"
    if name.endswith("A_log") or name.endswith("dt_bias"):
        return "small"
    return "normal"


@dataclass
class FullLayer:
    qkv: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    o: torch.Tensor
    kv_index: int


@dataclass
class LinearLayer:
    in_qkv: torch.Tensor
    in_zba: torch.Tensor  # rows: z (Hv*Dv), b (Hv), a (Hv)
    conv_w: torch.Tensor  # [C_local, K]
    dt_bias: torch.Tensor
    a_log: torch.Tensor
    norm_w: torch.Tensor  # f32 [Dv]
    out: torch.Tensor
    state_index: int


@dataclass
class HybridLayer:
    input_norm: torch.Tensor
    post_norm: torch.Tensor
    gate_up: torch.Tensor
    down: torch.Tensor
    full: Optional[FullLayer] = None
    linear: Optional[LinearLayer] = None


class RecurrentState:
    """Slot pool of per-request conv and delta-rule state (slot 0 is the padding slot)."""

    def __init__(self, num_slots: int, n_linear: int, channels: int, conv_k: int, hv: int, dk: int, dv: int, dtype, device):
        self.conv = torch.zeros((n_linear, num_slots, channels, conv_k - 1), dtype=dtype, device=device)
        self.ssm = torch.zeros((n_linear, num_slots, hv, dk, dv), dtype=torch.float32, device=device)
        self._free = list(range(num_slots - 1, 0, -1))
        self.by_rid: dict = {}

    def slot_for(self, rid: int, fresh: bool) -> int:
        s = self.by_rid.get(rid)
        if s is None:
            if not self._free:
                raise RuntimeError("recurrent-state slot pool exhausted")
            s = self._free.pop()
            self.by_rid[rid] = s
            fresh = True
        if fresh:
            self.conv[:, s].zero_()
            self.ssm[:, s].zero_()
        return s

    def release(self, rid: int) -> None:
        s = self.by_rid.pop(rid, None)
        if s is not None:
            self._free.append(s)


class Qwen35Model:
    family = "qwen35"
    supports_prefix_cache = False  # recurrent state is per request and not cached

    def __init__(self, cfg: ModelConfig, source: Optional[WeightSource] = None, device="cpu", dtype=torch.bfloat16, tp: TPContext = SINGLE, seed: int = 0, wp: str = "model.language_model"):
        self.cfg, self.device, self.dtype, self.tp = cfg, torch.device(device), dtype, tp
        w = tp.world
        for name, v in (("q heads", cfg.num_q_heads), ("kv heads", cfg.num_kv_heads), ("GDN k heads", cfg.gdn_num_k_heads), ("GDN v heads", cfg.gdn_num_v_heads), ("FFN", cfg.intermediate_size)):
            if v % w:
                raise ValueError(f"{name} ({v}) must divide tp={w}")
        self.q_heads, self.kv_heads = cfg.num_q_heads // w, cfg.num_kv_heads // w
        self.hk, self.hv = cfg.gdn_num_k_heads // w, cfg.gdn_num_v_heads // w
        self.dk = self.dv = cfg.gdn_head_dim
        self.channels = 2 * self.hk * self.dk + self.hv * self.dv
        self.wp = wp
        source = source or RandomSource(qwen35_shapes(cfg, wp), seed=seed, dtype=dtype, kind=_kind)
        self._load(source)
        self.cos, self.sin = rope_tables(min(cfg.max_position, 65536), cfg.rotary_dim, cfg.rope_theta, dtype, self.device)
        self.rec: Optional[RecurrentState] = None

    def _load(self, src):
        cfg, dev, dt, tp, wp = self.cfg, self.device, self.dtype, self.tp, self.wp
        d = cfg.head_dim
        self.embed = src.get(f"{wp}.embed_tokens.weight", dev, dt)
        self.lm_head = self.embed if cfg.tie_word_embeddings else src.get("lm_head.weight", dev, dt)
        self.final_norm = src.get(f"{wp}.norm.weight", dev, dt)
        qr = shard_range(cfg.num_q_heads, tp.rank, tp.world)
        kr = shard_range(cfg.num_kv_heads, tp.rank, tp.world)
        fr = shard_range(cfg.intermediate_size, tp.rank, tp.world)
        hkr = shard_range(cfg.gdn_num_k_heads, tp.rank, tp.world)
        hvr = shard_range(cfg.gdn_num_v_heads, tp.rank, tp.world)
        HK, dk, dv = cfg.gdn_num_k_heads, self.dk, self.dv
        self.layers, n_full, n_lin = [], 0, 0
        for i in range(cfg.num_layers):
            p = f"{wp}.layers.{i}."
            g = src.get(p + "mlp.gate_proj.weight", dev, dt, rows=fr)
            u = src.get(p + "mlp.up_proj.weight", dev, dt, rows=fr)
            L = HybridLayer(
                input_norm=src.get(p + "input_layernorm.weight", dev, dt),
                post_norm=src.get(p + "post_attention_layernorm.weight", dev, dt),
                gate_up=torch.cat([g, u], 0),
                down=src.get(p + "mlp.down_proj.weight", dev, dt, cols=fr),
            )
            if cfg.layer_type(i) == "full_attention":
                a = p + "self_attn."
                q = src.get(a + "q_proj.weight", dev, dt, rows=(qr[0] * d * 2, qr[1] * d * 2))
                k = src.get(a + "k_proj.weight", dev, dt, rows=(kr[0] * d, kr[1] * d))
                v = src.get(a + "v_proj.weight", dev, dt, rows=(kr[0] * d, kr[1] * d))
                L.full = FullLayer(torch.cat([q, k, v], 0), src.get(a + "q_norm.weight", dev, dt), src.get(a + "k_norm.weight", dev, dt), src.get(a + "o_proj.weight", dev, dt, cols=(qr[0] * d, qr[1] * d)), n_full)
                n_full += 1
            else:
                a = p + "linear_attn."
                # in_proj_qkv rows are [q (HK*dk) | k (HK*dk) | v (HV*dv)]; shard each part by heads
                rq = (hkr[0] * dk, hkr[1] * dk)
                rk = (HK * dk + hkr[0] * dk, HK * dk + hkr[1] * dk)
                rv = (2 * HK * dk + hvr[0] * dv, 2 * HK * dk + hvr[1] * dv)
                in_qkv = torch.cat([src.get(a + "in_proj_qkv.weight", dev, dt, rows=r) for r in (rq, rk, rv)], 0)
                conv_full = src.get(a + "conv1d.weight", dev, dt).reshape(-1, cfg.gdn_conv_kernel)
                conv_w = torch.cat([conv_full[r[0] : r[1]] for r in (rq, rk, rv)], 0).contiguous()
                z = src.get(a + "in_proj_z.weight", dev, dt, rows=(hvr[0] * dv, hvr[1] * dv))
                b = src.get(a + "in_proj_b.weight", dev, dt, rows=hvr)
                aa = src.get(a + "in_proj_a.weight", dev, dt, rows=hvr)
                L.linear = LinearLayer(
                    in_qkv=in_qkv,
                    in_zba=torch.cat([z, b, aa], 0),
                    conv_w=conv_w,
                    dt_bias=src.get(a + "dt_bias", dev, torch.float32)[hvr[0] : hvr[1]].contiguous(),
                    a_log=src.get(a + "A_log", dev, torch.float32)[hvr[0] : hvr[1]].contiguous(),
                    norm_w=src.get(a + "norm.weight", dev, torch.float32),
                    out=src.get(a + "out_proj.weight", dev, dt, cols=(hvr[0] * dv, hvr[1] * dv)),
                    state_index=n_lin,
                )
                n_lin += 1
            self.layers.append(L)
        self.n_full, self.n_lin = n_full, n_lin

    # -- geometry / executor ----------------------------------------------------------
    def kv_geometry(self) -> dict:
        return dict(num_layers=max(self.n_full, 1), kv_heads=self.kv_heads, head_dim=self.cfg.head_dim)

    def make_state(self, num_slots: int) -> RecurrentState:
        self.rec = RecurrentState(num_slots + 1, self.n_lin, self.channels, self.cfg.gdn_conv_kernel, self.hv, self.dk, self.dv, self.dtype, self.device)
        return self.rec

    @staticmethod
    def make_executor(model, kv, page_size, cuda_graph=False, max_decode_batch=256, max_blocks_per_seq=0, seed=0):
        return HybridExecutor(model, kv, page_size, cuda_graph=cuda_graph, max_decode_batch=min(max_decode_batch, 64), max_blocks_per_seq=max_blocks_per_seq, seed=seed)

    # -- blocks --------------------------------------------------------------------------
    def full_attention(self, F: FullLayer, x, meta, kv):
        cfg = self.cfg
        qkv = self.tp.col_linear(x, F.qkv)
        q, gate = ops.qk_norm_rope_append(qkv, F.q_norm, F.k_norm, self.cos, self.sin, meta, kv.layer(F.kv_index), self.q_heads, self.kv_heads, cfg.head_dim, cfg.rms_eps, offset=True, gated=True)
        a = ops.paged_attention(q, kv.layer(F.kv_index), meta)
        return ops.sigmoid_gate_mul(a, gate.reshape(a.shape))

    def linear_attention(self, Lp: LinearLayer, x, meta):
        t = x.shape[0]
        hk, hv, dk, dv = self.hk, self.hv, self.dk, self.dv
        mixed = self.tp.col_linear(x, Lp.in_qkv)
        zba = ops.linear(x, Lp.in_zba)
        z, b, a = zba[:, : hv * dv], zba[:, hv * dv : hv * dv + hv], zba[:, hv * dv + hv :]
        mixed = ops.gdn_conv1d(mixed, Lp.conv_w, self.rec.conv[Lp.state_index], meta)
        q = mixed[:, : hk * dk].reshape(t, hk, dk)
        k = mixed[:, hk * dk : 2 * hk * dk].reshape(t, hk, dk)
        v = mixed[:, 2 * hk * dk :].reshape(t, hv, dv)
        g, beta = ops.gdn_gates(a, b, Lp.a_log, Lp.dt_bias)
        o = ops.gdn_recurrent(q, k, v, g, beta, self.rec.ssm[Lp.state_index], meta)
        o = ops.gated_rms_norm(o, z.reshape(t, hv, dv), Lp.norm_w, self.cfg.rms_eps)
        return o.reshape(t, hv * dv)

    def forward_hidden(self, token_ids, meta: AttnMeta, kv, aux_layers=()):
        cfg, tp, eps = self.cfg, self.tp, self.cfg.rms_eps
        tp.begin_step()
        residual = ops.embedding(token_ids, self.embed)
        x = ops.rms_norm(residual, self.layers[0].input_norm, eps, offset=True)
        n = len(self.layers)
        for i, L in enumerate(self.layers):
            if L.full is not None:
                a = self.full_attention(L.full, x, meta, kv)
                x = tp.row_linear_add_norm(a, L.full.o, residual, L.post_norm, eps, offset=True)
            else:
                a = self.linear_attention(L.linear, x, meta)
                x = tp.row_linear_add_norm(a, L.linear.out, residual, L.post_norm, eps, offset=True)
            act = ops.swiglu(tp.col_linear(x, L.gate_up))
            nxt = self.layers[i + 1].input_norm if i + 1 < n else self.final_norm
            x = tp.row_linear_add_norm(act, L.down, residual, nxt, eps, offset=True)
        tp.sync()
        return x

    def logits(self, hidden, rows=None):
        if rows is not None:
            hidden = ops.gather_rows(hidden, rows)
        return ops.linear(hidden, self.lm_head)

    def forward(self, token_ids, meta, kv, logits_rows=None):
        return self.logits(self.forward_hidden(token_ids, meta, kv), logits_rows)


class HybridExecutor(TorchExecutor):
    """Adds recurrent-state slot management to the generic executor."""

    def __init__(self, model, kv, page_size, **kw):
        slots = kw.get("max_decode_batch", 64) + 8
        model.make_state(slots)
        super().__init__(model, kv, page_size, **kw)

    def prepare_meta(self, seqs, meta: AttnMeta) -> None:
        slots = [self.model.rec.slot_for(s.rid, s.fresh_state and s.start_pos == 0) for s in seqs]
        slots += [0] * (meta.num_seqs - len(slots))
        meta.h_state_slots = slots
        meta.state_slots = torch.tensor(slots, dtype=torch.int32, device=self.device)

    def release_request(self, rid: int) -> None:
        self.model.rec.release(rid)
