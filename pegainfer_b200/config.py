"""Model and engine configuration.

Model hyper-parameters come from a checkpoint's ``config.json`` (``from_hf``) or
from a named preset (random-init benchmarking).  ``EngineConfig`` carries the
serving knobs that the CLI exposes.

Reference parity: pegainfer-qwen3/src/config.rs:213-262,465-506;
pegainfer-qwen35/src/config.rs:26-215; pegainfer-deepseek-v2-lite/src/config.rs:69-190;
pegainfer-kimi-k2/src/config.rs:16-140; pegainfer-frontend/src/model_line.rs:93-206
(shared serving flags).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field, replace
from typing import Optional


@dataclass
class ModelConfig:
    family: str = "qwen3"  # qwen3 | qwen35 | deepseek_v2 | kimi_k2 | glm_dsa | gemma4 | kimi_k3
    vocab_size: int = 1024
    hidden_size: int = 256
    num_layers: int = 2
    num_q_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 64
    intermediate_size: int = 768
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position: int = 4096
    tie_word_embeddings: bool = False
    eos_token_ids: tuple = ()
    qk_norm: bool = True
    # Qwen3.5 hybrid
    layer_types: tuple = ()  # "linear_attention" | "full_attention" per layer
    partial_rotary_factor: float = 1.0
    attn_output_gate: bool = False
    norm_weight_offset: bool = False  # (1 + w) RMSNorm
    gdn_num_k_heads: int = 0
    gdn_num_v_heads: int = 0
    gdn_head_dim: int = 128
    gdn_conv_kernel: int = 4
    # MLA
    q_lora_rank: int = 0
    kv_lora_rank: int = 0
    qk_nope_head_dim: int = 0
    qk_rope_head_dim: int = 0
    v_head_dim: int = 0
    rope_scaling: Optional[dict] = None
    # MoE
    n_routed_experts: int = 0
    n_shared_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    first_k_dense_replace: int = 0
    scoring_func: str = "softmax"
    n_group: int = 1
    topk_group: int = 1
    norm_topk_prob: bool = False
    routed_scaling_factor: float = 1.0
    router_bias: bool = False
    expert_quant: str = "bf16"  # bf16 | int4_g32 | fp8_block128 | mxfp4 (Kimi-K3 checkpoints; dequantised to bf16 when loaded)
    quant_group_size: int = 32
    dense_quant: str = "bf16"  # bf16 | fp8_block128: projections outside the experts stay FP8 and run the FP8 GEMM
    # MTP
    num_mtp_layers: int = 0
    # sparse attention indexer (GLM-5 line): every query keeps its index_topk best-scoring keys
    index_topk: int = 0
    index_head_dim: int = 128
    index_n_heads: int = 0
    # Gemma 4 line: sliding-window layers (head_dim, num_kv_heads, rope_theta_local, full rotary) interleaved with global
    # layers (global_head_dim, num_global_kv_heads, rope_theta, partial_rotary_factor of the head rotated); layer_types
    # holds "sliding_attention" | "full_attention"
    sliding_window: int = 0
    global_head_dim: int = 0
    num_global_kv_heads: int = 0
    attention_k_eq_v: bool = False  # global layers have no v_proj: V is the key projection (before key norm and RoPE)
    final_logit_softcapping: float = 0.0
    rope_theta_local: float = 10000.0
    hidden_act: str = "silu"  # "silu" | "gelu_tanh" | "situ"
    # Kimi-K3 line: KDA linear-attention layers ("linear_attention", gdn_head_dim / gdn_conv_kernel give the head and the
    # short convolution) interleaved with NoPE MLA layers ("full_attention"), routed experts that work in a latent of
    # latent_moe_dim columns, and the attention-residual stream that snapshots the residual every attn_res_block layers
    latent_moe_dim: int = 0
    attn_res_block: int = 0
    kda_gate_rank: int = 0
    kda_gate_lower_bound: float = -5.0

    # -- derived ---------------------------------------------------------------
    @property
    def q_size(self) -> int:
        return self.num_q_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def is_mla(self) -> bool:
        return self.kv_lora_rank > 0

    @property
    def is_moe(self) -> bool:
        return self.n_routed_experts > 0

    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_head_dim + self.qk_rope_head_dim

    def layer_is_moe(self, i: int) -> bool:
        return self.is_moe and i >= self.first_k_dense_replace

    def layer_type(self, i: int) -> str:
        return self.layer_types[i] if self.layer_types else "full_attention"

    def mla_softmax_scale(self) -> float:
        scale = 1.0 / math.sqrt(self.qk_head_dim)
        rs = self.rope_scaling or {}
        if rs.get("type", rs.get("rope_type")) == "yarn":
            m = yarn_get_mscale(rs.get("factor", 1.0), rs.get("mscale_all_dim", 0.0))
            scale *= m * m
        return scale

    def param_count(self) -> int:
        """Approximate parameter count (for memory planning)."""
        h = self.hidden_size
        per_layer = 0
        if self.is_mla:
            q = (h * self.q_lora_rank + self.q_lora_rank * self.num_q_heads * self.qk_head_dim) if self.q_lora_rank else h * self.num_q_heads * self.qk_head_dim
            kv = h * (self.kv_lora_rank + self.qk_rope_head_dim) + self.kv_lora_rank * self.num_q_heads * (self.qk_nope_head_dim + self.v_head_dim)
            per_layer += q + kv + self.num_q_heads * self.v_head_dim * h
        else:
            per_layer += h * (self.q_size + 2 * self.kv_size) + self.q_size * h
        dense = 3 * h * self.intermediate_size
        moe = 3 * h * self.moe_intermediate_size * (self.n_routed_experts + self.n_shared_experts) + h * self.n_routed_experts
        n_moe = max(0, self.num_layers - self.first_k_dense_replace) if self.is_moe else 0
        total = self.num_layers * per_layer + (self.num_layers - n_moe) * dense + n_moe * moe
        total += self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        return total


def yarn_get_mscale(scale: float, mscale: float) -> float:
    """YaRN attention-scale correction (pegainfer-deepseek-v2-lite/src/host_ops.rs:377-386)."""
    if scale <= 1.0:
        return 1.0
    return 0.1 * mscale * math.log(scale) + 1.0


def _hybrid_pattern(n: int) -> tuple:
    return tuple("full_attention" if (i + 1) % 4 == 0 else "linear_attention" for i in range(n))


_YARN_DSV2 = {"type": "yarn", "factor": 40.0, "original_max_position_embeddings": 4096, "beta_fast": 32, "beta_slow": 1, "mscale": 0.707, "mscale_all_dim": 0.707}
_YARN_KIMI = {"type": "yarn", "factor": 64.0, "original_max_position_embeddings": 4096, "beta_fast": 32, "beta_slow": 1, "mscale": 1.0, "mscale_all_dim": 1.0}

PRESETS = {
    "tiny-qwen3": ModelConfig(),
    "qwen3-0.6b": ModelConfig(vocab_size=151936, hidden_size=1024, num_layers=28, num_q_heads=16, num_kv_heads=8, head_dim=128, intermediate_size=3072, max_position=40960, tie_word_embeddings=True),
    "qwen3-4b": ModelConfig(vocab_size=151936, hidden_size=2560, num_layers=36, num_q_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=9728, max_position=40960, tie_word_embeddings=True),
    "qwen3-8b": ModelConfig(vocab_size=151936, hidden_size=4096, num_layers=36, num_q_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=12288, max_position=40960),
    "tiny-qwen35": ModelConfig(family="qwen35", vocab_size=1024, hidden_size=256, num_layers=4, num_q_heads=4, num_kv_heads=2, head_dim=64, intermediate_size=512, layer_types=_hybrid_pattern(4), partial_rotary_factor=0.25, attn_output_gate=True, norm_weight_offset=True, gdn_num_k_heads=2, gdn_num_v_heads=4, gdn_head_dim=32, rope_theta=1e7),
    "qwen3.5-27b": ModelConfig(family="qwen35", vocab_size=248320, hidden_size=5120, num_layers=64, num_q_heads=24, num_kv_heads=4, head_dim=256, intermediate_size=17408, layer_types=_hybrid_pattern(64), partial_rotary_factor=0.25, attn_output_gate=True, norm_weight_offset=True, gdn_num_k_heads=16, gdn_num_v_heads=48, gdn_head_dim=128, rope_theta=1e7, max_position=262144),
    "tiny-dsv2": ModelConfig(family="deepseek_v2", vocab_size=1024, hidden_size=256, num_layers=3, num_q_heads=4, num_kv_heads=4, head_dim=48, intermediate_size=512, qk_norm=False, kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, n_routed_experts=8, n_shared_experts=2, num_experts_per_tok=2, moe_intermediate_size=128, first_k_dense_replace=1, rope_theta=10000.0, rope_scaling=dict(_YARN_DSV2)),
    "small-dsv2": ModelConfig(family="deepseek_v2", vocab_size=4096, hidden_size=1024, num_layers=3, num_q_heads=16, num_kv_heads=16, head_dim=192, intermediate_size=2048, qk_norm=False, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, n_routed_experts=16, n_shared_experts=2, num_experts_per_tok=4, moe_intermediate_size=256, first_k_dense_replace=1, rope_theta=10000.0, rope_scaling=dict(_YARN_DSV2), max_position=8192),
    "small-kimi": ModelConfig(family="kimi_k2", vocab_size=4096, hidden_size=1024, num_layers=3, num_q_heads=16, num_kv_heads=16, head_dim=192, intermediate_size=2048, qk_norm=False, q_lora_rank=512, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, n_routed_experts=32, n_shared_experts=1, num_experts_per_tok=4, moe_intermediate_size=256, first_k_dense_replace=1, scoring_func="sigmoid", n_group=4, topk_group=2, norm_topk_prob=True, routed_scaling_factor=2.827, router_bias=True, expert_quant="int4_g32", rope_theta=50000.0, rope_scaling=dict(_YARN_KIMI), rms_eps=1e-5, max_position=8192, num_mtp_layers=1),
    "small-qwen35": ModelConfig(family="qwen35", vocab_size=4096, hidden_size=1024, num_layers=4, num_q_heads=8, num_kv_heads=2, head_dim=256, intermediate_size=2048, layer_types=_hybrid_pattern(4), partial_rotary_factor=0.25, attn_output_gate=True, norm_weight_offset=True, gdn_num_k_heads=4, gdn_num_v_heads=8, gdn_head_dim=128, rope_theta=1e7, max_position=8192),
    "dsv2-lite": ModelConfig(family="deepseek_v2", vocab_size=102400, hidden_size=2048, num_layers=27, num_q_heads=16, num_kv_heads=16, head_dim=192, intermediate_size=10944, qk_norm=False, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, n_routed_experts=64, n_shared_experts=2, num_experts_per_tok=6, moe_intermediate_size=1408, first_k_dense_replace=1, rope_theta=10000.0, rope_scaling=dict(_YARN_DSV2), max_position=163840),
    "tiny-kimi": ModelConfig(family="kimi_k2", vocab_size=1024, hidden_size=256, num_layers=3, num_q_heads=4, num_kv_heads=4, head_dim=48, intermediate_size=512, qk_norm=False, q_lora_rank=96, kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, n_routed_experts=16, n_shared_experts=1, num_experts_per_tok=4, moe_intermediate_size=128, first_k_dense_replace=1, scoring_func="sigmoid", n_group=4, topk_group=2, norm_topk_prob=True, routed_scaling_factor=2.827, router_bias=True, expert_quant="int4_g32", rope_theta=50000.0, rope_scaling=dict(_YARN_KIMI), rms_eps=1e-5, num_mtp_layers=1),
    "kimi-k2": ModelConfig(family="kimi_k2", vocab_size=163840, hidden_size=7168, num_layers=61, num_q_heads=64, num_kv_heads=64, head_dim=192, intermediate_size=18432, qk_norm=False, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, n_routed_experts=384, n_shared_experts=1, num_experts_per_tok=8, moe_intermediate_size=2048, first_k_dense_replace=1, scoring_func="sigmoid", n_group=1, topk_group=1, norm_topk_prob=True, routed_scaling_factor=2.827, router_bias=True, expert_quant="int4_g32", rope_theta=50000.0, rope_scaling=dict(_YARN_KIMI), rms_eps=1e-5, max_position=131072, num_mtp_layers=1),
}
# the DeepSeek-V2 shapes with block-scaled FP8 e4m3 experts (128x128 scale blocks)
PRESETS["tiny-glm"] = ModelConfig(family="glm_dsa", vocab_size=1024, hidden_size=256, num_layers=3, num_q_heads=4, num_kv_heads=4, head_dim=48, intermediate_size=512, qk_norm=False, q_lora_rank=96,
                                  kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=48, n_routed_experts=8, n_shared_experts=1, num_experts_per_tok=2, moe_intermediate_size=128,
                                  first_k_dense_replace=1, scoring_func="sigmoid", n_group=1, topk_group=1, norm_topk_prob=True, routed_scaling_factor=2.5, router_bias=True, rope_theta=10000.0,
                                  rms_eps=1e-5, index_topk=24, index_head_dim=32, index_n_heads=4, num_mtp_layers=1)
PRESETS["small-glm"] = replace(PRESETS["tiny-glm"], vocab_size=4096, hidden_size=1024, num_q_heads=16, num_kv_heads=16, head_dim=256, intermediate_size=2048, q_lora_rank=512, kv_lora_rank=512,
                               qk_nope_head_dim=192, qk_rope_head_dim=64, v_head_dim=256, n_routed_experts=16, num_experts_per_tok=4, moe_intermediate_size=256, index_topk=256, index_head_dim=128,
                               index_n_heads=32, max_position=8192)
# GLM-5 (zai-org/GLM-5): 78 layers, 256 routed experts, MLA with 192 + 64 query dims and 256 value dims, 32-head indexer keeping 2048 keys
PRESETS["glm-5"] = replace(PRESETS["small-glm"], vocab_size=154880, hidden_size=6144, num_layers=78, num_q_heads=64, num_kv_heads=64, intermediate_size=12288, q_lora_rank=2048, n_routed_experts=256,
                           num_experts_per_tok=8, moe_intermediate_size=2048, first_k_dense_replace=3, index_topk=2048, max_position=202752, rope_theta=1e6, expert_quant="fp8_block128")
def _gemma_pattern(n: int) -> tuple:
    return tuple("sliding_attention" if (i + 1) % 6 else "full_attention" for i in range(n))


PRESETS["tiny-gemma4"] = ModelConfig(family="gemma4", vocab_size=1024, hidden_size=256, num_layers=6, num_q_heads=4, num_kv_heads=2, head_dim=64, global_head_dim=128, num_global_kv_heads=1,
                                     attention_k_eq_v=True, intermediate_size=512, sliding_window=32, layer_types=_gemma_pattern(6), rope_theta=1e6, rope_theta_local=1e4,
                                     partial_rotary_factor=0.25, final_logit_softcapping=30.0, hidden_act="gelu_tanh", tie_word_embeddings=True, max_position=4096)
# head dims of the released dense model (256 sliding, 512 global, 5 : 1), two global KV heads of 512 as wide as four local ones of 256
PRESETS["small-gemma4"] = replace(PRESETS["tiny-gemma4"], vocab_size=4096, hidden_size=1024, num_q_heads=8, num_kv_heads=4, head_dim=256, global_head_dim=512, num_global_kv_heads=2,
                                  intermediate_size=2048, sliding_window=128, max_position=8192)
# a 10 B-parameter shape of the line for benchmarks (not a released configuration): 30 sliding + 6 global layers, 16 local
# KV heads of 256 against 4 global KV heads of 512 (the narrower global layers pack their pages at the front of their slab)
PRESETS["gemma4-10b-shape"] = replace(PRESETS["small-gemma4"], vocab_size=262144, hidden_size=4096, num_layers=36, layer_types=_gemma_pattern(36), num_q_heads=32, num_kv_heads=16,
                                      num_global_kv_heads=4, intermediate_size=14336, sliding_window=1024, max_position=131072)


def _k3_pattern(n: int) -> tuple:
    """Full (MLA) attention on every fourth layer and on the last one, KDA elsewhere (pegainfer-k3/src/config.rs:108-114)."""
    return tuple("full_attention" if (i + 1 == n or i % 4 == 3) else "linear_attention" for i in range(n))


PRESETS["tiny-k3"] = ModelConfig(family="kimi_k3", vocab_size=1024, hidden_size=256, num_layers=5, layer_types=_k3_pattern(5), num_q_heads=4, num_kv_heads=4, head_dim=48, gdn_head_dim=32,
                                 gdn_conv_kernel=4, kda_gate_rank=32, intermediate_size=512, qk_norm=False, q_lora_rank=96, kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16,
                                 v_head_dim=32, n_routed_experts=8, n_shared_experts=2, num_experts_per_tok=3, moe_intermediate_size=64, latent_moe_dim=128, first_k_dense_replace=1,
                                 scoring_func="sigmoid", norm_topk_prob=True, router_bias=True, attn_res_block=2, hidden_act="situ", rms_eps=1e-5, max_position=4096)
# head and latent sizes of the released model (KDA heads of 128, MLA 128 + 64 / 128 over a 512-wide latent), few layers and experts
PRESETS["small-k3"] = replace(PRESETS["tiny-k3"], vocab_size=4096, hidden_size=1024, num_layers=6, layer_types=_k3_pattern(6), num_q_heads=16, num_kv_heads=16, head_dim=192, gdn_head_dim=128,
                              kda_gate_rank=128, intermediate_size=2048, q_lora_rank=512, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128, n_routed_experts=16,
                              num_experts_per_tok=4, moe_intermediate_size=256, latent_moe_dim=512, attn_res_block=3, max_position=8192)
# the released text tower (pegainfer-k3/src/config.rs:26-92): 93 layers, 96 heads, 896 routed experts (top 16) in a 3584-wide latent
PRESETS["kimi-k3"] = replace(PRESETS["small-k3"], vocab_size=163840, hidden_size=7168, num_layers=93, layer_types=_k3_pattern(93), num_q_heads=96, num_kv_heads=96, intermediate_size=33792,
                             q_lora_rank=1536, n_routed_experts=896, num_experts_per_tok=16, moe_intermediate_size=3072, latent_moe_dim=3584, attn_res_block=12, max_position=1048576)
# a one-GPU slice of the released shape for benchmarks (not a released configuration): full-width layers (6 KDA + 2 MLA, one dense
# and seven latent-MoE layers), 32 routed experts instead of 896, top 8
PRESETS["k3-8layer-shape"] = replace(PRESETS["kimi-k3"], num_layers=8, layer_types=_k3_pattern(8), n_routed_experts=32, num_experts_per_tok=8, attn_res_block=4, max_position=131072)
PRESETS["small-glm-fp8"] = replace(PRESETS["small-glm"], expert_quant="fp8_block128", dense_quant="fp8_block128")
for _name in ("tiny-dsv2", "small-dsv2", "dsv2-lite"):
    if _name in PRESETS:
        PRESETS[_name + "-fp8"] = replace(PRESETS[_name], expert_quant="fp8_block128")


def preset(name: str, **overrides) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}")
    return replace(PRESETS[name], **overrides)


def detect_family(cfg: dict) -> str:
    """Map a ``config.json`` to a model line (exactly one line must claim it)."""
    mt = cfg.get("model_type", "")
    archs = " ".join(cfg.get("architectures", []))
    if mt in ("qwen3",) or "Qwen3ForCausalLM" in archs:
        return "qwen3"
    if mt.startswith("qwen3_5") or mt in ("qwen3_next",) or "Qwen3_5" in archs or "Qwen3Next" in archs:
        return "qwen35"
    if mt == "deepseek_v2" or "DeepseekV2" in archs:
        return "deepseek_v2"
    if mt == "glm_moe_dsa" or "GlmMoeDsa" in archs:
        return "glm_dsa"
    if mt.startswith("gemma4") or "Gemma4" in archs:
        return "gemma4"
    if mt == "kimi_k3" or "KimiK3" in archs or cfg.get("text_config", {}).get("model_type") == "kimi_linear":
        return "kimi_k3"
    if mt in ("kimi_k2", "deepseek_v3", "kimi_k25") or "DeepseekV3" in archs or "Kimi" in archs:
        return "kimi_k2"
    raise ValueError(f"no model line recognises model_type={mt!r} architectures={archs!r}")


def _eos_ids(model_dir: Optional[str], cfg: dict) -> tuple:
    ids = None
    if model_dir:
        p = os.path.join(model_dir, "generation_config.json")
        if os.path.exists(p):
            with open(p) as f:
                ids = json.load(f).get("eos_token_id")
    if ids is None:
        ids = cfg.get("eos_token_id")
    if ids is None:
        return ()
    if isinstance(ids, int):
        ids = [ids]
    return tuple(dict.fromkeys(int(i) for i in ids))


def _k3_from_hf(cfg: dict, top: dict, model_dir: Optional[str]) -> ModelConfig:
    """Text tower of a Kimi-K3 ``config.json`` (keys as pegainfer-k3/src/config.rs:200-330 checks them)."""
    lin = cfg.get("linear_attn_config", {})
    n = cfg["num_hidden_layers"]
    full = lin.get("full_attn_layers")  # one-based in the checkpoint
    types = tuple("full_attention" if (i + 1) in full else "linear_attention" for i in range(n)) if full else _k3_pattern(n)
    for key, want in (("hidden_act", "situ"), ("moe_router_activation_func", "sigmoid")):
        if cfg.get(key, want) != want:
            raise ValueError(f"Kimi-K3 line: {key}={cfg.get(key)!r} is not supported (expected {want!r})")
    if not cfg.get("mla_use_nope", True) or not cfg.get("mla_use_output_gate", True):
        raise ValueError("Kimi-K3 line: MLA layers without positions (mla_use_nope) and with an output gate are the supported form")
    nope, rope = cfg["qk_nope_head_dim"], cfg["qk_rope_head_dim"]
    return ModelConfig(family="kimi_k3", vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"], num_layers=n, layer_types=types, num_q_heads=cfg["num_attention_heads"],
                       num_kv_heads=cfg.get("num_key_value_heads", cfg["num_attention_heads"]), head_dim=nope + rope, gdn_head_dim=lin.get("head_dim", 128),
                       gdn_conv_kernel=lin.get("short_conv_kernel_size", 4), kda_gate_rank=lin.get("gate_rank", lin.get("head_dim", 128)), kda_gate_lower_bound=float(lin.get("gate_lower_bound", -5.0)),
                       intermediate_size=cfg["intermediate_size"], qk_norm=False, q_lora_rank=cfg["q_lora_rank"], kv_lora_rank=cfg["kv_lora_rank"], qk_nope_head_dim=nope, qk_rope_head_dim=rope,
                       v_head_dim=cfg["v_head_dim"], n_routed_experts=cfg["num_experts"], n_shared_experts=cfg.get("num_shared_experts", 0), num_experts_per_tok=cfg["num_experts_per_token"],
                       moe_intermediate_size=cfg["moe_intermediate_size"], latent_moe_dim=cfg["routed_expert_hidden_size"], first_k_dense_replace=cfg.get("first_k_dense_replace", 1),
                       scoring_func="sigmoid", norm_topk_prob=bool(cfg.get("moe_renormalize", True)), routed_scaling_factor=float(cfg.get("routed_scaling_factor", 1.0)), router_bias=True,
                       expert_quant="mxfp4" if "quantization_config" in top or "quantization_config" in cfg else "bf16", attn_res_block=cfg["attn_res_block_size"], hidden_act="situ",
                       rms_eps=cfg.get("rms_norm_eps", 1e-5), max_position=cfg.get("max_position_embeddings", 4096), tie_word_embeddings=bool(top.get("tie_word_embeddings", False)),
                       eos_token_ids=_eos_ids(model_dir, top))


def from_hf(cfg: dict, model_dir: Optional[str] = None) -> ModelConfig:
    family = detect_family(cfg)
    top = cfg
    if family == "qwen35" and "text_config" in cfg:
        cfg = cfg["text_config"]
    if family == "kimi_k2" and "text_config" in cfg:
        cfg = cfg["text_config"]
    if family == "gemma4" and "text_config" in cfg:
        cfg = cfg["text_config"]
    if family == "kimi_k3":
        return _k3_from_hf(cfg.get("text_config", cfg), top, model_dir)
    common = dict(
        family=family,
        vocab_size=cfg["vocab_size"],
        hidden_size=cfg["hidden_size"],
        num_layers=cfg["num_hidden_layers"],
        num_q_heads=cfg["num_attention_heads"],
        num_kv_heads=cfg.get("num_key_value_heads", cfg["num_attention_heads"]),
        intermediate_size=cfg["intermediate_size"],
        rms_eps=cfg.get("rms_norm_eps", 1e-6),
        max_position=cfg.get("max_position_embeddings", 4096),
        tie_word_embeddings=bool(top.get("tie_word_embeddings", cfg.get("tie_word_embeddings", False))),
        eos_token_ids=_eos_ids(model_dir, top),
    )
    if family == "gemma4":
        for key in ("hidden_size_per_layer_input", "num_kv_shared_layers"):
            if cfg.get(key, 0):
                raise ValueError(f"gemma4: {key}={cfg[key]} (per-layer input embeddings / cross-layer KV sharing of the small variants) is not supported")
        if cfg.get("enable_moe_block"):
            raise ValueError("gemma4: the mixture-of-experts variant is not supported")
        rp = cfg.get("rope_parameters") or {}
        full, local = rp.get("full_attention", {}), rp.get("sliding_attention", {})
        n = cfg["num_hidden_layers"]
        types = cfg.get("layer_types") or ["sliding_attention" if (i + 1) % 6 else "full_attention" for i in range(n)]
        common["tie_word_embeddings"] = bool(top.get("tie_word_embeddings", cfg.get("tie_word_embeddings", True)))
        return ModelConfig(
            head_dim=cfg.get("head_dim", 256),
            global_head_dim=cfg.get("global_head_dim", 512) or cfg.get("head_dim", 256),
            num_global_kv_heads=cfg.get("num_global_key_value_heads") or common["num_kv_heads"],
            attention_k_eq_v=bool(cfg.get("attention_k_eq_v", False)),
            sliding_window=cfg.get("sliding_window", 512),
            layer_types=tuple(types),
            rope_theta=full.get("rope_theta", 1e6),
            partial_rotary_factor=full.get("partial_rotary_factor", 0.25),
            rope_theta_local=local.get("rope_theta", 1e4),
            final_logit_softcapping=cfg.get("final_logit_softcapping") or 0.0,
            hidden_act="gelu_tanh",
            qk_norm=True,
            **common,
        )
    if family == "qwen3":
        return ModelConfig(head_dim=cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"]), rope_theta=cfg.get("rope_theta", 1e6), **common)
    if family == "qwen35":
        rp = cfg.get("rope_parameters", {})
        return ModelConfig(
            head_dim=cfg.get("head_dim", 256),
            rope_theta=rp.get("rope_theta", cfg.get("rope_theta", 1e7)),
            partial_rotary_factor=rp.get("partial_rotary_factor", cfg.get("partial_rotary_factor", 0.25)),
            layer_types=tuple(cfg["layer_types"]),
            attn_output_gate=True,
            norm_weight_offset=True,
            gdn_num_k_heads=cfg["linear_num_key_heads"],
            gdn_num_v_heads=cfg["linear_num_value_heads"],
            gdn_head_dim=cfg.get("linear_key_head_dim", 128),
            gdn_conv_kernel=cfg.get("linear_conv_kernel_dim", 4),
            **common,
        )
    mla = dict(
        qk_norm=False,
        q_lora_rank=cfg.get("q_lora_rank") or 0,
        kv_lora_rank=cfg["kv_lora_rank"],
        qk_nope_head_dim=cfg["qk_nope_head_dim"],
        qk_rope_head_dim=cfg["qk_rope_head_dim"],
        v_head_dim=cfg["v_head_dim"],
        head_dim=cfg["qk_nope_head_dim"] + cfg["qk_rope_head_dim"],
        rope_theta=cfg.get("rope_theta") or (cfg.get("rope_parameters") or {}).get("rope_theta", 10000.0),
        rope_scaling=cfg.get("rope_scaling"),
        n_routed_experts=cfg.get("n_routed_experts", 0),
        n_shared_experts=cfg.get("n_shared_experts", 0),
        num_experts_per_tok=cfg.get("num_experts_per_tok", 0),
        moe_intermediate_size=cfg.get("moe_intermediate_size", 0),
        first_k_dense_replace=cfg.get("first_k_dense_replace", 0),
        scoring_func=cfg.get("scoring_func", "softmax"),
        n_group=cfg.get("n_group", 1) or 1,
        topk_group=cfg.get("topk_group", 1) or 1,
        norm_topk_prob=bool(cfg.get("norm_topk_prob", False)),
        routed_scaling_factor=cfg.get("routed_scaling_factor", 1.0),
    )
    q = cfg.get("quantization_config") or top.get("quantization_config") or {}
    quant = "bf16"
    if q.get("quant_method") == "compressed-tensors" or q.get("format") == "pack-quantized":
        quant = "int4_g32"
    elif q.get("quant_method") == "fp8":
        quant = "fp8_block128"
    mla.update(expert_quant=quant)
    if family == "kimi_k2":
        mla.update(router_bias=True, num_mtp_layers=cfg.get("num_nextn_predict_layers", 0))
    if family == "glm_dsa":
        types = cfg.get("mlp_layer_types")
        dense = cfg.get("first_k_dense_replace", 3) if types is None else next((i for i, t in enumerate(types) if t == "sparse"), len(types))
        mla.update(dense_quant="fp8_block128" if quant == "fp8_block128" else "bf16", router_bias=True, scoring_func="sigmoid", first_k_dense_replace=dense, num_mtp_layers=cfg.get("num_nextn_predict_layers", 0),
                   index_topk=cfg.get("index_topk", 2048), index_head_dim=cfg.get("index_head_dim", 128), index_n_heads=cfg.get("index_n_heads", 32))
    return ModelConfig(**common, **mla)


def load_model_config(model_dir: str) -> ModelConfig:
    with open(os.path.join(model_dir, "config.json")) as f:
        return from_hf(json.load(f), model_dir)


@dataclass
class EngineConfig:
    """Serving knobs (one per CLI flag)."""

    model_path: Optional[str] = None
    preset: Optional[str] = None
    served_model_name: Optional[str] = None
    port: int = 8000
    host: str = "127.0.0.1"
    cuda_graph: bool = True
    precapture_graphs: bool = False  # capture every decode bucket at start-up
    dump_graph_dot: Optional[str] = None
    device_ordinal: int = 0
    tp_size: int = 1
    dp_size: int = 1
    ep_size: int = 1
    kv_page_size: int = 16
    num_kv_blocks: Optional[int] = None
    gpu_memory_utilization: float = 0.90
    kv_cache_memory_margin_mib: int = 150
    no_prefix_cache: bool = False
    kv_offload: bool = False
    kv_offload_host_gib: float = 4.0
    kv_offload_l1_disabled: bool = False  # test mode: evict idle GPU blocks before every probe
    kv_offload_disk_dir: Optional[str] = None  # third tier: blocks evicted from host memory go to files here
    kv_offload_disk_gib: float = 0.0
    max_prefill_tokens: int = 1024
    max_decode_batch: int = 256
    max_model_len: Optional[int] = None
    batch_invariant: bool = False
    decode_overlap: bool = False
    run_ahead: bool = True  # greedy graph decode launches the next step before reading this one's tokens
    tune_gc: bool = False  # freeze start-up objects and raise the collector thresholds (utils/runtime.py); the server and the benches turn it on
    decode_sm_pct: int = 50
    decode_sm_split: bool = False  # --decode-sm-pct given: the prefill lane gets its own SM partition (green contexts)
    enable_lora: bool = False
    max_loras: int = 4
    max_lora_rank: int = 64
    lora_modules: tuple = ()
    spec_method: Optional[str] = None  # None | "mtp" | "draft" | "dflash" | "dspark" | "eagle3"
    spec_draft_len: int = 1
    draft_model_path: Optional[str] = None
    comm: str = "fused"  # fused | nccl
    gemm: str = "sm100"  # sm100 | cublas
    seed: int = 0
    dtype: str = "bfloat16"

    def validate(self) -> None:
        if self.kv_page_size not in (16, 32, 64):
            raise ValueError("--kv-page-size must be 16, 32 or 64")
        if not (0.05 <= self.gpu_memory_utilization <= 0.99):
            raise ValueError("--gpu-memory-utilization must be in [0.05, 0.99]")
        if self.max_prefill_tokens < 1:
            raise ValueError("--max-prefill-tokens must be positive")
        if self.comm not in ("fused", "nccl"):
            raise ValueError("--comm must be fused or nccl")
        if self.gemm not in ("sm100", "cublas"):
            raise ValueError("--gemm must be sm100 or cublas")
        for n in ("tp_size", "dp_size", "ep_size"):
            if getattr(self, n) < 1:
                raise ValueError(f"--{n.replace('_', '-')} must be >= 1")
