"""Model-line registry: one builder per architecture family.

Reference parity: pegainfer-server/src/main.rs:24-41 (compiled-in model lines),
pegainfer-frontend/src/model_line.rs:453-586 (registry, detect by config.json).
"""
from __future__ import annotations

from ..config import ModelConfig


def _qwen3(cfg, **kw):
    from .qwen3 import Qwen3Model

    kw.pop("ep", None)
    return Qwen3Model(cfg, **kw)


def _qwen35(cfg, **kw):
    from .qwen35 import Qwen35Model

    kw.pop("ep", None)
    return Qwen35Model(cfg, **kw)


def _mla_moe(cfg, **kw):
    from .mla_moe import MlaMoeModel

    return MlaMoeModel(cfg, **kw)


def _glm_dsa(cfg, **kw):
    from .glm_dsa import GlmDsaModel

    return GlmDsaModel(cfg, **kw)


def _gemma4(cfg, **kw):
    from .gemma4 import Gemma4Model

    kw.pop("ep", None)
    return Gemma4Model(cfg, **kw)


def _k3(cfg, **kw):
    from .k3 import K3Model

    return K3Model(cfg, **kw)


BUILDERS = {"kimi_k3": _k3, "gemma4": _gemma4, "glm_dsa": _glm_dsa, "qwen3": _qwen3, "qwen35": _qwen35, "deepseek_v2": _mla_moe, "kimi_k2": _mla_moe}


def build(cfg: ModelConfig, **kw):
    if cfg.family not in BUILDERS:
        raise ValueError(f"no model line for family {cfg.family!r}; known: {sorted(BUILDERS)}")
    return BUILDERS[cfg.family](cfg, **kw)


def shapes_for(cfg: ModelConfig) -> dict:
    """Full (unsharded) tensor shapes of a model family that has no entry in ``loader.export``."""
    if cfg.family == "glm_dsa":
        from .glm_dsa import glm_dsa_shapes

        return glm_dsa_shapes(cfg)
    if cfg.family == "gemma4":
        from .gemma4 import gemma4_shapes

        return gemma4_shapes(cfg)
    if cfg.family == "kimi_k3":
        from .k3 import k3_shapes

        return k3_shapes(cfg)
    raise ValueError(f"no tensor-shape table for family {cfg.family!r}")


def hf_config_extras(cfg: ModelConfig) -> dict:
    """Family-specific ``config.json`` keys for ``loader.export.to_hf_config``."""
    if cfg.family == "glm_dsa":
        return dict(model_type="glm_moe_dsa", architectures=["GlmMoeDsaForCausalLM"], q_lora_rank=cfg.q_lora_rank, kv_lora_rank=cfg.kv_lora_rank, qk_nope_head_dim=cfg.qk_nope_head_dim,
                    qk_rope_head_dim=cfg.qk_rope_head_dim, v_head_dim=cfg.v_head_dim, n_routed_experts=cfg.n_routed_experts, n_shared_experts=cfg.n_shared_experts,
                    num_experts_per_tok=cfg.num_experts_per_tok, moe_intermediate_size=cfg.moe_intermediate_size, n_group=cfg.n_group, topk_group=cfg.topk_group,
                    norm_topk_prob=cfg.norm_topk_prob, routed_scaling_factor=cfg.routed_scaling_factor, num_nextn_predict_layers=cfg.num_mtp_layers,
                    mlp_layer_types=["dense" if i < cfg.first_k_dense_replace else "sparse" for i in range(cfg.num_layers)], first_k_dense_replace=cfg.first_k_dense_replace,
                    index_topk=cfg.index_topk, index_head_dim=cfg.index_head_dim, index_n_heads=cfg.index_n_heads, rope_parameters=dict(rope_theta=cfg.rope_theta, rope_type="default"))
    if cfg.family == "gemma4":
        return dict(model_type="gemma4_text", architectures=["Gemma4ForCausalLM"], head_dim=cfg.head_dim, global_head_dim=cfg.global_head_dim or cfg.head_dim,
                    num_global_key_value_heads=cfg.num_global_kv_heads or cfg.num_kv_heads, attention_k_eq_v=cfg.attention_k_eq_v, sliding_window=cfg.sliding_window,
                    layer_types=list(cfg.layer_types), final_logit_softcapping=cfg.final_logit_softcapping or None, hidden_activation="gelu_pytorch_tanh",
                    hidden_size_per_layer_input=0, vocab_size_per_layer_input=cfg.vocab_size, num_kv_shared_layers=0, enable_moe_block=False, use_double_wide_mlp=False,
                    rope_parameters={"sliding_attention": {"rope_type": "default", "rope_theta": cfg.rope_theta_local},
                                     "full_attention": {"rope_type": "proportional", "partial_rotary_factor": cfg.partial_rotary_factor, "rope_theta": cfg.rope_theta}})
    if cfg.family == "kimi_k3":
        full = [i + 1 for i in range(cfg.num_layers) if cfg.layer_type(i) == "full_attention"]  # one-based in the checkpoint
        text = dict(model_type="kimi_linear", hidden_act="situ", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, num_hidden_layers=cfg.num_layers,
                    first_k_dense_replace=cfg.first_k_dense_replace, max_position_embeddings=cfg.max_position, intermediate_size=cfg.intermediate_size,
                    moe_intermediate_size=cfg.moe_intermediate_size, routed_expert_hidden_size=cfg.latent_moe_dim, attn_res_block_size=cfg.attn_res_block,
                    num_attention_heads=cfg.num_q_heads, num_key_value_heads=cfg.num_kv_heads, q_lora_rank=cfg.q_lora_rank, kv_lora_rank=cfg.kv_lora_rank,
                    qk_nope_head_dim=cfg.qk_nope_head_dim, qk_rope_head_dim=cfg.qk_rope_head_dim, v_head_dim=cfg.v_head_dim, mla_use_nope=True, mla_use_output_gate=True,
                    num_experts=cfg.n_routed_experts, num_experts_per_token=cfg.num_experts_per_tok, num_shared_experts=cfg.n_shared_experts, num_expert_group=1, topk_group=1,
                    moe_router_activation_func="sigmoid", moe_renormalize=cfg.norm_topk_prob, routed_scaling_factor=cfg.routed_scaling_factor, rms_norm_eps=cfg.rms_eps,
                    linear_attn_config=dict(num_heads=cfg.num_q_heads, head_dim=cfg.gdn_head_dim, short_conv_kernel_size=cfg.gdn_conv_kernel, gate_rank=cfg.kda_gate_rank,
                                            gate_lower_bound=cfg.kda_gate_lower_bound, full_attn_layers=full, use_full_rank_gate=True))
        return dict(model_type="kimi_k3", architectures=["KimiK3ForConditionalGeneration"], text_config=text)
    return {}
