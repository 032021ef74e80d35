"""Write a model as a Hugging Face style checkpoint directory.

``export_checkpoint`` materialises every tensor of a model configuration from a weight
source (by default the deterministic random source of that model family) and writes
``config.json`` plus sharded ``model-0000x-of-0000y.safetensors`` files with a
``model.safetensors.index.json`` weight map, in the tensor names and storage dtypes of the
real checkpoints: bf16 matrices, compressed-tensors INT4 (``weight_packed`` int32 +
``weight_scale`` bf16) and block-scaled FP8 (``weight`` e4m3 + ``weight_scale_inv`` f32).
It is what the loader tests read back, and it gives users a checkpoint of any preset shape
for dry runs without network access (``python -m pegainfer_b200.loader.export``).

``quantize_dense_to_fp8`` turns named bf16 matrices of such a directory's tensor dict into
the DeepSeek-V3 style FP8 pair, so that the load-boundary dequantisation can be exercised.

Reference parity: the checkpoint layouts consumed by pegainfer-core/src/weight_loader.rs:32-66
(index + shards), pegainfer-kimi-k2/src/weights/manifest.rs (INT4 names) and
pegainfer-glm52/src/fp8.rs (FP8 ``weight_scale_inv`` blocks).
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch

from ..config import ModelConfig


def default_source(cfg: ModelConfig, seed: int = 0, dtype=torch.bfloat16):
    """The deterministic random weight source a model of this family builds for itself."""
    from .sources import RandomSource

    if cfg.family == "qwen3":
        from ..models.qwen3 import qwen3_shapes

        return RandomSource(qwen3_shapes(cfg), seed=seed, dtype=dtype)
    if cfg.family == "qwen35":
        from ..models.qwen35 import _kind, qwen35_shapes

        return RandomSource(qwen35_shapes(cfg), seed=seed, dtype=dtype, kind=_kind)
    if cfg.family in ("deepseek_v2", "kimi_k2"):
        from ..models.mla_moe import _QuantRandomSource, mla_moe_shapes

        return _QuantRandomSource(mla_moe_shapes(cfg), seed=seed, dtype=dtype)
    if cfg.family == "gemma4":
        from ..models.gemma4 import gemma4_source

        return gemma4_source(cfg, seed=seed, dtype=dtype)
    from ..models import registry

    shapes = registry.shapes_for(cfg)
    if cfg.is_moe:
        from ..models.mla_moe import _QuantRandomSource

        return _QuantRandomSource(shapes, seed=seed, dtype=dtype)
    return RandomSource(shapes, seed=seed, dtype=dtype)


def to_hf_config(cfg: ModelConfig) -> dict:
    """``config.json`` contents that ``config.from_hf`` maps back to ``cfg``."""
    arch = {"qwen3": ("qwen3", "Qwen3ForCausalLM"), "qwen35": ("qwen3_5", "Qwen3_5ForCausalLM"), "deepseek_v2": ("deepseek_v2", "DeepseekV2ForCausalLM"),
            "kimi_k2": ("kimi_k2", "DeepseekV3ForCausalLM")}.get(cfg.family, (cfg.family, cfg.family))
    out = {
        "model_type": arch[0],
        "architectures": [arch[1]],
        "vocab_size": cfg.vocab_size,
        "hidden_size": cfg.hidden_size,
        "num_hidden_layers": cfg.num_layers,
        "num_attention_heads": cfg.num_q_heads,
        "num_key_value_heads": cfg.num_kv_heads,
        "intermediate_size": cfg.intermediate_size,
        "rms_norm_eps": cfg.rms_eps,
        "max_position_embeddings": cfg.max_position,
        "tie_word_embeddings": cfg.tie_word_embeddings,
        "rope_theta": cfg.rope_theta,
        "torch_dtype": "bfloat16",
    }
    if cfg.eos_token_ids:
        out["eos_token_id"] = list(cfg.eos_token_ids)
    if cfg.family == "qwen3":
        out["head_dim"] = cfg.head_dim
    elif cfg.family == "qwen35":
        out.update(head_dim=cfg.head_dim, partial_rotary_factor=cfg.partial_rotary_factor, layer_types=list(cfg.layer_types), linear_num_key_heads=cfg.gdn_num_k_heads,
                   linear_num_value_heads=cfg.gdn_num_v_heads, linear_key_head_dim=cfg.gdn_head_dim, linear_value_head_dim=cfg.gdn_head_dim, linear_conv_kernel_dim=cfg.gdn_conv_kernel)
    elif cfg.family in ("deepseek_v2", "kimi_k2"):
        out.update(q_lora_rank=cfg.q_lora_rank or None, kv_lora_rank=cfg.kv_lora_rank, qk_nope_head_dim=cfg.qk_nope_head_dim, qk_rope_head_dim=cfg.qk_rope_head_dim, v_head_dim=cfg.v_head_dim,
                   rope_scaling=cfg.rope_scaling, n_routed_experts=cfg.n_routed_experts, n_shared_experts=cfg.n_shared_experts, num_experts_per_tok=cfg.num_experts_per_tok,
                   moe_intermediate_size=cfg.moe_intermediate_size, first_k_dense_replace=cfg.first_k_dense_replace, scoring_func=cfg.scoring_func, n_group=cfg.n_group,
                   topk_group=cfg.topk_group, norm_topk_prob=cfg.norm_topk_prob, routed_scaling_factor=cfg.routed_scaling_factor, num_nextn_predict_layers=cfg.num_mtp_layers)
        if cfg.expert_quant == "int4_g32":
            out["quantization_config"] = {"quant_method": "compressed-tensors", "format": "pack-quantized", "config_groups": {"group_0": {"weights": {"num_bits": 4, "group_size": cfg.quant_group_size, "symmetric": True}}}}
        elif cfg.expert_quant == "fp8_block128":
            out["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128]}
    else:
        from ..models import registry

        out.update(registry.hf_config_extras(cfg))
    if cfg.family == "qwen35":
        # the released checkpoints are multimodal wrappers: the language model's keys sit in text_config
        text = dict(out, model_type="qwen3_5_text")
        text.pop("architectures")
        return {"model_type": "qwen3_5", "architectures": ["Qwen3_5ForConditionalGeneration"], "tie_word_embeddings": cfg.tie_word_embeddings, "text_config": text}
    return out


def storage_dtype(name: str, source, dtype):
    """Dtype a tensor has on disk in the real checkpoints."""
    if name.endswith("weight_packed"):
        return torch.int32
    if name.endswith("weight_scale_inv") or name.endswith("e_score_correction_bias"):
        return torch.float32
    if name.endswith(".weight") and source.has(name + "_scale_inv"):
        return torch.float8_e4m3fn
    return dtype


def materialize(cfg: ModelConfig, source=None, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """Every tensor of the model as a name -> CPU tensor dict, in checkpoint storage dtypes."""
    source = source or default_source(cfg, seed, dtype)
    return {name: source.get(name, "cpu", storage_dtype(name, source, dtype)).contiguous() for name in source.names()}


def quantize_dense_to_fp8(tensors: dict, names, block: int = 128) -> dict:
    """Replace the named 2-D matrices by the (e4m3 ``weight``, f32 ``weight_scale_inv``) pair with
    one scale per ``block`` x ``block`` tile.  Returns ``name -> dequantised f32`` (what a loader
    that widens the tensor must reproduce)."""
    expect = {}
    for name in names:
        w = tensors[name].float()
        rows, cols = w.shape
        nb_r, nb_c = (rows + block - 1) // block, (cols + block - 1) // block
        pad = torch.zeros((nb_r * block, nb_c * block))
        pad[:rows, :cols] = w
        tiles = pad.view(nb_r, block, nb_c, block)
        amax = tiles.abs().amax(dim=(1, 3)).clamp_(min=1e-12)
        scale_inv = amax / 448.0
        q = (tiles / scale_inv[:, None, :, None]).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn)
        deq = (q.float() * scale_inv[:, None, :, None]).reshape(nb_r * block, nb_c * block)[:rows, :cols]
        tensors[name] = q.reshape(nb_r * block, nb_c * block)[:rows, :cols].contiguous()
        tensors[name + "_scale_inv"] = scale_inv.contiguous()
        expect[name] = deq.contiguous()
    return expect


def write_checkpoint(tensors: dict, cfg: ModelConfig, out_dir: str, shards: int = 2) -> list:
    """Write ``tensors`` as ``shards`` safetensors files plus index and ``config.json``."""
    from safetensors.torch import save_file

    os.makedirs(out_dir, exist_ok=True)
    names = list(tensors)
    shards = max(1, min(shards, len(names)))
    total = sum(t.numel() * t.element_size() for t in tensors.values())
    files, weight_map = [], {}
    if shards == 1:
        save_file(tensors, os.path.join(out_dir, "model.safetensors"))
        files.append("model.safetensors")
    else:
        # contiguous name ranges of roughly equal bytes, like the hub's shards
        budget, cur, acc, groups = total / shards, [], 0, []
        for n in names:
            cur.append(n)
            acc += tensors[n].numel() * tensors[n].element_size()
            if acc >= budget and len(groups) < shards - 1:
                groups.append(cur)
                cur, acc = [], 0
        if cur:
            groups.append(cur)
        for i, grp in enumerate(groups):
            fn = f"model-{i + 1:05d}-of-{len(groups):05d}.safetensors"
            save_file({n: tensors[n] for n in grp}, os.path.join(out_dir, fn))
            files.append(fn)
            for n in grp:
                weight_map[n] = fn
        with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(to_hf_config(cfg), f, indent=1)
    return files


def export_checkpoint(cfg: ModelConfig, out_dir: str, seed: int = 0, dtype=torch.bfloat16, shards: int = 2, source=None) -> dict:
    tensors = materialize(cfg, source, seed, dtype)
    write_checkpoint(tensors, cfg, out_dir, shards)
    return tensors


def main(argv: Optional[list] = None) -> int:
    import argparse

    from ..config import preset

    ap = argparse.ArgumentParser(description="write a random-weight checkpoint of a preset shape")
    ap.add_argument("--preset", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--shards", type=int, default=2)
    a = ap.parse_args(argv)
    t = export_checkpoint(preset(a.preset), a.out, a.seed, shards=a.shards)
    print(f"wrote {len(t)} tensors to {a.out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
