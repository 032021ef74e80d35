"""LoRA: PEFT loading, per-request adapters in a mixed batch, HTTP routes, unload rules."""
import json
import os

import pytest
import torch
from safetensors.torch import save_file

from pegainfer_b200.config import EngineConfig, preset
from pegainfer_b200.engine.build import build_engine
from pegainfer_b200.engine.contract import Request
from pegainfer_b200.lora.manager import LoraError, LoraManager


def write_adapter(path, cfg, rank=4, alpha=8, seed=0, targets=("q_proj", "v_proj", "o_proj", "down_proj")):
    os.makedirs(path, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    d, h = cfg.head_dim, cfg.hidden_size
    dims = {"q_proj": (h, cfg.num_q_heads * d), "k_proj": (h, cfg.num_kv_heads * d), "v_proj": (h, cfg.num_kv_heads * d), "o_proj": (cfg.num_q_heads * d, h), "gate_proj": (h, cfg.intermediate_size), "up_proj": (h, cfg.intermediate_size), "down_proj": (cfg.intermediate_size, h)}
    t = {}
    for li in range(cfg.num_layers):
        for p in targets:
            k_in, m_out = dims[p]
            sub = "self_attn" if p in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
            base = f"base_model.model.model.layers.{li}.{sub}.{p}"
            t[base + ".lora_A.weight"] = torch.randn(rank, k_in, generator=g) * 0.3
            t[base + ".lora_B.weight"] = torch.randn(m_out, rank, generator=g) * 0.3
    save_file(t, os.path.join(path, "adapter_model.safetensors"))
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump({"r": rank, "lora_alpha": alpha, "target_modules": list(targets)}, f)
    return t


def merged_engine(cfg, tensors, rank, alpha):
    """Reference: fold the adapter into the dense weights of a fresh model."""
    eng = build_engine(EngineConfig(preset="tiny-qwen3", num_kv_blocks=128, cuda_graph=False), cfg, device="cpu", dtype=torch.float32)
    d = cfg.head_dim
    qs, ks = cfg.num_q_heads * d, cfg.num_kv_heads * d
    for li, l in enumerate(eng.model.layers):
        def delta(p):
            sub = "self_attn" if p in ("q_proj", "k_proj", "v_proj", "o_proj") else "mlp"
            a = tensors.get(f"base_model.model.model.layers.{li}.{sub}.{p}.lora_A.weight")
            b = tensors.get(f"base_model.model.model.layers.{li}.{sub}.{p}.lora_B.weight")
            return None if a is None else (alpha / rank) * (b @ a)
        for p, sl in (("q_proj", slice(0, qs)), ("k_proj", slice(qs, qs + ks)), ("v_proj", slice(qs + ks, None))):
            dl = delta(p)
            if dl is not None:
                l.qkv[sl] += dl
        for p, w in (("o_proj", l.o), ("down_proj", l.down)):
            dl = delta(p)
            if dl is not None:
                w += dl
        ff = cfg.intermediate_size
        for p, sl in (("gate_proj", slice(0, ff)), ("up_proj", slice(ff, None))):
            dl = delta(p)
            if dl is not None:
                l.gate_up[sl] += dl
    return eng


def test_mixed_batch_with_and_without_adapter(tmp_path):
    cfg = preset("tiny-qwen3")
    tensors = write_adapter(str(tmp_path / "a"), cfg, rank=4, alpha=8)
    eng = build_engine(EngineConfig(preset="tiny-qwen3", num_kv_blocks=128, cuda_graph=False, enable_lora=True), cfg, device="cpu", dtype=torch.float32)
    ref = merged_engine(cfg, tensors, 4, 8)
    base = build_engine(EngineConfig(preset="tiny-qwen3", num_kv_blocks=128, cuda_graph=False), cfg, device="cpu", dtype=torch.float32)
    try:
        mgr = LoraManager(eng, max_loras=2, max_rank=8)
        mgr.load("ada", str(tmp_path / "a"))
        p1, p2 = list(range(5, 30)), list(range(40, 60))
        s1 = eng.submit(Request(prompt_tokens=p1, max_tokens=6, lora_adapter="ada"))
        s2 = eng.submit(Request(prompt_tokens=p2, max_tokens=6))
        s3 = eng.submit(Request(prompt_tokens=p1, max_tokens=6, lora_adapter="nope"))
        t1, t2 = s1.collect(60)[0], s2.collect(60)[0]
        assert s3.collect(60)[1].kind == "rejected"
        assert t1 == ref.generate([p1], max_tokens=6)[0][0]
        assert t2 == base.generate([p2], max_tokens=6)[0][0]
        with pytest.raises(LoraError):
            mgr.load("ada", str(tmp_path / "a"))
        mgr.unload("ada")
        assert not mgr.has("ada") and eng.submit(Request(prompt_tokens=p1, max_tokens=2, lora_adapter="ada")).collect(60)[1].kind == "rejected"
        with pytest.raises(LoraError):
            mgr.load("big", str(tmp_path / "missing"))
    finally:
        for e in (eng, ref, base):
            e.shutdown()
