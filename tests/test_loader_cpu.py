"""Checkpoint loading from safetensors files on CPU: a tiny Hugging Face style directory
(config.json, two shards, index) is written for each storage format -- bf16, compressed-tensors
INT4 (``weight_packed`` / ``weight_scale``) and block-scaled FP8 (``weight`` / ``weight_scale_inv``)
-- and loaded through ``SafetensorsSource``; the model must match the one built from the same
tensors held in memory, at tensor-parallel size 1 (logits) and 2 (every rank's shards).

Mirrors the reference's loader checks (pegainfer-core/src/weight_loader.rs tests: shard index,
slices, dtype validation at the load boundary)."""
import dataclasses
import json
import os

import pytest
import torch

from pegainfer_b200.config import EngineConfig, load_model_config, preset
from pegainfer_b200.engine.build import build_engine
from pegainfer_b200.engine.contract import SamplingParams
from pegainfer_b200.loader import export
from pegainfer_b200.loader.sources import DictSource, SafetensorsSource, WeightError
from pegainfer_b200.models import registry
from pegainfer_b200.parallel.ep import EPContext
from pegainfer_b200.parallel.tp import TPContext


def _tensors_of(obj, prefix=""):
    """Every tensor reachable from a model's layers / attributes, by path."""
    out = {}
    items = vars(obj).items() if not isinstance(obj, dict) else obj.items()
    for k, v in items:
        if isinstance(v, torch.Tensor):
            out[prefix + str(k)] = v
        elif isinstance(v, (list, tuple)):
            for i, e in enumerate(v):
                if isinstance(e, torch.Tensor):
                    out[f"{prefix}{k}.{i}"] = e
                elif dataclasses.is_dataclass(e) or isinstance(e, dict):
                    out.update(_tensors_of(e, f"{prefix}{k}.{i}."))
        elif isinstance(v, dict):
            out.update(_tensors_of(v, f"{prefix}{k}."))
        elif dataclasses.is_dataclass(v):
            out.update(_tensors_of(v, f"{prefix}{k}."))
    return out


def _same_model(a, b):
    ta, tb = _tensors_of(a), _tensors_of(b)
    assert ta.keys() == tb.keys() and len(ta) > 4
    for k in ta:
        assert ta[k].dtype == tb[k].dtype and ta[k].shape == tb[k].shape, k
        assert torch.equal(ta[k].view(torch.uint8) if ta[k].dtype == torch.float8_e4m3fn else ta[k], tb[k].view(torch.uint8) if tb[k].dtype == torch.float8_e4m3fn else tb[k]), f"tensor {k} differs"


@pytest.mark.parametrize("name", ["tiny-qwen3", "tiny-kimi", "tiny-dsv2-fp8", "tiny-qwen35"])
def test_safetensors_directory_round_trip(tmp_path, name):
    cfg = preset(name)
    d = str(tmp_path / name)
    tensors = export.export_checkpoint(cfg, d, seed=3, dtype=torch.bfloat16, shards=2)
    assert os.path.exists(os.path.join(d, "model.safetensors.index.json"))
    wm = json.load(open(os.path.join(d, "model.safetensors.index.json")))["weight_map"]
    assert len(set(wm.values())) == 2 and set(wm) == set(tensors)
    if name == "tiny-kimi":
        assert any(n.endswith("weight_packed") and tensors[n].dtype == torch.int32 for n in tensors)
        assert any(n.endswith("weight_scale") and tensors[n].dtype == torch.bfloat16 for n in tensors)
    if name == "tiny-dsv2-fp8":
        assert any(n.endswith("weight_scale_inv") and tensors[n].dtype == torch.float32 for n in tensors)
        assert any(tensors[n].dtype == torch.float8_e4m3fn for n in tensors)
    # config.json maps back to the same model configuration
    back = load_model_config(d)
    for f in dataclasses.fields(cfg):
        if f.name in ("eos_token_ids",):
            continue
        assert getattr(back, f.name) == getattr(cfg, f.name), f.name
    # tensor-parallel / expert-parallel size 1: same weights, same logits, same greedy tokens
    moe = cfg.family in ("deepseek_v2", "kimi_k2")
    kw = dict(device="cpu", dtype=torch.float32, seed=0)
    ref = registry.build(cfg, source=DictSource(tensors), **kw)
    got = registry.build(cfg, source=SafetensorsSource(d, prefetch=False), **kw)
    _same_model(ref, got)
    ecfg = EngineConfig(model_path=d, kv_page_size=16, num_kv_blocks=64, cuda_graph=False, max_prefill_tokens=64)
    eng = build_engine(ecfg, device="cpu", dtype=torch.float32)
    ecfg2 = EngineConfig(preset=name, kv_page_size=16, num_kv_blocks=64, cuda_graph=False, max_prefill_tokens=64)
    eng2 = build_engine(ecfg2, cfg, device="cpu", dtype=torch.float32, model=ref)
    try:
        g = torch.Generator().manual_seed(5)
        ps = [torch.randint(0, cfg.vocab_size, (20 + 3 * i,), generator=g).tolist() for i in range(2)]
        sp = SamplingParams(temperature=0.0, ignore_eos=True)
        a = [o[0] for o in eng.generate(ps, sp, max_tokens=5, timeout=120)]
        b = [o[0] for o in eng2.generate(ps, sp, max_tokens=5, timeout=120)]
        assert a == b
    finally:
        eng.shutdown()
        eng2.shutdown()
    # size 2: every rank's shards are the same slices whichever source they come from
    for rank in range(2):
        par = dict(ep=EPContext(rank, 2, comm="nccl")) if moe else dict(tp=TPContext(rank, 2, comm="nccl"))
        r2 = registry.build(cfg, source=DictSource(tensors), **kw, **par)
        g2 = registry.build(cfg, source=SafetensorsSource(d, prefetch=False), **kw, **par)
        _same_model(r2, g2)


def test_dense_fp8_tensors_are_dequantised_at_the_load_boundary(tmp_path):
    """DeepSeek-V3 style checkpoints store dense projections as e4m3 + ``weight_scale_inv``; a
    loader that asks for them in a wider dtype gets ``fp8 * scale_inv[block]``, for whole tensors
    and for row / column shards that start inside a scale block."""
    cfg = preset("tiny-qwen3")
    d = str(tmp_path / "fp8dense")
    tensors = export.materialize(cfg, seed=1)
    names = ["model.layers.0.self_attn.q_proj.weight", "model.layers.1.mlp.down_proj.weight"]
    expect = export.quantize_dense_to_fp8(tensors, names)
    export.write_checkpoint(tensors, cfg, d, shards=2)
    src = SafetensorsSource(d, prefetch=False)
    for n in names:
        assert torch.equal(src.get(n, "cpu", torch.float32), expect[n])
        rows, cols = expect[n].shape
        r = (rows // 4, rows // 4 + rows // 2)
        c = (cols // 8, cols // 8 + cols // 2)
        assert torch.equal(src.get(n, "cpu", torch.float32, rows=r), expect[n][r[0] : r[1]])
        assert torch.equal(src.get(n, "cpu", torch.float32, cols=c), expect[n][:, c[0] : c[1]])
        assert src.get(n, "cpu", torch.float8_e4m3fn).dtype == torch.float8_e4m3fn  # kept as stored when asked for FP8
    # the widened tensors make a working model whose logits match the dequantised weights in memory
    plain = dict(tensors)
    for n in names:
        plain[n] = expect[n].to(torch.bfloat16)
        plain.pop(n + "_scale_inv")
    a = registry.build(cfg, source=src, device="cpu", dtype=torch.bfloat16)
    b = registry.build(cfg, source=DictSource(plain), device="cpu", dtype=torch.bfloat16)
    _same_model(a, b)


def test_missing_tensor_and_wrong_kind_are_errors(tmp_path):
    cfg = preset("tiny-qwen3")
    d = str(tmp_path / "m")
    export.export_checkpoint(cfg, d, shards=1)
    assert os.path.exists(os.path.join(d, "model.safetensors"))
    src = SafetensorsSource(d, prefetch=False)
    with pytest.raises(WeightError):
        src.get("model.layers.0.nope.weight", "cpu")
    with pytest.raises(WeightError):
        src.get("model.norm.weight", "cpu", torch.int32)  # a float tensor cannot load as integers
    with pytest.raises(WeightError):
        SafetensorsSource(str(tmp_path / "empty_dir_that_does_not_exist"))
