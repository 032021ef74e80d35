"""CLI flag ownership, model detection and small utilities (CPU only)."""
import json

import pytest

from pegainfer_b200 import serve
from pegainfer_b200.config import from_hf
from pegainfer_b200.utils.cpu_topology import parse_cpulist, plan_affinity
from pegainfer_b200.utils.stats import LatencyStats, percentile


def test_flag_a_line_does_not_read_is_rejected():
    ecfg, mcfg, line, _ = serve.resolve(["--preset", "tiny-qwen3", "--enable-lora", "--max-loras", "2"])
    assert line.name == "qwen3" and ecfg.enable_lora and ecfg.max_loras == 2
    with pytest.raises(SystemExit, match="not read by the qwen35 model line"):
        serve.resolve(["--preset", "tiny-qwen35", "--enable-lora"])
    with pytest.raises(SystemExit, match="not read by the qwen3 model line"):
        serve.resolve(["--preset", "tiny-qwen3", "--ep-backend", "nccl"])
    ecfg, _, line, _ = serve.resolve(["--preset", "tiny-kimi", "--spec-method", "mtp", "--ep-backend", "nccl"])
    assert line.name == "kimi-k2" and ecfg.spec_method == "mtp" and ecfg.comm == "nccl"
    with pytest.raises(SystemExit):
        serve.resolve([])
    with pytest.raises(ValueError):
        serve.resolve(["--preset", "tiny-qwen3", "--kv-page-size", "7"])


def test_model_detection_from_config_json(tmp_path):
    cfg = {"model_type": "qwen3", "architectures": ["Qwen3ForCausalLM"], "vocab_size": 1000, "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "rope_theta": 1e6, "eos_token_id": [1, 2, 1]}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 7}))
    ecfg, mcfg, line, _ = serve.resolve(["--model-path", str(tmp_path)])
    assert line.name == "qwen3" and mcfg.head_dim == 16 and mcfg.eos_token_ids == (7,)
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "llama", "architectures": ["LlamaForCausalLM"]}))
    with pytest.raises(SystemExit, match="supported model lines"):
        serve.resolve(["--model-path", str(tmp_path)])
    ds = from_hf({"model_type": "deepseek_v2", "vocab_size": 10, "hidden_size": 8, "num_hidden_layers": 2, "num_attention_heads": 2, "intermediate_size": 16, "kv_lora_rank": 4, "qk_nope_head_dim": 4, "qk_rope_head_dim": 2, "v_head_dim": 4, "n_routed_experts": 4, "num_experts_per_tok": 2, "moe_intermediate_size": 8, "first_k_dense_replace": 1})
    assert ds.family == "deepseek_v2" and ds.is_mla and ds.layer_is_moe(1) and not ds.layer_is_moe(0)


def test_percentiles_and_affinity_plan():
    v = [1, 2, 3, 4]
    assert percentile(v, 50) == 2.5 and percentile(v, 0) == 1 and percentile(v, 100) == 4
    st = LatencyStats.of([3, 1, 2])
    assert st.min == 1 and st.max == 3 and st.p50 == 2 and st.samples == 3
    assert parse_cpulist("0-3,8,10-11") == [0, 1, 2, 3, 8, 10, 11]
    assert plan_affinity(list(range(16)), 1, 4) == [4, 5, 6, 7]
    assert plan_affinity([], 0, 1) == []


def test_every_registered_family_has_exactly_one_model_line():
    from pegainfer_b200.models.registry import BUILDERS
    from pegainfer_b200.serve import detect_line

    for family in BUILDERS:
        assert detect_line(family).name
