"""Golden gate against the Hugging Face implementation of a model family.

``compare(dir, tokens)`` loads one checkpoint directory twice: through this package's loader
and engine (paged KV, chunked executor path) and through ``transformers``'
``AutoModelForCausalLM``, feeds both the same prompt and compares the logits of every
position.  It is the accuracy gate for a model line: same checkpoint, two independent
implementations, one tolerance.  The CLI writes a random-weight checkpoint of a preset shape
first when no directory is given, so the gate also runs without network access.

Reference parity: pegainfer-qwen3/tests/hf_golden_gate.rs (logits of the engine against a
stored Hugging Face run), tools/accuracy (per-position comparison with max and mean error).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from typing import Optional, Sequence

import torch


@dataclass
class ParityReport:
    positions: int
    max_abs_err: float
    mean_abs_err: float
    ref_abs_mean: float
    argmax_agreement: float
    worst_position: int

    def ok(self, atol: float, agree: float = 1.0) -> bool:
        return self.max_abs_err <= atol and self.argmax_agreement >= agree


def engine_prompt_logits(eng, tokens: Sequence[int], chunk: int = 0) -> torch.Tensor:
    """Logits of every prompt position through the engine's executor path (paged KV cache,
    optionally in chunks of ``chunk`` tokens).  The engine must be idle."""
    from ..kv.request_kv import KvView
    from ..sched.executor import SeqStep, build_meta

    ex, page = eng.executor, eng.executor.page_size
    n = len(tokens)
    pages = list(range(1, 2 + (n - 1) // page))
    if pages[-1] >= eng.pool.num_blocks:
        raise ValueError("prompt longer than the engine's KV pool")
    rid, out, start = -7, [], 0
    step = chunk or n
    try:
        while start < n:
            part = list(tokens[start : start + step])
            s = SeqStep(rid=rid, input_tokens=part, start_pos=start, view=KvView(pages, start + len(part), page), all_rows=True, fresh_state=(start == 0))
            tok, meta = build_meta([s], page, ex.device)
            ex.prepare_meta([s], meta)
            hidden = ex.model.forward_hidden(tok, meta, ex.kv)
            logits = ex.model.logits(hidden, torch.arange(len(part), dtype=torch.int32, device=ex.device))
            if hasattr(ex.model, "full_logits"):
                logits = ex.model.full_logits(logits)
            out.append(logits.float().cpu())
            start += len(part)
    finally:
        ex.release_request(rid)
    return torch.cat(out)


def _yarn_mscale_sq(rs: dict) -> float:
    from ..config import yarn_get_mscale

    if not rs or rs.get("type", rs.get("rope_type")) != "yarn" or not rs.get("mscale_all_dim"):
        return 1.0
    m = yarn_get_mscale(rs.get("factor", 1.0), rs["mscale_all_dim"])
    return m * m


def _as_deepseek_v3_dir(model_dir: str, cfg: dict, out_dir: str) -> str:
    """A Kimi-K2 checkpoint is the DeepSeek-V3 architecture with compressed-tensors INT4 experts and
    a model type ``transformers`` does not know: rewrite it as a plain ``deepseek_v3`` directory with
    the experts widened by the same dequantisation formula the loader uses."""
    import os

    from safetensors.torch import save_file

    from ..loader.sources import SafetensorsSource
    from ..ops.reference import dequant_int4_g32

    src = SafetensorsSource(model_dir)
    group = 32
    for g in (cfg.get("quantization_config", {}).get("config_groups", {}) or {}).values():
        group = g.get("weights", {}).get("group_size", group)
    tensors = {}
    mtp_prefix = f"model.layers.{cfg['num_hidden_layers']}."
    for name in src.names():
        plain = name[len("language_model.") :] if name.startswith("language_model.") else name  # multimodal wrapper prefix
        if name.endswith(".weight_scale") or name.endswith(".weight_shape") or plain.startswith(mtp_prefix):
            continue
        if name.endswith(".weight_packed"):
            base = name[: -len("_packed")]
            tensors[plain[: -len("_packed")]] = dequant_int4_g32(src.get(name, "cpu", torch.int32), src.get(base + "_scale", "cpu", torch.float32), group).float().contiguous()
        else:
            tensors[plain] = src.get(name, "cpu", torch.float32).contiguous()
    cfg = dict(cfg, model_type="deepseek_v3", architectures=["DeepseekV3ForCausalLM"])
    cfg.pop("quantization_config", None)
    os.makedirs(out_dir, exist_ok=True)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    return out_dir


def _qwen35_text_model(model_dir: str, cfg: dict, dtype):
    """The language model of a Qwen3.5 checkpoint (a multimodal wrapper whose text weights are named
    ``model.language_model.*``) as ``transformers``' text-only causal LM."""
    import transformers.models.qwen3_5.modeling_qwen3_5 as hf

    from ..loader.sources import SafetensorsSource

    text = dict(cfg.get("text_config", cfg))
    for k in ("model_type", "architectures", "torch_dtype"):
        text.pop(k, None)
    m = hf.Qwen3_5ForCausalLM(hf.Qwen3_5TextConfig(**text)).to(dtype)
    src = SafetensorsSource(model_dir)
    sd = {n.replace("model.language_model.", "model."): src.get(n, "cpu", dtype) for n in src.names() if not n.startswith("mtp.")}
    missing, unexpected = m.load_state_dict(sd, strict=False)
    if missing:
        raise RuntimeError(f"checkpoint lacks {missing[:4]} ...")
    return m


def hf_prompt_logits(model_dir: str, tokens: Sequence[int], dtype=torch.float32) -> torch.Tensor:
    import tempfile

    from transformers import AutoModelForCausalLM

    with open(f"{model_dir}/config.json") as f:
        cfg = json.load(f)
    with tempfile.TemporaryDirectory() as tmp:
        if cfg.get("model_type") == "qwen3_5":
            m = _qwen35_text_model(model_dir, cfg, dtype)
        else:
            path = _as_deepseek_v3_dir(model_dir, cfg, tmp) if cfg.get("model_type") == "kimi_k2" else model_dir
            m = AutoModelForCausalLM.from_pretrained(path, dtype=dtype, attn_implementation="eager")  # an explicit causal mask in every family
    m.eval()
    if cfg.get("model_type") == "deepseek_v2":
        # transformers' own DeepSeek-V2 leaves the YaRN mscale^2 off the softmax scale; DeepSeek's
        # modeling code (and its V3 port in transformers) applies it, and so does this package
        k = _yarn_mscale_sq(cfg.get("rope_scaling") or {})
        for layer in m.model.layers:
            layer.self_attn.scaling *= k
    with torch.no_grad():
        out = m(torch.tensor([list(tokens)], dtype=torch.long), use_cache=False)
    return out.logits[0].float()


def report(ours: torch.Tensor, ref: torch.Tensor) -> ParityReport:
    err = (ours - ref).abs()
    per_pos = err.amax(dim=-1)
    return ParityReport(
        positions=ours.shape[0],
        max_abs_err=float(err.max()),
        mean_abs_err=float(err.mean()),
        ref_abs_mean=float(ref.abs().mean()),
        argmax_agreement=float((ours.argmax(-1) == ref.argmax(-1)).float().mean()),
        worst_position=int(per_pos.argmax()),
    )


def compare(model_dir: str, tokens: Sequence[int], device: str = "cpu", dtype=torch.float32, chunk: int = 0, page_size: int = 16) -> ParityReport:
    from ..config import EngineConfig
    from ..engine.build import build_engine

    blocks = 4 + (len(tokens) + page_size - 1) // page_size
    ecfg = EngineConfig(model_path=model_dir, kv_page_size=page_size, num_kv_blocks=blocks, cuda_graph=False)
    eng = build_engine(ecfg, device=device, dtype=dtype, start=False)
    try:
        with torch.no_grad():
            ours = engine_prompt_logits(eng, tokens, chunk)
    finally:
        eng.shutdown()
    return report(ours, hf_prompt_logits(model_dir, tokens))


def main(argv: Optional[list] = None) -> int:
    import argparse
    import tempfile

    ap = argparse.ArgumentParser(description="compare prompt logits with the Hugging Face implementation")
    ap.add_argument("--model-path", help="checkpoint directory; default: a random-weight export of --preset")
    ap.add_argument("--preset", default="tiny-qwen3")
    ap.add_argument("--tokens", type=int, default=48)
    ap.add_argument("--chunk", type=int, default=0)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--atol", type=float, default=2e-3)
    a = ap.parse_args(argv)
    with tempfile.TemporaryDirectory() as tmp:
        path = a.model_path
        if not path:
            from ..config import preset
            from ..loader.export import export_checkpoint

            export_checkpoint(preset(a.preset), tmp, dtype=torch.float32)
            path = tmp
        with open(f"{path}/config.json") as f:
            cj = json.load(f)
        vocab = cj.get("text_config", cj)["vocab_size"]
        g = torch.Generator().manual_seed(1)
        toks = torch.randint(0, vocab, (a.tokens,), generator=g).tolist()
        dtype = torch.float32 if a.device == "cpu" else torch.bfloat16
        rep = compare(path, toks, a.device, dtype, a.chunk)
    print(json.dumps(asdict(rep)))
    return 0 if rep.ok(a.atol if a.device == "cpu" else 0.25, 1.0 if a.device == "cpu" else 0.9) else 1


if __name__ == "__main__":
    raise SystemExit(main())
