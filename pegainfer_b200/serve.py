"""``python -m pegainfer_b200.serve``: detect the model line, validate flags, launch the
engine, then serve the OpenAI API.

Flags are owned: shared flags are read by every model line, line-specific flags only by
the lines that declare them, and a flag the detected line does not consume is an error
rather than silently ignored.  The HTTP port opens only after the engine is ready.
Under ``torchrun`` every rank builds its shard of the model; rank 0 also hosts the
scheduler and HTTP server and replicates each step's events to the other ranks.

Reference parity: pegainfer-server/src/main.rs:24-258 (dispatch, feature hints, serve
paths), pegainfer-frontend/src/model_line.rs:93-206 (SharedArgs), :292-338 (ModelLine),
:453-616 (registry, consume-or-reject validation).
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import sys
from dataclasses import dataclass, field
from typing import Optional

from .config import PRESETS, EngineConfig, detect_family, load_model_config, preset
from .utils import logging as plog

log = logging.getLogger("pegainfer_b200.serve")

SHARED_FLAGS = {
    "model_path", "preset", "served_model_name", "port", "host", "cuda_graph", "precapture_graphs", "dump_graph_dot", "device_ordinal", "tp_size", "dp_size", "ep_size",
    "kv_offload", "kv_offload_host_gib", "kv_offload_disk_dir", "kv_offload_disk_gib", "no_prefix_cache", "max_prefill_tokens", "max_model_len", "num_kv_blocks", "gpu_memory_utilization",
    "kv_cache_memory_margin_mib", "kv_page_size", "max_decode_batch", "seed", "comm", "gemm", "tokenizer", "pd_prefill_device", "pd_store", "engine_process",
}


@dataclass
class ModelLine:
    """What one architecture family contributes to the CLI."""

    name: str
    families: tuple
    exclusive_flags: frozenset = frozenset()

    def validate(self, ns: argparse.Namespace, provided: set) -> None:
        pass


def _qwen3_validate(ns, provided):
    if ns.enable_lora and ns.cuda_graph:
        log.info("greedy decode steps with adapters replay adapter-aware CUDA graphs (the adapter slot of every row is a graph input); sampled or logprob steps with adapters run kernel by kernel")
    if ns.decode_overlap and ns.tp_size > 1:
        raise SystemExit("--decode-overlap is not available together with tensor parallelism")
    if "decode_sm_pct" in provided and not ns.decode_overlap:
        raise SystemExit("--decode-sm-pct splits the SMs between the decode stream and the prefill lane: it needs --decode-overlap")


LINES = [
    ModelLine("qwen3", ("qwen3",), frozenset({"enable_lora", "lora_modules", "max_loras", "max_lora_rank", "batch_invariant", "spec_method", "draft_model_path", "spec_draft_len", "decode_overlap", "decode_sm_pct"})),
    ModelLine("qwen35", ("qwen35",), frozenset({"max_batch"})),
    ModelLine("deepseek-v2-lite", ("deepseek_v2",), frozenset({"ep_backend"})),
    ModelLine("kimi-k2", ("kimi_k2",), frozenset({"ep_backend", "spec_method"})),
    ModelLine("glm-5", ("glm_dsa",), frozenset({"ep_backend", "spec_method"})),
    ModelLine("gemma4", ("gemma4",), frozenset()),
    ModelLine("kimi-k3", ("kimi_k3",), frozenset({"ep_backend"})),
]
LINES[0].validate = _qwen3_validate  # type: ignore[method-assign]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="pegainfer_b200.serve", description="B200-native OpenAI-compatible LLM server")
    g = ap.add_argument_group("model")
    g.add_argument("--model-path", help="Hugging Face checkpoint directory (config.json + safetensors)")
    g.add_argument("--preset", choices=sorted(PRESETS), help="random-init model of a named shape (benchmarks, tests)")
    g.add_argument("--served-model-name")
    g.add_argument("--tokenizer", default=None, help="'none' serves token-id prompts only")
    s = ap.add_argument_group("serving")
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--no-cuda-graph", dest="cuda_graph", action="store_false")
    s.add_argument("--precapture-graphs", action="store_true", help="capture every decode batch bucket at start-up")
    s.add_argument("--dump-graph-dot", help="write the captured decode graph as Graphviz DOT to this path")
    s.add_argument("--device-ordinal", type=int, default=0)
    s.add_argument("--tp-size", type=int, default=1)
    s.add_argument("--dp-size", type=int, default=1)
    s.add_argument("--ep-size", type=int, default=1)
    s.add_argument("--comm", choices=["fused", "nccl"], default="fused", help="fused = in-kernel collectives over peer memory; nccl = library baseline")
    s.add_argument("--gemm", choices=["sm100", "cublas"], default="sm100")
    s.add_argument("--seed", type=int, default=0)
    k = ap.add_argument_group("kv cache")
    k.add_argument("--kv-page-size", type=int, default=16)
    k.add_argument("--num-kv-blocks", type=int)
    k.add_argument("--gpu-memory-utilization", type=float, default=0.90)
    k.add_argument("--kv-cache-memory-margin-mib", type=int, default=150)
    k.add_argument("--no-prefix-cache", action="store_true")
    k.add_argument("--kv-offload", action="store_true", help="spill sealed KV blocks to a pinned host tier and restore them by content hash")
    k.add_argument("--kv-offload-host-gib", type=float, default=4.0)
    k.add_argument("--kv-offload-disk-dir", default=None, help="third KV tier: blocks evicted from host memory are kept as files in this directory")
    k.add_argument("--kv-offload-disk-gib", type=float, default=0.0)
    k.add_argument("--engine-process", action="store_true", help="run the engine in a process of its own, so that the HTTP frontend and the scheduler do not share one interpreter lock")
    k.add_argument("--pd-prefill-device", type=int, help="prefill / decode disaggregation: run prompts on this GPU and decode on --device-ordinal; KV blocks move by content hash")
    k.add_argument("--pd-store", choices=["peer", "host"], default="peer", help="where the handoff store lives: the decode GPU (one NVLink hop) or pinned host memory")
    k.add_argument("--max-prefill-tokens", type=int, default=1024)
    k.add_argument("--max-decode-batch", type=int, default=256)
    k.add_argument("--max-model-len", type=int)
    x = ap.add_argument_group("model-line specific")
    x.add_argument("--enable-lora", action="store_true")
    x.add_argument("--lora-modules", nargs="*", default=[], help="name=path pairs loaded at startup")
    x.add_argument("--max-loras", type=int, default=4)
    x.add_argument("--max-lora-rank", type=int, default=64)
    x.add_argument("--batch-invariant", action="store_true")
    x.add_argument("--spec-method", choices=["mtp", "draft", "dflash", "dspark", "eagle3"])
    x.add_argument("--draft-model-path")
    x.add_argument("--spec-draft-len", type=int, default=1)
    x.add_argument("--decode-overlap", action="store_true")
    x.add_argument("--no-run-ahead", action="store_true", help="read every decode step's tokens before launching the next step")
    x.add_argument("--no-gc-tuning", action="store_true", help="leave the interpreter's garbage collector at its defaults")
    x.add_argument("--decode-sm-pct", type=int, default=50)
    x.add_argument("--max-batch", type=int, default=64)
    x.add_argument("--ep-backend", choices=["fused", "nccl"], default=None)
    return ap


def provided_flags(argv: list, parser: argparse.ArgumentParser) -> set:
    out = set()
    for a in parser._actions:
        for opt in a.option_strings:
            if any(x == opt or x.startswith(opt + "=") for x in argv):
                out.add(a.dest)
    return out


def detect_line(model_cfg_family: str) -> ModelLine:
    hits = [l for l in LINES if model_cfg_family in l.families]
    if len(hits) != 1:
        raise SystemExit(f"expected exactly one model line for family {model_cfg_family!r}, found {[l.name for l in hits]}")
    return hits[0]


def validate_flags(line: ModelLine, provided: set) -> None:
    all_exclusive = set().union(*[l.exclusive_flags for l in LINES])
    for f in sorted(provided):
        if f in SHARED_FLAGS:
            continue
        if f in all_exclusive and f not in line.exclusive_flags:
            owners = [l.name for l in LINES if f in l.exclusive_flags]
            raise SystemExit(f"--{f.replace('_', '-')} is not read by the {line.name} model line (it belongs to: {', '.join(owners)})")


def engine_config_from(ns: argparse.Namespace) -> EngineConfig:
    return EngineConfig(
        model_path=ns.model_path, preset=ns.preset, served_model_name=ns.served_model_name, port=ns.port, host=ns.host, cuda_graph=ns.cuda_graph, precapture_graphs=ns.precapture_graphs,
        dump_graph_dot=ns.dump_graph_dot, device_ordinal=ns.device_ordinal, tp_size=ns.tp_size, dp_size=ns.dp_size, ep_size=ns.ep_size,
        kv_page_size=ns.kv_page_size, num_kv_blocks=ns.num_kv_blocks, gpu_memory_utilization=ns.gpu_memory_utilization,
        kv_cache_memory_margin_mib=ns.kv_cache_memory_margin_mib, no_prefix_cache=ns.no_prefix_cache, kv_offload=ns.kv_offload,
        kv_offload_host_gib=ns.kv_offload_host_gib, kv_offload_disk_dir=ns.kv_offload_disk_dir, kv_offload_disk_gib=ns.kv_offload_disk_gib, max_prefill_tokens=ns.max_prefill_tokens, max_decode_batch=ns.max_decode_batch,
        max_model_len=ns.max_model_len, batch_invariant=ns.batch_invariant, decode_overlap=ns.decode_overlap, run_ahead=not ns.no_run_ahead, tune_gc=not ns.no_gc_tuning, decode_sm_pct=ns.decode_sm_pct,
        enable_lora=ns.enable_lora, max_loras=ns.max_loras, max_lora_rank=ns.max_lora_rank, lora_modules=tuple(ns.lora_modules), spec_method=ns.spec_method,
        spec_draft_len=ns.spec_draft_len, draft_model_path=ns.draft_model_path, comm=ns.ep_backend or ns.comm, gemm=ns.gemm, seed=ns.seed,
    )


def resolve(argv: Optional[list] = None):
    """Parse + detect + validate; returns (EngineConfig, ModelConfig, ModelLine)."""
    argv = list(sys.argv[1:] if argv is None else argv)
    parser = build_parser()
    ns = parser.parse_args(argv)
    if not ns.model_path and not ns.preset:
        raise SystemExit("one of --model-path or --preset is required")
    if ns.model_path:
        cfg_path = os.path.join(ns.model_path, "config.json")
        if not os.path.exists(cfg_path):
            raise SystemExit(f"{ns.model_path}: config.json not found")
        with open(cfg_path) as f:
            raw = json.load(f)
        try:
            detect_family(raw)
        except ValueError as e:
            raise SystemExit(f"{e}; supported model lines: {', '.join(l.name for l in LINES)}")
        mcfg = load_model_config(ns.model_path)
    else:
        mcfg = preset(ns.preset)
    line = detect_line(mcfg.family)
    provided = provided_flags(argv, parser)
    validate_flags(line, provided)
    ecfg = engine_config_from(ns)
    ecfg.decode_sm_split = "decode_sm_pct" in provided
    ecfg.validate()
    line.validate(ns, provided)
    if mcfg.family == "qwen35":
        ecfg.max_decode_batch = min(ecfg.max_decode_batch, ns.max_batch)
    return ecfg, mcfg, line, ns


def main(argv: Optional[list] = None) -> int:
    plog.init_default()
    ecfg, mcfg, line, ns = resolve(argv)
    import torch

    from .engine.build import build_engine
    from .server.openai import serve
    from .server.tokenizer import load_tokenizer
    from .utils.tracing import tracer_from_env

    log.info("model line %s, family %s, %d layers, hidden %d", line.name, mcfg.family, mcfg.num_layers, mcfg.hidden_size)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        from .parallel.launch import launch_distributed

        return launch_distributed(ecfg, mcfg, ns)
    tok_dir = None if (ns.tokenizer == "none" or not ecfg.model_path) else ecfg.model_path
    tokenizer = load_tokenizer(tok_dir, mcfg.vocab_size)  # fails early when tokenizer.json is missing
    if ns.pd_prefill_device is not None:
        from .engine.pd import build_pd_engine

        if ecfg.enable_lora or ecfg.spec_method:
            raise SystemExit("--pd-prefill-device does not combine with LoRA or speculative decoding")
        dec = f"cuda:{ecfg.device_ordinal}" if torch.cuda.is_available() else "cpu"
        pre = f"cuda:{ns.pd_prefill_device}" if torch.cuda.is_available() else "cpu"
        eng = build_pd_engine(ecfg, mcfg, prefill_device=pre, decode_device=dec, store_device="cpu" if ns.pd_store == "host" else None)
        log.info("prefill on %s, decode on %s, %d store slots on %s", pre, dec, eng.store.num_slots, eng.store.slab.device)
        name = ecfg.served_model_name or ecfg.preset or os.path.basename(os.path.normpath(ecfg.model_path))
        try:
            serve(eng, tokenizer, name, ecfg.host, ecfg.port)
        finally:
            eng.shutdown()
        return 0
    if ns.engine_process:
        from .engine.remote import RemoteEngine

        if ecfg.enable_lora or ecfg.dump_graph_dot:
            raise SystemExit("--engine-process does not combine with LoRA routes or --dump-graph-dot")
        eng = RemoteEngine(ecfg, mcfg)
        name = ecfg.served_model_name or ecfg.preset or os.path.basename(os.path.normpath(ecfg.model_path))
        log.info("engine process up: %d KV blocks of %d tokens, max_model_len %d", eng.info.kv_capacity.num_blocks, eng.info.kv_capacity.block_size, eng.info.max_model_len)
        try:
            serve(eng, tokenizer, name, ecfg.host, ecfg.port)
        finally:
            eng.shutdown()
        return 0
    eng = build_engine(ecfg, mcfg)
    eng.scheduler.tracer = tracer_from_env()
    if ecfg.dump_graph_dot and getattr(eng.executor, "_graphs", None) is not None:
        eng.executor._graphs.dump_dot(ecfg.dump_graph_dot)
    name = ecfg.served_model_name or ecfg.preset or os.path.basename(os.path.normpath(ecfg.model_path))
    lora_mgr = None
    if ecfg.enable_lora:
        from .lora.manager import LoraManager

        lora_mgr = LoraManager(eng, ecfg.max_loras, ecfg.max_lora_rank)
        for spec in ecfg.lora_modules:
            n, p = spec.split("=", 1)
            lora_mgr.load(n, p)
    log.info("engine ready: %d KV blocks of %d tokens, max_model_len %d", eng.info.kv_capacity.num_blocks, eng.info.kv_capacity.block_size, eng.info.max_model_len)
    try:
        serve(eng, tokenizer, name, ecfg.host, ecfg.port, lora_manager=lora_mgr)
    finally:
        eng.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
