"""Assemble a serving engine: model -> KV buffer -> block pool -> executor ->
scheduler -> driver thread.

KV sizing on a GPU follows the reference's memory-profile pass: run one dummy
worst-case step, read the peak, and give the KV pool
``total * gpu_memory_utilization - non_kv_peak - margin``.

Reference parity: pegainfer-qwen3/src/lib.rs:257-346 (launch),
src/frontend_adapter.rs:84-211 (start_qwen3), src/weights.rs:662-790
(profiled KV budget), pegainfer-server/src/main.rs:122-258.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config import EngineConfig, ModelConfig, load_model_config, preset
from ..kv.block_pool import BlockPool
from ..kv.buffer import KvBuffer, KvLayout
from ..parallel.tp import SINGLE, TPContext
from ..sched.executor import TorchExecutor
from ..sched.scheduler import ContinuousScheduler, SchedulerConfig
from .contract import EngineInfo, KvCapacity
from .driver import Engine


def resolve_model_config(ecfg: EngineConfig) -> ModelConfig:
    if ecfg.model_path:
        return load_model_config(ecfg.model_path)
    if ecfg.preset:
        return preset(ecfg.preset)
    raise ValueError("either --model-path or --preset is required")


def build_model(mcfg: ModelConfig, ecfg: EngineConfig, device, dtype, tp: TPContext = SINGLE, ep=None):
    from ..models import registry

    source = None
    if ecfg.model_path:
        from ..loader.sources import SafetensorsSource

        source = SafetensorsSource(ecfg.model_path)
    return registry.build(mcfg, source=source, device=device, dtype=dtype, tp=tp, ep=ep, seed=ecfg.seed)


def profile_kv_blocks(model, ecfg: EngineConfig, page_size: int) -> int:
    """Number of KV blocks that fit next to the weights and activation peak."""
    geo = model.kv_geometry()
    elem = 2
    per_block = geo["num_layers"] * 2 * page_size * geo["kv_heads"] * geo["head_dim"] * elem
    if "bytes_per_block" in geo:
        per_block = geo["bytes_per_block"](page_size)
    draft = getattr(model, "draft_model", None)
    if draft is not None:  # the draft model's KV buffer shares the block ids
        dg = draft.kv_geometry()
        per_block += dg["bytes_per_block"](page_size) if "bytes_per_block" in dg else dg["num_layers"] * 2 * page_size * dg["kv_heads"] * dg["head_dim"] * elem
    if model.device.type != "cuda":
        return ecfg.num_kv_blocks or 512
    free, total = torch.cuda.mem_get_info(model.device)
    torch.cuda.reset_peak_memory_stats(model.device)
    base = torch.cuda.memory_allocated(model.device)
    # activation peak estimate: one worst-case unified step
    rows = ecfg.max_prefill_tokens + ecfg.max_decode_batch
    act = rows * (model.cfg.hidden_size * 8 + getattr(model.cfg, "intermediate_size", 0) * 6 // max(model.tp.world, 1)) * elem
    logits = ecfg.max_decode_batch * model.cfg.vocab_size * (2 + 4)
    budget = int(total * ecfg.gpu_memory_utilization) - base - act - logits - (ecfg.kv_cache_memory_margin_mib << 20)
    return max(0, budget // per_block)


def build_engine(ecfg: EngineConfig, mcfg: Optional[ModelConfig] = None, device=None, dtype=None, tp: TPContext = SINGLE, ep=None, model=None, start: bool = True):
    ecfg.validate()
    mcfg = mcfg or resolve_model_config(ecfg)
    if device is None:
        device = f"cuda:{ecfg.device_ordinal}" if torch.cuda.is_available() else "cpu"
    device = torch.device(device)
    if dtype is None:
        dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    if ecfg.gemm == "cublas" and device.type == "cuda":
        from .. import ops

        ops.set_mode("cublas")  # --gemm cublas: library GEMMs, everything else unchanged
    if ecfg.batch_invariant and device.type == "cuda":
        from ..ops import cuda as K

        K.set_batch_invariant(True)
    if model is None:
        model = build_model(mcfg, ecfg, device, dtype, tp, ep)
    if ecfg.spec_method == "draft" and getattr(model, "draft_model", None) is None:
        # built before the KV profile so that its weights and its share of every block are counted
        from ..spec.draft_model import load_draft_model

        model.draft_model = load_draft_model(ecfg, model)
    if ecfg.spec_method in ("dflash", "dspark") and getattr(model, "draft_model", None) is None:
        from ..spec.dflash import DFlashDraftModel

        model.draft_model = DFlashDraftModel.load(ecfg.draft_model_path or "random", model, seed=ecfg.seed + 1)
    if ecfg.spec_method == "eagle3" and getattr(model, "draft_model", None) is None:
        from ..spec.eagle3 import Eagle3DraftModel

        model.draft_model = Eagle3DraftModel.load(ecfg.draft_model_path or "random", model, seed=ecfg.seed + 1)
    page = ecfg.kv_page_size
    nblocks = ecfg.num_kv_blocks or profile_kv_blocks(model, ecfg, page)
    if nblocks < 2:
        raise RuntimeError("no memory left for the KV cache; lower --gpu-memory-utilization pressure or use more GPUs")
    max_len = ecfg.max_model_len or min(mcfg.max_position, (nblocks - 1) * page)
    kv = model.make_kv(nblocks, page) if hasattr(model, "make_kv") else KvBuffer(KvLayout(page_size=page, num_pages=nblocks, dtype=dtype, **model.kv_geometry()), device)
    pool = BlockPool(nblocks, page, enable_prefix_cache=not ecfg.no_prefix_cache and getattr(model, "supports_prefix_cache", True))
    max_blocks_per_seq = (max_len + page - 1) // page
    executor = (model.make_executor if hasattr(model, "make_executor") else TorchExecutor)(
        model, kv, page, cuda_graph=ecfg.cuda_graph, max_decode_batch=ecfg.max_decode_batch, max_blocks_per_seq=max_blocks_per_seq, seed=ecfg.seed
    )
    scfg = SchedulerConfig(
        max_prefill_tokens=ecfg.max_prefill_tokens,
        max_decode_batch=ecfg.max_decode_batch,
        max_model_len=max_len,
        eos_token_ids=tuple(mcfg.eos_token_ids),
        batch_invariant=ecfg.batch_invariant,
        decode_overlap=ecfg.decode_overlap and tp.world == 1,
        # ranks of a DP+EP group run different batches but must launch the same number of steps, so
        # only single-GPU and replicated (TP) schedulers may launch ahead
        run_ahead=ecfg.run_ahead and device.type == "cuda" and ep is None and not ecfg.kv_offload,
        vocab_size=mcfg.vocab_size,
    )
    host_tier = None
    if ecfg.kv_offload:
        if not getattr(model, "supports_prefix_cache", True):
            raise ValueError("KV offload needs whole pages per layer slab: this model's layers have different KV row widths (or keep recurrent state)")
        from ..kv.host_tier import HostTier

        host_tier = HostTier(kv, pool, int(ecfg.kv_offload_host_gib * (1 << 30)), l1_retention_disabled=ecfg.kv_offload_l1_disabled,
                             disk_dir=ecfg.kv_offload_disk_dir, disk_bytes=int(ecfg.kv_offload_disk_gib * (1 << 30)))
    spec = None
    if ecfg.spec_method:
        from ..spec.speculative import build_spec

        spec = build_spec(ecfg, model, executor)
        if hasattr(executor, "enable_verify_graph"):
            executor.enable_verify_graph(1 + int(getattr(spec, "draft_len", 1)))
    if ecfg.decode_overlap and getattr(ecfg, "decode_sm_split", False) and device.type == "cuda" and hasattr(executor, "enable_sm_split"):
        executor.enable_sm_split(ecfg.decode_sm_pct)
    if ecfg.precapture_graphs and getattr(executor, "_graphs", None) is not None:
        executor._graphs.precapture(True, ecfg.max_decode_batch)
    sched = ContinuousScheduler(executor, pool, scfg, spec=spec, host_tier=host_tier)
    info = EngineInfo(
        model_name=ecfg.served_model_name or ecfg.preset or (ecfg.model_path or "model"),
        max_model_len=max_len,
        kv_capacity=KvCapacity(nblocks - 1, page),
        dtype=str(dtype).replace("torch.", ""),
        vocab_size=mcfg.vocab_size,
        eos_token_ids=tuple(mcfg.eos_token_ids),
    )
    if ecfg.tune_gc and device.type == "cuda":
        from ..utils.runtime import tune_gc

        tune_gc()
    eng = Engine([sched], info, start=start)
    eng.model, eng.executor, eng.scheduler, eng.pool, eng.kv, eng.host_tier = model, executor, sched, pool, kv, host_tier
    return eng
