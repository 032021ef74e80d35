"""LoRA adapters: PEFT loading, tensor-parallel sharding, packed slots, hot load/unload.

Adapters are PEFT directories (``adapter_config.json`` + ``adapter_model.safetensors``)
targeting any of q/k/v/o/gate/up/down projections.  Every loaded adapter occupies a
*slot*; per layer and projection the A ([r, in]) and B ([out, r]) matrices of all slots
live in two packed tensors ``[slots, r_max, in]`` / ``[slots, out, r_max]`` (zero padded
to ``max_lora_rank``), so a mixed batch is one kernel launch per projection with a
per-token slot id.  Column-parallel projections shard B by output rows, row-parallel
ones shard A by input columns (their delta is added before the all-reduce).
Requests name an adapter; the prefix-cache hash is salted with it.

Reference parity: pegainfer-qwen3/src/lora.rs (PEFT manifest / loading),
src/weights.rs:130-330,418-560 (packed slots, TP sharding, decode delta),
pegainfer-frontend/src/vllm/lora.rs:72-200 (load / unload routes).
"""
from __future__ import annotations

import json
import os
import threading
from typing import Optional

import torch

from .. import ops
from ..loader.sources import shard_range

TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
COLUMN_PARALLEL = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")


class LoraError(RuntimeError):
    pass


def read_adapter(path: str):
    """Returns (rank, alpha, {(layer, proj): (A [r, in], B [out, r])})."""
    from safetensors import safe_open

    cfg_p = os.path.join(path, "adapter_config.json")
    w_p = os.path.join(path, "adapter_model.safetensors")
    if not os.path.exists(cfg_p) or not os.path.exists(w_p):
        raise LoraError(f"{path}: expected adapter_config.json and adapter_model.safetensors")
    with open(cfg_p) as f:
        cfg = json.load(f)
    rank, alpha = int(cfg["r"]), float(cfg.get("lora_alpha", cfg["r"]))
    for t in cfg.get("target_modules", []):
        if t not in TARGETS:
            raise LoraError(f"unsupported LoRA target module {t!r}")
    mats: dict = {}
    with safe_open(w_p, framework="pt") as f:
        for key in f.keys():
            parts = key.split(".")
            if "layers" not in parts:
                continue
            li = int(parts[parts.index("layers") + 1])
            proj = next((p for p in parts if p in TARGETS), None)
            if proj is None:
                raise LoraError(f"tensor {key} targets an unsupported module")
            which = "A" if "lora_A" in key else "B" if "lora_B" in key else None
            if which is None:
                continue
            mats.setdefault((li, proj), {})[which] = f.get_tensor(key)
    out = {}
    for k, v in mats.items():
        if "A" not in v or "B" not in v:
            raise LoraError(f"adapter is missing lora_A or lora_B for layer {k[0]} {k[1]}")
        if v["A"].shape[0] != rank or v["B"].shape[1] != rank:
            raise LoraError(f"layer {k[0]} {k[1]}: rank mismatch with adapter_config r={rank}")
        out[k] = (v["A"], v["B"])
    return rank, alpha, out


class LoraManager:
    def __init__(self, engine_or_model, max_loras: int = 4, max_rank: int = 64):
        model = getattr(engine_or_model, "model", engine_or_model)
        self.engine = engine_or_model if hasattr(engine_or_model, "scheduler") else None
        self.model = model
        self.max_loras = max_loras
        self.r_max = (max_rank + 7) // 8 * 8
        self._names: dict = {}  # name -> slot
        self._free = list(range(max_loras - 1, -1, -1))
        self._lock = threading.Lock()
        cfg, tp, dev, dt = model.cfg, model.tp, model.device, model.dtype
        d = cfg.head_dim
        self.scale = torch.zeros(max_loras, dtype=torch.float32, device=dev)
        q, kv, ff, h = cfg.num_q_heads * d // tp.world, cfg.num_kv_heads * d // tp.world, cfg.intermediate_size // tp.world, cfg.hidden_size
        self.dims = {"q_proj": (h, q), "k_proj": (h, kv), "v_proj": (h, kv), "o_proj": (q, h), "gate_proj": (h, ff), "up_proj": (h, ff), "down_proj": (ff, h)}
        self.A = {}
        self.B = {}
        for li in range(cfg.num_layers):
            for p, (k_in, m_out) in self.dims.items():
                self.A[(li, p)] = torch.zeros((max_loras, self.r_max, k_in), dtype=dt, device=dev)
                self.B[(li, p)] = torch.zeros((max_loras, m_out, self.r_max), dtype=dt, device=dev)
        model.lora = self
        if hasattr(model, "set_gate_up_layout"):
            # adapter deltas address the gate and up halves of the fused projection
            model.fused_decode = False
            model.set_gate_up_layout(False)
        if self.engine is not None:
            self.engine.scheduler.lora = self

    # -- registry ------------------------------------------------------------------------
    def has(self, name: str) -> bool:
        return name in self._names

    def names(self) -> list:
        return sorted(self._names)

    def slot_of(self, name: str) -> int:
        return self._names[name]

    def _in_use(self, name: str) -> bool:
        if self.engine is None:
            return False
        s = self.engine.scheduler
        return any(r.q.request.lora_adapter == name for r in list(s.running.values())) or any(q.request.lora_adapter == name for q in list(s.waiting))

    def load(self, name: str, path: str) -> int:
        rank, alpha, mats = read_adapter(path)
        if rank > self.r_max:
            raise LoraError(f"adapter rank {rank} exceeds --max-lora-rank {self.r_max}")
        with self._lock:
            if name in self._names:
                raise LoraError(f"adapter {name!r} is already loaded")
            if not self._free:
                raise LoraError(f"all {self.max_loras} adapter slots are in use")
            slot = self._free.pop()
            cfg, tp = self.model.cfg, self.model.tp
            d = cfg.head_dim
            ranges = {
                "q_proj": shard_range(cfg.num_q_heads, tp.rank, tp.world), "k_proj": shard_range(cfg.num_kv_heads, tp.rank, tp.world),
                "v_proj": shard_range(cfg.num_kv_heads, tp.rank, tp.world), "o_proj": shard_range(cfg.num_q_heads, tp.rank, tp.world),
            }
            ffr = shard_range(cfg.intermediate_size, tp.rank, tp.world)
            for key in self.A:
                self.A[key][slot].zero_()
                self.B[key][slot].zero_()
            for (li, p), (a, b) in mats.items():
                if li >= cfg.num_layers:
                    raise LoraError(f"adapter names layer {li}, model has {cfg.num_layers}")
                if p in ("q_proj", "k_proj", "v_proj"):
                    r0, r1 = ranges[p][0] * d, ranges[p][1] * d
                    b = b[r0:r1]
                elif p == "o_proj":
                    r0, r1 = ranges[p][0] * d, ranges[p][1] * d
                    a = a[:, r0:r1]
                elif p in ("gate_proj", "up_proj"):
                    b = b[ffr[0] : ffr[1]]
                else:
                    a = a[:, ffr[0] : ffr[1]]
                k_in, m_out = self.dims[p]
                if a.shape[1] != k_in or b.shape[0] != m_out:
                    raise LoraError(f"layer {li} {p}: adapter shapes {tuple(a.shape)} / {tuple(b.shape)} do not fit the model ({k_in} in, {m_out} out)")
                self.A[(li, p)][slot, :rank].copy_(a.to(self.A[(li, p)].dtype))
                self.B[(li, p)][slot, :, :rank].copy_(b.to(self.B[(li, p)].dtype))
            self.scale[slot] = alpha / rank
            self._names[name] = slot
            return slot

    def unload(self, name: str) -> None:
        with self._lock:
            if name not in self._names:
                raise LoraError(f"adapter {name!r} is not loaded")
            if self._in_use(name):
                raise LoraError(f"adapter {name!r} is in use by running or queued requests")
            slot = self._names.pop(name)
            self.scale[slot] = 0.0
            self._free.append(slot)

    # -- application ------------------------------------------------------------------------
    def apply_shared(self, layer: int, projs, x: torch.Tensor, ys, slots: Optional[torch.Tensor]) -> None:
        """``apply`` for projections that read the same ``x`` (q / k / v, gate / up): one pair of launches for all."""
        if slots is None:
            return
        ops.lora_delta_multi_(list(ys), x, [self.A[(layer, p)] for p in projs], [self.B[(layer, p)] for p in projs], self.scale, slots)

    def apply(self, layer: int, proj: str, x: torch.Tensor, y: torch.Tensor, slots: Optional[torch.Tensor]) -> None:
        """``y += scale * B (A x)`` for rows whose request uses an adapter; ``y`` may be a column slice."""
        if slots is None:
            return
        ops.lora_delta_(y, x, self.A[(layer, proj)], self.B[(layer, proj)], self.scale, slots)
