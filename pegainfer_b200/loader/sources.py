"""Weight sources: where named tensors come from.

``SafetensorsSource`` reads a Hugging Face checkpoint directory
(``model.safetensors`` or ``model.safetensors.index.json`` + shards), validates
dtype/shape at the load boundary and stages host->device copies through a pair of
pinned buffers so disk reads overlap PCIe transfers.  ``RandomSource`` synthesises
deterministic N(0, 0.02) matrices / unit norm vectors directly on the device, keyed
by tensor name, so every rank and every run sees the same full tensor regardless
of load order.  ``DictSource`` wraps in-memory tensors (tests).

Reference parity: pegainfer-core/src/weight_loader.rs:32-66 (shard index),
:69-180 (page-cache prefetch), :359-613 (StagedWeightLoader: record plan, then
``finish()`` uploads through pinned double buffers), weight_loader/staging.rs:19-350.
"""
from __future__ import annotations

import hashlib
import json
import os
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Callable, Optional, Sequence

import torch

PREFETCH_THREADS = 8
PREFETCH_CHUNK = 16 << 20
STAGING_BYTES = 32 << 20


class WeightError(RuntimeError):
    pass


class WeightSource:
    def has(self, name: str) -> bool:
        raise NotImplementedError

    def shape(self, name: str) -> tuple:
        raise NotImplementedError

    def get(self, name: str, device, dtype=None, rows: Optional[tuple] = None, cols: Optional[tuple] = None) -> torch.Tensor:
        """Return tensor ``name`` (optionally the ``rows``/``cols`` half-open slice of a
        2-D tensor) on ``device``."""
        raise NotImplementedError

    def names(self) -> list:
        raise NotImplementedError


def _slice(t, rows, cols):
    if rows is not None:
        t = t[rows[0] : rows[1]]
    if cols is not None:
        t = t[:, cols[0] : cols[1]]
    return t


class DictSource(WeightSource):
    def __init__(self, tensors: dict):
        self.tensors = tensors

    def has(self, name):
        return name in self.tensors

    def shape(self, name):
        return tuple(self.tensors[name].shape)

    def names(self):
        return list(self.tensors)

    def get(self, name, device, dtype=None, rows=None, cols=None):
        if name not in self.tensors:
            raise WeightError(f"missing tensor {name}")
        t = _slice(self.tensors[name], rows, cols)
        return t.to(device=device, dtype=dtype or t.dtype).contiguous()


class RandomSource(WeightSource):
    """Deterministic synthetic weights.  ``shapes`` maps tensor name -> shape; a
    callable ``kind(name)`` picks the distribution: ``"normal"`` (std 0.02),
    ``"ones"``, ``"zeros"``, ``"const:<value>"`` or ``"small"`` (N(0, 0.02) vectors, e.g. biases)."""

    def __init__(self, shapes: dict, seed: int = 0, std: float = 0.02, kind: Optional[Callable[[str], str]] = None, dtype=torch.bfloat16):
        self.shapes = shapes
        self.seed = seed
        self.std = std
        self.dtype = dtype
        self._kind = kind or self._default_kind

    @staticmethod
    def _default_kind(name: str) -> str:
        if name.endswith("norm.weight") or "layernorm" in name or name.endswith("_norm.weight") or name.endswith("layer_scalar"):
            return "ones"
        if name.endswith("A_log") or name.endswith("dt_bias") or name.endswith("e_score_correction_bias"):
            return "small"
        return "normal"

    def has(self, name):
        return name in self.shapes

    def shape(self, name):
        return tuple(self.shapes[name])

    def names(self):
        return list(self.shapes)

    def _seed_for(self, name: str) -> int:
        h = hashlib.blake2b(f"{self.seed}:{name}".encode(), digest_size=8).digest()
        return int.from_bytes(h, "little") & 0x7FFFFFFFFFFFFFFF

    def get(self, name, device, dtype=None, rows=None, cols=None):
        if name not in self.shapes:
            raise WeightError(f"missing tensor {name}")
        shape = tuple(self.shapes[name])
        dtype = dtype or self.dtype
        kind = self._kind(name)
        if kind == "ones":
            t = torch.ones(shape, dtype=dtype, device=device)
        elif kind == "zeros":
            t = torch.zeros(shape, dtype=dtype, device=device)
        elif kind.startswith("const:"):
            t = torch.full(shape, float(kind[6:]), dtype=dtype, device=device)
        else:
            dev = torch.device(device)
            g = torch.Generator(device=dev)
            g.manual_seed(self._seed_for(name))
            # 2-D tensors are generated in fixed 1024-row blocks, each with its own
            # stream, so a row slice never materialises the full matrix and equals
            # the same rows of the full tensor.
            if len(shape) == 2:
                t = self._rows_normal(shape, rows or (0, shape[0]), g, dev).to(dtype)
                return _slice(t, None, cols).contiguous()
            t = torch.empty(shape, dtype=torch.float32, device=dev).normal_(0.0, self.std, generator=g).to(dtype)
        return _slice(t, rows, cols).contiguous()

    def _rows_normal(self, shape, rows, g, dev):
        # Row r of the full tensor is a fixed function of (name, r // BLOCK): generate
        # whole 1024-row blocks with per-block offsets into the same generator stream.
        block = 1024
        r0, r1 = rows
        out = []
        b0, b1 = r0 // block, (r1 + block - 1) // block
        base = g.initial_seed()
        for b in range(b0, b1):
            gb = torch.Generator(device=dev)
            gb.manual_seed((base + 0x9E3779B97F4A7C15 * (b + 1)) & 0x7FFFFFFFFFFFFFFF)
            nrows = min(block, shape[0] - b * block)
            blk = torch.empty((nrows, shape[1]), dtype=torch.float32, device=dev).normal_(0.0, self.std, generator=gb)
            lo = max(r0 - b * block, 0)
            hi = min(r1 - b * block, nrows)
            out.append(blk[lo:hi])
        return torch.cat(out, 0)


class SafetensorsSource(WeightSource):
    def __init__(self, model_dir: str, prefetch: bool = True):
        from safetensors import safe_open

        self.model_dir = model_dir
        self._open = safe_open
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self.name_to_file: dict = {}
        if os.path.exists(index):
            with open(index) as f:
                wm = json.load(f)["weight_map"]
            for name, fn in wm.items():
                self.name_to_file[name] = os.path.join(model_dir, fn)
        elif os.path.exists(single):
            with safe_open(single, framework="pt") as f:
                for name in f.keys():
                    self.name_to_file[name] = single
        else:
            raise WeightError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")
        self._handles: dict = {}
        self._lock = threading.Lock()
        self._staging = None
        if prefetch:
            self._prefetch_thread = threading.Thread(target=self._prefetch_all, daemon=True)
            self._prefetch_thread.start()

    # page-cache warmup: sequentially read every shard in 16 MiB chunks on 8 threads
    def _prefetch_all(self):
        files = sorted(set(self.name_to_file.values()))

        def read(fn):
            try:
                with open(fn, "rb", buffering=0) as f:
                    while f.read(PREFETCH_CHUNK):
                        pass
            except OSError:
                pass

        with ThreadPoolExecutor(PREFETCH_THREADS) as ex:
            list(ex.map(read, files))

    def _handle(self, fn):
        with self._lock:
            h = self._handles.get(fn)
            if h is None:
                h = self._open(fn, framework="pt")
                self._handles[fn] = h
            return h

    def has(self, name):
        return name in self.name_to_file

    def names(self):
        return list(self.name_to_file)

    def shape(self, name):
        return tuple(self._handle(self.name_to_file[name]).get_slice(name).get_shape())

    def get(self, name, device, dtype=None, rows=None, cols=None):
        if name not in self.name_to_file:
            raise WeightError(f"missing tensor {name}")
        sl = self._handle(self.name_to_file[name]).get_slice(name)
        if rows is not None and cols is not None:
            t = sl[rows[0] : rows[1], cols[0] : cols[1]]
        elif rows is not None:
            t = sl[rows[0] : rows[1]]
        elif cols is not None:
            t = sl[:, cols[0] : cols[1]]
        else:
            t = sl[:]
        if dtype is not None and t.dtype != dtype and t.dtype.is_floating_point != dtype.is_floating_point:
            raise WeightError(f"{name}: dtype {t.dtype} cannot load as {dtype}")
        if t.dtype == torch.float8_e4m3fn and dtype not in (None, torch.float8_e4m3fn) and (name + "_scale_inv") in self.name_to_file:
            # block-scaled FP8 checkpoint, tensor wanted in a wider type: dequantise at the load boundary
            t = self._dequant_fp8(name, t, rows, cols)
        return staged_upload(t.contiguous(), device, dtype)

    def _dequant_fp8(self, name, t, rows, cols, block: int = 128):
        """``w = fp8 * scale_inv[row // block, col // block]`` for the requested slice."""
        sname = name + "_scale_inv"
        scale = self._handle(self.name_to_file[sname]).get_slice(sname)[:].float()
        full_rows, full_cols = self.shape(name)
        r0 = rows[0] if rows is not None else 0
        c0 = cols[0] if cols is not None else 0
        ridx = (torch.arange(r0, r0 + t.shape[0]) // block).clamp_(max=scale.shape[0] - 1)
        cidx = (torch.arange(c0, c0 + t.shape[1]) // block).clamp_(max=scale.shape[1] - 1)
        return t.float() * scale[ridx][:, cidx]


_STAGING = {}


def staged_upload(t: torch.Tensor, device, dtype=None) -> torch.Tensor:
    """Host->device copy through two pinned staging buffers (double buffered)."""
    dev = torch.device(device)
    if dev.type != "cuda":
        return t.to(dtype=dtype or t.dtype)
    out = torch.empty(t.shape, dtype=t.dtype, device=dev)
    nbytes = t.numel() * t.element_size()
    src = t.reshape(-1).view(torch.uint8)
    dst = out.reshape(-1).view(torch.uint8)
    key = dev.index
    if key not in _STAGING:
        _STAGING[key] = [torch.empty(STAGING_BYTES, dtype=torch.uint8).pin_memory() for _ in range(2)]
        _STAGING[key].append([torch.cuda.Event(), torch.cuda.Event()])
    bufs, events = _STAGING[key][:2], _STAGING[key][2]
    stream = torch.cuda.current_stream(dev)
    off, i = 0, 0
    used = [False, False]
    while off < nbytes:
        n = min(STAGING_BYTES, nbytes - off)
        b = i & 1
        if used[b]:
            events[b].synchronize()
        bufs[b][:n].copy_(src[off : off + n])
        dst[off : off + n].copy_(bufs[b][:n], non_blocking=True)
        events[b].record(stream)
        used[b] = True
        off += n
        i += 1
    for b in range(2):
        if used[b]:
            events[b].synchronize()
    return out.to(dtype) if dtype is not None and dtype != out.dtype else out


def shard_range(total: int, rank: int, world: int) -> tuple:
    """Half-open range of ``total`` owned by ``rank`` (must divide evenly)."""
    if total % world:
        raise WeightError(f"dimension {total} is not divisible by tensor-parallel size {world}")
    per = total // world
    return rank * per, (rank + 1) * per
