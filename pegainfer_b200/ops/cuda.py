"""ctypes front end of the sm_100a kernels: same signatures as ``ops.reference``.

Every function validates dtypes/shapes, takes the current CUDA stream and calls the
C API of ``libpegainfer_b200.so``.  Per-device scratch (GEMM split-K workspace and tile
counters, argmax partials, split-KV partials, the device status word) is allocated
once with a fixed size so its addresses stay valid inside captured CUDA graphs.
"""
from __future__ import annotations

import ctypes
import os
import math
from typing import Optional

import torch

from .. import _native
from .reference import AttnMeta

_c = ctypes
_vp = ctypes.c_void_p
_ll = ctypes.c_longlong
_ci = ctypes.c_int
_cf = ctypes.c_float

GEMM_WS_BYTES = 96 << 20
GEMM_COUNTERS = 1 << 16
ATTN_PART_BYTES = 64 << 20


def _ptr(t: Optional[torch.Tensor]):
    return _vp(t.data_ptr()) if t is not None else _vp(0)


def _stream():
    return _vp(torch.cuda.current_stream().cuda_stream)


class _DeviceCtx:
    def __init__(self, device: torch.device):
        self.device = device
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.gemm_ws = torch.empty(GEMM_WS_BYTES, dtype=torch.uint8, device=device)
        self.gemm_counters = torch.zeros(GEMM_COUNTERS, dtype=torch.int32, device=device)
        self.argmax_scratch = torch.empty(8 << 20, dtype=torch.uint8, device=device)
        self.attn_part = torch.empty(ATTN_PART_BYTES, dtype=torch.uint8, device=device)
        self.sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.launches = 0


_CTX: dict = {}
_LANE = [0]  # 1 while ops are being queued on the prefill lane (second stream)


class lane_scratch:
    """Ops launched inside this block use a second set of per-device scratch buffers (split-K
    workspace and counters, attention partials, argmax scratch), because they run on another
    stream concurrently with ops that use the first set.  The status word is shared."""

    def __enter__(self):
        _LANE[0] += 1

    def __exit__(self, *exc):
        _LANE[0] -= 1


def ctx(device) -> _DeviceCtx:
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if torch.cuda.current_device() != idx:
        # kernels launched through the C API and torch.cuda.current_stream() follow the calling
        # thread's current device, which starts at 0 in every new thread
        torch.cuda.set_device(idx)
    key = (idx, 1 if _LANE[0] else 0)
    c = _CTX.get(key)
    if c is None:
        with torch.cuda.device(idx):
            c = _DeviceCtx(torch.device("cuda", idx))
        if key[1]:  # one status word per device
            main = _CTX.get((idx, 0))
            if main is not None:
                c.status = main.status
        _CTX[key] = c
    return c


_TUNED = False


def lib():
    global _TUNED
    l = _native.load()
    if not _TUNED:
        import os

        _TUNED = True
        stages = os.environ.get("PEGAINFER_ATTN_STAGES")
        if stages:
            l.pg_attn_set_decode_stages(_ci(int(stages)))
    return l


def _check(rc, c: Optional[_DeviceCtx] = None, n: int = 1):
    if rc != 0:
        _native.check(rc)
    if c is not None:
        c.launches += n


def launch_count(device=None) -> int:
    """Kernels of this library launched so far on ``device`` (eager calls; a graph
    replay re-launches what was captured without passing through here)."""
    if device is None:
        return sum(c.launches for c in _CTX.values())
    return ctx(device).launches


def read_status(device) -> int:
    """Device status word: 0 = clean; low byte 1 = a bounded wait expired, 2 = an index
    was out of range; bits 8.. identify the kernel site.  Synchronises."""
    return int(ctx(device).status[0].item()) & 0xFFFFFFFF


def clear_status(device) -> None:
    ctx(device).status.zero_()


# ----------------------------------------------------------------------------------
def _bf16(t):
    if t.dtype != torch.bfloat16:
        raise TypeError(f"sm_100a kernels take bfloat16 activations/weights, got {t.dtype}")
    return t


def embedding(ids, table):
    return gather_rows(table, ids)


def gather_rows(x, idx):
    _bf16(x)
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    idx = idx.to(torch.int32).contiguous()
    out = torch.empty((idx.numel(), x2.shape[1]), dtype=x.dtype, device=x.device)
    c = ctx(x.device)
    _check(lib().pg_gather_rows(_ptr(x2), _ptr(idx), _ptr(out), _ci(idx.numel()), _ci(x2.shape[1]), _ll(x2.shape[0]), _ptr(c.status), _stream()), c)
    return out


def gather_words(src: torch.Tensor, idx: torch.Tensor, dst: torch.Tensor) -> None:
    """``dst[i] = src[idx[i]]`` for int32 tensors (views allowed, unit stride)."""
    assert src.dtype == dst.dtype == idx.dtype == torch.int32 and src.stride(0) == 1 and dst.stride(0) == 1 and idx.stride(0) == 1
    c = ctx(src.device)
    _check(lib().pg_gather_words(_ptr(src), _ptr(idx), _ptr(dst), _ci(dst.numel()), _ci(src.numel()), _ptr(c.status), _stream()), c)


def _rows2d(x):
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    return x2


def rms_norm(x, w, eps, offset=False):
    _bf16(x)
    x2 = _rows2d(x)
    if x2.shape[1] % 8 != 0:
        raise ValueError(f"rms_norm: the sm_100a kernel takes rows of a multiple of 8 elements, got {x2.shape[1]}")
    y = torch.empty((x2.shape[0], x2.shape[1]), dtype=x.dtype, device=x.device)
    c = ctx(x.device)
    _check(lib().pg_rms_norm(_ptr(x2), _vp(0), _ptr(w), _ptr(y), _ci(x2.shape[0]), _ci(x2.shape[1]), _cf(eps), _ci(int(offset)), _ci(0), _ll(x2.stride(0)), _ll(0), _ll(y.stride(0)), _stream()), c)
    return y.view(x.shape)


def add_rms_norm(x, residual, w, eps, offset=False, round_before_norm=True):
    _bf16(x)
    x2, r2 = _rows2d(x), residual.reshape(-1, residual.shape[-1])
    assert r2.stride(-1) == 1 and r2.data_ptr() == residual.data_ptr(), "residual must be updatable in place"
    y = torch.empty((x2.shape[0], x2.shape[1]), dtype=x.dtype, device=x.device)
    c = ctx(x.device)
    _check(lib().pg_rms_norm(_ptr(x2), _ptr(r2), _ptr(w), _ptr(y), _ci(x2.shape[0]), _ci(x2.shape[1]), _cf(eps), _ci(int(offset)), _ci(int(round_before_norm)), _ll(x2.stride(0)), _ll(r2.stride(0)), _ll(y.stride(0)), _stream()), c)
    return y.view(x.shape)


def gated_rms_norm(x, gate, w, eps, act: str = "silu"):
    """Per-head ``rms_norm(x) * w * silu(gate)``; ``act="sigmoid"``: ``bf16(rms_norm(x) * w) * bf16(sigmoid(gate))``."""
    _bf16(x)
    x = x.contiguous()
    gate = gate.contiguous()
    w = w.float().contiguous()
    y = torch.empty_like(x)
    rows = x.numel() // x.shape[-1]
    c = ctx(x.device)
    _check(lib().pg_gated_rms_norm_act(_ptr(x), _ptr(gate), _ptr(w), _ptr(y), _ll(rows), _ci(x.shape[-1]), _cf(eps), _ci({"silu": 0, "sigmoid": 1}[act]), _stream()), c)
    return y


def swiglu(gate_up, interleaved: bool = False):
    """``bf16(silu(gate)) * up``; ``interleaved``: columns are (gate_0, up_0, gate_1, up_1, ...)."""
    _bf16(gate_up)
    g2 = _rows2d(gate_up)
    inter = g2.shape[1] // 2
    out = torch.empty((g2.shape[0], inter), dtype=g2.dtype, device=g2.device)
    c = ctx(g2.device)
    _check(lib().pg_swiglu(_ptr(g2), _ptr(out), _ci(g2.shape[0]), _ci(inter), _ll(g2.stride(0)), _ll(out.stride(0)), _ci(int(interleaved)), _stream()), c)
    return out.view(*gate_up.shape[:-1], inter)


def geglu(gate_up):
    """``bf16(gelu_tanh(gate)) * up`` on a fused ``[T, 2 I]`` buffer, gate half first."""
    _bf16(gate_up)
    g2 = _rows2d(gate_up)
    inter = g2.shape[1] // 2
    out = torch.empty((g2.shape[0], inter), dtype=g2.dtype, device=g2.device)
    _check(lib().pg_swiglu(_ptr(g2), _ptr(out), _ci(g2.shape[0]), _ci(inter), _ll(g2.stride(0)), _ll(out.stride(0)), _ci(2), _stream()), ctx(g2.device))
    return out.view(*gate_up.shape[:-1], inter)


def situ(gate_up):
    """``bf16(4 tanh(g / 4) sigmoid(g) * 25 tanh(u / 25))`` on a fused ``[T, 2 I]`` buffer, gate half first."""
    _bf16(gate_up)
    g2 = _rows2d(gate_up)
    inter = g2.shape[1] // 2
    out = torch.empty((g2.shape[0], inter), dtype=g2.dtype, device=g2.device)
    _check(lib().pg_swiglu(_ptr(g2), _ptr(out), _ci(g2.shape[0]), _ci(inter), _ll(g2.stride(0)), _ll(out.stride(0)), _ci(4), _stream()), ctx(g2.device))
    return out.view(*gate_up.shape[:-1], inter)


def attnres_mix(cur, snaps, nb: int, score_w, eps: float):
    """Softmax mix of each token's first ``nb`` snapshot rows (``snaps`` [T, cap, H]) and its current row ``cur`` [T, H],
    scored by ``dot(x / rms(x), score_w)`` (``score_w`` f32 [H])."""
    _bf16(cur)
    t, h = cur.shape
    assert snaps.is_contiguous() and snaps.shape[0] == t and snaps.shape[2] == h and nb <= snaps.shape[1] and cur.stride(1) == 1
    assert score_w.dtype == torch.float32 and score_w.is_contiguous()
    out = torch.empty((t, h), dtype=cur.dtype, device=cur.device)
    rc = lib().pg_attnres_mix(_ptr(cur), _ll(cur.stride(0)), _ptr(snaps), _ll(snaps.stride(0)), _ptr(score_w), _ptr(out), _ll(out.stride(0)), _ci(t), _ci(nb), _ci(h), _cf(eps), _stream())
    _check(rc, ctx(cur.device))
    return out


def softcap(logits, cap: float):
    """``cap * tanh(logits / cap)``."""
    _bf16(logits)
    x = logits.contiguous()
    y = torch.empty_like(x)
    _check(lib().pg_softcap(_ptr(x), _ptr(y), _ll(x.numel()), _cf(cap), _stream()), ctx(x.device))
    return y


class DeferredNorm:
    """Activations whose RMSNorm is still owed its per-token scale: ``xw = h * norm_w`` plus the
    per-(token, weight tile) sums of squares of ``h`` (``ssp[:, :parts]``).  The GEMM that consumes
    ``xw`` applies ``rsqrt(sum(ssp[n, :parts]) / width + eps)`` to every output element of token n."""

    __slots__ = ("xw", "ssp", "parts", "width", "eps")

    def __init__(self, xw, ssp, parts, width, eps):
        self.xw, self.ssp, self.parts, self.width, self.eps = xw, ssp, parts, width, eps


FUSED_MAX_ROWS = 64
EPI_PLAIN, EPI_SWIGLU, EPI_RESID_NORMW = 0, 1, 2


def fused_plan_ok(t: int, m: int, k: int) -> bool:
    """Does ``linear_fused`` run this problem on the on-chip split-K path (fused epilogues live there)?"""
    return t <= FUSED_MAX_ROWS and not _BATCH_INVARIANT and gemm_plan(t, m, k)["cluster"] > 1


def linear_fused(x, w, epilogue: int = EPI_PLAIN, residual=None, norm_w=None, norm_offset: bool = False, eps: float = 0.0):
    """Decode-chain GEMM.  ``x``: a bf16 ``[T, K]`` tensor or a ``DeferredNorm``.  ``epilogue``:
    ``EPI_PLAIN`` -> ``[T, M]``; ``EPI_SWIGLU`` (interleaved gate/up weight rows) -> ``[T, M / 2]``;
    ``EPI_RESID_NORMW`` -> updates ``residual`` in place and returns a ``DeferredNorm`` for the norm
    with weight ``norm_w`` (its consumer completes it)."""
    dn = x if isinstance(x, DeferredNorm) else None
    xin = dn.xw if dn is not None else x
    _bf16(xin)
    _bf16(w)
    t, k = xin.shape
    m = w.shape[0]
    assert w.shape[1] == k and xin.stride(-1) == 1 and w.stride(-1) == 1
    c = ctx(xin.device)
    out = torch.empty((t, m // 2 if epilogue == EPI_SWIGLU else m), dtype=torch.bfloat16, device=xin.device)
    ssp = None
    if epilogue == EPI_RESID_NORMW:
        assert residual is not None and norm_w is not None and residual.stride(-1) == 1
        parts = (m + 127) // 128
        ssp = torch.empty((t, (parts + 3) // 4 * 4), dtype=torch.float32, device=xin.device)
    GemmTrace.arm(f"fused{epilogue} {t}x{m}x{k}")
    rc = lib().pg_gemm_bf16_tn_fused(
        _ptr(xin), _ptr(w), _ptr(out), _ci(t), _ci(m), _ci(k), _ll(xin.stride(0)), _ll(w.stride(0)), _ll(out.stride(0)),
        _ptr(dn.ssp) if dn is not None else _vp(0), _ci(dn.parts if dn is not None else 0), _ci(dn.ssp.stride(0) if dn is not None else 0), _ci(dn.width if dn is not None else 0),
        _cf(dn.eps if dn is not None else 0.0),
        _ci(epilogue), _ptr(residual), _ll(residual.stride(0) if residual is not None else 0), _ptr(norm_w), _ci(int(norm_offset)), _ptr(ssp), _ci(ssp.stride(0) if ssp is not None else 0),
        _ptr(c.gemm_ws), _ll(c.gemm_ws.numel()), _ptr(c.gemm_counters), _ll(c.gemm_counters.numel() * 4), _ptr(c.status), _stream(),
    )
    _check(rc, c)
    if epilogue == EPI_RESID_NORMW:
        return DeferredNorm(out, ssp, parts, m, eps)
    return out


class GemmTrace:
    """Debug aid (``PEGAINFER_GEMM_TRACE=1``): every GEMM launch gets its own slot of a device
    buffer for the kernel's globaltimer phase stamps, so a captured decode step can be read back
    as one timeline (``dump``).  Off by default; the stamps cost a few stores per CTA."""

    enabled = os.environ.get("PEGAINFER_GEMM_TRACE") == "1"
    slots = 1024
    buf = None
    names: list = []

    @classmethod
    def arm(cls, label: str) -> None:
        if not cls.enabled:
            return
        if cls.buf is None:
            cls.buf = torch.zeros((cls.slots, 148 * 16), dtype=torch.int64, device="cuda")
        i = len(cls.names) % cls.slots
        cls.names.append(label)
        if label.startswith("chain"):
            lib().pg_decode_chain_set_timing(_vp(cls.buf[i].data_ptr()))
        else:
            lib().pg_gemm_set_timing(_vp(cls.buf[i].data_ptr()))

    @classmethod
    def chain_rows(cls, first: int, end: int) -> list:
        """Stamps of the decode-chain launches among the armed launches ``first .. end``: per launch the
        medians over the CTAs of [entry, predecessor complete, then per phase: tiles stored, partials
        visible, fix-up done], microseconds from the first launch's entry, and the last CTA's last stamp."""
        import numpy as np

        torch.cuda.synchronize()
        rows, t0 = [], None
        for i in range(first, end):
            if not cls.names[i].startswith("chain"):
                continue
            tm = cls.buf[i % cls.slots].view(148, 16).cpu().numpy().astype(np.float64)
            if t0 is None:
                t0 = np.median(tm[:, 0])
            med = [(np.median(tm[:, j]) - t0) / 1e3 if (tm[:, j] > 0).all() else float("nan") for j in range(14)]
            last = (tm[:, :14].max() - t0) / 1e3
            rows.append((cls.names[i], med, last))
        return rows

    @classmethod
    def reset(cls) -> None:
        cls.names = []
        if cls.buf is not None:
            cls.buf.zero_()

    @classmethod
    def dump(cls, first: int, end: int, detail: bool = False) -> list:
        """(label, entry, x ready, first MMA, last MMA, exit) in microseconds from the first entry,
        medians over the CTAs, for the armed launches ``first .. end``."""
        import numpy as np

        torch.cuda.synchronize()
        rows = []
        t0 = None
        for i in range(first, end):
            tm = cls.buf[i % cls.slots].view(148, 16).cpu().numpy().astype(np.float64)
            tm = tm[tm[:, 0] > 0]
            if not len(tm):
                continue
            if t0 is None:
                t0 = tm[:, 0].min()
            med = lambda j: (np.median(tm[:, j][tm[:, j] > 0]) - t0) / 1e3 if (tm[:, j] > 0).any() else float("nan")
            rows.append((cls.names[i], (tm[:, 0].min() - t0) / 1e3, med(2), med(4), med(5), (max(tm[:, 10].max(), tm[:, 11].max()) - t0) / 1e3))
            if detail:
                base = np.median(tm[:, 2][tm[:, 2] > 0])
                det = {}
                for j in range(2, 12):
                    col = tm[:, j][tm[:, j] >= base - 1e6]
                    col = col[col > 0]
                    if len(col):
                        det[j] = (round((col.min() - base) / 1e3, 2), round((np.median(col) - base) / 1e3, 2), round((col.max() - base) / 1e3, 2))
                rows[-1] = rows[-1] + (det,)
        return rows


def linear(x, w, out_dtype=None, force_splits: int = 0, out: Optional[torch.Tensor] = None):
    """``x[T, K] @ w[M, K].T`` on the tcgen05 GEMM (f32 accumulation)."""
    _bf16(x)
    _bf16(w)
    x2 = _rows2d(x)
    if w.stride(-1) != 1:
        w = w.contiguous()
    t, k = x2.shape
    m = w.shape[0]
    assert w.shape[1] == k, f"linear: x has K={k}, w has K={w.shape[1]}"
    f32 = out_dtype == torch.float32
    if out is None:
        out = torch.empty((t, m), dtype=torch.float32 if f32 else torch.bfloat16, device=x.device)
    if t == 0:
        return out.view(*x.shape[:-1], m)
    if _BATCH_INVARIANT and force_splits == 0:
        force_splits = 1
    c = ctx(x.device)
    GemmTrace.arm(f"linear {t}x{m}x{k}")
    rc = lib().pg_gemm_bf16_tn(
        _ptr(x2), _ptr(w), _ptr(out), _ci(int(f32)), _ci(t), _ci(m), _ci(k), _ll(x2.stride(0)), _ll(w.stride(0)), _ll(out.stride(0)),
        _ptr(c.gemm_ws), _ll(c.gemm_ws.numel()), _ptr(c.gemm_counters), _ll(c.gemm_counters.numel() * 4), _ptr(c.status), _ci(force_splits), _stream(),
    )
    _check(rc, c)
    res = out.view(*x.shape[:-1], m)
    if out_dtype is not None and res.dtype != out_dtype:
        res = res.to(out_dtype)
    return res


def linear_2sm(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` through the two-SM (``cta_group::2``) kernel regardless of the size
    heuristic of ``linear`` (tests and benchmarks)."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    t, k = x2.shape
    m = w.shape[0]
    out = torch.empty((t, m), dtype=torch.bfloat16, device=x.device)
    c = ctx(x.device)
    rc = lib().pg_gemm2sm_bf16_tn(_ptr(x2), _ptr(w), _ptr(out), _ci(t), _ci(m), _ci(k), _ll(x2.stride(0)), _ll(w.stride(0)), _ll(out.stride(0)), _ptr(c.status), _stream())
    _check(rc, c)
    return out.view(*x.shape[:-1], m)


def linear_swiglu_2sm(x: torch.Tensor, w: torch.Tensor) -> Optional[torch.Tensor]:
    """``swiglu(x @ w.T)`` for a gate_up weight whose rows alternate (gate_i, up_i), with SwiGLU in the epilogue of the
    two-SM GEMM (prefill-sized steps); ``None`` when the two-SM kernel does not take the problem."""
    _bf16(x)
    x2 = _rows2d(x)
    t, k = x2.shape
    m = w.shape[0]
    if not lib().pg_gemm2sm_eligible(_ci(t), _ci(m), _ci(k)) or _BATCH_INVARIANT or w.stride(-1) != 1:
        return None
    out = torch.empty((t, m // 2), dtype=torch.bfloat16, device=x.device)
    c = ctx(x.device)
    rc = lib().pg_gemm2sm_bf16_tn_swiglu(_ptr(x2), _ptr(w), _ptr(out), _ci(t), _ci(m), _ci(k), _ll(x2.stride(0)), _ll(w.stride(0)), _ll(out.stride(0)), _ptr(c.status), _stream())
    _check(rc, c)
    return out.view(*x.shape[:-1], m // 2)


class _ChainPhase(ctypes.Structure):
    _fields_ = [("x", _vp), ("ldx", _ll), ("w", _vp), ("ldw", _ll), ("M", _ci), ("K", _ci), ("epi", _ci), ("out", _vp), ("ld_out", _ll), ("norm_w", _vp), ("norm_offset", _ci),
                ("in_ssp", _vp), ("in_parts", _ci), ("in_ld", _ci), ("in_width", _ci), ("in_eps", _cf), ("out_ssp", _vp), ("out_ld", _ci),
                ("q_w", _vp), ("k_w", _vp), ("cos", _vp), ("sin", _vp), ("positions", _vp), ("slots", _vp), ("kv", _vp), ("hq", _ci), ("hkv", _ci), ("rot", _ci), ("page_size", _ci),
                ("max_pos", _ci), ("num_slots", _ll), ("qk_eps", _cf)]


CHAIN_MAX_ROWS = 64
CH_PLAIN, CH_SWIGLU, CH_RESID_NORM, CH_QKV_ROPE = 0, 1, 2, 3


def decode_chain(x, phases, residual=None, eps: float = 0.0, tp=None):
    """Up to four dependent GEMMs of a decode step (at most 64 rows) in one persistent kernel.

    ``x``: bf16 ``[T, K0]`` or a ``DeferredNorm``; it feeds the first phase, each later phase reads
    the previous phase's output.  ``phases``: list of ``(weight [M, K], epilogue, norm_weight_or_None,
    norm_offset)`` with epilogue ``CH_PLAIN`` (output [T, M]), ``CH_SWIGLU`` (weight rows interleaved
    gate/up; output [T, M / 2]) or ``CH_RESID_NORM`` (``residual`` += GEMM; the output is a
    ``DeferredNorm``: ``residual * norm_weight`` plus the sums of squares from which the next phase, or
    a later ``linear_fused`` / ``decode_chain``, takes the per-token RMSNorm scale).  A last phase
    ``(qkv_weight, CH_QKV_ROPE, spec, norm_offset)`` finishes the fused qkv projection of a model with
    128-wide heads: per-head QK RMSNorm, rotary embedding and the paged KV append happen in its epilogue;
    ``spec`` is a dict with ``q_norm``, ``k_norm`` (or None), ``cos``, ``sin``, ``meta`` (positions, slot
    mapping), ``kv_layer``, ``hq``, ``hkv``, ``eps``; the output is q ``[T, hq, 128]``.
    ``tp``: a ``parallel.chain_tp.ChainTP``; the residual + norm phases then sum over the ranks
    through NVSwitch multicast memory.  Returns the list of phase outputs."""
    dn = x if isinstance(x, DeferredNorm) else None
    cur = dn.xw if dn is not None else x
    _bf16(cur)
    t = cur.shape[0]
    assert 1 <= t <= CHAIN_MAX_ROWS and 1 <= len(phases) <= 4 and cur.stride(-1) == 1
    c = ctx(cur.device)
    if not hasattr(c, "chain_ws"):
        c.chain_ws = torch.empty(int(lib().pg_decode_chain_ws_bytes(_ci(c.device.index or 0))), dtype=torch.uint8, device=cur.device)
        c.chain_counters = torch.zeros(16, dtype=torch.int32, device=cur.device)
    arr = (_ChainPhase * len(phases))()
    results = []
    for i, (w, epi, norm_w, norm_offset) in enumerate(phases):
        _bf16(w)
        m, k = w.shape
        assert cur.shape[1] == k and w.stride(-1) == 1, f"chain phase {i}: input has {cur.shape[1]} features, weight wants {k}"
        width = m // 2 if epi == CH_SWIGLU else m
        spec = norm_w if epi == CH_QKV_ROPE else None
        if spec is not None:
            norm_w = None
            out = torch.empty((t, spec["hq"], 128), dtype=torch.bfloat16, device=cur.device)
        else:
            out = torch.empty((t, width), dtype=torch.bfloat16, device=cur.device)
        ph = _ChainPhase()
        ph.x, ph.ldx, ph.w, ph.ldw, ph.M, ph.K, ph.epi, ph.out, ph.ld_out = cur.data_ptr(), cur.stride(0), w.data_ptr(), w.stride(0), m, k, epi, out.data_ptr(), out.stride(0)
        ph.norm_w, ph.norm_offset = (norm_w.data_ptr() if norm_w is not None else 0), int(bool(norm_offset))
        if dn is not None:
            ph.in_ssp, ph.in_parts, ph.in_ld, ph.in_width, ph.in_eps = dn.ssp.data_ptr(), dn.parts, dn.ssp.stride(0), dn.width, dn.eps
        dn = None
        if spec is not None:
            meta, kvl = spec["meta"], spec["kv_layer"]
            assert kvl.is_contiguous() and kvl.shape[-1] == 128 and spec["cos"].shape[-1] * 2 == 128, "the fused qkv epilogue is built for 128-wide heads with full rotary"
            ph.q_w = spec["q_norm"].data_ptr() if spec.get("q_norm") is not None else 0
            ph.k_w = spec["k_norm"].data_ptr() if spec.get("k_norm") is not None else 0
            ph.cos, ph.sin = spec["cos"].data_ptr(), spec["sin"].data_ptr()
            ph.positions, ph.slots, ph.kv = meta.positions.data_ptr(), meta.slot_mapping.data_ptr(), kvl.data_ptr()
            ph.hq, ph.hkv, ph.rot, ph.page_size, ph.max_pos = spec["hq"], spec["hkv"], spec["cos"].shape[-1] * 2, kvl.shape[2], spec["cos"].shape[0]
            ph.num_slots, ph.qk_eps = kvl.shape[0] * kvl.shape[2], spec["eps"]
        if epi == CH_RESID_NORM:
            assert residual is not None and norm_w is not None and residual.shape == (t, m) and residual.stride(-1) == 1
            parts = (m + 127) // 128
            ssp = torch.empty((t, (parts + 3) // 4 * 4), dtype=torch.float32, device=cur.device)
            ph.out_ssp, ph.out_ld = ssp.data_ptr(), ssp.stride(0)
            dn = DeferredNorm(out, ssp, parts, m, eps)
            results.append(dn)
        else:
            results.append(out)
        arr[i] = ph
        cur = out
    GemmTrace.arm(f"chain x{len(phases)} T{t}")
    if tp is not None and tp.world > 1:
        rc = lib().pg_decode_chain_tp(arr, _ci(len(phases)), _ci(t), _ptr(residual), _ll(residual.stride(0) if residual is not None else 0), _cf(eps), _ptr(c.chain_ws), _ll(c.chain_ws.numel()),
                                      _ptr(c.chain_counters), _ptr(c.status), ctypes.byref(tp.spec), _stream())
    else:
        rc = lib().pg_decode_chain(arr, _ci(len(phases)), _ci(t), _ptr(residual), _ll(residual.stride(0) if residual is not None else 0), _cf(eps), _ptr(c.chain_ws), _ll(c.chain_ws.numel()),
                                   _ptr(c.chain_counters), _ptr(c.status), _stream())
    _check(rc, c)
    return results


_PREFETCH_CAP = int(float(os.environ.get("PEGAINFER_GEMM_PREFETCH_MB", "8")) * (1 << 20))


def prefetch_weights(w: torch.Tensor) -> None:
    """Hint for the next ``linear`` launched from this thread: while it runs, its idle
    producer lanes pull the leading part of ``w`` (the weights of the GEMM that follows)
    into L2, so the launch gap and the small kernel in between find HBM busy."""
    if _PREFETCH_CAP <= 0 or not w.is_cuda:
        return
    lib().pg_gemm_prefetch_next(_ptr(w), _ll(min(w.numel() * w.element_size(), _PREFETCH_CAP) & ~15))


def gemm_plan(t: int, m: int, k: int, force_splits: int = 0) -> dict:
    """Launch plan of ``linear`` for a problem size on the current device."""
    import ctypes

    out = (ctypes.c_int * 6)()
    _check(lib().pg_gemm_plan(_ci(t), _ci(m), _ci(k), _ci(force_splits), out), None)
    return dict(zip(("bn", "splits", "cluster", "grid", "stages", "max_clusters"), list(out)))


def qk_norm_rope_append(qkv, q_norm_w, k_norm_w, cos, sin, meta: AttnMeta, kv_layer, num_q_heads, num_kv_heads, head_dim, eps, offset=False, gated=False, v_norm=False):
    _bf16(qkv)
    t = qkv.shape[0]
    assert qkv.stride(-1) == 1
    q = torch.empty((t, num_q_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    gate = torch.empty_like(q) if gated else None
    assert kv_layer.is_contiguous()
    num_pages, _, page_size = kv_layer.shape[0], kv_layer.shape[1], kv_layer.shape[2]
    c = ctx(qkv.device)
    rc = lib().pg_qk_norm_rope_append(
        _ptr(qkv), _ll(qkv.stride(0)), _ptr(q_norm_w), _ptr(k_norm_w), _ptr(cos), _ptr(sin), _ptr(meta.positions), _ptr(meta.slot_mapping),
        _ptr(q), _ptr(gate), _ptr(kv_layer), _ci(t), _ci(num_q_heads), _ci(num_kv_heads), _ci(head_dim), _ci(cos.shape[-1] * 2), _ci(page_size),
        _ll(num_pages), _ci(cos.shape[0]), _ci(int(gated)), _ci(int(offset)), _cf(eps), _ci(int(v_norm)), _ptr(c.status), _stream(),
    )
    _check(rc, c)
    return (q, gate) if gated else q


_BATCH_INVARIANT = False
INVARIANT_KV_SPLITS = 4
_WIDE_MMA = os.environ.get("PEGAINFER_WIDE_MMA", "1") != "0"  # head dim 512 on the mma.sync kernel (0: the CUDA-core kernel)
_PREFILL_TC = os.environ.get("PEGAINFER_PREFILL_TC", "1") != "0"  # tcgen05 prefill attention for head dims 128 and 256
_PREFILL_TC_MIN_ROWS = int(os.environ.get("PEGAINFER_PREFILL_TC_MIN_ROWS", "64"))  # shorter chunks keep the 64-row mma.sync tiles
# the tcgen05 kernel wins from a few hundred keys on (head dim 128, against the mma.sync kernel: 1.0x at 256 keys, 1.3x at 512,
# 1.9x at 1024, 3.2x at 4096, 3.8x at 16384)
_PREFILL_TC_MIN_KV = int(os.environ.get("PEGAINFER_PREFILL_TC_MIN_KV", "512"))


# how often each tcgen05 prefill kernel was chosen (tests assert that long prompts really take them)
PREFILL_TC_CALLS = {"hd128": 0, "hd256": 0, "mla": 0}


def set_prefill_tc(min_kv: int) -> int:
    """KV length from which prefill attention of head dim 128 takes the tcgen05 kernel; returns the previous value."""
    global _PREFILL_TC_MIN_KV
    prev, _PREFILL_TC_MIN_KV = _PREFILL_TC_MIN_KV, int(min_kv)
    return prev


def set_batch_invariant(on: bool) -> None:
    """Numeric policy for ``--batch-invariant`` serving: a row's result must not depend on what
    else rides in the batch.  GEMMs run with one k-split (the k order inside a CTA is fixed and
    independent of the token tile), decode attention uses a constant number of KV splits (the
    split boundaries then depend on the sequence's own length only); the default policy picks
    both from the batch shape.  Reference: pegainfer-kernels/src/ops/linear.rs NumericPolicy,
    pegainfer-qwen3/src/lib.rs:498-548."""
    global _BATCH_INVARIANT
    _BATCH_INVARIANT = bool(on)


def batch_invariant() -> bool:
    return _BATCH_INVARIANT


_MIXED_DECODE_MIN = 4  # fewer trailing decode rows than this stay in the prefill kernel of a unified step


def plan_decode_splits(num_seqs: int, hkv: int, max_kv_len: int, device) -> int:
    if _BATCH_INVARIANT:
        return INVARIANT_KV_SPLITS
    return int(lib().pg_decode_splits(_ci(num_seqs), _ci(hkv), _ci(max(max_kv_len, 1)), _ci(ctx(device).sms)))


def paged_attention(q, kv_layer, meta: AttnMeta, scale=None, window=0, out: Optional[torch.Tensor] = None):
    _bf16(q)
    t, hq, d = q.shape
    hkv = kv_layer.shape[-2]
    page_size = kv_layer.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if out is None:
        out = torch.empty((t, hq * d), dtype=q.dtype, device=q.device)
    c = ctx(q.device)
    table = meta.block_table
    if d == 512:
        # wide heads (global layers of the Gemma 4 line): one block per (query row, KV head), csrc/attention_wide.cu
        assert q.is_contiguous() and kv_layer.is_contiguous()
        group = hq // hkv
        q_tiles = 0
        if _WIDE_MMA and 32 % group == 0:  # tensor-core kernel: 32 / group query tokens of a sequence x the group's heads per block
            tpt = 32 // group
            if meta.decode_only:
                q_tiles = meta.num_seqs
            else:
                qh = meta.h_q_indptr if meta.h_q_indptr is not None else meta.q_indptr.tolist()
                q_tiles = sum((qh[b + 1] - qh[b] + tpt - 1) // tpt for b in range(meta.num_seqs))
        # decode steps: split the keys of a sequence over several blocks until the launch fills the GPU about twice
        splits = 1
        if q_tiles > 0 and meta.decode_only:
            splits = max(1, min(8, (2 * c.sms) // max(1, q_tiles * hkv), (max(meta.max_kv_len, 1) + 255) // 256))
            while splits > 1 and t * hq * splits * (d + 2) * 4 > c.attn_part.numel():
                splits -= 1
        ml_off = t * hq * splits * d * 4
        rc = lib().pg_attention_wide(_ptr(q), _ptr(kv_layer), _ptr(out), _ptr(_unit_seq(meta, q.device)), _ptr(meta.q_indptr), _ptr(meta.kv_lens), _ptr(table),
                                     _ci(table.stride(0)), _ci(t), _ci(meta.num_seqs), _ci(q_tiles), _ci(hq), _ci(hkv), _ci(d), _ci(page_size), _ll(kv_layer.shape[0]), _cf(scale),
                                     _ci(window), _ci(splits), _ptr(c.attn_part), _ptr(c.attn_part[ml_off:]), _ptr(c.status), _stream())
        _check(rc, c, 2 if splits > 1 else 1)
        return out

    def decode_rows(first: int, n: int, plan=None):
        """Decode kernel (one query row per sequence, the Q heads of a KV head packed into one MMA
        tile, split KV) over sequences ``first .. first + n``; rows are found through q_indptr."""
        splits = plan if isinstance(plan, int) else plan_decode_splits(n, hkv, meta.max_kv_len, q.device)
        need = n * hq * splits * (d + 1) * 4
        if need > c.attn_part.numel():
            splits = max(1, c.attn_part.numel() // (n * hq * (d + 1) * 4))
        lse_off = n * hq * splits * d * 4
        rc = lib().pg_paged_attention(
            _ptr(q), _ptr(kv_layer), _ptr(out), _ptr(meta.q_indptr[first:]), _ptr(meta.kv_lens[first:]), _ptr(table[first:]), _ci(table.stride(0)), _ci(n),
            _ci(hq), _ci(hkv), _ci(d), _ci(page_size), _ll(kv_layer.shape[0]), _cf(scale), _ci(0), _ci(splits), _ptr(c.attn_part), _ptr(c.attn_part[lse_off:]),
            _ci(0), _ci(window), _ptr(c.status), _stream(),
        )
        _check(rc, c, 2 if splits > 1 else 1)

    if window > 0 and meta.h_kv_lens is not None and max(meta.h_kv_lens[: meta.num_seqs], default=0) <= window:
        window = 0  # no sequence of this step is longer than the window: plain causal attention (and its faster kernels)
    if meta.decode_only:  # with a sliding window the decode kernel walks the last `window` keys of every sequence
        decode_rows(0, meta.num_seqs, meta.plan)
        return out
    qi = meta.h_q_indptr if meta.h_q_indptr is not None else meta.q_indptr.tolist()
    n_pf = meta.num_seqs
    # A unified step lists its prompt chunks first and its decode rows last.  Through the prefill
    # kernel a decode row is a 64-row query tile with one live row per Q head, and 63 of them cost
    # several times the chunk itself; the trailing single-row sequences take the decode kernel.
    while n_pf > 0 and qi[n_pf] - qi[n_pf - 1] == 1:
        n_pf -= 1
    # batch-invariant serving: a single-row sequence ALWAYS takes the decode kernel (same KV
    # splits and merge order as in a pure decode step or a graph replay), however few there are
    if meta.num_seqs - n_pf < (1 if _BATCH_INVARIANT else _MIXED_DECODE_MIN):
        n_pf = meta.num_seqs
    # (not under the batch-invariant policy: which kernel runs would depend on the other sequences of the step)
    if (n_pf > 0 and (d == 256 or (d == 128 and window == 0)) and _PREFILL_TC and not _BATCH_INVARIANT and (128 if d == 128 else 64) % page_size == 0 and q.is_contiguous() and max(qi[b + 1] - qi[b] for b in range(n_pf)) >= _PREFILL_TC_MIN_ROWS
            and (meta.h_kv_lens is None or max(meta.h_kv_lens[:n_pf]) >= _PREFILL_TC_MIN_KV)):
        # tcgen05 kernel: 256 (head dim 128) or 128 (head dim 256) query rows of one head per CTA, S and P V on the
        # tensor cores, accumulators in TMEM
        rows_per_cta = 256 if d == 128 else 128
        PREFILL_TC_CALLS["hd128" if d == 128 else "hd256"] += 1
        q_tiles = sum((qi[b + 1] - qi[b] + rows_per_cta - 1) // rows_per_cta for b in range(n_pf))
        rc = lib().pg_prefill_attention_tc(_ptr(q), _ptr(kv_layer), _ptr(out), _ptr(meta.q_indptr), _ptr(meta.kv_lens), _ptr(table), _ci(table.stride(0)), _ci(n_pf), _ci(qi[n_pf]),
                                           _ci(hq), _ci(hkv), _ci(d), _ci(page_size), _ll(kv_layer.shape[0]), _cf(scale), _ci(q_tiles), _ci(window), _ptr(c.status), _stream())
        _check(rc, c)
    elif n_pf > 0:
        q_tiles = sum((qi[b + 1] - qi[b] + 63) // 64 for b in range(n_pf))
        rc = lib().pg_paged_attention(
            _ptr(q), _ptr(kv_layer), _ptr(out), _ptr(meta.q_indptr), _ptr(meta.kv_lens), _ptr(table), _ci(table.stride(0)), _ci(n_pf),
            _ci(hq), _ci(hkv), _ci(d), _ci(page_size), _ll(kv_layer.shape[0]), _cf(scale), _ci(1), _ci(1), _vp(0), _vp(0), _ci(q_tiles), _ci(window),
            _ptr(c.status), _stream(),
        )
        _check(rc, c)
    if n_pf < meta.num_seqs:
        decode_rows(n_pf, meta.num_seqs - n_pf)
    return out


def sigmoid_gate_mul_(x, gate):
    c = ctx(x.device)
    assert x.is_contiguous() and gate.is_contiguous()
    _check(lib().pg_sigmoid_gate_mul(_ptr(x), _ptr(gate), _ll(x.numel()), _stream()), c)
    return x


def argmax(logits, out: Optional[torch.Tensor] = None):
    rows, vocab = logits.shape
    assert logits.stride(-1) == 1
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    c = ctx(logits.device)
    f32 = logits.dtype == torch.float32
    if not f32:
        _bf16(logits)
    rc = lib().pg_argmax(_ptr(logits), _ci(int(f32)), _ci(rows), _ci(vocab), _ll(logits.stride(0)), _ptr(c.argmax_scratch), _ll(c.argmax_scratch.numel()), _ptr(out), _stream())
    _check(rc, c, 2)
    return out


def markov_step_argmax(base, bias, block: int, step: int, next_tokens, drafts):
    """``next_tokens[r] = drafts[r, step] = argmax_v base[r * block + step, v] + bias[r, v]``."""
    rows, vocab = bias.shape
    assert base.shape[0] == rows * block and base.shape[1] == vocab and base.stride(-1) == 1 and bias.stride(-1) == 1 and base.dtype == bias.dtype
    c = ctx(base.device)
    f32 = base.dtype == torch.float32
    if not f32:
        _bf16(base)
    rc = lib().pg_markov_step_argmax(_ptr(base), _ci(int(f32)), _ci(rows), _ci(block), _ci(step), _ci(vocab), _ll(base.stride(0)), _ptr(bias), _ll(bias.stride(0)),
                                     _ptr(c.argmax_scratch), _ll(c.argmax_scratch.numel()), _ptr(next_tokens), _ptr(drafts), _stream())
    _check(rc, c, 2)
    return next_tokens


def sample(logits, temperature, top_k, top_p, min_p, u):
    rows, vocab = logits.shape
    if logits.stride(-1) != 1:
        logits = logits.contiguous()
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    f32 = logits.dtype == torch.float32
    c = ctx(logits.device)
    rc = lib().pg_sample(
        _ptr(logits), _ci(int(f32)), _ci(rows), _ci(vocab), _ll(logits.stride(0)), _ptr(temperature.float().contiguous()), _ptr(top_k.to(torch.int32).contiguous()),
        _ptr(top_p.float().contiguous()), _ptr(min_p.float().contiguous()), _ptr(u.float().contiguous()), _ptr(out), _stream(),
    )
    _check(rc, c)
    return out


def logprobs_topk(logits, picked, k):
    rows, vocab = logits.shape
    if logits.stride(-1) != 1:
        logits = logits.contiguous()
    f32 = logits.dtype == torch.float32
    dev = logits.device
    chosen = torch.empty(rows, dtype=torch.float32, device=dev)
    tv = torch.empty((rows, max(k, 1)), dtype=torch.float32, device=dev)
    ti = torch.empty((rows, max(k, 1)), dtype=torch.int32, device=dev)
    c = ctx(dev)
    rc = lib().pg_logprob_topk(_ptr(logits), _ci(int(f32)), _ci(rows), _ci(vocab), _ll(logits.stride(0)), _ptr(picked.to(torch.int32).contiguous()), _ci(k), _ptr(chosen), _ptr(tv), _ptr(ti), _stream())
    _check(rc, c)
    if k == 0:
        return chosen, None, None
    return chosen, tv, ti


# ----------------------------------------------------------------------------------
# Gated DeltaNet
# ----------------------------------------------------------------------------------
def sigmoid_gate_mul(x, gate):
    return sigmoid_gate_mul_(x.contiguous(), gate.contiguous())


def gdn_conv1d(x, conv_w, conv_state, meta: AttnMeta):
    _bf16(x)
    assert x.stride(-1) == 1 and conv_w.is_contiguous() and conv_state.is_contiguous()
    t, ch = x.shape
    out = torch.empty((t, ch), dtype=x.dtype, device=x.device)
    c = ctx(x.device)
    k = conv_w.shape[1]
    rc = lib().pg_gdn_conv1d(_ptr(x), _ll(x.stride(0)), _ptr(conv_w), _ptr(conv_state), _ptr(out), _ll(out.stride(0)), _ptr(meta.q_indptr), _ptr(meta.state_slots),
                             _ci(meta.num_seqs), _ci(ch), _ci(k), _ll(conv_state.stride(0)), _stream())
    _check(rc, c)
    return out


def gdn_gates(a, b, a_log, dt_bias):
    t, hv = a.shape
    g = torch.empty((t, hv), dtype=torch.float32, device=a.device)
    beta = torch.empty_like(g)
    c = ctx(a.device)
    assert a.stride(-1) == 1 and b.stride(-1) == 1
    rc = lib().pg_gdn_gates(_ptr(a), _ll(a.stride(0)), _ptr(b), _ll(b.stride(0)), _ptr(a_log), _ptr(dt_bias), _ptr(g), _ptr(beta), _ci(t), _ci(hv), _stream())
    _check(rc, c)
    return g, beta


_GDN_CHUNKED = os.environ.get("PEGAINFER_GDN_CHUNKED", "1") != "0"
_GDN_CHUNK_MIN = 32  # sequences of at least this many tokens in a step take the chunk-wise kernel


def gdn_recurrent(q, k, v, g, beta, state, meta: AttnMeta, chunked: Optional[bool] = None):
    t, hk, dk = q.shape
    hv, dv = v.shape[1], v.shape[2]
    assert q.stride(2) == 1 and q.stride(1) == dk and k.stride(1) == dk and v.stride(1) == dv and q.stride(0) == k.stride(0)
    assert state.is_contiguous() and state.dtype == torch.float32
    out = torch.empty((t, hv, dv), dtype=q.dtype, device=q.device)
    c = ctx(q.device)
    g, beta = g.contiguous(), beta.contiguous()
    # prompt chunks go through the chunk-wise tensor-core scan, short rows (decode) through the recurrence
    chunked = (_GDN_CHUNKED if chunked is None else chunked) and int(meta.max_q_len) >= _GDN_CHUNK_MIN and dk == 128 and dv % 64 == 0 and q.stride(0) % 8 == 0 and v.stride(0) % 8 == 0
    args = (_ptr(q), _ptr(k), _ll(q.stride(0)), _ptr(v), _ll(v.stride(0)), _ptr(g), _ptr(beta), _ptr(state), _ptr(out),
            _ptr(meta.q_indptr), _ptr(meta.state_slots), _ci(meta.num_seqs), _ci(hk), _ci(hv), _ci(dk), _ci(dv))
    if chunked:
        rc = lib().pg_gdn_chunked(*args, _ci(_GDN_CHUNK_MIN), _stream())
        _check(rc, c)
    short_rows = True  # is there a sequence below the chunk threshold (decode rows in a unified step)?
    if chunked and meta.h_q_indptr is not None:
        qi = meta.h_q_indptr
        short_rows = any(qi[i + 1] - qi[i] < _GDN_CHUNK_MIN for i in range(meta.num_seqs))
    if not chunked or short_rows:
        rc = lib().pg_gdn_recurrent(*args, _ci(int(meta.max_q_len)), _ci(_GDN_CHUNK_MIN if chunked else 0), _stream())
        _check(rc, c)
    return out


def kda_recurrent(q, k, v, f, b, a_log, dt_bias, lower: float, state, meta: AttnMeta):
    """Delta rule with one decay per key channel; the decay and beta arithmetic on the raw gate projections ``f`` [T, H * Dk]
    and ``b`` [T, H] runs inside the kernel.  ``q, k, v`` [T, H, D] share one row stride (slices of the fused convolution
    output); ``state`` [slots, H, Dk, Dv] f32 is updated in place."""
    _bf16(q)
    t, h, dk = q.shape
    dv = v.shape[2]
    assert q.stride(2) == 1 and q.stride(1) == dk and k.stride(1) == dk and v.stride(1) == dv and q.stride(0) == k.stride(0) == v.stride(0)
    assert f.stride(1) == 1 and b.stride(1) == 1 and f.shape[1] == h * dk and b.shape[1] == h
    assert state.is_contiguous() and state.dtype == torch.float32 and a_log.dtype == torch.float32 and dt_bias.dtype == torch.float32
    out = torch.empty((t, h, dv), dtype=q.dtype, device=q.device)
    rc = lib().pg_kda_recurrent(_ptr(q), _ptr(k), _ptr(v), _ll(q.stride(0)), _ptr(f), _ll(f.stride(0)), _ptr(b), _ll(b.stride(0)), _ptr(a_log), _ptr(dt_bias), _cf(lower),
                                _ptr(state), _ptr(out), _ptr(meta.q_indptr), _ptr(meta.state_slots), _ci(meta.num_seqs), _ci(h), _ci(dk), _ci(dv), _ci(int(meta.max_q_len)), _stream())
    _check(rc, ctx(q.device))
    return out


# ----------------------------------------------------------------------------------
# mixture of experts
# ----------------------------------------------------------------------------------
def router_topk(logits, top_k, scoring="softmax", bias=None, n_group=1, topk_group=1, norm_topk_prob=False, scale=1.0):
    assert logits.dtype == torch.float32 and logits.stride(-1) == 1
    t, e = logits.shape
    ids = torch.empty((t, top_k), dtype=torch.int32, device=logits.device)
    w = torch.empty((t, top_k), dtype=torch.float32, device=logits.device)
    c = ctx(logits.device)
    b = bias.float().contiguous() if bias is not None else None
    rc = lib().pg_router_topk(_ptr(logits), _ll(logits.stride(0)), _ptr(b), _ptr(ids), _ptr(w), _ci(t), _ci(e), _ci(top_k), _ci(int(scoring == "sigmoid")), _ci(n_group),
                              _ci(topk_group), _ci(int(norm_topk_prob)), _cf(scale), _stream())
    _check(rc, c)
    return ids, w


def _token_tile(routes: int, experts: int) -> int:
    avg = max(1, (routes + experts - 1) // experts)
    bn = 16
    while bn < avg and bn < 128:
        bn *= 2
    return bn


def moe_route_plan(ids, e0: int, e_local: int):
    """Stable sort of the routes that hit experts [e0, e0 + e_local)."""
    routes = ids.numel()
    dev = ids.device
    offsets = torch.empty(e_local + 1, dtype=torch.int32, device=dev)
    sorted_src = torch.empty(max(routes, 1), dtype=torch.int32, device=dev)
    route_pos = torch.empty(max(routes, 1), dtype=torch.int32, device=dev)
    c = ctx(dev)
    _check(lib().pg_moe_align(_ptr(ids.contiguous()), _ci(routes), _ci(e0), _ci(e_local), _ptr(offsets), _ptr(sorted_src), _ptr(route_pos), _stream()), c)
    return offsets, sorted_src, route_pos


def quant_code(w) -> int:
    """Weight storage mode of the grouped GEMM: 0 bf16, 1 packed INT4 group-32, 2 block-scaled FP8 e4m3."""
    if w.dtype == torch.int32:
        return 1
    if w.dtype in (torch.float8_e4m3fn, torch.uint8):
        return 2
    return 0


def paired_int4(w):
    """INT4 expert weights in the nibble order the grouped GEMM reads (pair-interleaved).  Model
    loaders repack once at load; a tensor that still has the checkpoint order is repacked here
    and the copy is kept on it."""
    if w.dtype != torch.int32 or getattr(w, "_pg_nibbles", None) == "paired":
        return w
    cp = getattr(w, "_pg_paired_copy", None)
    if cp is None:
        cp = repack_int4_pairs(w)
        w._pg_paired_copy = cp
    return cp


def repack_int4_pairs(packed):
    """Load-time repack of compressed-tensors INT4 words (int32, eight nibbles each) into the pair-interleaved nibble
    order of the grouped GEMM, on the device."""
    assert packed.dtype == torch.int32 and packed.is_cuda
    src = packed.contiguous()
    out = torch.empty_like(src)
    _check(lib().pg_repack_int4_pairs(_ptr(src), _ptr(out), _ll(src.numel()), _stream()), ctx(src.device))
    out._pg_nibbles = "paired"
    return out


def grouped_gemm(xs, offsets, w, scales=None, bn: int = 16):
    """``xs`` [rows, K] sorted by expert; ``w`` bf16 [E, M, K], packed int32 [E, M, K/8] with bf16
    scales [E, M, K/32], or FP8 e4m3 [E, M, K] with f32 ``scale_inv`` [E, ceil(M/128), ceil(K/128)]."""
    rows, k = xs.shape
    e, m = w.shape[0], w.shape[1]
    mode = quant_code(w)
    assert (mode == 0) == (scales is None), "quantised expert weights need their scales"
    if mode == 1:
        w = paired_int4(w)
    if mode == 2:
        assert scales.dtype == torch.float32 and scales.shape == (e, (m + 127) // 128, (k + 127) // 128), "FP8 experts need f32 scale_inv per 128x128 block"
    y = torch.empty((rows, m), dtype=torch.bfloat16, device=xs.device)
    c = ctx(xs.device)
    rc = lib().pg_moe_grouped_gemm(_ptr(xs), _ll(xs.stride(0)), _ll(rows), _ptr(w), _ptr(scales), _ci(mode), _ptr(y), _ll(y.stride(0)), _ptr(offsets), _ci(e), _ci(m),
                                   _ci(k), _ci(bn), _ptr(c.status), _stream())
    _check(rc, c)
    return y


_MOE_FP8_TC = os.environ.get("PEGAINFER_MOE_FP8_TC", "1") != "0"  # FP8 experts on the FP8 tensor-core path (activations quantised per token group)


def grouped_gemm_fp8(xq, x_scale, offsets, w_fp8, w_scale, bn: int = 16):
    """``xq`` e4m3 [rows, K] sorted by expert with ``x_scale`` [K / 128, ld] (``quant_fp8_1x128``), ``w_fp8`` e4m3 [E, M, K] with
    f32 ``w_scale`` [E, M / 128, K / 128]; bf16 [rows, M] on tcgen05 kind::f8f6f4."""
    rows, k = xq.shape
    e, m = w_fp8.shape[0], w_fp8.shape[1]
    assert w_fp8.is_contiguous() and w_scale.is_contiguous() and w_scale.dtype == torch.float32 and w_scale.shape == (e, m // 128, k // 128)
    y = torch.empty((rows, m), dtype=torch.bfloat16, device=xq.device)
    c = ctx(xq.device)
    rc = lib().pg_moe_grouped_gemm_fp8(_ptr(xq), _ll(rows), _ptr(x_scale), _ll(x_scale.stride(0)), _ptr(w_fp8), _ptr(w_scale), _ptr(y), _ll(m), _ptr(offsets), _ci(e), _ci(m),
                                       _ci(k), _ci(min(64, max(16, bn))), _ptr(c.status), _stream())
    _check(rc, c)
    return y


def _moe_pipeline(x, ids, weights, w13, s13, w2, s2, expert_offset, act: str = "swiglu"):
    _bf16(x)
    t, h = x.shape
    k = ids.shape[1]
    e_local = w13.shape[0]
    routes = t * k
    c = ctx(x.device)
    offsets, sorted_src, route_pos = moe_route_plan(ids, expert_offset, e_local)
    xs = torch.empty((routes, h), dtype=x.dtype, device=x.device)
    _check(lib().pg_moe_gather(_ptr(x), _ll(x.stride(0)), _ptr(sorted_src), _ptr(offsets), _ci(e_local), _ci(k), _ptr(xs), _ci(h), _ci(routes), _stream()), c)
    bn = _token_tile(routes, e_local)
    assert act == "swiglu" or quant_code(w13) == 0, "the situ activation is wired for bf16 expert weights"
    if quant_code(w13) == 2 and _MOE_FP8_TC and h % 128 == 0 and w13.shape[1] % 256 == 0 and w2.shape[1] % 128 == 0:
        # both GEMMs on the FP8 tensor-core path: activations quantised per row and 128-wide k group
        xq, xsc = quant_fp8_1x128(xs)
        aq, asc = swiglu_quant_fp8_1x128(grouped_gemm_fp8(xq, xsc, offsets, w13, s13, bn))
        y2 = grouped_gemm_fp8(aq, asc, offsets, w2, s2, bn)
    else:
        y1 = grouped_gemm(xs, offsets, w13, s13, bn)
        mid = situ(y1) if act == "situ" else swiglu(y1)
        y2 = grouped_gemm(mid, offsets, w2, s2, bn)
    out = torch.empty((t, h), dtype=torch.float32, device=x.device)
    _check(lib().pg_moe_combine(_ptr(y2), _ll(y2.stride(0)), _ptr(route_pos), _ptr(weights.contiguous()), _ci(t), _ci(k), _ptr(out), _ci(h), _ci(0), _stream()), c)
    return out


def moe_experts(x, ids, weights, w13, w2, expert_offset=0, act: str = "swiglu"):
    return _moe_pipeline(x, ids, weights, w13, None, w2, None, expert_offset, act)


def moe_experts_int4(x, ids, weights, w13_packed, w13_scale, w2_packed, w2_scale, expert_offset=0, group=32):
    assert group == 32, "the int4 grouped GEMM is built for group size 32"
    return _moe_pipeline(x, ids, weights, w13_packed, w13_scale, w2_packed, w2_scale, expert_offset)


def moe_experts_fp8(x, ids, weights, w13_fp8, w13_scale, w2_fp8, w2_scale, expert_offset=0, block=128):
    assert block == 128, "the FP8 grouped GEMM is built for 128x128 scale blocks"
    return _moe_pipeline(x, ids, weights, w13_fp8, w13_scale, w2_fp8, w2_scale, expert_offset)


# ----------------------------------------------------------------------------------
# multi-head latent attention
# ----------------------------------------------------------------------------------
def mla_append(kv_a, kv_norm_w, cos, sin, meta: AttnMeta, latent_layer, kv_lora, eps):
    _bf16(kv_a)
    assert kv_a.stride(-1) == 1 and latent_layer.is_contiguous()
    t = kv_a.shape[0]
    rope = kv_a.shape[1] - kv_lora
    c = ctx(kv_a.device)
    num_slots = latent_layer.shape[0] * latent_layer.shape[1]
    rc = lib().pg_mla_append(_ptr(kv_a), _ll(kv_a.stride(0)), _ptr(kv_norm_w), _ptr(cos), _ptr(sin), _ptr(meta.positions), _ptr(meta.slot_mapping), _ptr(latent_layer), _ci(t),
                             _ci(kv_lora), _ci(rope), _ci(cos.shape[0]), _ll(num_slots), _cf(eps), _ptr(c.status), _stream())
    _check(rc, c)


class _MlaQ:
    """Query after RoPE in the layout the absorbed attention wants."""

    def __init__(self, nope_hm, pe, tokens, heads, nope):
        self.nope_hm, self.pe, self.tokens, self.heads, self.nope = nope_hm, pe, tokens, heads, nope


def mla_rope_q(q, cos, sin, meta: AttnMeta, nope):
    _bf16(q)
    t, h, d = q.shape
    rope = d - nope
    q = q.contiguous()
    nope_hm = torch.empty((h, t, nope), dtype=q.dtype, device=q.device)
    pe = torch.empty((t, h, rope), dtype=q.dtype, device=q.device)
    c = ctx(q.device)
    _check(lib().pg_mla_q_prep(_ptr(q), _ptr(cos), _ptr(sin), _ptr(meta.positions), _ptr(nope_hm), _ptr(pe), _ci(t), _ci(h), _ci(nope), _ci(rope), _ci(cos.shape[0]), _stream()), c)
    return _MlaQ(nope_hm, pe, t, h, nope)


_HEAD_OFFSETS: dict = {}


def _head_offsets(heads: int, tokens: int, device):
    key = (heads, tokens, device.index)
    o = _HEAD_OFFSETS.get(key)
    if o is None:
        o = (torch.arange(heads + 1, dtype=torch.int32, device=device) * tokens).contiguous()
        if len(_HEAD_OFFSETS) < 512:
            _HEAD_OFFSETS[key] = o
    return o


def _mla_expanded_seqs(q: "_MlaQ", w_uk, w_uv, meta: AttnMeta, kv_lora) -> int:
    """How many leading sequences of the step take the expanded-form tcgen05 prefill: the prefill chunks (at least
    two rows each) in front of the step's single-row decodes, when they have the 128 + 64 / 128 head shape and are
    long enough for the tensor-core kernel to pay for expanding K and V; 0 when the step stays on the absorbed kernel."""
    if meta.decode_only or not _PREFILL_TC or _BATCH_INVARIANT or meta.h_q_indptr is None or meta.h_kv_lens is None:
        return 0
    if not (isinstance(w_uk, torch.Tensor) and isinstance(w_uv, torch.Tensor)) or w_uk.dtype != torch.bfloat16 or w_uv.dtype != torch.bfloat16:
        return 0
    if q.nope != 128 or q.pe.shape[-1] != 64 or w_uv.shape[1] != 128:
        return 0
    qi = meta.h_q_indptr
    n_pf = meta.num_seqs
    while n_pf > 0 and qi[n_pf] - qi[n_pf - 1] == 1:
        n_pf -= 1
    if n_pf == 0:
        return 0
    rows = [qi[b + 1] - qi[b] for b in range(n_pf)]
    if min(rows) < 2 or max(rows) < _PREFILL_TC_MIN_ROWS or max(meta.h_kv_lens[:n_pf]) < _PREFILL_TC_MIN_KV:
        return 0
    return n_pf


def _mla_expanded_ok(q: "_MlaQ", w_uk, w_uv, meta: AttnMeta, kv_lora) -> bool:
    return _mla_expanded_seqs(q, w_uk, w_uv, meta, kv_lora) > 0


def _mla_split_step(q: "_MlaQ", w_uk, w_uv, latent_layer, meta: AttnMeta, scale, kv_lora, n_pf: int):
    """A unified step: the leading prefill chunks through the expanded form, the single-row decodes behind them
    through the absorbed kernel, each on its own slice of the step."""
    from dataclasses import replace

    qi, kvl = meta.h_q_indptr, meta.h_kv_lens
    n, t, h = meta.num_seqs, q.tokens, q.heads
    t_pf, n_dec = qi[n_pf], n - n_pf
    vdim = w_uv.shape[1]
    out = torch.empty((t, h * vdim), dtype=torch.bfloat16, device=latent_layer.device)
    meta_pf = replace(meta, q_indptr=meta.q_indptr[: n_pf + 1], kv_lens=meta.kv_lens[:n_pf], block_table=meta.block_table[:n_pf], num_seqs=n_pf, num_tokens=t_pf,
                      max_q_len=max(qi[b + 1] - qi[b] for b in range(n_pf)), max_kv_len=max(kvl[:n_pf]), decode_only=False, h_q_indptr=list(qi[: n_pf + 1]), h_kv_lens=list(kvl[:n_pf]),
                      plan=None)
    q_pf = _MlaQ(q.nope_hm[:, :t_pf], q.pe[:t_pf], t_pf, h, q.nope)
    out[:t_pf] = _mla_prefill_expanded(q_pf, w_uk, w_uv, latent_layer, meta_pf, scale, kv_lora)
    meta_dec = replace(meta, q_indptr=(meta.q_indptr[n_pf : n + 1] - t_pf).contiguous(), kv_lens=meta.kv_lens[n_pf:n], block_table=meta.block_table[n_pf:n], num_seqs=n_dec,
                       num_tokens=n_dec, max_q_len=1, max_kv_len=max(kvl[n_pf:n]), decode_only=True, h_q_indptr=list(range(n_dec + 1)), h_kv_lens=list(kvl[n_pf:n]), plan=None)
    q_dec = _MlaQ(q.nope_hm[:, t_pf:].contiguous(), q.pe[t_pf:], n_dec, h, q.nope)
    out[t_pf:] = mla_attention(q_dec, w_uk, w_uv, latent_layer, meta_dec, scale, kv_lora)
    return out


def _mla_prefill_expanded(q: "_MlaQ", w_uk, w_uv, latent_layer, meta: AttnMeta, scale, kv_lora):
    """Prefill in the expanded form: the latent rows of every key of the step are gathered through the page table,
    K (nope part) and V are expanded per head with the two up-projection GEMMs, and attention runs on the tcgen05
    kernel with 128 + 64 query / key and 128 value columns per head (a quarter of the absorbed form's FLOPs).
    Reference: pegainfer-kernels/csrc/k3/k3_flash_mla_prefill.cu (gather / expand + dense FMHA)."""
    PREFILL_TC_CALLS["mla"] += 1
    t, h = q.tokens, q.heads
    dev = latent_layer.device
    c = ctx(dev)
    n = meta.num_seqs
    kvl = [int(x) for x in meta.h_kv_lens[:n]]
    kv_ind = [0]
    for x in kvl:
        kv_ind.append(kv_ind[-1] + x)
    total = kv_ind[-1]
    kv_indptr = torch.tensor(kv_ind, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
    width = latent_layer.shape[-1]
    page_size = latent_layer.shape[1]
    dense = torch.empty((total, width), dtype=torch.bfloat16, device=dev)
    _check(lib().pg_mla_gather_latent(_ptr(latent_layer), _ci(page_size), _ll(latent_layer.shape[0]), _ci(width), _ptr(meta.block_table), _ci(meta.block_table.stride(0)),
                                      _ptr(kv_indptr), _ci(n), _ci(total), _ptr(dense), _ptr(c.status), _stream()), c)
    nope, vdim = q.nope, w_uv.shape[1]
    c_lat = dense[:, :kv_lora]
    k_nope = linear(c_lat, w_uk.reshape(h * nope, kv_lora))   # [total, h * 128]
    v = linear(c_lat, w_uv.reshape(h * vdim, kv_lora))         # [total, h * 128]
    out = torch.empty((t, h * vdim), dtype=torch.bfloat16, device=dev)
    qi = meta.h_q_indptr
    q_tiles = sum((qi[b + 1] - qi[b] + 255) // 256 for b in range(n))
    assert q.nope_hm.stride(2) == 1 and q.nope_hm.stride(1) == nope and q.pe.is_contiguous()
    rc = lib().pg_mla_prefill_tc(_ptr(q.nope_hm), _ll(q.nope_hm.stride(0)), _ptr(q.pe), _ptr(k_nope), _ptr(dense), _ci(width), _ci(kv_lora), _ptr(v), _ptr(out), _ptr(meta.q_indptr), _ptr(kv_indptr),
                                 _ptr(meta.kv_lens), _ci(n), _ci(t), _ci(total), _ci(h), _ci(nope), _ci(q.pe.shape[-1]), _ci(vdim), _cf(scale), _ci(q_tiles), _ptr(c.status),
                                 _stream())
    _check(rc, c)
    return out


def mla_attention(q: "_MlaQ", w_uk, w_uv, latent_layer, meta: AttnMeta, scale, kv_lora):
    """``w_uk`` [H, nope, kv_lora], ``w_uv`` [H, v, kv_lora].  The absorb GEMM wants W_UK as
    an [out = kv_lora, in = nope] weight per head; that transposed copy is made once per
    layer and kept."""
    w_uk_t = getattr(w_uk, "_pg_transposed", None)  # lives and dies with the weight tensor
    if w_uk_t is None:
        w_uk_t = w_uk.transpose(1, 2).contiguous()
        w_uk._pg_transposed = w_uk_t
    t, h = q.tokens, q.heads
    dev = latent_layer.device
    c = ctx(dev)
    if t == 0:
        return torch.empty((0, h * w_uv.shape[1]), dtype=torch.bfloat16, device=dev)
    n_pf = _mla_expanded_seqs(q, w_uk, w_uv, meta, kv_lora)
    if n_pf == meta.num_seqs:
        return _mla_prefill_expanded(q, w_uk, w_uv, latent_layer, meta, scale, kv_lora)
    if n_pf > 0:
        return _mla_split_step(q, w_uk, w_uv, latent_layer, meta, scale, kv_lora, n_pf)
    offs = _head_offsets(h, t, dev)
    bn = _token_tile(h * t, h)
    q_abs = grouped_gemm(q.nope_hm.view(h * t, q.nope), offs, w_uk_t, None, bn)  # [H*T, kv_lora]
    rope = q.pe.shape[-1]
    page_size = latent_layer.shape[1]
    if meta.decode_only:
        unit_seq = meta.q_indptr  # one row per sequence: q_indptr[i] == i
    else:
        qi = meta.h_q_indptr if meta.h_q_indptr is not None else meta.q_indptr.tolist()
        seq_of = []
        for b in range(meta.num_seqs):
            seq_of.extend([b] * (qi[b + 1] - qi[b]))
        unit_seq = torch.tensor(seq_of, dtype=torch.int32, device=dev)
    groups = h // 16
    if meta.decode_only:
        splits = max(1, min(16, (4 * c.sms) // max(1, t * groups), (min(meta.max_kv_len, 4096) + 127) // 128))
    else:
        splits = 1
    need = t * h * splits * (kv_lora + 1) * 4
    if need > c.attn_part.numel():
        splits = 1
    part_o = c.attn_part
    part_lse = c.attn_part[t * h * splits * kv_lora * 4 :]
    lat_out = torch.empty((h * t, kv_lora), dtype=torch.bfloat16, device=dev)
    rc = lib().pg_mla_attention(_ptr(q_abs), _ptr(q.pe), _ptr(latent_layer), _ptr(lat_out), _ptr(meta.q_indptr), _ptr(meta.kv_lens), _ptr(meta.block_table),
                                _ci(meta.block_table.stride(0)), _ptr(unit_seq), _ci(meta.num_seqs), _ci(t), _ci(h), _ci(kv_lora), _ci(rope), _ci(page_size), _cf(scale),
                                _ci(splits), _ptr(part_o), _ptr(part_lse), _ptr(c.status), _stream())
    _check(rc, c, 2 if splits > 1 else 1)
    v_hm = grouped_gemm(lat_out, offs, w_uv, None, bn)  # [H*T, v]
    vdim = w_uv.shape[1]
    out = torch.empty((t, h * vdim), dtype=torch.bfloat16, device=dev)
    _check(lib().pg_permute_021(_ptr(v_hm), _ptr(out), _ci(h), _ci(t), _ci(vdim), _stream()), c)
    return out


# ---- block-scaled FP8 GEMM (csrc/gemm_fp8_sm100.cu) -------------------------------------------------
def quant_fp8_1x128(x):
    """bf16 ``[T, K]`` -> (e4m3 ``[T, K]``, f32 scales ``[K / 128, T padded to 64]``): one scale per token and 128-wide k group."""
    _bf16(x)
    assert x.stride(-1) == 1
    t, k = x.shape
    xq = torch.empty((t, k), dtype=torch.float8_e4m3fn, device=x.device)
    lds = (t + 63) // 64 * 64
    scale = torch.zeros((k // 128, lds), dtype=torch.float32, device=x.device)
    _check(lib().pg_quant_fp8_1x128(_ptr(x), _ll(x.stride(0)), _ci(t), _ci(k), _ptr(xq), _ll(k), _ptr(scale), _ll(lds), _stream()), ctx(x.device))
    return xq, scale


def swiglu_quant_fp8_1x128(gate_up):
    """SwiGLU of a fused ``[T, 2 K]`` buffer (gate half first) and the per-token, per-k-group e4m3 quantiser in one kernel;
    the same values as ``quant_fp8_1x128(swiglu(gate_up))``."""
    _bf16(gate_up)
    assert gate_up.stride(-1) == 1
    t, k2 = gate_up.shape
    k = k2 // 2
    xq = torch.empty((t, k), dtype=torch.float8_e4m3fn, device=gate_up.device)
    lds = (t + 63) // 64 * 64
    scale = torch.zeros((k // 128, lds), dtype=torch.float32, device=gate_up.device)
    _check(lib().pg_swiglu_quant_fp8_1x128(_ptr(gate_up), _ll(gate_up.stride(0)), _ci(t), _ci(k), _ptr(xq), _ll(k), _ptr(scale), _ll(lds), _stream()), ctx(gate_up.device))
    return xq, scale


_FP8_WS: dict = {}


def linear_fp8_block(x, wq, w_scale, xq=None, x_scale=None):
    """``x [T, K]`` bf16 (quantised here per token and k group, unless ``xq`` / ``x_scale`` are given) times the
    block-scaled e4m3 weight ``wq [M, K]`` with ``w_scale [M / 128, K / 128]``; bf16 ``[T, M]``."""
    if xq is None:
        xq, x_scale = quant_fp8_1x128(x)
    t, k = xq.shape
    m = wq.shape[0]
    assert wq.is_contiguous() and w_scale.is_contiguous() and w_scale.dtype == torch.float32 and w_scale.shape == (m // 128, k // 128)
    dev = xq.device
    c = ctx(dev)
    y = torch.empty((t, m), dtype=torch.bfloat16, device=dev)
    ws = _FP8_WS.get(dev.index)
    need = lib().pg_gemm_fp8_ws_bytes(_ci(min(t, 64)), _ci(m))  # split K only happens for one narrow token tile
    if ws is None or ws.numel() < need:
        ws = torch.empty(int(need), dtype=torch.uint8, device=dev)
        _FP8_WS[dev.index] = ws
    # one launch for any number of rows: token tiles of 64 are the grid's second dimension
    rc = lib().pg_gemm_fp8_block(_ptr(xq), _ll(k), _ptr(x_scale), _ll(x_scale.stride(0)), _ptr(wq), _ll(k), _ptr(w_scale), _ptr(y), _ll(m), _ci(t), _ci(m), _ci(k), _ptr(ws),
                                 _ll(ws.numel()), _ptr(c.status), _stream())
    _check(rc, c, 3)
    return y


# ---- sparse-attention indexer (csrc/dsa.cu) ---------------------------------------------------------
def dsa_index_append(k, norm_w, norm_b, cos, sin, meta: AttnMeta, index_layer, eps=1e-6):
    _bf16(k)
    assert k.stride(-1) == 1 and index_layer.is_contiguous() and norm_w.dtype == torch.float32 and norm_b.dtype == torch.float32
    t, d = k.shape
    c = ctx(k.device)
    num_slots = index_layer.shape[0] * index_layer.shape[1]
    rc = lib().pg_dsa_k_append(_ptr(k), _ll(k.stride(0)), _ptr(norm_w), _ptr(norm_b), _ptr(cos), _ptr(sin), _ptr(meta.positions), _ptr(meta.slot_mapping), _ptr(index_layer),
                               _ci(t), _ci(d), _ci(cos.shape[-1] * 2), _ci(cos.shape[0]), _ll(num_slots), _cf(eps), _ptr(c.status), _stream())
    _check(rc, c)


def dsa_rope_q(q, cos, sin, meta: AttnMeta):
    _bf16(q)
    q = q.contiguous()
    t, h, d = q.shape
    _check(lib().pg_dsa_q_rope(_ptr(q), _ptr(cos), _ptr(sin), _ptr(meta.positions), _ci(t), _ci(h), _ci(d), _ci(cos.shape[-1] * 2), _ci(cos.shape[0]), _stream()), ctx(q.device))
    return q


def _unit_seq(meta: AttnMeta, device):
    """Sequence index of every query row."""
    if meta.decode_only:
        return meta.q_indptr  # one row per sequence: q_indptr[i] == i
    cached = getattr(meta, "_pg_unit_seq", None)  # one upload per step, shared by the layers (and made before any capture)
    if cached is not None:
        return cached
    qi = meta.h_q_indptr if meta.h_q_indptr is not None else meta.q_indptr.tolist()
    seq_of = []
    for b in range(meta.num_seqs):
        seq_of.extend([b] * (qi[b + 1] - qi[b]))
    out = torch.tensor(seq_of, dtype=torch.int32).pin_memory().to(device, non_blocking=True) if torch.device(device).type == "cuda" else torch.tensor(seq_of, dtype=torch.int32)
    try:
        meta._pg_unit_seq = out
    except Exception:
        pass
    return out


def dsa_index_scores(q, w, index_layer, meta: AttnMeta):
    """``[T, width]`` f32 with ``width`` = the step's longest sequence rounded up to the 128-key tile."""
    _bf16(q)
    t, h, d = q.shape
    assert q.is_contiguous() and w.dtype == torch.float32 and w.is_contiguous() and index_layer.is_contiguous()
    dev = q.device
    c = ctx(dev)
    width = (max(meta.max_kv_len, 1) + 127) // 128 * 128
    scores = torch.empty((t, width), dtype=torch.float32, device=dev)
    rc = lib().pg_dsa_scores(_ptr(q), _ptr(w), _ptr(index_layer), _ptr(_unit_seq(meta, dev)), _ptr(meta.q_indptr), _ptr(meta.kv_lens), _ptr(meta.block_table),
                             _ci(meta.block_table.stride(0)), _ci(index_layer.shape[1]), _ll(index_layer.shape[0]), _ci(t), _ci(h), _ci(d), _ptr(scores), _ci(width),
                             _ptr(c.status), _stream())
    _check(rc, c)
    return scores


def dsa_topk(scores, k: int):
    """``[T, k]`` int32 positions in increasing order, ``-1`` padded; the number of live entries per row rides
    along as ``._pg_counts``."""
    t, width = scores.shape
    assert scores.is_contiguous() and scores.dtype == torch.float32
    k = min(k, width)
    out = torch.empty((t, k), dtype=torch.int32, device=scores.device)
    counts = torch.empty((t,), dtype=torch.int32, device=scores.device)
    _check(lib().pg_dsa_topk(_ptr(scores), _ci(t), _ci(width), _ci(k), _ptr(out), _ptr(counts), _stream()), ctx(scores.device))
    out._pg_counts = counts
    return out


def mla_attention_sparse(q: "_MlaQ", w_uk, w_uv, latent_layer, meta: AttnMeta, scale, kv_lora, select):
    """Latent attention over the selected keys only: the chosen latent rows of every query are copied into pages
    of a scratch cache (row ``t`` owns pages ``t * kp .. (t + 1) * kp``) and the dense kernel runs with every
    query as a sequence of its own.  Key order does not matter to attention, and the rotary phase is part of
    the cached key.  Long steps go through in slices so that the scratch stays under 1 GiB."""
    t, k = select.shape
    dev = latent_layer.device
    c = ctx(dev)
    ps, width = latent_layer.shape[1], latent_layer.shape[2]
    kp = (k + ps - 1) // ps
    counts = getattr(select, "_pg_counts", None)
    if counts is None:
        counts = (select >= 0).sum(1, dtype=torch.int32)
    unit = _unit_seq(meta, dev)
    per = max(1, min(t, (1 << 30) // (kp * ps * width * 2)))
    outs = []
    for r0 in range(0, t, per):
        n = min(per, t - r0)
        scratch = torch.empty((n * kp, ps, width), dtype=latent_layer.dtype, device=dev)
        rc = lib().pg_dsa_gather(_ptr(latent_layer), _ptr(select[r0:]), _ci(k), _ptr(unit[r0:]), _ptr(meta.block_table), _ci(meta.block_table.stride(0)), _ci(ps),
                                 _ll(latent_layer.shape[0]), _ci(width * 2), _ci(n), _ptr(scratch), _ci(kp * ps), _ptr(c.status), _stream())
        _check(rc, c)
        ar = torch.arange(n * kp + 1, dtype=torch.int32, device=dev)
        sub = AttnMeta(q_indptr=ar[: n + 1], kv_lens=counts[r0 : r0 + n], block_table=ar[: n * kp].view(n, kp), slot_mapping=None, positions=None, page_size=ps, num_seqs=n,
                       num_tokens=n, max_q_len=1, max_kv_len=k, decode_only=True)
        if n == t:
            subq = q
        else:
            subq = _MlaQ(q.nope_hm[:, r0 : r0 + n].contiguous(), q.pe[r0 : r0 + n], n, q.heads, q.nope)
        outs.append(mla_attention(subq, w_uk, w_uv, scratch, sub, scale, kv_lora))
    return outs[0] if len(outs) == 1 else torch.cat(outs)


def lora_delta_multi_(ys, x, As, Bs, scale, slots):
    """``lora_delta_`` for up to three projections that read the same ``x`` (q / k / v, gate / up): one shrink and one
    expand launch for all of them."""
    import ctypes

    _bf16(x)
    n = len(ys)
    assert 1 <= n <= 3 and x.stride(-1) == 1 and all(y.stride(-1) == 1 for y in ys) and all(a.is_contiguous() for a in As) and all(b.is_contiguous() for b in Bs)
    t, k = x.shape
    r = As[0].shape[1]
    tvec = torch.empty((n, t, r), dtype=torch.float32, device=x.device)
    vp = ctypes.c_void_p * n
    rc = lib().pg_lora_delta_multi(_ptr(x), _ll(x.stride(0)), _ci(n), vp(*[a.data_ptr() for a in As]), vp(*[b.data_ptr() for b in Bs]), vp(*[y.data_ptr() for y in ys]),
                                   (ctypes.c_longlong * n)(*[y.stride(0) for y in ys]), (ctypes.c_int * n)(*[y.shape[1] for y in ys]), _ptr(scale), _ptr(slots), _ci(t), _ci(k), _ci(r),
                                   _ci(As[0].shape[0]), _ptr(tvec), _stream())
    _check(rc, ctx(x.device), 2)
    return ys


def lora_delta_(y, x, A, B, scale, slots):
    """In place: ``y[t] += scale[s] * B[s] @ (A[s] @ x[t])`` with ``s = slots[t]`` (negative = skip)."""
    _bf16(x)
    assert x.stride(-1) == 1 and y.stride(-1) == 1 and A.is_contiguous() and B.is_contiguous()
    t, k = x.shape
    m = y.shape[1]
    c = ctx(x.device)
    tvec = torch.empty((t, A.shape[1]), dtype=torch.float32, device=x.device)  # A x per token, between the shrink and the expand kernel
    rc = lib().pg_lora_delta(_ptr(x), _ll(x.stride(0)), _ptr(A), _ptr(B), _ptr(scale), _ptr(slots), _ptr(y), _ll(y.stride(0)), _ci(t), _ci(k), _ci(m), _ci(A.shape[1]),
                             _ci(A.shape[0]), _ptr(tvec), _stream())
    _check(rc, c, 2)
    return y
