"""Op entry points used by every model.

CUDA tensors run the hand-written sm_100a kernels (``ops.cuda``); CPU tensors run the
PyTorch restatement (``ops.reference``).  ``set_mode("library")`` sends CUDA tensors
through PyTorch/cuBLAS instead: that is the comparison arm (the reference's
GEMM -> collective -> norm decomposition on vendor libraries), never a silent
fallback: with mode ``sm100`` a missing extension raises.
"""
from __future__ import annotations

import contextlib

from . import reference
from .reference import AttnMeta  # noqa: F401

_MODE = "sm100"  # sm100 | cublas | library


def set_mode(mode: str) -> None:
    """``sm100``: every op is a kernel of this repository.  ``cublas``: dense projections go
    through ``torch.nn.functional.linear`` (cuBLAS) and everything else stays on this
    repository's kernels; with NCCL all-reduce this is the library build of the GEMM ->
    collective -> norm decomposition, and it can be captured in CUDA graphs.  ``library``:
    every op is its PyTorch restatement (the oracle; host-synchronising, not capturable)."""
    global _MODE
    if mode not in ("sm100", "cublas", "library"):
        raise ValueError("mode must be 'sm100', 'cublas' or 'library'")
    _MODE = mode


def get_mode() -> str:
    return _MODE


@contextlib.contextmanager
def mode(m: str):
    prev = _MODE
    set_mode(m)
    try:
        yield
    finally:
        set_mode(prev)


def _impl(t):
    if t.is_cuda and _MODE != "library":
        from . import cuda

        return cuda
    return reference


def embedding(ids, table):
    return _impl(table).embedding(ids, table)


def rms_norm(x, w, eps, offset=False):
    return _impl(x).rms_norm(x, w, eps, offset)


def add_rms_norm(x, residual, w, eps, offset=False, round_before_norm=True):
    return _impl(x).add_rms_norm(x, residual, w, eps, offset, round_before_norm)


def gated_rms_norm(x, gate, w, eps, act="silu"):
    if act != "silu":
        return _impl(x).gated_rms_norm(x, gate, w, eps, act)
    return _impl(x).gated_rms_norm(x, gate, w, eps)


def swiglu(gate_up, interleaved=False):
    return _impl(gate_up).swiglu(gate_up, interleaved)


class Fp8Weight:
    """A dense matrix kept as block-scaled FP8: ``q`` e4m3 ``[M, K]`` and one f32 scale per 128 x 128 block.
    ``linear`` quantises the activations per token and 128-wide k group and runs the FP8 tensor-core GEMM."""

    __slots__ = ("q", "scale")

    def __init__(self, q, scale):
        self.q, self.scale = q.contiguous(), scale.float().contiguous()

    @property
    def shape(self):
        return self.q.shape

    def numel(self):
        return self.q.numel()

    @staticmethod
    def cat(parts):
        """Stack matrices by rows (each part's rows a multiple of 128, so its scale rows stack too)."""
        import torch

        return Fp8Weight(torch.cat([p.q for p in parts], 0), torch.cat([p.scale for p in parts], 0))


def linear(x, w, out_dtype=None):
    if isinstance(w, Fp8Weight):
        y = _impl(x).linear_fp8_block(x, w.q, w.scale)
        return y if out_dtype is None or y.dtype == out_dtype else y.to(out_dtype)
    if _MODE == "cublas" and x.is_cuda:
        import torch

        y = torch.nn.functional.linear(x, w)
        return y if out_dtype is None or y.dtype == out_dtype else y.to(out_dtype)
    return _impl(x).linear(x, w, out_dtype)


def gather_rows(x, idx):
    return _impl(x).gather_rows(x, idx)


def qk_norm_rope_append(qkv, q_norm_w, k_norm_w, cos, sin, meta, kv_layer, num_q_heads, num_kv_heads, head_dim, eps, offset=False, gated=False, v_norm=False):
    if v_norm:
        return _impl(qkv).qk_norm_rope_append(qkv, q_norm_w, k_norm_w, cos, sin, meta, kv_layer, num_q_heads, num_kv_heads, head_dim, eps, offset, gated, True)
    return _impl(qkv).qk_norm_rope_append(qkv, q_norm_w, k_norm_w, cos, sin, meta, kv_layer, num_q_heads, num_kv_heads, head_dim, eps, offset, gated)


def paged_attention(q, kv_layer, meta, scale=None, window=0):
    return _impl(q).paged_attention(q, kv_layer, meta, scale, window)


def argmax(logits):
    return _impl(logits).argmax(logits)


def sample(logits, temperature, top_k, top_p, min_p, u):
    return _impl(logits).sample(logits, temperature, top_k, top_p, min_p, u)


def logprobs_topk(logits, picked, k):
    return _impl(logits).logprobs_topk(logits, picked, k)


# Load-time and test helpers that are plain tensor arithmetic on whatever device their inputs
# live on (quantisers, repackers, RoPE tables, the dense-attention oracle): these have no kernel.
_HOST_UTILS = frozenset(
    ("rope_tables", "dense_causal_attention", "filtered_probs", "dequant_int4_g32", "quant_int4_g32", "repack_int4_pairs", "unrepack_int4_pairs", "plain_int4", "dequant_fp8_block", "quant_fp8_block", "dequant_mxfp4", "quant_mxfp4")
)


def __getattr__(name):
    # ops added by later model families (MLA, MoE, GDN) resolve lazily
    if hasattr(reference, name):
        def _dispatch(*args, **kwargs):
            import torch

            first = next((a for a in args if isinstance(a, torch.Tensor)), None)
            impl = _impl(first) if first is not None else reference
            fn = getattr(impl, name, None)
            if fn is None:
                if name not in _HOST_UTILS:
                    raise NotImplementedError(f"ops.{name}: no sm_100a kernel for this op; refusing to run the PyTorch restatement on a CUDA tensor (use ops.mode('library') for the comparison arm)")
                fn = getattr(reference, name)
            return fn(*args, **kwargs)

        return _dispatch
    raise AttributeError(name)
