"""Tensor-parallel context: who am I, and how partial sums are combined.

Two arms share one interface.  ``comm="nccl"`` is the library arm: a row-parallel
projection is a local GEMM, ``ncclAllReduce`` through ``torch.distributed``, then a
separate residual-add + RMSNorm kernel (the reference's decomposition,
pegainfer-qwen3/src/batch_decode.rs:320-347, weights.rs:616-644).  ``comm="fused"``
routes the same call to the peer-memory kernels in ``parallel.fused`` where the GEMM
partials are reduce-scattered, normalised and all-gathered inside hand-written
kernels over NVLink peer pointers.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


class TPContext:
    def __init__(self, rank: int = 0, world: int = 1, group=None, comm: str = "nccl", fused=None):
        self.rank = rank
        self.world = world
        self.group = group
        self.comm = comm if world > 1 else "none"
        self.fused = fused  # parallel.fused.FusedTP when comm == "fused"

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(x, group=self.group)
        return x

    def row_linear_add_norm(self, a, w, residual, norm_w, eps, offset=False):
        """``residual += all_reduce(a @ w.T)``; returns ``rms_norm(residual)``."""
        if self.comm == "fused" and a.is_cuda:
            return self.fused.row_linear_add_norm(a, w, residual, norm_w, eps, offset)
        y = ops.linear(a, w)
        y = self.all_reduce(y)
        return ops.add_rms_norm(y, residual, norm_w, eps, offset)

    def begin_step(self) -> None:
        """Called at the start of every forward pass (fused mode numbers its sites)."""

    def describe(self, rows: int) -> dict:
        """Which collective path a step of ``rows`` token rows takes on this context."""
        return {"path": "none" if self.world == 1 else "nccl", "fused_sites_per_step": 0, "library_sites_per_step": 0}

    def close(self) -> None:
        """Release communication buffers (nothing to release for the library arm)."""

    def col_linear(self, x, w, out_dtype=None):
        """Column-parallel projection of (possibly just all-gathered) activations."""
        return ops.linear(x, w, out_dtype)

    def sync(self) -> None:
        """Gathered activations become readable by kernels that do not wait on flags."""

    def row_linear(self, a, w):
        """``all_reduce(a @ w.T)`` without the norm tail (last layer, MoE shared path)."""
        return self.all_reduce(ops.linear(a, w))


SINGLE = TPContext()
