"""Expert parallelism: routed experts live on their owner rank, tokens travel.

``EPContext.moe`` returns the routed-expert output for this rank's tokens.

* world 1: all experts are local.
* ``comm="nccl"`` (library arm): tokens, ids and weights are all-gathered, every rank
  runs its local experts over all tokens, and the f32 outputs are reduce-scattered
  back (``tokens="dp"``: every rank holds different tokens) or all-reduced
  (``tokens="replicated"``) through ``torch.distributed``.
* ``comm="fused"``: the peer-memory dispatch / grouped-GEMM / combine kernels in
  ``parallel.fused_ep``.

Reference decomposition: DeepEP dispatch -> Marlin W13 -> SwiGLU -> Marlin W2 -> DeepEP
combine (pegainfer-kimi-k2/src/runner/moe_deepep.rs:243-397) and the NCCL pair
all-reduce backend (pegainfer-deepseek-v2-lite/src/nccl_backend.rs:838-1060).
"""
from __future__ import annotations

import torch

from .. import ops


def _local_experts(x, ids, wts, experts, cfg):
    if "w13_fp8" in experts:
        return ops.moe_experts_fp8(x, ids, wts, experts["w13_fp8"], experts["w13_scale"], experts["w2_fp8"], experts["w2_scale"], experts["offset"])
    if "w13_packed" in experts:
        return ops.moe_experts_int4(x, ids, wts, experts["w13_packed"], experts["w13_scale"], experts["w2_packed"], experts["w2_scale"], experts["offset"], cfg.quant_group_size)
    if getattr(cfg, "hidden_act", "silu") == "situ":
        return ops.moe_experts(x, ids, wts, experts["w13"], experts["w2"], experts["offset"], act="situ")
    return ops.moe_experts(x, ids, wts, experts["w13"], experts["w2"], experts["offset"])


class EPContext:
    def __init__(self, rank: int = 0, world: int = 1, group=None, comm: str = "nccl", tokens: str = "dp", fused=None):
        self.rank, self.world, self.group = rank, world, group
        self.comm = comm if world > 1 else "none"
        self.tokens = tokens
        self.fused = fused

    def begin_step(self) -> None:
        """Start of a forward pass (the fused path numbers its MoE layers)."""

    def moe(self, x, ids, wts, experts, cfg):
        if self.world == 1 and self.comm != "fused":
            return _local_experts(x, ids, wts, experts, cfg)
        if self.comm == "fused" and x.is_cuda:
            return self.fused.moe(x, ids, wts, experts, cfg)
        import torch.distributed as dist

        if self.tokens == "replicated":
            y = _local_experts(x, ids, wts, experts, cfg).float()
            dist.all_reduce(y, group=self.group)
            return y
        t = x.shape[0]
        xs = torch.empty((self.world * t, x.shape[1]), dtype=x.dtype, device=x.device)
        idg = torch.empty((self.world * t, ids.shape[1]), dtype=ids.dtype, device=x.device)
        wg = torch.empty((self.world * t, wts.shape[1]), dtype=wts.dtype, device=x.device)
        dist.all_gather_into_tensor(xs, x.contiguous(), group=self.group)
        dist.all_gather_into_tensor(idg, ids.contiguous(), group=self.group)
        dist.all_gather_into_tensor(wg, wts.contiguous(), group=self.group)
        y = _local_experts(xs, idg, wg, experts, cfg).float()
        if dist.get_backend(self.group) == "gloo":  # no reduce-scatter on gloo (CPU runs): all-reduce, keep this rank's rows
            dist.all_reduce(y, group=self.group)
            return y[self.rank * t : (self.rank + 1) * t].contiguous()
        out = torch.empty((t, x.shape[1]), dtype=torch.float32, device=x.device)
        dist.reduce_scatter_tensor(out, y, group=self.group)
        return out


LOCAL_EP = EPContext()
