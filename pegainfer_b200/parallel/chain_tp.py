"""Tensor parallelism for the decode chain: partial sums meet inside the NVSwitch.

``ChainTP`` owns one buffer per rank that is mapped on every rank AND bound to an NVSwitch
multicast object (allocated and exchanged through ``torch.distributed._symmetric_memory``:
the framework layer does the plumbing -- allocation, handle exchange, multicast binding).
The decode-chain kernel (``csrc/decode_chain.cu``) does the rest itself: each rank's
row-parallel phase leaves a bf16 partial ``[T, hidden]`` in that buffer, announces it with
release stores into the peers' flag words, and reads the sum over ranks with
``multimem.ld_reduce`` (the switch adds the eight copies, f32 accumulation), then finishes
residual + RMSNorm on its own replicated residual.  No NCCL call sits on the decode path.

Steps with more than 64 rows (prompt chunks) use GEMM + ``ncclAllReduce`` + add/RMSNorm, the
reference's decomposition (pegainfer-qwen3/src/batch_decode.rs:320-347,378-396).

Teardown: ``close()`` must run on every rank, after a barrier, before any rank exits -- a
process that dies while its memory is bound to a multicast object can fault the peers.
"""
from __future__ import annotations

import ctypes

import torch

from .tp import TPContext

_vp, _ci, _ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong
MAX_ROWS = 64


class _ChainTpSpec(ctypes.Structure):
    _fields_ = [("world", _ci), ("rank", _ci), ("y_local", _vp * 2), ("y_mc", _vp * 2), ("flags_peer", _vp * 8), ("wait_ns", _ull), ("y_peer", (_vp * 2) * 8), ("use_multimem", _ci)]


class ChainTP(TPContext):
    def __init__(self, rank: int, world: int, device, hidden: int, group=None, wait_s: float = 5.0):
        super().__init__(rank, world, group, comm="chain")
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        self.device = torch.device(device)
        self.hidden = hidden
        grp = group if group is not None else dist.group.WORLD
        y_bytes = (MAX_ROWS * hidden * 2 + 255) // 256 * 256
        self._off_flags = 2 * y_bytes
        nbytes = self._off_flags + 8192  # 8 x 160 arrival words (source rank x CTA) and the exchange counter
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm_mem.rendezvous(self.buf, grp)
        if not self.handle.multicast_ptr:
            raise RuntimeError("this system exposes no NVSwitch multicast mapping; use --comm nccl")
        spec = _ChainTpSpec()
        spec.world, spec.rank, spec.wait_ns = world, rank, int(wait_s * 1e9)
        for i in range(2):
            spec.y_local[i] = self.handle.buffer_ptrs[rank] + i * y_bytes
            spec.y_mc[i] = self.handle.multicast_ptr + i * y_bytes
        import os

        # how the partial sums meet: "pull" = every rank reads every rank's copy with plain peer loads and adds in
        # rank order; "multimem" = multimem.ld_reduce, the NVSwitch adds the copies
        self.mode = os.environ.get("PEGAINFER_CHAIN_TP", "pull")
        spec.use_multimem = int(self.mode == "multimem")
        for q in range(world):
            spec.flags_peer[q] = self.handle.buffer_ptrs[q] + self._off_flags
            for i in range(2):
                spec.y_peer[q][i] = self.handle.buffer_ptrs[q] + i * y_bytes
        self.spec = spec
        self.sites_by_rows: dict = {}
        dist.barrier(group=grp)
        torch.cuda.synchronize(self.device)

    def describe(self, rows: int) -> dict:
        """Collective path of a step with ``rows`` token rows: up to 64 rows run the chain kernel with
        the in-switch reduction (two exchanges per layer), larger steps the library all-reduce."""
        keys = sorted(k for k in self.sites_by_rows if k >= rows) or sorted(self.sites_by_rows)
        fused, libs = self.sites_by_rows[keys[0]] if keys else (0, 0)
        path = f"fused-{self.mode}" if fused and not libs else "nccl" if libs and not fused else "fused+nccl" if fused else "none"
        return {"path": path, "fused_sites_per_step": fused, "library_sites_per_step": libs}

    def close(self) -> None:
        """Drop the multicast-bound buffer.  Call on every rank after a barrier, before exit."""
        self.spec = None
        self.handle = None
        self.buf = None
