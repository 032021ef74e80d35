"""Tensor parallelism with the collective fused into the GEMM kernels.

A row-parallel projection (o_proj, down_proj) runs as ONE kernel launch per rank:
the epilogue of every tcgen05 GEMM tile pushes its f32 partial straight into the receive
buffer of the rank that owns those token rows (posted NVLink stores, so the transfer of
a tile overlaps the MMAs of the tiles still being computed); once every rank has
signalled its tiles (epoch flags), each rank sums the partials of its rows from local
memory in fixed rank order (reduce-scatter), adds the residual, applies RMSNorm and
stores the normalised rows into every rank's activation buffer (all-gather).  With few
rows (decode) every rank receives all partials and reduces all rows itself: one hop.  The following column-parallel GEMM (qkv, gate_up) streams its first
weight tiles while those rows travel and only then waits on the delivery flags, so the
gather overlaps the GEMM's ramp-up.  Flags are monotonic epochs kept in device memory,
so captured CUDA graphs replay without any reset.

Reference decomposition this replaces: GEMM, ncclAllReduce, fused_add_rms_norm
(pegainfer-qwen3/src/batch_decode.rs:320-347,378-396; weights.rs:616-644).
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _native
from ..ops import cuda as K
from .symm import SymmetricBuffer
from .tp import TPContext

FLAG_WORDS_PER_SITE = 32
MAX_SITES = 1024
_vp, _ll, _ci, _cf, _ull = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float, ctypes.c_ulonglong


class FusedTP(TPContext):
    def __init__(self, rank: int, world: int, device, hidden: int, max_tokens: int, group=None, wait_s: float = 5.0, fused_max_rows: int = 256, site_max_world: int = 4):
        super().__init__(rank, world, group, comm="fused")
        # Steps with more token rows than this (prefill chunks) take the library all-reduce:
        # measured at 1024 rows on 2 GPUs the fused site is ~30 us slower than GEMM + NCCL +
        # norm, while up to a few hundred rows (decode) it is at parity or ahead.
        self.fused_max_rows = int(os.environ.get("PEGAINFER_TP_FUSED_MAX_ROWS", fused_max_rows))
        # This class is the PER-SITE fused kernel (GEMM + peer-store reduce-scatter + norm + all-gather), which the
        # models that do not run on the decode-chain kernel use (the chain kernel carries its own cross-GPU reduction,
        # peer pull or multimem, at every world size).  Measured at 64 rows the site kernel is within 1-2 % of GEMM +
        # NCCL + norm on 2 and 4 GPUs but 27 % behind on 8, where NCCL reduces inside the switch and the two-hop
        # peer-store protocol pays the skew of eight ranks twice: above `site_max_world` ranks a site takes the
        # library all-reduce.
        self.fused_max_world = int(site_max_world)
        import torch.distributed as dist

        self.device = torch.device(device)
        self.hidden = hidden
        self.max_tokens = max_tokens
        self.wait_ns = int(wait_s * 1e9)
        self.lib = _native.load()
        self.one_shot_rows = 256  # one-shot all-reduce while tokens * world stays below this
        # receive buffer [source rank][rows][hidden] f32, double buffered by site parity: a fast
        # rank may already push the next site's tiles while this rank still reduces the current one
        self._part_elems = max(self.one_shot_rows, max_tokens + world) * hidden
        part_b = 2 * self._part_elems * 4
        x_b = max_tokens * hidden * 2
        flag_b = MAX_SITES * FLAG_WORDS_PER_SITE * 4
        self._off_x = (part_b + 255) // 256 * 256
        self._off_f = self._off_x + (x_b + 255) // 256 * 256
        self.buf = SymmetricBuffer(self._off_f + flag_b, rank, world, self.device, group)
        self.part_table = self.buf.sub_table(0)
        self.x_table = self.buf.sub_table(self._off_x)
        self.flag_table = self.buf.sub_table(self._off_f)
        self.x = self.buf.view(torch.bfloat16, (max_tokens, hidden), self._off_x)
        self.flags = self.buf.view(torch.int32, (MAX_SITES, FLAG_WORDS_PER_SITE), self._off_f)
        self._site = 0
        self._pending_site = -1
        self._lib_sites = 0
        self._rows = 0
        self.sites_by_rows: dict = {}  # token rows of a step -> (fused sites, library all-reduce sites) of its last forward
        self.fused = self
        if world > 1:
            dist.barrier(group=group)
        torch.cuda.synchronize(self.device)

    def begin_step(self) -> None:
        if self._site & 1:
            raise RuntimeError("fused TP needs an even number of row-parallel projections per step (partial buffers alternate)")
        self._site = 0
        self._pending_site = -1
        self._lib_sites = 0

    def describe(self, rows: int) -> dict:
        """What the last forward pass of a step with ``rows`` token rows (or the next larger one
        seen) actually ran: the fused kernels, the library all-reduce, or both."""
        keys = sorted(k for k in self.sites_by_rows if k >= rows) or sorted(self.sites_by_rows)
        fused, libs = self.sites_by_rows[keys[0]] if keys else (0, 0)
        path = "fused" if fused and not libs else "nccl" if libs and not fused else "fused+nccl" if fused else "none"
        return {"path": path, "fused_sites_per_step": fused, "library_sites_per_step": libs}

    def close(self) -> None:
        """Unmap the peers' buffers and free the local one.  Every rank must be past its last
        kernel that touches them (callers put a barrier in front)."""
        if self.buf is not None:
            self.x = self.flags = None
            self.buf.close()
            self.buf = None

    def _flag_ptr(self, site: int) -> int:
        return self.buf.local_ptr + self._off_f + site * FLAG_WORDS_PER_SITE * 4

    def row_linear_add_norm(self, a, w, residual, norm_w, eps, offset=False):
        t, k = a.shape
        if t > self.fused_max_rows or self.world > self.fused_max_world:
            import torch.distributed as dist

            from .. import ops

            self._lib_sites += 1
            self._rows = t
            y = K.linear(a, w)
            dist.all_reduce(y, group=self.group)
            return ops.add_rms_norm(y, residual, norm_w, eps, offset)
        if t > self.max_tokens:
            raise ValueError(f"fused TP buffers hold {self.max_tokens} tokens, step has {t}")
        if a.stride(-1) != 1:
            a = a.contiguous()
        site = self._site
        self._site += 1
        self._rows = t
        if self._site >= MAX_SITES:
            raise RuntimeError("too many fused collective sites in one step")
        one_shot = t * self.world <= self.one_shot_rows
        part_offset = (site & 1) * self._part_elems
        c = K.ctx(a.device)
        rc = self.lib.pg_tp_gemm_rs_norm_ag(
            _vp(a.data_ptr()), _vp(w.data_ptr()), _ci(t), _ci(self.hidden), _ci(k), _ll(a.stride(0)), _ll(w.stride(0)), self.part_table, self.x_table,
            self.flag_table, _ci(self.rank), _ci(self.world), _ci(site), _vp(residual.data_ptr()), _ll(residual.stride(0)), _vp(norm_w.data_ptr()),
            _cf(eps), _ci(int(offset)), _ci(int(one_shot)), _ll(part_offset), _ull(self.wait_ns), _vp(c.gemm_ws.data_ptr()), _ll(c.gemm_ws.numel()), _vp(c.gemm_counters.data_ptr()),
            _ll(c.gemm_counters.numel() * 4), _vp(c.status.data_ptr()), _vp(torch.cuda.current_stream().cuda_stream),
        )
        K._check(rc, c)
        self._pending_site = -1 if one_shot else site  # one-shot rows are local: stream order is enough
        return self.x[:t]

    def col_linear(self, x, w, out_dtype=None):
        if self._pending_site < 0 or x.data_ptr() != self.x.data_ptr():
            return K.linear(x, w, out_dtype)
        site, self._pending_site = self._pending_site, -1
        t, k = x.shape
        m = w.shape[0]
        f32 = out_dtype == torch.float32
        out = torch.empty((t, m), dtype=torch.float32 if f32 else torch.bfloat16, device=x.device)
        c = K.ctx(x.device)
        rc = self.lib.pg_gemm_bf16_tn_after_gather(
            _vp(x.data_ptr()), _vp(w.data_ptr()), _vp(out.data_ptr()), _ci(int(f32)), _ci(t), _ci(m), _ci(k), _ll(x.stride(0)), _ll(w.stride(0)),
            _ll(out.stride(0)), _vp(c.gemm_ws.data_ptr()), _ll(c.gemm_ws.numel()), _vp(c.gemm_counters.data_ptr()), _ll(c.gemm_counters.numel() * 4),
            _vp(c.status.data_ptr()), _vp(self._flag_ptr(site)), _ci(self.world), _ull(self.wait_ns), _vp(torch.cuda.current_stream().cuda_stream),
        )
        K._check(rc, c)
        return out

    def sync(self) -> None:
        """Make the last gathered rows safe to read by kernels that do not wait themselves."""
        if self._rows:
            self.sites_by_rows[self._rows] = (self._site, self._lib_sites)
        if self._pending_site < 0:
            return
        site, self._pending_site = self._pending_site, -1
        c = K.ctx(self.device)
        rc = self.lib.pg_tp_wait(_vp(self._flag_ptr(site)), _ci(self.world), _ull(self.wait_ns), _vp(c.status.data_ptr()), _vp(torch.cuda.current_stream().cuda_stream))
        K._check(rc, c)


def make_fused_tp(rank: int, world: int, device, mcfg, max_tokens: int, group=None, wait_s: float = 5.0, site_max_world: int = 4) -> FusedTP:
    return FusedTP(rank, world, device, mcfg.hidden_size, max_tokens, group, wait_s, site_max_world=site_max_world)
