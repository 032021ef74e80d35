"""Expert parallelism with dispatch and combine inside our own kernels.

Per MoE layer: ``ep_dispatch`` stores every routed token row into the owner rank's
receive slab over NVLink and publishes the wanted local-expert ids; the owner sorts what
it received, runs the grouped tcgen05 GEMMs (W13, SwiGLU, W2) and the W2 epilogue
stores each output row straight back into the source rank's combine buffer;
``ep_combine`` sums a token's k rows in slot order.  No NCCL call on the path; the only
coupling between ranks is the pair of epoch flags per layer.

Every rank must run every MoE layer of every step (idle ranks run padding tokens), and
all ranks use the same token bucket per step so slab slots line up.

Reference decomposition this replaces: pegainfer-kimi-k2/src/runner/moe_deepep.rs:243-397
(router, DeepEP dispatch, Marlin W13, SwiGLU, Marlin W2, DeepEP combine).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from ..ops import cuda as K
from .ep import EPContext
from .symm import SymmetricBuffer

FLAG_WORDS = 32
MAX_SITES = 256
_vp, _ll, _ci, _ull = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_ulonglong


class FusedEP(EPContext):
    def __init__(self, rank: int, world: int, device, hidden: int, top_k: int, max_tokens: int, group=None, wait_s: float = 5.0):
        super().__init__(rank, world, group, comm="fused", tokens="dp")
        self.comm = "fused"
        import torch.distributed as dist

        self.device = torch.device(device)
        self.hidden, self.k = hidden, top_k
        self.max_tokens = max_tokens
        self.cap = max_tokens * top_k
        self.wait_ns = int(wait_s * 1e9)
        self.lib = _native.load()
        al = lambda n: (n + 255) // 256 * 256
        slab_b = al(world * self.cap * hidden * 2)
        ids_b = al(world * self.cap * 4)
        comb_b = al(self.cap * hidden * 2)
        flag_b = MAX_SITES * FLAG_WORDS * 4
        self._off_ids = slab_b
        self._off_comb = slab_b + ids_b
        self._off_flags = self._off_comb + comb_b
        self.buf = SymmetricBuffer(self._off_flags + flag_b, rank, world, self.device, group)
        self.slab_table = self.buf.sub_table(0)
        self.ids_table = self.buf.sub_table(self._off_ids)
        self.comb_table = self.buf.sub_table(self._off_comb)
        self.flag_table = self.buf.sub_table(self._off_flags)
        self.slab = self.buf.view(torch.bfloat16, (world * self.cap, hidden), 0)
        self.recv_ids = self.buf.view(torch.int32, (world * self.cap,), self._off_ids)
        self.recv_ids.fill_(-1)
        self.comb = self.buf.view(torch.bfloat16, (self.cap, hidden), self._off_comb)
        self.valid_tokens = None  # optional device int: live prefix of a padded bucket
        self._site = 0
        self.fused = self
        torch.cuda.synchronize(self.device)
        if world > 1:
            dist.barrier(group=group)

    def begin_step(self) -> None:
        self._site = 0

    def _flags(self, site: int) -> int:
        return self.buf.local_ptr + self._off_flags + site * FLAG_WORDS * 4

    def moe(self, x, ids, wts, experts, cfg):
        t, h = x.shape
        k = ids.shape[1]
        assert k == self.k and h == self.hidden
        if t > self.max_tokens:
            raise ValueError(f"fused EP buffers hold {self.max_tokens} tokens per rank, step has {t}")
        site = self._site
        self._site += 1
        if site >= MAX_SITES:
            raise RuntimeError("too many MoE layers for the EP flag table")
        key = "_packed" if "w13_packed" in experts else "_fp8" if "w13_fp8" in experts else ""
        w13, w2 = experts["w13" + key], experts["w2" + key]
        mode = K.quant_code(w13)
        if mode == 1:
            w13, w2 = K.paired_int4(w13), K.paired_int4(w2)
        s13 = experts.get("w13_scale")
        s2 = experts.get("w2_scale")
        e_local = w13.shape[0]
        c = K.ctx(x.device)
        st = _vp(torch.cuda.current_stream().cuda_stream)
        ids = ids.contiguous()
        vt = _vp(self.valid_tokens.data_ptr()) if self.valid_tokens is not None else _vp(0)
        rc = self.lib.pg_ep_dispatch(_vp(x.data_ptr()), _ll(x.stride(0)), _vp(ids.data_ptr()), _ci(t), vt, _ci(k), _ci(h), _ci(e_local), _ci(self.cap), self.slab_table,
                                     self.ids_table, self.flag_table, _ci(self.rank), _ci(self.world), _ci(site), _ull(self.wait_ns), st)
        K._check(rc, c)
        dev = x.device
        offsets = torch.empty(e_local + 1, dtype=torch.int32, device=dev)
        sorted_src = torch.empty(self.world * t * k, dtype=torch.int32, device=dev)
        rc = self.lib.pg_ep_align(_vp(self.recv_ids.data_ptr()), _ci(self.world), _ci(self.cap), _ci(t * k), _ci(e_local), _vp(offsets.data_ptr()), _vp(sorted_src.data_ptr()),
                                  _vp(self._flags(site)), _ull(self.wait_ns), _vp(c.status.data_ptr()), st)
        K._check(rc, c)
        # rows this rank can receive at most: every route of every rank of this step's bucket
        max_rows = self.world * t * k
        xs = torch.empty((max_rows, h), dtype=x.dtype, device=dev)
        rc = self.lib.pg_moe_gather(_vp(self.slab.data_ptr()), _ll(h), _vp(sorted_src.data_ptr()), _vp(offsets.data_ptr()), _ci(e_local), _ci(1), _vp(xs.data_ptr()), _ci(h),
                                    _ci(max_rows), st)
        K._check(rc, c)
        bn = K._token_tile(max_rows, e_local)
        if mode == 2 and K._MOE_FP8_TC and h % 128 == 0 and w13.shape[1] % 256 == 0:
            # FP8 experts: W13 on the FP8 tensor-core path (received rows quantised per row and k group); rows past the
            # live routes are whatever the buffer held, and their products are never read
            xq, xsc = K.quant_fp8_1x128(xs)
            y1 = K.grouped_gemm_fp8(xq, xsc, offsets, w13, s13, bn)
        else:
            y1 = K.grouped_gemm(xs, offsets, w13, s13, bn)
        m = w2.shape[1]
        kk = y1.shape[1] // 2
        fp8_w2 = mode == 2 and K._MOE_FP8_TC and kk % 128 == 0 and m % 128 == 0
        act = None if fp8_w2 else K.swiglu(y1)
        if fp8_w2:
            bn8 = 16 if bn <= 16 else 32 if bn <= 32 else 64
            # W2 on the FP8 tensor-core path as well (SwiGLU and the quantiser in one kernel), with the same
            # scatter-return epilogue
            aq, asc = K.swiglu_quant_fp8_1x128(y1)
            rc = self.lib.pg_moe_grouped_gemm_fp8_return(_vp(aq.data_ptr()), _ll(max_rows), _vp(asc.data_ptr()), _ll(asc.stride(0)), _vp(w2.data_ptr()), _vp(s2.data_ptr()), _ll(h),
                                                         _vp(offsets.data_ptr()), _ci(e_local), _ci(m), _ci(kk), _ci(bn8), _vp(c.status.data_ptr()), _vp(sorted_src.data_ptr()),
                                                         self.comb_table, self.flag_table, _ci(self.cap), _ci(self.rank), _ci(self.world), _ci(site), st)
        else:
            rc = self.lib.pg_moe_grouped_gemm_return(_vp(act.data_ptr()), _ll(act.stride(0)), _ll(max_rows), _vp(w2.data_ptr()), _vp(s2.data_ptr()) if s2 is not None else _vp(0),
                                                     _ci(mode), _ll(h), _vp(offsets.data_ptr()), _ci(e_local), _ci(m), _ci(kk), _ci(bn), _vp(c.status.data_ptr()),
                                                     _vp(sorted_src.data_ptr()), self.comb_table, self.flag_table, _ci(self.cap), _ci(self.rank), _ci(self.world), _ci(site), st)
        K._check(rc, c)
        out = torch.empty((t, h), dtype=torch.float32, device=dev)
        wts = wts.contiguous()
        rc = self.lib.pg_ep_combine(_vp(self.comb.data_ptr()), _vp(ids.data_ptr()), _vp(wts.data_ptr()), _ci(t), _ci(k), _vp(out.data_ptr()), _ci(h), vt, _vp(self._flags(site)),
                                    _ci(self.world), _ull(self.wait_ns), _vp(c.status.data_ptr()), st)
        K._check(rc, c)
        return out


def make_fused_ep(rank: int, world: int, device, mcfg, max_tokens: int, group=None, wait_s: float = 5.0) -> FusedEP:
    return FusedEP(rank, world, device, mcfg.hidden_size, mcfg.num_experts_per_tok, max_tokens, group, wait_s)
