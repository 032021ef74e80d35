"""CUDA-graph decode: one captured graph per batch bucket.

Inputs live in pointer-stable device buffers that are refreshed from pinned host
mirrors before each replay; rows beyond the live batch are padding rows that point at
page 0 with ``kv_len == 0`` so they attend to nothing and their KV write lands in the
reserved padding page.  The greedy variant captures the argmax too, so a replay
yields token ids directly.  ``dump_dot`` writes the captured graph as Graphviz text.

Reference parity: pegainfer-core/src/cuda_graph.rs:42-234 (capture / replay state),
pegainfer-qwen3/src/batch_decode.rs:99-167 (bucket padding, graph per bucket and
attention path), pegainfer-core/src/cuda_graph/dump.rs:24-135 (DOT export).
"""
from __future__ import annotations

import os
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..ops.reference import AttnMeta


def _K():
    from ..ops import cuda

    return cuda


class DecodeGraphs:
    def __init__(self, executor, max_batch: int, max_blocks_per_seq: int):
        from ..sched.executor import DECODE_BUCKETS, bucket_for

        self.ex = executor
        self.device = executor.device
        self.buckets = [b for b in DECODE_BUCKETS if b <= max(bucket_for(max_batch), 1)]
        self.max_b = self.buckets[-1]
        self.width = max(max_blocks_per_seq, 1)
        self.page_size = executor.page_size
        B, W, dev = self.max_b, self.width, self.device
        # one int32 arena: tokens | positions | slots | kv_lens, mirrored in pinned memory
        self.h_small = torch.zeros(4 * B, dtype=torch.int32).pin_memory()
        self.d_small = torch.zeros(4 * B, dtype=torch.int32, device=dev)
        self.h_table = torch.zeros((B, W), dtype=torch.int32).pin_memory()
        self.d_table = torch.zeros((B, W), dtype=torch.int32, device=dev)
        self.np_small = self.h_small.numpy()
        self.np_table = self.h_table.numpy()
        self.q_indptr = torch.arange(B + 1, dtype=torch.int32, device=dev)
        self.out_tokens = torch.zeros(B, dtype=torch.int32, device=dev)
        self.h_slots = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.d_slots = torch.zeros(B, dtype=torch.int32, device=dev)
        self.uses_state = hasattr(executor.model, "rec")
        self.h_out = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.graphs: dict = {}
        self.logits: dict = {}
        self.pool = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.replays = 0
        self.kernels_per_graph: dict = {}
        self.invalidate_table()

    def invalidate_table(self) -> None:
        """Forget what ``stage`` knows about the block-table mirror (call after writing it directly)."""
        self._row_state = [(-1, 0)] * self.max_b
        self._table_b = 0
        self._table_w = 0

    # views of the arena for a bucket
    def _views(self, b: int):
        B = self.max_b
        s = self.d_small
        return s[0:b], s[B : B + b], s[2 * B : 2 * B + b], s[3 * B : 3 * B + b]

    def _meta(self, b: int, splits: int) -> AttnMeta:
        tok, pos, slot, kvl = self._views(b)
        return AttnMeta(
            q_indptr=self.q_indptr[: b + 1],
            kv_lens=kvl,
            block_table=self.d_table[:b],
            slot_mapping=slot,
            positions=pos,
            page_size=self.page_size,
            num_seqs=b,
            num_tokens=b,
            max_q_len=1,
            max_kv_len=self.width * self.page_size,
            decode_only=True,
            plan=splits,
            state_slots=self.d_slots[:b] if self.uses_state else None,
        )

    def _forward(self, b: int, greedy: bool, splits: int):
        tok = self._views(b)[0]
        meta = self._meta(b, splits)
        hidden = self.ex.model.forward_hidden(tok, meta, self.ex.kv)
        logits = self.ex.model.logits(hidden)
        if greedy:
            _K().argmax(logits, out=self.out_tokens[:b])
        return logits

    def _splits_for(self, b: int) -> int:
        geo = self.ex.model.kv_geometry()
        # fixed per bucket so the captured launch shape never changes; sized for ~2k context
        return _K().plan_decode_splits(b, geo["kv_heads"], min(self.width * self.page_size, 2048), self.device)

    def capture(self, b: int, greedy: bool):
        """Capture bucket ``b``.  The warm-up pass and the capture run on padding inputs
        (page 0, kv_len 0, state slot 0), so capturing never touches live KV or
        recurrent state; the caller stages real inputs afterwards."""
        key = (b, greedy)
        splits = self._splits_for(b)
        self.d_small.zero_()
        self.d_slots.zero_()
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            before = _K().launch_count(self.device)
            self._forward(b, greedy, splits)
            self.kernels_per_graph[key] = _K().launch_count(self.device) - before
            s.synchronize()
            g = torch.cuda.CUDAGraph()
            if self.pool is None:
                self.pool = torch.cuda.graph_pool_handle()
            g.capture_begin(pool=self.pool)
            try:
                logits = self._forward(b, greedy, splits)
            finally:
                g.capture_end()
        torch.cuda.current_stream(self.device).wait_stream(s)
        self.graphs[key] = g
        self.logits[key] = logits
        return g

    def precapture(self, greedy: bool = True, max_batch: int = 0) -> int:
        """Capture every bucket up front so serving never pays a capture on the request
        path (pegainfer-qwen3/src/executor.rs:1428-1496 pre-capture sweep)."""
        n = 0
        for b in self.buckets:
            if max_batch and b > max_batch:
                break
            if (b, greedy) not in self.graphs:
                self.capture(b, greedy)
                n += 1
        torch.cuda.synchronize(self.device)
        return n

    def stage(self, seqs, b: int) -> None:
        """Fill the pinned mirrors for ``seqs`` padded to bucket ``b`` and start the
        host->device copies on the current stream."""
        n = len(seqs)
        B = self.max_b
        sm, tb = self.np_small, self.np_table
        wmax = 1
        rows = self._row_state  # per table row: (request id, pages already written): a decode step adds at most one page
        dirty = False
        ps = self.page_size
        toks, poss, slots = [0] * n, [0] * n, [0] * n
        for i, s in enumerate(seqs):
            pos = s.start_pos
            pages = s.view.page_indices
            toks[i] = s.input_tokens[0]
            poss[i] = pos
            slots[i] = pages[pos // ps] * ps + pos % ps
            np_ = len(pages)
            rid, have = rows[i]
            if rid != s.rid or have > np_:
                tb[i, :np_] = pages
                rows[i] = (s.rid, np_)
                dirty = True
            elif have < np_:
                tb[i, have:np_] = pages[have:]
                rows[i] = (s.rid, np_)
                dirty = True
            if np_ > wmax:
                wmax = np_
        sm[:n] = toks
        sm[B : B + n] = poss
        sm[2 * B : 2 * B + n] = slots
        sm[3 * B : 3 * B + n] = poss
        sm[3 * B : 3 * B + n] += 1
        if n < b:
            sm[n:b] = 0
            sm[B + n : B + b] = 0
            sm[2 * B + n : 2 * B + b] = 0
            sm[3 * B + n : 3 * B + b] = 0
        if self.uses_state:
            hs = self.h_slots.numpy()
            for i, s in enumerate(seqs):
                hs[i] = self.ex.model.rec.slot_for(s.rid, False)
            hs[n:b] = 0
            self.d_slots.copy_(self.h_slots, non_blocking=True)
        self.d_small.copy_(self.h_small, non_blocking=True)
        self.h2d_bytes += self.h_small.numel() * 4
        if dirty or b != self._table_b or wmax > self._table_w:
            # the block table only changes when a sequence crosses a page boundary or rows change hands
            self.d_table[:b, :wmax].copy_(self.h_table[:b, :wmax], non_blocking=True)
            self.h2d_bytes += b * wmax * 4
            self._table_b, self._table_w = b, wmax

    def run(self, seqs, greedy: bool = True) -> torch.Tensor:
        from ..sched.executor import bucket_for

        n = len(seqs)
        b = bucket_for(n, self.buckets)
        key = (b, greedy)
        g = self.graphs.get(key)
        if g is None:
            g = self.capture(b, greedy)
        self.stage(seqs, b)
        g.replay()
        self.replays += 1
        if greedy:
            self.h_out[:n].copy_(self.out_tokens[:n], non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()
            self.d2h_bytes += n * 4
            return self.h_out[:n]
        return self.logits[key][:n]

    def dump_dot(self, path: str, b: Optional[int] = None, greedy: bool = True) -> str:
        """Write the captured graph of bucket ``b`` as Graphviz DOT text."""
        b = b if b is not None else self.buckets[0]
        g = self.graphs.get((b, greedy)) or self.capture(b, greedy)
        g.enable_debug_mode() if hasattr(g, "enable_debug_mode") else None
        try:
            g.debug_dump(path)
        except Exception:
            with open(path, "w") as f:
                f.write("digraph decode { /* this torch build cannot export graph nodes */ }\n")
        return path
