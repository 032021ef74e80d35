"""CUDA-graph decode: one captured graph per batch bucket.

Inputs live in pointer-stable device buffers that are refreshed from pinned host
mirrors before each replay; rows beyond the live batch are padding rows that point at
page 0 with ``kv_len == 0`` so they attend to nothing and their KV write lands in the
reserved padding page.  The greedy variant captures the argmax too, so a replay
yields token ids directly.  ``dump_dot`` writes the captured graph as Graphviz text.

Run-ahead: a greedy decode step can be followed at once by the launch of the NEXT step,
before the host has read this step's tokens.  The next step's positions, slots and KV
lengths are known on the host (every sequence advances by one; its next page is already
in the block table), and its input tokens are gathered on the device from the tokens the
running step is about to write.  The scheduler's host work between two steps then
overlaps the GPU work of the step that is already running.  A sequence that turns out to
have finished just wastes its row of the step that ran ahead; a step whose rows nobody
claims is dropped, its only side effect being KV written at positions that are not yet
committed.

Reference parity: pegainfer-core/src/cuda_graph.rs:42-234 (capture / replay state),
pegainfer-qwen3/src/batch_decode.rs:99-167 (bucket padding, graph per bucket and
attention path), pegainfer-core/src/cuda_graph/dump.rs:24-135 (DOT export).
"""
from __future__ import annotations

import os
import time
from typing import Optional

import numpy as np
import torch

from .. import ops
from ..ops.reference import AttnMeta


def _K():
    from ..ops import cuda

    return cuda


class _InFlight:
    """A decode step that has been launched: where each request's token will appear."""

    __slots__ = ("rows", "pos", "event", "host", "n")

    def __init__(self, rows, pos, event, host, n):
        self.rows = rows  # rid -> row of the step
        self.pos = pos  # rid -> position of the token the step feeds
        self.event = event
        self.host = host  # pinned int32 buffer the tokens are copied into
        self.n = n


class DecodeGraphs:
    def __init__(self, executor, max_batch: int, max_blocks_per_seq: int, with_lora: bool = False):
        from ..sched.executor import DECODE_BUCKETS, bucket_for

        self.ex = executor
        self.device = executor.device
        self.buckets = [b for b in DECODE_BUCKETS if b <= max(bucket_for(max_batch), 1)]
        self.max_b = self.buckets[-1]
        self.width = max(max_blocks_per_seq, 1)
        self.page_size = executor.page_size
        B, W, dev = self.max_b, self.width, self.device
        # one int32 arena: tokens | positions | slots | kv_lens | source rows (run-ahead), mirrored in pinned memory
        self.h_small = torch.zeros(5 * B, dtype=torch.int32).pin_memory()
        self.d_small = torch.zeros(5 * B, dtype=torch.int32, device=dev)
        self.h_table = torch.zeros((B, W), dtype=torch.int32).pin_memory()
        self.d_table = torch.zeros((B, W), dtype=torch.int32, device=dev)
        self.np_small = self.h_small.numpy()
        self.np_table = self.h_table.numpy()
        self.q_indptr = torch.arange(B + 1, dtype=torch.int32, device=dev)
        self.out_tokens = torch.zeros(B, dtype=torch.int32, device=dev)
        self.h_slots = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.d_slots = torch.zeros(B, dtype=torch.int32, device=dev)
        self.uses_state = hasattr(executor.model, "rec")
        # graphs whose steps carry an adapter slot per row (-1: no adapter); a separate set from the adapter-free graphs,
        # which keep the fused decode path
        self.with_lora = with_lora
        self.h_lora = torch.full((B,), -1, dtype=torch.int32).pin_memory()
        self.d_lora = torch.full((B,), -1, dtype=torch.int32, device=dev)
        self.h_out = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.h_out2 = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.pending: Optional[_InFlight] = None  # the step that is running ahead, if any
        self._staged = None  # event behind the last host->device copies out of the pinned mirrors
        self.ahead_launches = 0
        self.ahead_claimed = 0
        self._timing = [] if os.environ.get("PEGAINFER_GRAPH_TIMING") == "1" else None  # (start, end) events of every replay
        self._host_ms = []  # (stage, replay call) host milliseconds per replay, with the timing switch
        self.wait_s = 0.0  # host time spent waiting for a step's tokens
        self.launch_s = 0.0  # host time spent staging and launching steps
        self.graphs: dict = {}
        self.logits: dict = {}
        self.aux_layers: tuple = ()  # target layers whose residual stream every captured step also returns (drafters read them)
        self.aux: dict = {}  # graph key -> the step's tapped hidden states (graph outputs, overwritten by the next replay)
        self.pool = None
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.replays = 0
        self.kernels_per_graph: dict = {}
        self.trace_range: dict = {}
        self.invalidate_table()
        # first use of a framework kernel loads its module (tens of milliseconds): do that now for the
        # two copies the run-ahead path issues between replays, not on a live decode step
        _K().gather_words(self.out_tokens, self.d_small[4 * B : 4 * B + 1], self.d_small[:1])
        self.d_small[:1].copy_(self.out_tokens[:1], non_blocking=True)
        self.h_out[:1].copy_(self.out_tokens[:1], non_blocking=True)
        torch.cuda.synchronize(dev)

    def release(self) -> None:
        """Drop every captured graph (each pins its kernels' buffers and a share of the graph
        memory pool), so that the process can unmap peer memory and exit in order."""
        self.pending = None
        self.graphs.clear()
        self.logits.clear()
        self.aux.clear()
        self._last_aux = None
        self.pool = None

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
            lora_slots=self.d_lora[:b] if self.with_lora else None,
        )

    def _forward(self, b: int, greedy: bool, splits: int):
        tok = self._views(b)[0]
        meta = self._meta(b, splits)
        model = self.ex.model
        if self.aux_layers:
            hidden = model.forward_hidden(tok, meta, self.ex.kv, aux_layers=self.aux_layers)
            self._last_aux = list(model.last_aux)
        else:
            hidden = model.forward_hidden(tok, meta, self.ex.kv)
        logits = model.logits(hidden)
        if greedy:
            if hasattr(model, "greedy_tokens"):
                model.greedy_tokens(logits, out=self.out_tokens[:b])
            else:
                _K().argmax(logits, out=self.out_tokens[:b])
            return logits
        return model.full_logits(logits) if hasattr(model, "full_logits") else logits

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
            trace0 = len(_K().GemmTrace.names)
            g.capture_begin(pool=self.pool)
            try:
                logits = self._forward(b, greedy, splits)
            finally:
                g.capture_end()
            self.trace_range[key] = (trace0, len(_K().GemmTrace.names))  # GEMM trace slots of this graph (debug aid)
            # The first launch of an instantiated graph uploads it to the device (measured: 50 - 70 ms
            # for a whole-step graph).  Pay that here, on the padding inputs the capture ran on, and not
            # on the first decode step that lands in this bucket.
            g.replay()
        torch.cuda.current_stream(self.device).wait_stream(s)
        self.graphs[key] = g
        self.logits[key] = logits
        if self.aux_layers:
            self.aux[key] = self._last_aux
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

    def stage(self, seqs, b: int, ahead_of: Optional[_InFlight] = None) -> None:
        """Fill the pinned mirrors for ``seqs`` padded to bucket ``b`` and start the
        host->device copies on the current stream.  With ``ahead_of`` the step fed is the
        one AFTER ``seqs``' own (every position one further) and the input tokens do not
        come from the host: they are gathered on the device from the rows of the step
        ``ahead_of`` that is still running."""
        n = len(seqs)
        B = self.max_b
        sm, tb = self.np_small, self.np_table
        wmax = 1
        rows = self._row_state  # per table row: (request id, pages already written): a decode step adds at most one page
        dirty = False
        ps = self.page_size
        adv = 0 if ahead_of is None else 1
        if self._staged is not None:
            self._staged.synchronize()  # the previous copies have read the mirrors (long done in practice)
        toks, poss, slots = [0] * n, [0] * n, [0] * n
        for i, s in enumerate(seqs):
            pos = s.start_pos + adv
            pages = s.table_pages if s.table_pages is not None else s.view.page_indices
            toks[i] = ahead_of.rows[s.rid] if adv else s.input_tokens[0]
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
        t0 = 4 * B if adv else 0  # run-ahead: the list holds source rows, not tokens
        sm[t0 : t0 + n] = toks
        sm[B : B + n] = poss
        sm[2 * B : 2 * B + n] = slots
        sm[3 * B : 3 * B + n] = poss
        sm[3 * B : 3 * B + n] += 1
        if n < b:
            sm[t0 + n : t0 + b] = 0
            sm[B + n : B + b] = 0
            sm[2 * B + n : 2 * B + b] = 0
            sm[3 * B + n : 3 * B + b] = 0
        if self.uses_state:
            hs = self.h_slots.numpy()
            for i, s in enumerate(seqs):
                hs[i] = self.ex.model.rec.slot_for(s.rid, False)
            hs[n:b] = 0
            self.d_slots.copy_(self.h_slots, non_blocking=True)
        if adv:
            self.d_small[B:].copy_(self.h_small[B:], non_blocking=True)
            self.h2d_bytes += 4 * B * 4
            # rows keep their place unless a sequence left the batch: a plain copy then, else a gather
            if toks == list(range(n)):
                self.d_small[:n].copy_(self.out_tokens[:n], non_blocking=True)
            else:
                _K().gather_words(self.out_tokens, self.d_small[4 * B : 4 * B + n], self.d_small[:n])
        else:
            self.d_small[: 4 * B].copy_(self.h_small[: 4 * B], non_blocking=True)
            self.h2d_bytes += 4 * B * 4
        if dirty or b != self._table_b or wmax > self._table_w:
            # the block table only changes when a sequence crosses a page boundary or rows change hands
            self.d_table[:b, :wmax].copy_(self.h_table[:b, :wmax], non_blocking=True)
            self.h2d_bytes += b * wmax * 4
            self._table_b, self._table_w = b, wmax
        if self._staged is None:
            self._staged = torch.cuda.Event()
        self._staged.record(torch.cuda.current_stream(self.device))  # never "the current device's" stream: that is per thread

    def _launch(self, seqs, b: int, key, ahead_of: Optional[_InFlight] = None) -> _InFlight:
        """Stage, replay and queue the copy of the picked tokens into pinned memory."""
        t0 = time.perf_counter()
        self.stage(seqs, b, ahead_of)
        if self._timing is not None:
            t1 = time.perf_counter()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(torch.cuda.current_stream(self.device))
            self.graphs[key].replay()
            e1.record(torch.cuda.current_stream(self.device))
            self._timing.append((e0, e1))
            self._host_ms.append((round(1e3 * (t1 - t0), 3), round(1e3 * (time.perf_counter() - t1), 3)))
        else:
            self.graphs[key].replay()
        self.replays += 1
        n = len(seqs)
        host = self.h_out2 if (ahead_of is not None and ahead_of.host is self.h_out) else self.h_out
        host[:n].copy_(self.out_tokens[:n], non_blocking=True)
        self.d2h_bytes += n * 4
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        adv = 0 if ahead_of is None else 1
        self.launch_s += time.perf_counter() - t0
        return _InFlight({s.rid: i for i, s in enumerate(seqs)}, {s.rid: s.start_pos + adv for s in seqs}, ev, host, n)

    def timing_summary(self, last: int = 0) -> dict:
        """With ``PEGAINFER_GRAPH_TIMING=1``: device time of the replays and of the gaps between
        consecutive replays (copies, launch latency, a GPU waiting for the host), over the last
        ``last`` replays (0 = all)."""
        if not self._timing or len(self._timing) < 2:
            return {}
        torch.cuda.synchronize(self.device)
        ev = self._timing[-last:] if last else self._timing
        run = [a.elapsed_time(b) for a, b in ev]
        gap = [ev[i][1].elapsed_time(ev[i + 1][0]) for i in range(len(ev) - 1)]
        srt = sorted(gap)
        return dict(replays=len(ev), graph_ms_mean=sum(run) / len(run), gap_ms_mean=sum(gap) / len(gap), gap_ms_p50=srt[len(srt) // 2], gap_ms_max=srt[-1],
                    graph_ms=[round(x, 3) for x in run], gap_ms=[round(x, 3) for x in gap], host_stage_replay_ms=self._host_ms[-len(ev):])

    def covers(self, s) -> bool:
        """True if the step that is running ahead computes exactly this decode row."""
        p = self.pending
        return p is not None and len(s.input_tokens) == 1 and p.pos.get(s.rid, -1) == s.start_pos

    def claim(self, seqs) -> dict:
        """Take the tokens of the rows among ``seqs`` that the step running ahead has
        computed (``rid -> token``) and forget that step.  Nothing is waited for when no
        row matches: whatever the dropped step writes is ordered before later work on the
        stream."""
        p = self.pending
        if p is None:
            return {}
        hit = [s for s in seqs if self.covers(s)]
        self.pending = None
        if not hit:
            return {}
        p.event.synchronize()
        self.ahead_claimed += 1
        return {s.rid: int(p.host[p.rows[s.rid]]) for s in hit}

    def _launch_ahead(self, seqs, cur: _InFlight) -> None:
        """Launch the step after ``cur`` for every sequence that will still be running."""
        from ..sched.executor import bucket_for

        ps = self.page_size
        nxt = [s for s in seqs if not s.final]
        if not nxt or any(s.table_pages is None or (s.start_pos + 1) // ps >= len(s.table_pages) for s in nxt):
            return
        b = bucket_for(len(nxt), self.buckets)
        key = (b, True)
        if key not in self.graphs:
            return  # captured by the next ordinary step
        self.pending = self._launch(nxt, b, key, ahead_of=cur)
        self.ahead_launches += 1

    def run(self, seqs, greedy: bool = True, ahead: bool = False):
        """One decode step for ``seqs``: token ids (a list) when ``greedy``, else the logits.
        If a step is running ahead, the caller has checked that it covers every row."""
        from ..sched.executor import bucket_for

        n = len(seqs)
        cur, self.pending = self.pending, None
        if cur is not None:  # the executor has checked that it covers every row (``covers``)
            self.ahead_claimed += 1
        else:
            b = bucket_for(n, self.buckets)
            key = (b, greedy)
            if key not in self.graphs:
                self.capture(b, greedy)
            if not greedy:
                self.stage(seqs, b)
                self.graphs[key].replay()
                self.replays += 1
                return self.logits[key][:n]
            cur = self._launch(seqs, b, key)
        if ahead and not self.uses_state:
            self._launch_ahead(seqs, cur)
        t0 = time.perf_counter()
        cur.event.synchronize()
        self.wait_s += time.perf_counter() - t0
        host = cur.host.tolist()
        return [host[cur.rows[s.rid]] for s in seqs]

    def run_rows(self, rows):
        """A verify step as a widened decode step.  ``rows``: one-token steps, several of them per request
        (consecutive positions of the same block table).  Row ``j`` of a request is a sequence of its own
        whose KV length ends at its position: the layer's K/V append runs over all rows before its
        attention, so the row sees the request's earlier rows of the same step, and causality inside the
        span needs no mask.  Returns ``(tokens, tapped hidden states or None)`` for the rows in order."""
        from ..sched.executor import bucket_for

        n = len(rows)
        self.pending = None
        b = bucket_for(n, self.buckets)
        key = (b, True)
        if key not in self.graphs:
            self.capture(b, True)
        self.invalidate_table()  # rows of one request share a request id: the per-row table cache does not apply
        self.stage(rows, b)
        if self.with_lora:
            self.h_lora[:n] = torch.tensor([getattr(r, "lora_slot", -1) for r in rows], dtype=torch.int32)
            self.h_lora[n:b] = -1
            self.d_lora[:b].copy_(self.h_lora[:b], non_blocking=True)
            self.h2d_bytes += b * 4
        self.graphs[key].replay()
        self.replays += 1
        self.invalidate_table()
        self.h_out[:n].copy_(self.out_tokens[:n], non_blocking=True)
        self.d2h_bytes += n * 4
        torch.cuda.current_stream(self.device).synchronize()
        return self.h_out[:n].tolist(), self.aux.get(key)

    def dump_dot(self, path: str, b: Optional[int] = None, greedy: bool = True, png: bool = False) -> dict:
        """Write the decode graph of bucket ``b`` as Graphviz DOT text: every kernel node with its
        name and launch shape, every dependency edge (programmatic-launch edges dashed) and a
        per-kernel launch count in the header.  The bucket is captured once more into a graph
        object that keeps its ``cudaGraph_t``, which the C library walks.  With ``png`` and a
        ``dot`` binary on the PATH a PNG is rendered beside it.  Returns the node / edge counts."""
        import ctypes
        import shutil
        import subprocess

        from .. import _native

        b = b if b is not None else self.buckets[0]
        splits = self._splits_for(b)
        self.d_small.zero_()
        self.d_slots.zero_()
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self._forward(b, greedy, splits)
            s.synchronize()
            g = torch.cuda.CUDAGraph(keep_graph=True)
            g.capture_begin()
            try:
                self._forward(b, greedy, splits)
            finally:
                g.capture_end()
        torch.cuda.current_stream(self.device).wait_stream(s)
        counts = (ctypes.c_longlong * 4)()
        lib = _native.load()
        _native.check(lib.pg_graph_export_dot(ctypes.c_void_p(g.raw_cuda_graph()), path.encode(), f"decode step, batch bucket {b}".encode(), counts))
        out = dict(path=path, nodes=counts[0], edges=counts[1], kernels=counts[2], programmatic_edges=counts[3], png=None)
        if png and shutil.which("dot"):
            target = os.path.splitext(path)[0] + ".png"
            if subprocess.run(["dot", "-Tpng", path, "-o", target], capture_output=True).returncode == 0:
                out["png"] = target
        del g
        return out
