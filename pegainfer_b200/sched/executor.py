"""Step batches and the model executor.

The scheduler decides *what* runs (which requests, how many tokens, which pages);
the executor turns one :class:`StepBatch` into device tensors, runs the model and
the sampler, and returns one :class:`StepResult`.  Pure-decode batches replay a
CUDA graph captured per batch bucket: inputs live in pointer-stable buffers and
padding rows point at page 0.

Reference parity: pegainfer-qwen3/src/executor.rs:2467-2603 (execute_prefill /
execute_decode), src/batch_decode.rs:62-182 (bucket padding, graph replay),
src/batch_decode_buffers.rs:26-200 (bucket list, pointer-stable buffers),
src/scheduler/test_support.rs:27-289 (FakeExecutor for scheduler tests).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..engine.contract import SamplingParams
from ..kv.request_kv import KvView
from ..ops.reference import AttnMeta
from ..sample.select import batch_logprobs, select_batch

DECODE_BUCKETS = tuple(list(range(1, 9)) + list(range(10, 33, 2)) + list(range(36, 65, 4)) + list(range(72, 129, 8)) + list(range(144, 257, 16)))


def bucket_for(n: int, buckets: Sequence[int] = DECODE_BUCKETS) -> int:
    for b in buckets:
        if b >= n:
            return b
    raise ValueError(f"batch {n} exceeds the largest decode bucket {buckets[-1]}")


@dataclass
class SeqStep:
    rid: int
    input_tokens: list
    start_pos: int
    view: KvView
    sample: bool = True
    params: SamplingParams = field(default_factory=SamplingParams)
    step_index: int = 0
    logprobs: int = 0
    all_rows: bool = False  # speculative verify: a token for every input row
    lora_slot: int = -1
    state_slot: int = -1  # recurrent-state slot (hybrid models)
    next_token: int = -1  # token following the last input row when it is known (non-final prefill chunk)
    fresh_state: bool = False
    table_pages: Optional[list] = None  # decode run-ahead: the request's pages including the one for the next position
    final: bool = False  # decode run-ahead: this step's token is the request's last (length limit)


@dataclass
class StepBatch:
    seqs: list
    kind: str = "unified"  # prefill | decode | unified | verify
    run_ahead: bool = False  # a greedy graph decode step may launch the following step before it returns

    @property
    def num_tokens(self) -> int:
        return sum(len(s.input_tokens) for s in self.seqs)

    def is_decode(self) -> bool:
        return all(len(s.input_tokens) == 1 for s in self.seqs)


@dataclass
class StepResult:
    tokens: dict = field(default_factory=dict)  # rid -> [token, ...]
    logprobs: dict = field(default_factory=dict)  # rid -> [TokenLogprob, ...]
    drafts: dict = field(default_factory=dict)  # rid -> [draft token per sampled row] (MTP)
    elapsed_s: float = 0.0


class ModelExecutor:
    """Interface the scheduler drives."""

    vocab_size: int = 0

    def execute(self, batch: StepBatch) -> StepResult:
        raise NotImplementedError

    def release_request(self, rid: int) -> None:
        """Forget per-request executor state (recurrent slots, LoRA pins)."""


def build_meta(seqs: Sequence[SeqStep], page_size: int, device, pad_to: int = 0, table_width: int = 0, pinned: bool = False):
    """Flatten a list of per-sequence steps into ``(token_ids, AttnMeta)``."""
    n = len(seqs)
    b = max(n, pad_to)
    q_indptr = np.zeros(b + 1, dtype=np.int32)
    kv_lens = np.zeros(b, dtype=np.int32)
    width = max([len(s.view.page_indices) for s in seqs] + [1, table_width])
    table = np.zeros((b, width), dtype=np.int32)
    toks, pos, slots = [], [], []
    max_q = max_kv = 0
    for i, s in enumerate(seqs):
        nt = len(s.input_tokens)
        q_indptr[i + 1] = q_indptr[i] + nt
        kv_lens[i] = s.start_pos + nt
        pages = s.view.page_indices
        table[i, : len(pages)] = pages
        toks.extend(s.input_tokens)
        p = np.arange(s.start_pos, s.start_pos + nt, dtype=np.int64)
        pos.append(p)
        pg = np.asarray(pages, dtype=np.int64)
        slots.append(pg[p // page_size] * page_size + p % page_size)
        max_q = max(max_q, nt)
        max_kv = max(max_kv, s.start_pos + nt)
    t_real = int(q_indptr[n])
    # padding sequences: one row each, zero KV, slot in page 0
    for i in range(n, b):
        q_indptr[i + 1] = q_indptr[i] + 1
    t = int(q_indptr[b])
    tok = np.zeros(t, dtype=np.int32)
    tok[:t_real] = toks
    posa = np.zeros(t, dtype=np.int32)
    slota = np.zeros(t, dtype=np.int32)
    if t_real:
        posa[:t_real] = np.concatenate(pos)
        slota[:t_real] = np.concatenate(slots)

    def dev(a):
        x = torch.from_numpy(a)
        if torch.device(device).type == "cuda":
            return x.pin_memory().to(device, non_blocking=True) if pinned else x.to(device)
        return x

    meta = AttnMeta(
        q_indptr=dev(q_indptr),
        kv_lens=dev(kv_lens),
        block_table=dev(table),
        slot_mapping=dev(slota),
        positions=dev(posa),
        page_size=page_size,
        num_seqs=b,
        num_tokens=t,
        max_q_len=max(max_q, 1),
        max_kv_len=max_kv,
        decode_only=(max_q <= 1),
        h_q_indptr=q_indptr.tolist(),
        h_kv_lens=kv_lens.tolist(),
    )
    return dev(tok), meta


class TorchExecutor(ModelExecutor):
    """Runs a model object exposing ``forward_hidden`` / ``logits`` on CPU or GPU."""

    def __init__(self, model, kv, page_size: int, cuda_graph: bool = False, max_decode_batch: int = 256, max_blocks_per_seq: int = 0, seed: int = 0):
        self.model = model
        self.kv = kv
        self.page_size = page_size
        self.device = model.device
        self.vocab_size = model.cfg.vocab_size
        self.seed = seed
        self.steps = 0
        self.use_graph = bool(cuda_graph) and self.device.type == "cuda"
        self.max_decode_batch = max_decode_batch
        self.max_blocks_per_seq = max_blocks_per_seq
        self.mtp = None  # set by spec.MtpSpec
        self.aux_sink = None  # set by drafters that read target hidden states: .aux_layers, .observe(kind, seqs, meta, aux)
        self._lane_stream = None  # second stream of the decode-overlap prefill lane
        self.sm_split = None  # utils.green_ctx.SmSplit when the lane is confined to its own SM partition
        self._graphs = None
        if self.use_graph:
            from ..utils.cuda_graph import DecodeGraphs

            self._graphs = DecodeGraphs(self, max_decode_batch, max_blocks_per_seq)

    def prepare_meta(self, seqs, meta) -> None:
        """Hook for model lines that carry extra per-sequence state (recurrent slots)."""

    # -- sampling ----------------------------------------------------------------
    def _sample(self, logits, seqs, rows_per_seq):
        params, steps = [], []
        for s, nrows in zip(seqs, rows_per_seq):
            for j in range(nrows):
                params.append(s.params)
                steps.append(s.step_index + j)
        toks = select_batch(logits, params, steps, base_seed=self.seed + self.steps)
        want_lp = max((s.logprobs for s in seqs), default=0)
        lps = None
        if any(s.logprobs > 0 for s in seqs):
            lps = batch_logprobs(logits, toks, want_lp)
        return toks, lps

    @property
    def supports_run_ahead(self) -> bool:
        return self._graphs is not None and self.mtp is None and not self._graphs.uses_state

    def _graph_decode(self, batch: StepBatch) -> bool:
        seqs = batch.seqs
        return (self._graphs is not None and self.mtp is None and self.aux_sink is None and batch.is_decode() and len(seqs) <= self.max_decode_batch
                and all(s.sample and s.logprobs == 0 and s.lora_slot < 0 for s in seqs))

    def _graph_lora_decode(self, batch: StepBatch) -> bool:
        """A greedy decode step in which at least one request uses an adapter: replayed from the adapter-aware graphs
        (the adapter slot of every row is a graph input), not run kernel by kernel."""
        seqs = batch.seqs
        return (self._graphs is not None and not self._graphs.uses_state and self.mtp is None and self.aux_sink is None and getattr(self.model, "lora", None) is not None
                and batch.is_decode() and len(seqs) <= self.max_decode_batch and any(s.lora_slot >= 0 for s in seqs)
                and all(s.sample and s.logprobs == 0 and s.params.effectively_greedy(self.vocab_size) for s in seqs))

    def _lora_graphs(self):
        g = getattr(self, "_graphs_lora", None)
        if g is None:
            from ..utils.cuda_graph import DecodeGraphs

            g = self._graphs_lora = DecodeGraphs(self, self.max_decode_batch, self.max_blocks_per_seq, with_lora=True)
        return g

    def enable_sm_split(self, decode_pct: int) -> None:
        """Confine the prefill lane to ``100 - decode_pct`` percent of the SMs (green contexts)."""
        from ..utils.green_ctx import SmSplit

        self.sm_split = SmSplit(self.device, decode_pct)
        self._lane_stream = self.sm_split.prefill_stream

    def enable_verify_graph(self, span: int) -> None:
        """Size the decode graphs for verify steps of ``span`` rows per request (speculative decoding):
        a verify step replays the decode graph of ``requests * span`` rows."""
        self.verify_span = span
        if self._graphs is None or self._graphs.uses_state:
            return
        from ..utils.cuda_graph import DecodeGraphs

        want = min(DECODE_BUCKETS[-1], self.max_decode_batch * span)
        if want > self._graphs.max_b:
            self._graphs.release()
            self._graphs = DecodeGraphs(self, want, self.max_blocks_per_seq)
        if self.aux_sink is not None:
            self._graphs.aux_layers = tuple(self.aux_sink.aux_layers)

    def _graph_verify(self, batch: StepBatch) -> bool:
        g, seqs = self._graphs, batch.seqs
        return (batch.kind == "verify" and g is not None and not g.uses_state and self.mtp is None and getattr(self, "verify_span", 0) > 0
                and batch.num_tokens <= g.max_b and all(s.sample and s.all_rows and s.logprobs == 0 and s.lora_slot < 0 and s.params.effectively_greedy(self.vocab_size) for s in seqs))

    def _execute_verify_graph(self, batch: StepBatch, t0: float) -> StepResult:
        from types import SimpleNamespace

        rows, indptr = [], [0]
        for s in batch.seqs:
            for j, tok in enumerate(s.input_tokens):
                rows.append(SeqStep(rid=s.rid, input_tokens=[tok], start_pos=s.start_pos + j, view=s.view))
            indptr.append(len(rows))
        toks, aux = self._graphs.run_rows(rows)
        if self.aux_sink is not None:
            self.aux_sink.observe("verify", batch.seqs, SimpleNamespace(num_tokens=len(rows), h_q_indptr=indptr), aux)
        return StepResult(tokens={s.rid: toks[indptr[i] : indptr[i + 1]] for i, s in enumerate(batch.seqs)}, elapsed_s=time.perf_counter() - t0)

    def execute(self, batch: StepBatch) -> StepResult:
        g = self._graphs
        if g is not None and g.pending is not None:
            # A decode step is already running ahead.  If it is exactly this batch the graph
            # path below picks it up; otherwise (a prompt chunk came along, a request joined,
            # sampling changed) take the rows it did compute and run only the rest.
            seqs = batch.seqs
            whole = self._graph_decode(batch) and all(g.covers(s) for s in seqs) and all(s.params.effectively_greedy(self.vocab_size) for s in seqs)
            if not whole:
                claimed = g.claim(seqs)
                if claimed:
                    rest = [s for s in seqs if s.rid not in claimed]
                    res = self._execute(StepBatch(seqs=rest, kind=batch.kind)) if rest else StepResult()
                    for rid, tok in claimed.items():
                        res.tokens[rid] = [tok]
                    return res
        return self._execute(batch)

    def _execute(self, batch: StepBatch) -> StepResult:
        t0 = time.perf_counter()
        self.steps += 1
        seqs = batch.seqs
        if self._graph_verify(batch):
            return self._execute_verify_graph(batch, t0)
        if self._graph_lora_decode(batch):
            toks, _ = self._lora_graphs().run_rows(batch.seqs)
            return StepResult(tokens={s.rid: [toks[i]] for i, s in enumerate(batch.seqs)}, elapsed_s=time.perf_counter() - t0)
        if self._graph_decode(batch):
            all_greedy = all(s.params.effectively_greedy(self.vocab_size) for s in seqs)
            out = self._graphs.run(seqs, greedy=all_greedy, ahead=batch.run_ahead and all_greedy)
            if all_greedy:
                toks = out
            else:
                toks, _ = self._sample(out[: len(seqs)], seqs, [1] * len(seqs))
                toks = toks.tolist()
            return StepResult(tokens={s.rid: [toks[i]] for i, s in enumerate(seqs)}, elapsed_s=time.perf_counter() - t0)
        token_ids, meta = build_meta(seqs, self.page_size, self.device)
        if meta.decode_only and self.device.type == "cuda" and self.max_blocks_per_seq:
            # the same KV-split plan a captured graph of this batch size uses (it depends on the batch
            # size and the longest sequence the engine admits, not on the live lengths), so an eager
            # decode step and a graph replay of the same batch are bit-identical
            from ..ops import cuda as K

            geo = self.model.kv_geometry()
            meta.plan = K.plan_decode_splits(len(seqs), geo["kv_heads"], min(self.max_blocks_per_seq * self.page_size, 2048), self.device)
        if any(s.lora_slot >= 0 for s in seqs):
            rows = []
            for s in seqs:
                rows.extend([s.lora_slot] * len(s.input_tokens))
            rows += [-1] * (meta.num_tokens - len(rows))
            meta.lora_slots = torch.tensor(rows, dtype=torch.int32, device=self.device)
        self.prepare_meta(seqs, meta)
        if self.aux_sink is not None:
            hidden = self.model.forward_hidden(token_ids, meta, self.kv, aux_layers=self.aux_sink.aux_layers)
            self.aux_sink.observe(batch.kind, seqs, meta, self.model.last_aux)
        else:
            hidden = self.model.forward_hidden(token_ids, meta, self.kv)
        # rows that need logits
        rows, rows_per_seq, sample_seqs = [], [], []
        for i, s in enumerate(seqs):
            if not s.sample:
                continue
            q0, q1 = meta.h_q_indptr[i], meta.h_q_indptr[i + 1]
            r = list(range(q0, q1)) if s.all_rows else [q1 - 1]
            rows.extend(r)
            rows_per_seq.append(len(r))
            sample_seqs.append(s)
        res = StepResult()
        if rows:
            idx = torch.tensor(rows, dtype=torch.int32, device=self.device)
            logits = self.model.logits(hidden, idx)
            if hasattr(self.model, "full_logits"):
                logits = self.model.full_logits(logits)  # vocabulary-sharded output projection: gather before sampling
            toks, lps = self._sample(logits, sample_seqs, rows_per_seq)
            toks = toks.tolist()
            k = 0
            for s, nrows in zip(sample_seqs, rows_per_seq):
                res.tokens[s.rid] = toks[k : k + nrows]
                if lps is not None and s.logprobs > 0:
                    res.logprobs[s.rid] = lps[k : k + nrows]
                k += nrows
        if self.mtp is not None:
            self._mtp_drafts(seqs, meta, res)
        res.elapsed_s = time.perf_counter() - t0
        return res

    # -- prefill lane (decode overlap) -----------------------------------------------
    def launch_async(self, batch: StepBatch):
        """Start a prompt-chunk batch on the executor's second CUDA stream and return without
        waiting: the forward pass, the greedy pick of every sampled row and the copy of the
        picked tokens into pinned memory are queued behind each other on that stream, followed
        by an event.  Decode steps keep running on the main stream meanwhile (shared SMs).
        On CPU the batch simply runs here and now.  Reference: pegainfer-qwen3
        src/executor.rs:490-589 (decode-overlap prefill lane, polled through an event)."""
        if self.device.type != "cuda":
            return ("done", self.execute(batch))
        self.steps += 1
        if self._lane_stream is None:
            self._lane_stream = torch.cuda.Stream(self.device)
        lane = self._lane_stream
        lane.wait_stream(torch.cuda.current_stream(self.device))
        seqs = batch.seqs
        from ..ops import cuda as K

        with torch.cuda.stream(lane), K.lane_scratch():
            token_ids, meta = build_meta(seqs, self.page_size, self.device, pinned=True)
            self.prepare_meta(seqs, meta)
            hidden = self.model.forward_hidden(token_ids, meta, self.kv)
            rows, owners = [], []
            for i, s in enumerate(seqs):
                if s.sample:
                    rows.append(meta.h_q_indptr[i + 1] - 1)
                    owners.append(s.rid)
            host = None
            keep = [token_ids, meta, hidden]
            if rows:
                idx = torch.tensor(rows, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
                lg = self.model.logits(hidden, idx)
                toks = self.model.greedy_tokens(lg) if hasattr(self.model, "greedy_tokens") else ops.argmax(lg)
                host = torch.empty(len(rows), dtype=toks.dtype).pin_memory()
                host.copy_(toks, non_blocking=True)
                keep += [idx, toks]
            ev = torch.cuda.Event()
            ev.record(lane)
        return ("cuda", ev, owners, host, keep)

    def finish_async(self, pending, wait: bool = False) -> Optional[StepResult]:
        """The result of ``launch_async`` once its event has fired (``None`` before that)."""
        if pending[0] == "done":
            return pending[1]
        _, ev, owners, host, _keep = pending
        if wait:
            ev.synchronize()
        elif not ev.query():
            return None
        res = StepResult()
        if host is not None:
            for rid, tok in zip(owners, host.tolist()):
                res.tokens[rid] = [tok]
        return res

    def _mtp_drafts(self, seqs, meta, res: StepResult) -> None:
        """Run the MTP block over every row of the step: it fills the MTP KV layer for
        those positions and drafts one token after each sampled row."""
        nxt, draft_rows, owners = [], [], []
        for i, s in enumerate(seqs):
            q0, n = meta.h_q_indptr[i], len(s.input_tokens)
            sampled = res.tokens.get(s.rid)
            for j in range(n):
                if sampled is not None and s.all_rows:
                    nxt.append(sampled[j])
                elif j + 1 < n:
                    nxt.append(s.input_tokens[j + 1])
                elif sampled is not None:
                    nxt.append(sampled[-1])
                else:
                    nxt.append(max(s.next_token, 0))
            if sampled is not None:
                rows = list(range(q0, q0 + n)) if s.all_rows else [q0 + n - 1]
                draft_rows.extend(rows)
                owners.append((s.rid, len(rows)))
        nt = torch.tensor(nxt + [0] * (meta.num_tokens - len(nxt)), dtype=torch.int32, device=self.device)
        h = self.mtp.forward(nt, self.model.last_residual, meta, self.kv)
        if not draft_rows:
            return
        idx = torch.tensor(draft_rows, dtype=torch.int32, device=self.device)
        toks = ops.argmax(self.model.logits(h, idx)).tolist()
        k = 0
        for rid, n in owners:
            res.drafts[rid] = toks[k : k + n]
            k += n
