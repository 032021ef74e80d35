"""Multi-GPU serving: one process per GPU, rank 0 hosts the HTTP frontend.

Two layouts share one control loop (``drive_replicated``):

* tensor parallel (Qwen3, Qwen3.5): every rank runs an identical scheduler over its
  weight shard.  Rank 0 owns the requests; at the top of every iteration it broadcasts
  the new requests and aborts of that iteration over a gloo group, every rank applies
  them in the same order, and since admission, chunking and greedy / seeded sampling are
  deterministic functions of that event stream, all ranks issue the same kernels and
  collectives in the same order.  Only rank 0's ledger talks to clients.
* data-parallel attention + expert parallel (DeepSeek-V2-Lite, Kimi-K2): every rank runs
  its own scheduler partition in lock-step (``parallel.dp``); rank 0 routes each request
  to the partition with the most free slots and every rank returns its step's updates to
  rank 0 with one ``gather_object``.

The event broadcast doubles as the failure detector: a rank that died between steps
makes the next broadcast raise on the others (process-group timeout), which fail their
open requests instead of entering a device-side collective that can never complete.

Reference parity: pegainfer-qwen3/src/executor.rs:3513-3895 (StepCommand broadcast to
rank workers, only rank 0 collects), pegainfer-kimi-k2/src/runner/scheduler/dp.rs,
pegainfer-glm52/src/rendezvous.rs (multi-process bring-up).
"""
from __future__ import annotations

import logging
import os
import queue
import threading
import time
from datetime import timedelta
from typing import Optional

from ..engine.contract import EngineInfo, KvCapacity, QueuedRequest, RequestUpdate, StepOutputs, Terminal
from ..engine.driver import Engine, SchedulerHandle
from ..engine.ledger import RequestLedger

log = logging.getLogger("pegainfer_b200.launch")


def drive_replicated(scheduler, handle: SchedulerHandle, stop: threading.Event, group, rank: int, world: int, mode: str = "tp", partition_of=None) -> None:
    """Control loop of one rank.  ``mode``: "tp" (replicated scheduler) or "dp" (own partition)."""
    import torch.distributed as dist

    from ..engine.driver import _bind_thread_to_device

    _bind_thread_to_device(scheduler)  # the current CUDA device is per thread and starts at 0
    collected: list = []
    direct = rank == 0 and mode == "tp"
    ledger = RequestLedger(sink=handle.dispatch if direct else collected.append)
    mine: dict = {}  # rid -> QueuedRequest registered with this rank's scheduler
    tracked: dict = {}  # rank 0 only: rid -> QueuedRequest of every open request (abort flags, failure reporting)
    known_aborts: set = set()
    try:
        while True:
            payload = None
            if rank == 0:
                new = []
                while True:
                    try:
                        q = handle._submit_q.get_nowait()
                    except queue.Empty:
                        break
                    tracked[q.id] = q
                    new.append((q.id, q.request, q.queued_at, None if mode == "tp" else partition_of(q)))
                aborts = [rid for rid, q in tracked.items() if q.is_aborted() and rid not in known_aborts]
                payload = (new, aborts, stop.is_set())
            box = [payload]
            dist.broadcast_object_list(box, src=0, group=group)
            new, aborts, stopping = box[0]
            if stopping:
                break
            for rid, req, queued_at, target in new:
                if target is not None and target != rank:
                    continue
                # Every rank, rank 0 included, gives its scheduler a PRIVATE copy whose abort flag is set
                # from the broadcast list only.  The client-facing request (whose flag an HTTP thread may
                # set at any moment) stays in `tracked`; if the scheduler saw that flag directly, rank 0
                # could retire a request one iteration before the other ranks and run a different batch.
                q = QueuedRequest(id=rid, request=req, queued_at=queued_at)
                mine[rid] = q
                ledger.register(q)
                scheduler.submit(q)
            for rid in aborts:
                known_aborts.add(rid)
                if rid in mine:
                    mine[rid].abort_flag.set()
            busy = scheduler.step(ledger)
            if rank == 0:
                handle.metrics_cell.publish(scheduler.metrics())
            ledger.commit_step()
            for rid in [r for r in mine if not ledger.is_open(r)]:
                mine.pop(rid, None)
                if direct:
                    tracked.pop(rid, None)
                    known_aborts.discard(rid)
            if mode == "dp":
                # every rank's updates of this step go back to the frontend on rank 0
                gathered = [None] * world if rank == 0 else None
                dist.gather_object(collected[:], gathered, dst=0, group=group)
                if rank == 0:
                    for outs in gathered:
                        for so in outs or []:
                            for upd in so.updates:
                                if upd.terminal is not None:
                                    tracked.pop(upd.id, None)
                                    known_aborts.discard(upd.id)
                            handle.dispatch(so)
            collected.clear()
            if not busy and not new:
                time.sleep(0.001)
    except Exception as exc:  # a lost rank or a fatal step: fail-stop for every open request
        log.error("control loop ended: %r", exc)
        if rank == 0:
            upd = [RequestUpdate(id=rid, terminal=Terminal.failed(f"engine failure: {exc!r}")) for rid in list(tracked)]
            if upd:
                handle.dispatch(StepOutputs(updates=upd))
        raise
    finally:
        handle.alive = False
        if rank == 0:  # nothing submitted after the loop stopped may hang
            while True:
                try:
                    q = handle._submit_q.get_nowait()
                except queue.Empty:
                    break
                handle.dispatch(StepOutputs(updates=[RequestUpdate(id=q.id, terminal=Terminal.failed("engine shut down"))]))


class ReplicatedEngine(Engine):
    """Engine whose single partition is driven by ``drive_replicated`` on every rank."""

    def __init__(self, scheduler, info: EngineInfo, group, rank: int, world: int, mode: str = "tp", partition_of=None):
        super().__init__([scheduler], info, start=False)
        self._rep = (group, rank, world, mode, partition_of)

    def start(self) -> None:
        if self._threads:
            return
        group, rank, world, mode, partition_of = self._rep
        t = threading.Thread(target=self._run_rep, name="scheduler-replicated", daemon=True)
        t.start()
        self._threads.append(t)

    def _run_rep(self):
        group, rank, world, mode, partition_of = self._rep
        try:
            drive_replicated(self._schedulers[0], self._handles[0], self._stop, group, rank, world, mode, partition_of)
        except Exception as exc:
            self._errors.append(exc)


def build_replicated_engine(ecfg, mcfg, rank: int, world: int, device, dtype, control, tp=None, ep=None) -> ReplicatedEngine:
    """This rank's engine for a multi-process deployment.  ``tp`` (dense model lines) or
    ``ep`` (MLA + MoE lines: data-parallel attention, experts spread over the ranks) is the
    rank's communication context; ``control`` is the host-side (gloo) group that carries
    the event broadcast, the lock-step agreement and the result gather."""
    from ..engine.build import build_engine
    from .tp import TPContext

    moe = mcfg.family in ("deepseek_v2", "kimi_k2")
    eng = build_engine(ecfg, mcfg, device=device, dtype=dtype, tp=tp or TPContext(), ep=ep, start=False)
    sched = eng.scheduler
    partition_of = None
    if moe:
        from .dp import DpScheduler, LockstepExecutor

        sched.__class__ = DpScheduler
        sched.ex = LockstepExecutor(eng.executor, control, world)
        rr = [-1]

        def partition_of(q):  # rank 0 decides; round-robin is load-balanced for equal-cost requests
            rr[0] = (rr[0] + 1) % world
            return rr[0]

    rep = ReplicatedEngine(sched, eng.info, control, rank, world, "dp" if moe else "tp", partition_of)
    rep.model, rep.executor, rep.scheduler, rep.pool, rep.kv = eng.model, eng.executor, sched, eng.pool, eng.kv
    return rep


def launch_distributed(ecfg, mcfg, ns) -> int:
    """Entry point under torchrun: build this rank's shard, then serve (rank 0) or follow."""
    import torch
    import torch.distributed as dist

    from ..server.openai import serve
    from ..server.tokenizer import load_tokenizer
    from .tp import TPContext

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=device)
    control = dist.new_group(backend="gloo", timeout=timedelta(seconds=float(os.environ.get("PEGAINFER_CONTROL_TIMEOUT_S", "60"))))
    moe = mcfg.family in ("deepseek_v2", "kimi_k2")
    tp, ep = None, None
    if moe:
        if ecfg.comm == "fused":
            from .fused_ep import make_fused_ep

            ep = make_fused_ep(rank, world, device, mcfg, max_tokens=max(ecfg.max_prefill_tokens, ecfg.max_decode_batch))
        else:
            from .ep import EPContext

            ep = EPContext(rank, world, comm="nccl", tokens="dp")
    elif ecfg.comm == "fused" and mcfg.family == "qwen3":
        # decode: one chain kernel per layer that sums over the ranks inside the NVSwitch (multimem)
        from .chain_tp import ChainTP

        tp = ChainTP(rank, world, device, mcfg.hidden_size)
    elif ecfg.comm == "fused":
        from .fused import make_fused_tp

        tp = make_fused_tp(rank, world, device, mcfg, max_tokens=ecfg.max_prefill_tokens + ecfg.max_decode_batch)
    else:
        tp = TPContext(rank, world, comm="nccl")
    rep = build_replicated_engine(ecfg, mcfg, rank, world, device, torch.bfloat16, control, tp=tp, ep=ep)
    dist.barrier()
    rep.start()
    if rank == 0:
        tok_dir = None if (ns.tokenizer == "none" or not ecfg.model_path) else ecfg.model_path
        tokenizer = load_tokenizer(tok_dir, mcfg.vocab_size)
        name = ecfg.served_model_name or ecfg.preset or os.path.basename(os.path.normpath(ecfg.model_path))
        try:
            serve(rep, tokenizer, name, ecfg.host, ecfg.port)
        finally:
            rep.shutdown()
    else:
        while rep.healthy():
            time.sleep(0.2)
    return 0
