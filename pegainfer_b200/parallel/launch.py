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

    collected: list = []
    ledger = RequestLedger(sink=(handle.dispatch if (rank == 0 and mode == "tp") else collected.append))
    local: dict = {}  # rid -> QueuedRequest on this rank
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
                    target = None if mode == "tp" else partition_of(q)
                    local[q.id] = q
                    new.append((q.id, q.request, q.queued_at, target))
                aborts = [rid for rid, q in local.items() if q.is_aborted() and rid not in known_aborts]
                payload = (new, aborts, stop.is_set())
            box = [payload]
            dist.broadcast_object_list(box, src=0, group=group)
            new, aborts, stopping = box[0]
            if stopping:
                break
            for rid, req, queued_at, target in new:
                if target is not None and target != rank:
                    continue
                q = local.get(rid) if rank == 0 else None
                if q is None:
                    q = QueuedRequest(id=rid, request=req, queued_at=queued_at)
                    local[rid] = q
                ledger.register(q)
                scheduler.submit(q)
            for rid in aborts:
                known_aborts.add(rid)
                if rid in local:
                    local[rid].abort_flag.set()
            busy = scheduler.step(ledger)
            if rank == 0:
                handle.metrics_cell.publish(scheduler.metrics())
            ledger.commit_step()
            for rid in [r for r in local if not ledger.is_open(r)]:
                local.pop(rid, None)
            if mode == "dp":
                # every rank's updates of this step go back to the frontend on rank 0
                gathered = [None] * world if rank == 0 else None
                dist.gather_object(collected[:], gathered, dst=0, group=group)
                collected.clear()
                if rank == 0:
                    for outs in gathered:
                        for so in outs or []:
                            handle.dispatch(so)
            else:
                collected.clear()
            if not busy and not new:
                time.sleep(0.001)
    except Exception as exc:  # a lost rank or a fatal step: fail-stop for every open request
        log.error("control loop ended: %r", exc)
        if rank == 0:
            upd = [RequestUpdate(id=rid, terminal=Terminal.failed(f"engine failure: {exc!r}")) for rid in list(local)]
            if upd:
                handle.dispatch(StepOutputs(updates=upd))
        handle.alive = False
        raise
    finally:
        handle.alive = False


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


def launch_distributed(ecfg, mcfg, ns) -> int:
    """Entry point under torchrun: build this rank's shard, then serve (rank 0) or follow."""
    import torch
    import torch.distributed as dist

    from ..engine.build import build_engine
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
    tp, ep, mode = TPContext(), None, "tp"
    if moe:
        mode = "dp"
        if ecfg.comm == "fused":
            from .fused_ep import make_fused_ep

            ep = make_fused_ep(rank, world, device, mcfg, max_tokens=max(ecfg.max_prefill_tokens, ecfg.max_decode_batch))
        else:
            from .ep import EPContext

            ep = EPContext(rank, world, comm="nccl", tokens="dp")
    elif ecfg.comm == "fused":
        from .fused import make_fused_tp

        tp = make_fused_tp(rank, world, device, mcfg, max_tokens=ecfg.max_prefill_tokens + ecfg.max_decode_batch)
    else:
        tp = TPContext(rank, world, comm="nccl")
    eng = build_engine(ecfg, mcfg, device=device, dtype=torch.bfloat16, tp=tp, ep=ep, start=False)
    sched = eng.scheduler
    partition_of = None
    if moe:
        from .dp import DpScheduler, LockstepExecutor

        lock = LockstepExecutor(eng.executor, control, world)
        sched.__class__ = DpScheduler
        sched.ex = lock
        rr = [0]

        def partition_of(q):  # round-robin is load-balanced for equal-cost requests; rank 0 decides
            rr[0] = (rr[0] + 1) % world
            return rr[0]

    rep = ReplicatedEngine(sched, eng.info, control, rank, world, mode, partition_of)
    rep.model, rep.executor, rep.scheduler, rep.pool, rep.kv = eng.model, eng.executor, sched, eng.pool, eng.kv
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
