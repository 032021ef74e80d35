"""Worker for the multi-process CPU tests (gloo): ``python -m torch.distributed.run ... tests/mp_worker.py MODE OUT``.

Modes
  tp        tiny Qwen3 with tensor parallelism over the ranks (replicated schedulers,
            rank 0 owns the requests); rank 0 writes the generated tokens
  dp_ep     tiny DeepSeek-V2 shape: data-parallel attention, experts spread over the ranks,
            lock-step executor; rank 0 routes requests and collects every rank's updates
  rank_loss like tp, but the last rank leaves between steps (no collective in flight): the
            others must fail their open requests on the host instead of hanging
  abort     like tp with long outputs; a client thread on rank 0 aborts two requests in the
            middle of decoding.  Every rank logs the composition of every batch it executes
            (OUT for rank 0, OUT.rankN for the others): the logs must be identical
"""
import json
import os
import sys
import threading
import time
from datetime import timedelta

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

from pegainfer_b200.config import EngineConfig, preset
from pegainfer_b200.engine.contract import Request, SamplingParams
from pegainfer_b200.parallel.ep import EPContext
from pegainfer_b200.parallel.launch import build_replicated_engine
from pegainfer_b200.parallel.tp import TPContext


def main():
    mode, out_path = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=timedelta(seconds=8 if mode == "rank_loss" else 120))
    control = dist.group.WORLD
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, 1024, (18 + 5 * i,), generator=g).tolist() for i in range(4)]
    if mode in ("dp_ep", "dp_ep_k3"):
        name, tp, ep = ("tiny-dsv2" if mode == "dp_ep" else "tiny-k3"), None, EPContext(rank, world, group=control, comm="nccl", tokens="dp")
    else:
        name, tp, ep = "tiny-qwen3", TPContext(rank, world, group=control, comm="nccl"), None
    ecfg = EngineConfig(preset=name, kv_page_size=16, num_kv_blocks=128, cuda_graph=False, max_prefill_tokens=32)
    eng = build_replicated_engine(ecfg, preset(name), rank, world, "cpu", torch.float32, control, tp=tp, ep=ep)
    result = {"rank": rank}
    batches = []
    if mode == "abort":
        ex = eng.scheduler.ex
        inner = ex.execute

        def logged(batch):
            batches.append([batch.kind] + [[s.rid, s.start_pos, len(s.input_tokens)] for s in batch.seqs])
            time.sleep(0.002)  # widen the window between the abort broadcast and the step
            return inner(batch)

        ex.execute = logged
    if rank == 0:
        n_tok = 400 if mode == "rank_loss" else 120 if mode == "abort" else 6
        streams = [eng.submit(Request(prompt_tokens=p, params=SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=n_tok)) for p in prompts]
    if mode == "rank_loss" and rank == world - 1:
        # leave between steps: stop the local loop after a few iterations, then exit without telling anyone
        eng.start()
        time.sleep(0.4)
        os._exit(0)
    eng.start()
    if mode == "abort" and rank == 0:
        def client():
            # abort as soon as the request has produced a few tokens, from a thread of its own
            for victim, after in ((streams[1], 5), (streams[3], 17)):
                seen = 0
                while seen < after:
                    seen += len(victim.get(timeout=60).tokens)
                victim.abort()

        threading.Thread(target=client, daemon=True).start()
        outs = []
        for i, s in enumerate(streams):
            if i in (1, 3):
                # the client thread consumes these; wait for the stream to close
                deadline = time.monotonic() + 60
                while not s.closed and time.monotonic() < deadline:
                    time.sleep(0.01)
                outs.append(([], type("T", (), {"kind": "aborted" if s.closed else "open", "message": ""})(), []))
            else:
                outs.append(s.collect(60))
        result["batches"] = batches
    elif rank == 0:
        outs = [s.collect(60) for s in streams]
    if rank == 0:
        result["tokens"] = [o[0] for o in outs]
        result["terminals"] = [o[1].kind if hasattr(o[1], "kind") else str(o[1]) for o in outs]
        result["messages"] = [getattr(o[1], "message", "") for o in outs]
        if mode != "rank_loss":
            eng.shutdown()
        with open(out_path, "w") as f:
            json.dump(result, f)
    else:
        deadline = time.monotonic() + 90
        while eng.healthy() and time.monotonic() < deadline:
            time.sleep(0.05)
        if mode == "abort":
            with open(f"{out_path}.rank{rank}", "w") as f:
                json.dump({"rank": rank, "batches": batches}, f)
    sys.stdout.flush()
    os._exit(0)  # a peer may be gone: skip the process-group teardown


if __name__ == "__main__":
    main()
