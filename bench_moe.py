#!/usr/bin/env python
"""Decode benchmark for the MLA + MoE model line with expert parallelism.

    python -m torch.distributed.run --nproc-per-node N bench_moe.py --model dsv2-lite --conc 64 --prompt-len 512 --steps 64
    python bench_moe.py --model dsv2-lite            # one GPU, all experts local

Data-parallel attention (each rank decodes conc/N sequences, attention weights
replicated) with routed experts spread over the N ranks; ``--comm fused`` uses the
peer-memory dispatch / grouped-GEMM / combine kernels, ``--comm nccl`` the
all-gather + reduce-scatter baseline.  Device-timed (CUDA events, max over ranks) over
K CUDA-graph decode steps; prints one JSON line on rank 0.  Synthetic uniform-random
prompts, random-init weights (INT4 group-32 experts for the Kimi-K2 shape).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="dsv2-lite")
    ap.add_argument("--conc", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--layers", type=int, default=0, help="truncate the model (marks the result as a reduced configuration)")
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()

    import numpy as np
    import torch

    from bench import ClockSampler, barrier, init_dist, max_over_ranks
    from pegainfer_b200.config import preset
    from pegainfer_b200.kv.block_pool import BlockPool
    from pegainfer_b200.kv.request_kv import KvView
    from pegainfer_b200.models.mla_moe import MlaMoeModel
    from pegainfer_b200.ops import cuda as K
    from pegainfer_b200.parallel.ep import EPContext
    from pegainfer_b200.sched.executor import SeqStep, StepBatch, TorchExecutor, bucket_for

    rank, local, world = init_dist(args)
    device = torch.device("cuda", local)
    mcfg = preset(args.model)
    mcfg.num_mtp_layers = 0
    if args.layers:
        mcfg.num_layers = args.layers
    n_local = max(1, args.conc // world)
    page = 16
    chunk_tokens = 1024
    if world > 1 and args.comm == "fused":
        from pegainfer_b200.parallel.fused_ep import make_fused_ep

        ep = make_fused_ep(rank, world, device, mcfg, max_tokens=chunk_tokens)
    else:
        ep = EPContext(rank, world, comm="nccl", tokens="dp")
    t0 = time.perf_counter()
    model = MlaMoeModel(mcfg, device=device, dtype=torch.bfloat16, ep=ep)
    torch.cuda.synchronize(device)
    load_s = time.perf_counter() - t0
    total = args.warmup + args.steps
    need_pages = (args.prompt_len + total + page) // page + 1
    nblocks = n_local * need_pages + 8
    kv = model.make_kv(nblocks, page)
    pool = BlockPool(nblocks, page, enable_prefix_cache=False)
    ex = TorchExecutor(model, kv, page, cuda_graph=not args.no_graph, max_decode_batch=max(n_local, 8), max_blocks_per_seq=need_pages + 1)
    g = torch.Generator().manual_seed(100 + rank)
    prompts = torch.randint(0, mcfg.vocab_size, (n_local, args.prompt_len), generator=g)
    pages = [pool.allocate(need_pages) for _ in range(n_local)]
    per = max(1, chunk_tokens // args.prompt_len)
    first = [0] * n_local
    barrier(world, device)
    tp0 = time.perf_counter()
    for i in range(0, n_local, per):
        seqs = [SeqStep(rid=j, input_tokens=prompts[j].tolist(), start_pos=0, view=KvView(pages[j][: (args.prompt_len + page - 1) // page], args.prompt_len, page)) for j in range(i, min(n_local, i + per))]
        # every rank runs the same number of equally sized prefill batches, so the MoE collectives line up
        res = ex.execute(StepBatch(seqs=seqs, kind="prefill"))
        for j in range(i, min(n_local, i + per)):
            first[j] = res.tokens[j][0]
    torch.cuda.synchronize(device)
    prefill_s = time.perf_counter() - tp0
    graphs = ex._graphs
    pg = np.asarray(pages, dtype=np.int64)
    if graphs is not None:
        b = bucket_for(n_local, graphs.buckets)
        B = graphs.max_b
        if hasattr(ep, "valid_tokens"):
            ep.valid_tokens = torch.tensor([n_local], dtype=torch.int32, device=device)
        barrier(world, device)
        graphs.capture(b, True)  # capture runs on padding inputs and clears the input arena
        sched = torch.zeros((total, 3, b), dtype=torch.int32).pin_memory()
        sn = sched.numpy()
        for s in range(total):
            pos = args.prompt_len + s
            sn[s, 0, :n_local] = pos
            sn[s, 1, :n_local] = pg[:, pos // page] * page + pos % page
            sn[s, 2, :n_local] = pos + 1
        graphs.np_table[:n_local, :need_pages] = pg
        graphs.d_table.copy_(graphs.h_table)
        graphs.invalidate_table()
        graphs.d_small.zero_()
        graphs.d_small[:n_local].copy_(torch.tensor(first, dtype=torch.int32))
        graphs.d_small[B : B + b].copy_(sched[0, 0])
        graphs.d_small[2 * B : 2 * B + b].copy_(sched[0, 1])
        graphs.d_small[3 * B : 3 * B + b].copy_(sched[0, 2])
        gr = graphs.graphs[(b, True)]
        kernels = graphs.kernels_per_graph.get((b, True), 0)

        def step(s):
            graphs.d_small[B : B + b].copy_(sched[s, 0], non_blocking=True)
            graphs.d_small[2 * B : 2 * B + b].copy_(sched[s, 1], non_blocking=True)
            graphs.d_small[3 * B : 3 * B + b].copy_(sched[s, 2], non_blocking=True)
            gr.replay()
            graphs.d_small[:b].copy_(graphs.out_tokens[:b], non_blocking=True)
    else:
        cur = list(first)
        kernels = 0

        def step(s):
            pos = args.prompt_len + s
            seqs = [SeqStep(rid=j, input_tokens=[cur[j]], start_pos=pos, view=KvView(pages[j], pos + 1, page)) for j in range(n_local)]
            res = ex.execute(StepBatch(seqs=seqs, kind="decode"))
            for j in range(n_local):
                cur[j] = res.tokens[j][0]

    for s in range(args.warmup):
        step(s)
    barrier(world, device)
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    stream = torch.cuda.current_stream(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for s in range(args.warmup, total):
        step(s)
    e1.record(stream)
    barrier(world, device)
    clocks = sampler.stop()
    ms = max_over_ranks(e0.elapsed_time(e1), world, device)
    status = K.read_status(device)
    assert status == 0, f"device status word set: {status:#x}"
    if rank == 0:
        conc = n_local * world
        print(json.dumps({
            "metric": f"decode out tok/s per box @conc {conc} ({args.model} EP{world})",
            "value": round(conc * args.steps / (ms / 1e3), 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "strong", "dtype": "bf16" + ("+int4 experts" if mcfg.expert_quant == "int4_g32" else ""),
            "data": "synthetic uniform-random token prompts, random-init weights",
            "config": {"model": args.model + (f"[{args.layers} of {preset(args.model).num_layers} layers]" if args.layers else ""), "global_batch": conc, "seq_len": args.prompt_len,
                       "parallelism": f"dp{world}xep{world}-{args.comm if world > 1 else 'local'}", "cuda_graph": graphs is not None, "prefill_s": round(prefill_s, 3), "load_s": round(load_s, 1)},
            "clocks": clocks, "gpu_launches": kernels * args.steps,
        }))
    # orderly exit: the captured graphs pin kernels and buffers, peers' memory is unmapped only after every rank is past
    # its last kernel, then the process group goes
    import gc

    from bench import leave_group

    if graphs is not None:
        graphs.release()
    gr = None
    del ex, model, kv
    gc.collect()
    torch.cuda.synchronize(device)
    barrier(world, device)
    if hasattr(ep, "close"):
        ep.close()
    leave_group(world)


if __name__ == "__main__":
    main()
