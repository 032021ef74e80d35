"""Worker for the multi-GPU decode-chain tensor-parallel test (launched by torchrun, one rank per GPU).

The chain kernel sums the row-parallel projections over the ranks with multimem.ld_reduce on memory bound
to an NVSwitch multicast object.  A rank must not leave while that binding is live and peers still run, so
a failed check is recorded and the rank carries on through the same sequence of launches and collectives
as everybody else; the verdict is agreed at the end, the buffers are released after a barrier."""
import os
import sys
import traceback

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from pegainfer_b200.config import EngineConfig, preset
    from pegainfer_b200.engine.build import build_engine
    from pegainfer_b200.engine.contract import Request, SamplingParams
    from pegainfer_b200.kv.buffer import KvBuffer, KvLayout
    from pegainfer_b200.kv.request_kv import KvView
    from pegainfer_b200.models.qwen3 import Qwen3Model
    from pegainfer_b200.ops import cuda as K
    from pegainfer_b200.parallel.chain_tp import ChainTP
    from pegainfer_b200.parallel.tp import SINGLE, TPContext
    from pegainfer_b200.sched.executor import SeqStep, build_meta

    failures = []

    def note(msg):
        print(f"[rank {rank}] {msg}", flush=True)

    def expect(cond, msg):
        if not cond:
            failures.append(msg)

    mcfg = preset("qwen3-0.6b", num_layers=3, vocab_size=4096, num_q_heads=16, num_kv_heads=8)
    page, npages = 16, 96
    tp_c = ChainTP(rank, world, dev, mcfg.hidden_size, wait_s=3.0)
    note("symmetric buffer ready")
    models = {
        "single": Qwen3Model(mcfg, device=dev, tp=SINGLE),
        "nccl": Qwen3Model(mcfg, device=dev, tp=TPContext(rank, world, comm="nccl")),
        "chain": Qwen3Model(mcfg, device=dev, tp=tp_c),
    }
    expect(models["chain"].vocab_sharded and models["chain"].fused_decode, "the chain model should shard lm_head and run the fused decode path")
    kvs = {k: KvBuffer(KvLayout(page_size=page, num_pages=npages, dtype=torch.bfloat16, **m.kv_geometry()), dev) for k, m in models.items()}
    g = torch.Generator().manual_seed(5)
    lens = [170, 33, 5]
    prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in lens]
    pages = [list(range(1, 12)), [12, 13, 14], [15]]

    def run(name, seqs):
        tok, meta = build_meta(seqs, page, dev)
        return models[name].forward(tok, meta, kvs[name]).float()

    def check(tag, seqs):
        note(f"check {tag}")
        try:
            ref = run("single", seqs)
            out = {k: run(k, seqs) for k in ("nccl", "chain")}
            again = run("chain", seqs)
            torch.cuda.synchronize()
            expect(torch.equal(out["chain"], again), f"{tag}: the chain path is not bit-reproducible")
            for k, v in out.items():
                err = (v - ref).abs()
                expect(err.mean().item() < 0.03 and err.max().item() < 0.4, f"{tag} {k}: mean err {err.mean().item():.4f} max {err.max().item():.4f}")
            mine = out["chain"].contiguous()
            gathered = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(gathered, mine)
            expect(all(torch.equal(gathered[0], t) for t in gathered), f"{tag}: ranks hold different logits")
        except Exception:
            failures.append(f"{tag}: " + traceback.format_exc()[-1500:])

    prefill = [SeqStep(rid=i, input_tokens=p, start_pos=0, view=KvView(pages[i], len(p), page)) for i, p in enumerate(prompts)]
    check("prefill (library all-reduce)", prefill)
    decode = [SeqStep(rid=i, input_tokens=[7 + i], start_pos=lens[i], view=KvView(pages[i], lens[i] + 1, page)) for i in range(3)]
    check("decode3", decode)
    check("decode1", decode[:1])
    wide = [SeqStep(rid=20 + i, input_tokens=[3 + i], start_pos=0, view=KvView([40 + i], 1, page)) for i in range(40)]
    check("decode40", wide)
    expect(tp_c.sites_by_rows.get(3) == (2 * mcfg.num_layers, 0), f"decode steps should take the in-switch reduction: {tp_c.sites_by_rows}")
    note("graph replay")
    # CUDA-graph replay (exchange numbers live on the device: no reset between replays)
    try:
        tok, meta = build_meta(decode, page, dev)
        eager = models["chain"].forward(tok, meta, kvs["chain"]).float()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            captured = models["chain"].forward(tok, meta, kvs["chain"])
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize()
        expect(torch.equal(captured.float(), eager), "graph replay differs from eager")
        # a captured graph keeps a reference on the NCCL communicator of the collectives inside it (the
        # logits all-gather); the process group cannot be destroyed while such a graph is alive
        del gr, captured
    except Exception:
        failures.append("graph: " + traceback.format_exc()[-1500:])
    expect(K.read_status(dev) == 0, f"status {K.read_status(dev):#x}")
    dist.barrier()

    note("engine")
    # the whole engine on every rank: CUDA-graph decode with the sharded argmax, run-ahead, rows leaving
    try:
        ecfg = EngineConfig(preset="qwen3-0.6b", num_kv_blocks=256, cuda_graph=True, max_decode_batch=8, max_model_len=512, max_prefill_tokens=256, no_prefix_cache=True)
        eng = build_engine(ecfg, mcfg, device=dev, dtype=torch.bfloat16, tp=tp_c, model=models["chain"], start=False)
        limits = [24, 7, 15, 24, 11]
        reqs = [torch.randint(0, 4096, (20 + 9 * i,), generator=g).tolist() for i in range(len(limits))]
        streams = [eng.submit(Request(prompt_tokens=p, params=SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=n)) for p, n in zip(reqs, limits)]
        eng.start()
        outs = [s.collect(120)[0] for s in streams]
        torch.cuda.synchronize()
        expect([len(o) for o in outs] == limits, "wrong output lengths")
        flat = torch.tensor([t for o in outs for t in o], dtype=torch.int64, device=dev)
        gathered = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(gathered, flat)
        expect(all(torch.equal(gathered[0], t) for t in gathered), "ranks read different tokens on the host")
        eng.shutdown()
        graphs = eng.executor._graphs
        expect(graphs.replays > 10, "the decode graphs did not run")
        graphs.release()
    except Exception:
        failures.append("engine: " + traceback.format_exc()[-1500:])
    expect(K.read_status(dev) == 0, f"status after the engine run {K.read_status(dev):#x}")

    note("verdict")
    import faulthandler

    faulthandler.dump_traceback_later(25, exit=False)  # if the teardown below stalls, say where
    # agree on the verdict, then release the multicast-bound memory together
    torch.cuda.synchronize()
    bad = torch.tensor([len(failures)], dtype=torch.int32, device=dev)
    dist.all_reduce(bad)
    for f in failures:
        print(f"[rank {rank}] FAILED: {f}", flush=True)
    del models, kvs
    import gc

    gc.collect()
    dist.barrier()
    tp_c.close()
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0 and int(bad.item()) == 0:
        print("CHAIN_TP_OK", flush=True)
    note("leaving the process group")
    dist.destroy_process_group()
    note("exit")
    faulthandler.cancel_dump_traceback_later()
    sys.exit(0 if int(bad.item()) == 0 else 1)


if __name__ == "__main__":
    main()
