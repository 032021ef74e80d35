"""Worker for the multi-GPU tensor-parallel test (launched by torchrun, one rank per GPU)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from pegainfer_b200.config import preset
    from pegainfer_b200.kv.buffer import KvBuffer, KvLayout
    from pegainfer_b200.kv.request_kv import KvView
    from pegainfer_b200.models.qwen3 import Qwen3Model
    from pegainfer_b200.ops import cuda as K
    from pegainfer_b200.parallel.fused import make_fused_tp
    from pegainfer_b200.parallel.tp import SINGLE, TPContext
    from pegainfer_b200.sched.executor import SeqStep, build_meta

    mcfg = preset("qwen3-0.6b", num_layers=3, vocab_size=4096)
    page, npages = 16, 64
    tp_f = make_fused_tp(rank, world, dev, mcfg, max_tokens=512, wait_s=20.0, site_max_world=8)  # exercise the site kernels at every world size
    models = {
        "single": Qwen3Model(mcfg, device=dev, tp=SINGLE),
        "nccl": Qwen3Model(mcfg, device=dev, tp=TPContext(rank, world, comm="nccl")),
        "fused": Qwen3Model(mcfg, device=dev, tp=tp_f),
    }

    def kv_for(m):
        return KvBuffer(KvLayout(page_size=page, num_pages=npages, dtype=torch.bfloat16, **m.kv_geometry()), dev)

    kvs = {k: kv_for(m) for k, m in models.items()}
    g = torch.Generator().manual_seed(5)
    lens = [170, 33, 5]  # 208 rows: two-shot (reduce-scatter + all-gather) on 2..8 ranks; the decode steps below are one-shot
    prompts = [torch.randint(0, 4096, (n,), generator=g).tolist() for n in lens]
    pages = [list(range(1, 12)), [12, 13, 14], [15]]

    def run(name, seqs):
        tok, meta = build_meta(seqs, page, dev)
        return models[name].forward(tok, meta, kvs[name]).float()

    def check(tag, seqs):
        ref = run("single", seqs)
        out = {k: run(k, seqs) for k in ("nccl", "fused")}
        again = run("fused", seqs)
        torch.cuda.synchronize()
        assert torch.equal(out["fused"], again), f"{tag}: fused TP is not bit-reproducible"
        for k, v in out.items():
            err = (v - ref).abs()
            assert err.mean().item() < 0.03 and err.max().item() < 0.4, (tag, k, err.mean().item(), err.max().item())
        # every rank must hold the same logits (the reduction order is fixed, rows are broadcast)
        mine = out["fused"].contiguous()
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        assert all(torch.equal(gathered[0], t) for t in gathered), f"{tag}: ranks disagree"
        return ref, out

    prefill = [SeqStep(rid=i, input_tokens=p, start_pos=0, view=KvView(pages[i], len(p), page)) for i, p in enumerate(prompts)]
    check("prefill", prefill)
    # a chunk above the fused row limit takes the library all-reduce; results must agree as well
    big = [SeqStep(rid=9, input_tokens=torch.randint(0, 4096, (300,), generator=g).tolist(), start_pos=0, view=KvView(list(range(20, 39)), 300, page))]
    check("prefill300", big)
    decode = [SeqStep(rid=i, input_tokens=[7 + i], start_pos=lens[i], view=KvView(pages[i], lens[i] + 1, page)) for i in range(3)]
    check("decode3", decode)
    check("decode1", decode[:1])  # fewer rows than ranks: some ranks own nothing
    # CUDA-graph replay of the fused path (epoch flags need no reset)
    tok, meta = build_meta(decode, page, dev)
    eager = models["fused"].forward(tok, meta, kvs["fused"]).float()
    torch.cuda.synchronize()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        captured = models["fused"].forward(tok, meta, kvs["fused"])
    for _ in range(3):
        gr.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured.float(), eager), "graph replay differs from eager"
    assert K.read_status(dev) == 0, f"status {K.read_status(dev):#x}"
    dist.barrier()

    # The whole engine on every rank: scheduler thread, CUDA-graph decode with run-ahead, requests
    # that end at different lengths (rows are squeezed out between steps).  Every rank must read the
    # same tokens on the host: the scheduler thread of a rank other than 0 starts with GPU 0 as its
    # current device, and anything that follows "the current device" there goes wrong quietly.
    from pegainfer_b200.config import EngineConfig
    from pegainfer_b200.engine.build import build_engine
    from pegainfer_b200.engine.contract import Request, SamplingParams

    ecfg = EngineConfig(preset="qwen3-0.6b", num_kv_blocks=256, cuda_graph=True, max_decode_batch=8, max_model_len=512, max_prefill_tokens=256, no_prefix_cache=True)
    eng = build_engine(ecfg, mcfg, device=dev, dtype=torch.bfloat16, tp=tp_f, model=models["fused"], start=False)
    limits = [24, 7, 15, 24, 11]
    streams = [
        eng.submit(Request(prompt_tokens=torch.randint(0, 4096, (20 + 9 * i,), generator=g).tolist(), params=SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=n))
        for i, n in enumerate(limits)
    ]
    eng.start()  # all requests queued first: the replicated schedulers see the same admission order
    outs = [s.collect(120)[0] for s in streams]
    torch.cuda.synchronize()
    assert [len(o) for o in outs] == limits
    assert eng.executor._graphs.ahead_claimed > 10
    flat = torch.tensor([t for o in outs for t in o], dtype=torch.int64, device=dev)
    gathered = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    assert all(torch.equal(gathered[0], t) for t in gathered), "ranks read different tokens on the host"
    assert K.read_status(dev) == 0, f"status {K.read_status(dev):#x}"
    eng.shutdown()
    dist.barrier()
    if rank == 0:
        print("TP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
