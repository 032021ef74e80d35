"""Worker for the multi-GPU expert-parallel test (one process per GPU, torchrun).

Every rank holds a different batch (data-parallel attention) and 1/world of the routed
experts.  The fused path (dispatch / grouped GEMM with scatter-return / combine over peer
memory) must agree with the NCCL all-gather + reduce-scatter path and with a single-GPU
model that holds every expert, for bf16, INT4-g32 and block-scaled FP8 experts, eagerly
and under CUDA-graph replay."""
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
    from pegainfer_b200.kv.request_kv import KvView
    from pegainfer_b200.models.mla_moe import MlaMoeModel
    from pegainfer_b200.ops import cuda as K
    from pegainfer_b200.parallel.ep import LOCAL_EP, EPContext
    from pegainfer_b200.parallel.fused_ep import make_fused_ep
    from pegainfer_b200.sched.executor import SeqStep, build_meta

    page, npages = 16, 64
    for name in ("small-dsv2", "small-kimi", "small-dsv2-fp8"):
        mcfg = preset(name)
        mcfg.num_mtp_layers = 0
        ep_f = make_fused_ep(rank, world, dev, mcfg, max_tokens=128, wait_s=20.0)
        models = {
            "single": MlaMoeModel(mcfg, device=dev, dtype=torch.bfloat16, ep=LOCAL_EP),
            "nccl": MlaMoeModel(mcfg, device=dev, dtype=torch.bfloat16, ep=EPContext(rank, world, comm="nccl", tokens="dp")),
            "fused": MlaMoeModel(mcfg, device=dev, dtype=torch.bfloat16, ep=ep_f),
        }
        kvs = {k: m.make_kv(npages, page) for k, m in models.items()}
        g = torch.Generator().manual_seed(100 + rank)  # every rank decodes its own sequences
        lens = [40, 9, 23]
        prompts = [torch.randint(0, mcfg.vocab_size, (n,), generator=g).tolist() for n in lens]
        pages = [[1, 2, 3], [4], [5, 6]]

        def run(kind, seqs, pad_to=0):
            tok, meta = build_meta(seqs, page, dev, pad_to=pad_to)
            return models[kind].forward(tok, meta, kvs[kind]).float()

        def check(tag, seqs):
            ref = run("single", seqs)
            out = {k: run(k, seqs) for k in ("nccl", "fused")}
            again = run("fused", seqs)
            torch.cuda.synchronize()
            assert torch.equal(out["fused"], again), f"{name} {tag}: fused EP is not bit-reproducible"
            for k, v in out.items():
                err = (v - ref).abs()
                assert err.mean().item() < 0.03 and err.max().item() < 0.5, (name, tag, k, err.mean().item(), err.max().item())

        prefill = [SeqStep(rid=i, input_tokens=p, start_pos=0, view=KvView(pages[i], len(p), page)) for i, p in enumerate(prompts)]
        check("prefill", prefill)
        decode = [SeqStep(rid=i, input_tokens=[7 + i + rank], start_pos=lens[i], view=KvView(pages[i], lens[i] + 1, page)) for i in range(3)]
        check("decode", decode)
        # CUDA-graph replay of the fused path (epoch flags need no reset between replays)
        tok, meta = build_meta(decode, page, dev)
        eager = models["fused"].forward(tok, meta, kvs["fused"]).float()
        torch.cuda.synchronize()
        dist.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            captured = models["fused"].forward(tok, meta, kvs["fused"])
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize()
        assert torch.equal(captured.float(), eager), f"{name}: graph replay differs from eager"
        assert K.read_status(dev) == 0, f"{name}: status {K.read_status(dev):#x}"
        dist.barrier()
        del models, kvs, ep_f, gr
        torch.cuda.empty_cache()
    if rank == 0:
        print("EP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
