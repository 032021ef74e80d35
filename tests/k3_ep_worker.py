"""Worker for the multi-GPU test of the Kimi-K3 line (one process per GPU, torchrun).

Every rank holds a different batch and 1/world of the routed experts; tokens, expert ids and weights are gathered over
NCCL, every rank runs its local latent experts, and the f32 outputs are reduce-scattered.  One prefill step and one decode
step must agree with a single-GPU model that holds every expert.  The routed output of this line is RMS-normalised, so
an expert choice that flips under a different summation order moves that token's logits by O(1): the check is on the
typical token (median of the per-token maximum error) and on the mean."""
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
    from pegainfer_b200.models.k3 import K3Model
    from pegainfer_b200.ops import cuda as K
    from pegainfer_b200.parallel.ep import LOCAL_EP, EPContext
    from pegainfer_b200.sched.executor import SeqStep, build_meta

    mcfg = preset("small-k3")
    page, npages = 16, 64
    models = {"single": K3Model(mcfg, device=dev, dtype=torch.bfloat16, ep=LOCAL_EP),
              "nccl": K3Model(mcfg, device=dev, dtype=torch.bfloat16, ep=EPContext(rank, world, comm="nccl", tokens="dp"))}
    assert models["nccl"].layers[1].experts["w13"].shape[0] == mcfg.n_routed_experts // world
    kvs = {k: m.make_kv(npages, page) for k, m in models.items()}
    for m in models.values():
        m.make_state(8)
    g = torch.Generator().manual_seed(100 + rank)  # every rank decodes its own sequences
    lens = [40, 9, 23]
    prompts = [torch.randint(0, mcfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    pages = [[1, 2, 3], [4], [5, 6]]

    def run(kind, seqs):
        tok, meta = build_meta(seqs, page, dev)
        meta.h_state_slots = [1, 2, 3]
        meta.state_slots = torch.tensor([1, 2, 3], dtype=torch.int32, device=dev)
        return models[kind].forward(tok, meta, kvs[kind]).float()

    def check(tag, seqs):
        ref, out = run("single", seqs), run("nccl", seqs)
        torch.cuda.synchronize()
        err = (out - ref).abs()
        typical = err.max(-1).values.median().item()
        assert typical < 0.12 and err.mean().item() < 0.05, (tag, typical, err.mean().item(), err.max().item())

    check("prefill", [SeqStep(rid=i, input_tokens=p, start_pos=0, view=KvView(pages[i], len(p), page)) for i, p in enumerate(prompts)])
    check("decode", [SeqStep(rid=i, input_tokens=[7 + i + rank], start_pos=lens[i], view=KvView(pages[i], lens[i] + 1, page)) for i in range(3)])
    assert K.read_status(dev) == 0, f"status {K.read_status(dev):#x}"
    dist.barrier()
    if rank == 0:
        print("K3_EP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
