"""Speculative decoding throughput and acceptance on one GPU.

Runs the same greedy workload through the engine without drafts and with each drafter, and prints one JSON line
per arm: output tokens per second over the decode phase, draft rounds, mean accepted drafts per round and the
share of verify steps that were CUDA-graph replays.  Weights are random (there is no checkpoint here), so the
block / chain drafters propose tokens the target almost never accepts: those arms show what a round costs.
``draft-self`` drafts with a copy of the target itself (every draft is accepted): it shows the acceptance
accounting and the upper end of the tokens-per-verify-step range.  Token-for-token equality with plain decoding is
what the tests check (under the batch-invariant policy); with random weights the logits are nearly flat, so the arms
here, which run different kernel shapes, need not pick the same tokens.

    python bench_spec.py --preset qwen3-8b --conc 16 --prompt-len 512 --max-tokens 96
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def run(args, method, path, draft_len):
    from pegainfer_b200.config import EngineConfig, preset
    from pegainfer_b200.engine.build import build_engine
    from pegainfer_b200.engine.contract import SamplingParams

    kw = {}
    if method:
        kw = dict(spec_method=method, draft_model_path=path, spec_draft_len=draft_len)
    mcfg = preset(args.preset)
    ecfg = EngineConfig(preset=args.preset, cuda_graph=True, max_decode_batch=args.conc, max_model_len=args.prompt_len + args.max_tokens + 64, max_prefill_tokens=4096,
                        num_kv_blocks=args.conc * ((args.prompt_len + args.max_tokens + 64) // 16 + 2) + 8, **kw)
    eng = build_engine(ecfg, mcfg, device="cuda:0", dtype=torch.bfloat16)
    try:
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, mcfg.vocab_size, (args.prompt_len,), generator=g).tolist() for _ in range(args.conc)]
        sp = SamplingParams(temperature=0.0, ignore_eos=True)
        warm = [torch.randint(0, mcfg.vocab_size, (args.prompt_len,), generator=g).tolist() for _ in range(args.conc)]
        eng.generate(warm, sp, max_tokens=8)  # warm-up with a full batch of other prompts: every graph bucket the timed run uses is captured here
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        first = eng.generate(prompts, sp, max_tokens=1)
        torch.cuda.synchronize()
        t_prefill = time.perf_counter() - t0
        t0 = time.perf_counter()
        outs = eng.generate(prompts, sp, max_tokens=args.max_tokens)
        torch.cuda.synchronize()
        t_all = time.perf_counter() - t0
        toks = sum(len(o[0]) for o in outs)
        c = eng.scheduler._metrics.spec_decode
        spec = eng.scheduler.spec
        g_ = eng.executor._graphs
        row = dict(arm=method or "none", drafter=path, tok_per_s=round((toks - len(first)) / max(t_all - t_prefill, 1e-9), 1), out_tokens=toks, total_s=round(t_all, 3),
                   prefill_s=round(t_prefill, 3), rounds=c.num_drafts, drafts_per_round=(c.num_draft_tokens / c.num_drafts if c.num_drafts else 0),
                   accepted_per_round=round(c.num_accepted_tokens / c.num_drafts, 3) if c.num_drafts else 0.0, tokens_per_round=round(1 + c.num_accepted_tokens / c.num_drafts, 3) if c.num_drafts else 1.0,
                   graph_replays=g_.replays if g_ is not None else 0, verify_span=getattr(eng.executor, "verify_span", 0), first_tokens=outs[0][0][:6])
        print(json.dumps(row), flush=True)
        return row
    finally:
        eng.shutdown()
        del eng
        torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="qwen3-8b")
    ap.add_argument("--conc", type=int, default=16)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--max-tokens", type=int, default=96)
    ap.add_argument("--arms", default="none,draft-self,dflash,dspark,eagle3")
    a = ap.parse_args()
    arms = {
        "none": (None, None, 0),
        "draft-self": ("draft", f"preset:{a.preset}:seed=0", 3),  # the target's own weights (engine seed 0): every draft is accepted
        "dflash": ("dflash", "random:layers=2,block=4", 3),
        "dspark": ("dspark", "random:layers=2,block=4,markov=64", 4),
        "eagle3": ("eagle3", "random:draft_vocab=32768", 3),
    }
    for name in a.arms.split(","):
        run(a, *arms[name])


if __name__ == "__main__":
    main()
