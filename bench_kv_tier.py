#!/usr/bin/env python
"""Time to first token with a warm prefix: GPU prefix cache, host-tier restore, cold prefill.

    python bench_kv_tier.py [--preset qwen3-4b] [--lens 1024,4096,16384] [--reps 3]

For each prompt length three requests are timed through ``Engine.submit`` (TTFT = submit to first
token on the host): cold (nothing cached), GPU-warm (same prompt again: prefix-cache hit on the GPU),
host-warm (the prompt's blocks were saved to pinned host memory and evicted from the GPU pool, so
they are copied back before the remaining tokens prefill).  The prompt's last 16 tokens differ between
the runs of one length so that at least one chunk is always computed.

The reference reports the same three numbers for Qwen3-4B on an RTX 5090
(docs/models/qwen3/serving-performance.md:90-110: warm 9.2 / 12.7 / 26.3 ms, host restore
15.4 / 37.5 / 125.5 ms, cold 44.0 / 211.5 / 1143.9 ms at 1k / 4k / 16k tokens).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main() -> int:
    import torch

    from pegainfer_b200.config import EngineConfig, preset
    from pegainfer_b200.engine.build import build_engine
    from pegainfer_b200.engine.contract import Request, SamplingParams

    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="qwen3-4b")
    ap.add_argument("--lens", default="1024,4096,16384")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    lens = [int(v) for v in a.lens.split(",")]
    mcfg = preset(a.preset)
    page = 16
    blocks = 3 * (max(lens) // page + 8)
    ecfg = EngineConfig(preset=a.preset, num_kv_blocks=blocks, kv_page_size=page, cuda_graph=True, max_decode_batch=8, max_model_len=max(lens) + 64, max_prefill_tokens=4096, kv_offload=True,
                        kv_offload_host_gib=max(4.0, 3e-9 * max(lens) * 40 * 2 * 8 * 128 * 2))
    eng = build_engine(ecfg, mcfg, device="cuda:0", dtype=torch.bfloat16)
    ht = eng.host_tier
    g = torch.Generator().manual_seed(0)

    def ttft(tokens):
        t0 = time.perf_counter()
        s = eng.submit(Request(prompt_tokens=tokens, params=SamplingParams(temperature=0.0, ignore_eos=True), max_tokens=2))
        first = None
        for upd in s:
            if upd.tokens and first is None:
                first = time.perf_counter() - t0
            if upd.terminal is not None:
                break
        return 1e3 * first

    rows = []
    try:
        ttft(torch.randint(0, mcfg.vocab_size, (256,), generator=g).tolist())  # warm-up: graphs, kernels
        for n in lens:
            cold, warm, host = [], [], []
            for _ in range(a.reps):
                base = torch.randint(0, mcfg.vocab_size, (n,), generator=g).tolist()
                tail = lambda k: base[:-16] + torch.randint(0, mcfg.vocab_size, (16,), generator=g).tolist()
                ht.l1_retention_disabled = False
                cold.append(ttft(tail(0)))
                warm.append(ttft(tail(1)))
                ht.flush_saves_then(lambda: None)
                ht.l1_retention_disabled = True  # the next probe first evicts idle GPU blocks: only the host copy is left
                host.append(ttft(tail(2)))
            med = lambda xs: sorted(xs)[len(xs) // 2]
            rows.append({"prompt_tokens": n, "cold_ttft_ms": round(med(cold), 2), "gpu_warm_ttft_ms": round(med(warm), 2), "host_restore_ttft_ms": round(med(host), 2)})
            print(rows[-1], flush=True)
        print(json.dumps({"model": a.preset, "rows": rows, "host_tier": {"saves": ht.stats.saves, "loads": ht.stats.loads, "host_hits": ht.stats.host_hits, "load_failures": ht.stats.load_failures}}))
        if a.json:
            json.dump(rows, open(a.json, "w"), indent=1)
    finally:
        eng.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
