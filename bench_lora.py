"""Decode throughput with LoRA adapters, end to end through ``Engine.submit``.

Arms, same engine, same prompts, greedy, ``--conc`` requests of ``--prompt-len`` tokens generating ``--gen`` tokens:

  none      no request names an adapter (the adapter machinery is loaded but idle)
  one       every request uses the same adapter
  spread    the requests are spread over ``--adapters`` adapters
  mixed     half of the requests use an adapter, half do not

Adapters are random rank-``--rank`` matrices on q / k / v / o / gate / up / down of every layer, written as PEFT
directories and loaded through ``LoraManager``.  Prints one JSON line per arm (tokens per second over the whole run,
prefill included, and the decode-phase rate from the inter-token times).

    python bench_lora.py --model qwen3-8b --conc 64 --prompt-len 1024 --gen 128 --rank 16 --adapters 4

Reference parity: the reference's LoRA serving path (pegainfer-qwen3/src/lora.rs, per-request adapter slots in the
batched decode); it publishes no throughput figure for it.
"""
import argparse
import json
import os
import tempfile
import time

import torch


def write_adapter(path, cfg, rank, alpha, seed):
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    g = torch.Generator().manual_seed(seed)
    d, h = cfg.head_dim, cfg.hidden_size
    dims = {"q_proj": (h, cfg.num_q_heads * d), "k_proj": (h, cfg.num_kv_heads * d), "v_proj": (h, cfg.num_kv_heads * d), "o_proj": (cfg.num_q_heads * d, h),
            "gate_proj": (h, cfg.intermediate_size), "up_proj": (h, cfg.intermediate_size), "down_proj": (cfg.intermediate_size, h)}
    t = {}
    for li in range(cfg.num_layers):
        for p, (k_in, m_out) in dims.items():
            sub = "self_attn" if p.endswith(("q_proj", "k_proj", "v_proj", "o_proj")) else "mlp"
            base = f"base_model.model.model.layers.{li}.{sub}.{p}"
            t[base + ".lora_A.weight"] = (torch.randn(rank, k_in, generator=g) * 0.01).to(torch.bfloat16)
            t[base + ".lora_B.weight"] = (torch.randn(m_out, rank, generator=g) * 0.01).to(torch.bfloat16)
    save_file(t, os.path.join(path, "adapter_model.safetensors"))
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump({"r": rank, "lora_alpha": alpha, "target_modules": list(dims)}, f)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--conc", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--gen", type=int, default=128)
    ap.add_argument("--rank", type=int, default=16)
    ap.add_argument("--adapters", type=int, default=4)
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model")
    args = ap.parse_args()

    from pegainfer_b200.config import EngineConfig, preset
    from pegainfer_b200.engine.build import build_engine
    from pegainfer_b200.engine.contract import Request, SamplingParams
    from pegainfer_b200.lora.manager import LoraManager

    mcfg = preset(args.model, **({"num_layers": args.layers} if args.layers else {}))
    page = 16
    blocks = args.conc * ((args.prompt_len + args.gen + page) // page + 1) + 64
    ecfg = EngineConfig(preset=args.model, num_kv_blocks=blocks, kv_page_size=page, cuda_graph=True, max_decode_batch=max(args.conc, 8), max_model_len=args.prompt_len + args.gen + page,
                        max_prefill_tokens=4096, no_prefix_cache=True, enable_lora=True, max_loras=args.adapters, max_lora_rank=args.rank)
    eng = build_engine(ecfg, mcfg, device="cuda:0", dtype=torch.bfloat16)
    try:
        mgr = getattr(eng, "lora", None) or LoraManager(eng, max_loras=args.adapters, max_rank=args.rank)
        with tempfile.TemporaryDirectory() as tmp:
            for a in range(args.adapters):
                write_adapter(os.path.join(tmp, f"a{a}"), mcfg, args.rank, 2 * args.rank, seed=a)
                mgr.load(f"a{a}", os.path.join(tmp, f"a{a}"))
        g = torch.Generator().manual_seed(1)
        prompts = torch.randint(0, mcfg.vocab_size, (args.conc, args.prompt_len), generator=g).tolist()
        params = SamplingParams(temperature=0.0, ignore_eos=True)

        def run(pick):
            times = [[] for _ in prompts]

            def listener(i):
                def fn(upd):
                    if upd.tokens:
                        times[i].append(time.perf_counter())
                return fn

            torch.cuda.synchronize()
            t0 = time.perf_counter()
            streams = [eng.submit(Request(prompt_tokens=p, params=params, max_tokens=args.gen, lora_adapter=pick(i)), listener=listener(i)) for i, p in enumerate(prompts)]
            outs = [s.collect(600) for s in streams]
            dt = time.perf_counter() - t0
            ntok = sum(len(o[0]) for o in outs)
            assert all(o[1].kind == "finished" for o in outs), [o[1] for o in outs if o[1].kind != "finished"][:1]
            gaps = sorted(b - a for ts in times for a, b in zip(ts[len(ts) // 4 :], ts[len(ts) // 4 + 1 :]))
            itl = gaps[len(gaps) // 2] if gaps else 0.0
            return ntok / dt, itl

        arms = {"none": lambda i: None, "one": lambda i: "a0", "spread": lambda i: f"a{i % args.adapters}", "mixed": lambda i: ("a0" if i % 2 else None)}
        run(arms["spread"])  # warm-up: graph capture of both decode variants
        for name, pick in arms.items():
            tps, itl = run(pick)
            print(json.dumps({"arm": name, "model": args.model, "conc": args.conc, "prompt_len": args.prompt_len, "gen": args.gen, "rank": args.rank, "adapters": args.adapters,
                              "tok_per_s_end_to_end": round(tps, 1), "inter_token_ms_p50": round(itl * 1e3, 3), "decode_tok_per_s": round(args.conc / itl, 1) if itl else None}), flush=True)
    finally:
        eng.shutdown()


if __name__ == "__main__":
    main()
