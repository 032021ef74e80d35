#!/usr/bin/env python
"""HTTP serving benchmark against an OpenAI-compatible ``/v1/completions`` endpoint.

    python bench_serving.py --url http://127.0.0.1:8000 --num-prompts 256 --input-len 1024 --output-len 256 --concurrency 64
    python bench_serving.py --url ... --request-rate 8            # open loop, Poisson arrivals
    python bench_serving.py --url ... --qps-sweep 1,2,4,8,16      # one open-loop run per rate, one table row each
    python bench_serving.py --spawn sim --num-prompts 64           # self-contained: serves the CPU fake engine

Prompts are uniform-random token ids sent as ``prompt: [int, ...]`` (no tokenizer in the
loop), ``ignore_eos`` so that every request produces exactly ``--output-len`` tokens, and
``stream: true`` so that time to first token (TTFT) and inter-token latency (ITL) are seen
from the client.  Closed loop = ``--concurrency`` requests in flight; open loop =
``--request-rate`` requests per second with exponential gaps (``--concurrency`` then caps
the number in flight).  Definitions: TTFT = first content chunk minus send; TPOT =
(last chunk minus first chunk) / (output tokens - 1); ITL = gap between consecutive
content chunks; E2EL = last chunk minus send; output throughput = all output tokens /
wall time of the run.  Prints a table and one JSON line; ``--json`` also writes it.

Takes the place of the reference's scripts/bench_http_serving.py, bench_http_common.py
and tools/bench/run_serving_bench.sh (same metrics, same percentile set).
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import random
import sys
import threading
import time
from dataclasses import dataclass, field

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


@dataclass
class RequestTrace:
    send: float = 0.0
    first: float = 0.0
    last: float = 0.0
    chunks: list = field(default_factory=list)  # arrival time of every content chunk
    out_tokens: int = 0
    prompt_tokens: int = 0
    cached_tokens: int = 0
    ok: bool = False
    error: str = ""


def percentiles(xs, ps=(50, 90, 95, 99)):
    if not xs:
        return {f"p{p}": None for p in ps} | {"mean": None}
    s = sorted(xs)
    out = {"mean": sum(s) / len(s)}
    for p in ps:
        k = min(len(s) - 1, max(0, int(round(p / 100.0 * (len(s) - 1)))))
        out[f"p{p}"] = s[k]
    return out


def summarize(traces, wall_s: float) -> dict:
    good = [t for t in traces if t.ok]
    ttft = [(t.first - t.send) * 1e3 for t in good if t.first > 0]
    tpot = [(t.last - t.first) * 1e3 / (t.out_tokens - 1) for t in good if t.out_tokens > 1 and t.first > 0]
    itl = [(b - a) * 1e3 for t in good for a, b in zip(t.chunks, t.chunks[1:])]
    e2el = [(t.last - t.send) * 1e3 for t in good]
    out_tok = sum(t.out_tokens for t in good)
    in_tok = sum(t.prompt_tokens for t in good)
    return {
        "completed": len(good),
        "failed": len(traces) - len(good),
        "duration_s": wall_s,
        "request_throughput": len(good) / wall_s if wall_s > 0 else 0.0,
        "output_tok_s": out_tok / wall_s if wall_s > 0 else 0.0,
        "total_tok_s": (out_tok + in_tok) / wall_s if wall_s > 0 else 0.0,
        "input_tokens": in_tok,
        "output_tokens": out_tok,
        "cached_tokens": sum(t.cached_tokens for t in good),
        "ttft_ms": percentiles(ttft),
        "tpot_ms": percentiles(tpot),
        "itl_ms": percentiles(itl),
        "e2el_ms": percentiles(e2el),
        "errors": sorted({t.error for t in traces if t.error})[:5],
    }


async def one_request(session, url: str, model: str, prompt: list, output_len: int, trace: RequestTrace, extra: dict) -> None:
    body = {"model": model, "prompt": prompt, "max_tokens": output_len, "stream": True, "ignore_eos": True, "temperature": 0.0,
            "stream_options": {"include_usage": True}}
    body.update(extra)
    trace.send = time.perf_counter()
    try:
        async with session.post(url + "/v1/completions", json=body) as resp:
            if resp.status != 200:
                trace.error = f"HTTP {resp.status}: {(await resp.text())[:200]}"
                return
            buf = b""
            async for chunk in resp.content.iter_any():
                now = time.perf_counter()
                buf += chunk
                while b"\n\n" in buf:
                    event, buf = buf.split(b"\n\n", 1)
                    if not event.startswith(b"data:"):
                        continue
                    data = event[5:].strip()
                    if data == b"[DONE]":
                        continue
                    obj = json.loads(data)
                    if obj.get("usage"):
                        u = obj["usage"]
                        trace.out_tokens = int(u.get("completion_tokens", trace.out_tokens))
                        trace.prompt_tokens = int(u.get("prompt_tokens", 0))
                        trace.cached_tokens = int((u.get("prompt_tokens_details") or {}).get("cached_tokens", 0))
                    if obj.get("choices"):
                        if not trace.first:
                            trace.first = now
                        trace.chunks.append(now)
                        trace.last = now
            if not trace.out_tokens:
                trace.out_tokens = len(trace.chunks)
            trace.ok = trace.first > 0
            if not trace.ok:
                trace.error = "no content chunk"
    except Exception as exc:  # connection errors are results, not crashes
        trace.error = repr(exc)[:200]


async def run_load(url: str, model: str, prompts: list, output_len: int, concurrency: int, request_rate: float, seed: int, extra: dict):
    import aiohttp

    traces = [RequestTrace() for _ in prompts]
    sem = asyncio.Semaphore(max(1, concurrency))
    rng = random.Random(seed)
    timeout = aiohttp.ClientTimeout(total=None, sock_read=600)
    conn = aiohttp.TCPConnector(limit=0)
    async with aiohttp.ClientSession(timeout=timeout, connector=conn) as session:

        async def guarded(i):
            async with sem:
                await one_request(session, url, model, prompts[i], output_len, traces[i], extra)

        t0 = time.perf_counter()
        tasks = []
        for i in range(len(prompts)):
            tasks.append(asyncio.create_task(guarded(i)))
            if request_rate > 0:
                await asyncio.sleep(rng.expovariate(request_rate))
        await asyncio.gather(*tasks)
        wall = time.perf_counter() - t0
    return traces, wall


def make_prompts(n: int, input_len: int, vocab: int, seed: int, shared_prefix: int = 0) -> list:
    rng = random.Random(seed)
    prefix = [rng.randrange(vocab) for _ in range(shared_prefix)]
    return [prefix + [rng.randrange(vocab) for _ in range(input_len - shared_prefix)] for _ in range(n)]


def spawn_sim(port: int):
    """Serve the CPU fake engine in a background thread (self-contained runs and tests)."""
    import uvicorn

    from pegainfer_b200.server.openai import Frontend, create_app
    from pegainfer_b200.server.tokenizer import IdTokenizer
    from pegainfer_b200.sim.fake import SimConfig, make_sim_engine

    eng = make_sim_engine(SimConfig(), model_name="sim")
    fe = Frontend(eng, IdTokenizer(), "sim")
    server = uvicorn.Server(uvicorn.Config(create_app(fe), host="127.0.0.1", port=port, log_level="warning"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    for _ in range(200):
        if server.started:
            break
        time.sleep(0.05)
    return eng, server, th


def print_table(r: dict) -> None:
    print(f"completed {r['completed']}  failed {r['failed']}  duration {r['duration_s']:.2f} s")
    print(f"request throughput {r['request_throughput']:.2f} req/s   output {r['output_tok_s']:.1f} tok/s   total {r['total_tok_s']:.1f} tok/s")
    print(f"{'':10s} {'mean':>9s} {'p50':>9s} {'p90':>9s} {'p95':>9s} {'p99':>9s}")
    for k in ("ttft_ms", "tpot_ms", "itl_ms", "e2el_ms"):
        v = r[k]
        f = lambda x: f"{x:9.2f}" if x is not None else f"{'-':>9s}"
        print(f"{k:10s} {f(v['mean'])} {f(v['p50'])} {f(v['p90'])} {f(v['p95'])} {f(v['p99'])}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="default")
    ap.add_argument("--num-prompts", type=int, default=128)
    ap.add_argument("--input-len", type=int, default=1024)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--concurrency", type=int, default=64)
    ap.add_argument("--request-rate", type=float, default=0.0, help="requests/s, Poisson arrivals (0 = closed loop)")
    ap.add_argument("--qps-sweep", default=None, help="comma-separated request rates: run the open-loop benchmark once per rate (fresh prompts each) and print one row per rate")
    ap.add_argument("--vocab", type=int, default=32000, help="prompt token ids are drawn from [0, vocab)")
    ap.add_argument("--shared-prefix", type=int, default=0, help="leading tokens shared by all prompts (prefix-cache runs)")
    ap.add_argument("--warmup", type=int, default=2, help="untimed requests sent first")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--extra", default="{}", help="JSON merged into every request body")
    ap.add_argument("--spawn", choices=["sim"], help="serve the CPU fake engine in-process and benchmark it")
    ap.add_argument("--json", help="write the result object to this path")
    args = ap.parse_args(argv)

    server = None
    if args.spawn == "sim":
        port = 18000 + os.getpid() % 2000
        _, server, _ = spawn_sim(port)
        args.url = f"http://127.0.0.1:{port}"
        args.model = "sim"
    extra = json.loads(args.extra)
    prompts = make_prompts(args.num_prompts, args.input_len, args.vocab, args.seed, args.shared_prefix)
    if args.warmup > 0:
        warm = make_prompts(args.warmup, min(args.input_len, 64), args.vocab, args.seed + 1)
        asyncio.run(run_load(args.url, args.model, warm, min(args.output_len, 4), args.warmup, 0.0, args.seed, extra))
    if args.qps_sweep:
        # the reference's QPS sweep (tools/bench/run_serving_bench.sh, scripts/qps_sweep.sh): Poisson arrivals at each
        # rate, different prompts per rate so that the prefix cache of one run does not serve the next
        rows = []
        for i, rate in enumerate(float(v) for v in args.qps_sweep.split(",")):
            ps = make_prompts(args.num_prompts, args.input_len, args.vocab, args.seed + 100 * (i + 1), args.shared_prefix)
            traces, wall = asyncio.run(run_load(args.url, args.model, ps, args.output_len, args.concurrency, rate, args.seed + i, extra))
            r = summarize(traces, wall)
            r["request_rate"] = rate
            rows.append(r)
        print(f"{'QPS':>6s} {'out tok/s':>10s} {'TTFT p50':>9s} {'TTFT p99':>9s} {'TPOT p50':>9s} {'TPOT p99':>9s} {'failed':>6s}   (ms)")
        for r in rows:
            ms = lambda d, k: "-" if d.get(k) is None else f"{d[k]:.1f}"
            print(f"{r['request_rate']:6.1f} {r['output_tok_s']:10.1f} {ms(r['ttft_ms'], 'p50'):>9s} {ms(r['ttft_ms'], 'p99'):>9s} {ms(r['tpot_ms'], 'p50'):>9s} {ms(r['tpot_ms'], 'p99'):>9s} {r['failed']:6d}")
        res = {"sweep": rows, "config": {"url": args.url, "num_prompts": args.num_prompts, "input_len": args.input_len, "output_len": args.output_len, "concurrency": args.concurrency}}
        print(json.dumps(res))
        if args.json:
            os.makedirs(os.path.dirname(os.path.abspath(args.json)) or ".", exist_ok=True)
            with open(args.json, "w") as f:
                json.dump(res, f, indent=1)
        if server is not None:
            server.should_exit = True
        return 0 if all(r["failed"] == 0 for r in rows) else 1
    traces, wall = asyncio.run(run_load(args.url, args.model, prompts, args.output_len, args.concurrency, args.request_rate, args.seed, extra))
    res = summarize(traces, wall)
    res["config"] = {"url": args.url, "num_prompts": args.num_prompts, "input_len": args.input_len, "output_len": args.output_len,
                     "concurrency": args.concurrency, "request_rate": args.request_rate, "shared_prefix": args.shared_prefix}
    print_table(res)
    print(json.dumps(res))
    if args.json:
        os.makedirs(os.path.dirname(os.path.abspath(args.json)) or ".", exist_ok=True)
        with open(args.json, "w") as f:
            json.dump(res, f, indent=1)
    if server is not None:
        server.should_exit = True
    return 0 if res["failed"] == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
