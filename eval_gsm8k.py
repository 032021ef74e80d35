#!/usr/bin/env python
"""GSM8K-style accuracy check against an OpenAI-compatible endpoint.

    python eval_gsm8k.py --url http://127.0.0.1:8000 --model qwen3-4b --data gsm8k_test.jsonl --limit 200
    python eval_gsm8k.py --spawn sim --data my.jsonl            # self-contained plumbing check on the CPU fake engine

``--data`` is a local JSON-lines file with ``question`` and ``answer`` fields (the GSM8K layout: the gold
answer ends in ``#### <number>``); nothing is downloaded.  Each question is sent to
``/v1/chat/completions`` (or ``/v1/completions`` with ``--raw``) with greedy decoding; the model's final
number is extracted with the strict rule (the number after the last ``####``, else after "answer is", else
the last number in the text) and compared with the gold number after normalisation (commas, ``$``,
trailing ``.0``).  Thinking models: everything up to ``</think>`` is dropped before extraction.
Prints accuracy, the number of requests that failed, and writes per-sample records with ``--out``.

Takes the place of the reference's scripts/eval_gsm8k_thinking.py (strict-match GSM8K, reported in
docs/benchmarks/accuracy-eval-results.md).
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import json
import os
import re
import sys
import urllib.request

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

_NUM = re.compile(r"-?\$?\d[\d,]*\.?\d*")


def normalize(num: str):
    s = num.replace(",", "").replace("$", "").strip().rstrip(".")
    try:
        v = float(s)
    except ValueError:
        return None
    return int(v) if v == int(v) else v


def gold_answer(answer: str):
    tail = answer.split("####")[-1]
    m = _NUM.search(tail)
    return normalize(m.group(0)) if m else None


def extract_answer(text: str):
    """Strict-first extraction of the final number from a completion."""
    if "</think>" in text:
        text = text.split("</think>")[-1]
    if "####" in text:
        m = _NUM.search(text.split("####")[-1])
        if m:
            return normalize(m.group(0))
    m = re.search(r"answer is[^\d\-$]*(-?\$?\d[\d,]*\.?\d*)", text, flags=re.I)
    if m:
        return normalize(m.group(1))
    nums = _NUM.findall(text)
    return normalize(nums[-1]) if nums else None


PROMPT = "Solve the problem step by step and finish with a line of the form '#### <number>'.\n\nQuestion: {q}\nAnswer:"


def ask(url: str, model: str, question: str, max_tokens: int, raw: bool, timeout: float) -> str:
    if raw:
        body = {"model": model, "prompt": PROMPT.format(q=question), "max_tokens": max_tokens, "temperature": 0.0}
        path = "/v1/completions"
    else:
        body = {"model": model, "messages": [{"role": "user", "content": PROMPT.format(q=question)}], "max_tokens": max_tokens, "temperature": 0.0}
        path = "/v1/chat/completions"
    req = urllib.request.Request(url.rstrip("/") + path, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        out = json.loads(r.read())
    ch = out["choices"][0]
    return ch["text"] if raw else (ch["message"].get("content") or "")


def evaluate(url: str, model: str, rows: list, max_tokens: int = 1024, raw: bool = False, workers: int = 16, timeout: float = 600.0) -> dict:
    records = []

    def one(row):
        gold = gold_answer(row["answer"])
        try:
            text = ask(url, model, row["question"], max_tokens, raw, timeout)
            pred = extract_answer(text)
            return {"question": row["question"], "gold": gold, "pred": pred, "correct": pred is not None and gold is not None and abs(float(pred) - float(gold)) < 1e-6, "error": None, "completion": text}
        except Exception as exc:  # a failed request counts as wrong and is reported
            return {"question": row["question"], "gold": gold, "pred": None, "correct": False, "error": repr(exc), "completion": ""}

    with cf.ThreadPoolExecutor(workers) as ex:
        records = list(ex.map(one, rows))
    n = len(records)
    return {"n": n, "correct": sum(r["correct"] for r in records), "accuracy": (sum(r["correct"] for r in records) / n) if n else 0.0, "failed_requests": sum(r["error"] is not None for r in records),
            "records": records}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="strict-match GSM8K-style evaluation over HTTP")
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="default")
    ap.add_argument("--data", required=True, help="JSON lines with `question` and `answer` (gold ends in '#### <number>')")
    ap.add_argument("--limit", type=int, default=0)
    ap.add_argument("--max-tokens", type=int, default=1024)
    ap.add_argument("--workers", type=int, default=16)
    ap.add_argument("--raw", action="store_true", help="use /v1/completions instead of the chat route")
    ap.add_argument("--spawn", choices=["sim"], help="serve the CPU fake engine in-process (plumbing check)")
    ap.add_argument("--out", help="write per-sample records (JSON lines)")
    a = ap.parse_args(argv)
    rows = [json.loads(l) for l in open(a.data) if l.strip()]
    if a.limit:
        rows = rows[: a.limit]
    server = None
    if a.spawn == "sim":
        from bench_serving import spawn_sim

        port = 21000 + os.getpid() % 2000
        _, server, _ = spawn_sim(port)
        a.url, a.model, a.raw = f"http://127.0.0.1:{port}", "sim", True
    res = evaluate(a.url, a.model, rows, a.max_tokens, a.raw, a.workers)
    print(f"GSM8K strict match: {res['correct']} / {res['n']} = {100 * res['accuracy']:.2f} %   (failed requests: {res['failed_requests']})")
    if a.out:
        with open(a.out, "w") as f:
            for r in res["records"]:
                f.write(json.dumps(r) + "\n")
    if server is not None:
        server.should_exit = True
    return 0


if __name__ == "__main__":
    sys.exit(main())
