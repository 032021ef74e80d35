"""HTTP behaviour against the simulated engine (no GPU, token-id prompts)."""
import json
import threading
import time

import pytest
from fastapi.testclient import TestClient

from pegainfer_b200.server.openai import Frontend, create_app
from pegainfer_b200.server.tokenizer import IdTokenizer
from pegainfer_b200.sim.fake import SimConfig, make_sim_engine


def make(cfg=None, partitions=1, declared=None):
    eng = make_sim_engine(cfg or SimConfig(), partitions=partitions, model_name="sim-model")
    fe = Frontend(eng, IdTokenizer(), "sim-model", declared_engines=declared)
    return eng, TestClient(create_app(fe))


def sse_events(text):
    return [blk[len("data: "):] for blk in text.split("\n\n") if blk.startswith("data: ")]


def test_health_models_and_completion():
    eng, c = make()
    try:
        assert c.get("/health").status_code == 200
        assert any(m["id"] == "sim-model" for m in c.get("/v1/models").json()["data"])
        r = c.post("/v1/completions", json={"prompt": [1, 2], "max_tokens": 4, "temperature": 0.0, "ignore_eos": True})
        assert r.status_code == 200
        body = r.json()
        assert body["choices"][0]["text"] == "<1><2><1><2>"
        assert body["choices"][0]["finish_reason"] == "length"
        assert body["usage"] == {"prompt_tokens": 2, "completion_tokens": 4, "total_tokens": 6, "prompt_tokens_details": {"cached_tokens": 0}}
    finally:
        eng.shutdown()


def test_streaming_has_exactly_one_done_and_usage_chunk():
    eng, c = make()
    try:
        r = c.post("/v1/completions", json={"prompt": [5, 6, 7], "max_tokens": 5, "stream": True, "stream_options": {"include_usage": True}})
        assert r.headers["content-type"].startswith("text/event-stream")
        ev = sse_events(r.text)
        assert ev.count("[DONE]") == 1 and ev[-1] == "[DONE]"
        chunks = [json.loads(e) for e in ev[:-1]]
        usage_chunks = [ch for ch in chunks if ch.get("usage")]
        assert len(usage_chunks) == 1 and usage_chunks[0]["choices"] == [] and chunks[-1] is usage_chunks[0]
        assert "".join(ch["choices"][0]["text"] for ch in chunks if ch["choices"]) == "<5><6><7><5><6>"
        assert chunks[-2]["choices"][0]["finish_reason"] == "length"
    finally:
        eng.shutdown()


def test_chat_completion_and_stream():
    eng, c = make(SimConfig(script=[72, 105]))
    try:
        msgs = [{"role": "user", "content": "hi"}]
        r = c.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 3}).json()
        assert r["object"] == "chat.completion"
        ch = r["choices"][0]
        assert ch["message"]["role"] == "assistant" and ch["message"]["content"] and ch["finish_reason"] == "length"
        u = r["usage"]
        assert u["prompt_tokens"] > 0 and u["completion_tokens"] == 3 and u["total_tokens"] == u["prompt_tokens"] + 3
        rs = c.post("/v1/chat/completions", json={"messages": msgs, "max_tokens": 3, "stream": True})
        ev = sse_events(rs.text)
        assert ev[-1] == "[DONE]" and ev.count("[DONE]") == 1
        chunks = [json.loads(e) for e in ev[:-1]]
        assert all(x["object"] == "chat.completion.chunk" for x in chunks)
        assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
        text = "".join(x["choices"][0]["delta"].get("content") or "" for x in chunks)
        assert text == ch["message"]["content"]
        assert chunks[-1]["choices"][0]["finish_reason"] == "length"
    finally:
        eng.shutdown()


def test_unsupported_params_are_rejected_not_ignored():
    eng, c = make()
    try:
        base = {"prompt": [1], "max_tokens": 1}
        for extra in ({"frequency_penalty": 0.5}, {"presence_penalty": 1.0}, {"repetition_penalty": 1.2}, {"min_p": 1.5}, {"n": 2}, {"vllm_xargs": {"pegainfer_lora_adapter": 7}}):
            assert c.post("/v1/completions", json={**base, **extra}).status_code == 400, extra
        # the server keeps serving after a bad request
        assert c.post("/v1/completions", json=base).status_code == 200
        # unknown adapter fails only that request
        assert c.post("/v1/completions", json={**base, "vllm_xargs": {"pegainfer_lora_adapter": "nope"}}).status_code == 400
        assert c.post("/v1/completions", json=base).status_code == 200
        assert c.post("/v1/completions", json={"prompt": [], "max_tokens": 1}).status_code == 400
    finally:
        eng.shutdown()


def test_metrics_gauges_and_partitions():
    eng, c = make(SimConfig(base_ttft_s=3.0, tpot_s=0.1), partitions=2, declared=2)  # a window of seconds: the polls below share the machine with other tests
    try:
        out = {}

        def slow():
            out["r"] = c.post("/v1/completions", json={"prompt": [1, 2, 3], "max_tokens": 3})

        t = threading.Thread(target=slow)
        t.start()
        # deadlines, not iteration counts: on a loaded machine the poster thread may start late.  The gauges are read
        # through a client of their own: one test client runs its requests one after the other, so a GET behind the slow
        # POST on the same client would only be answered once the request is over
        watcher = TestClient(c.app)
        seen_running, polls, m, t_start = False, 0, "", time.monotonic()
        deadline = time.monotonic() + 20.0
        while time.monotonic() < deadline and t.is_alive():
            m = watcher.get("/metrics").text
            polls += 1
            if 'vllm:num_requests_running{engine="0",model_name="sim-model"} 1' in m or 'vllm:num_requests_running{engine="1",model_name="sim-model"} 1' in m:
                seen_running = True
                break
            time.sleep(0.01)
        t.join()
        assert seen_running and out["r"].status_code == 200, (seen_running, polls, time.monotonic() - t_start, out["r"].status_code, out["r"].text[:200], m[-600:])
        idle = ['vllm:num_requests_running{engine="%d",model_name="sim-model"} 0' % i for i in (0, 1)]
        deadline = time.monotonic() + 10.0
        m = c.get("/metrics").text
        while not all(line in m for line in idle) and time.monotonic() < deadline:  # gauges are published once per driver iteration
            time.sleep(0.02)
            m = c.get("/metrics").text
        for eng_idx in (0, 1):
            assert f'vllm:num_requests_running{{engine="{eng_idx}",model_name="sim-model"}} 0' in m
            assert f'vllm:num_requests_waiting{{engine="{eng_idx}",model_name="sim-model"}}' in m
            assert f'vllm:kv_cache_usage_perc{{engine="{eng_idx}",model_name="sim-model"}}' in m
        assert 'vllm:generation_tokens_total{model_name="sim-model"} 3' in m
        assert "vllm:time_to_first_token_seconds_count" in m
        # explicit partition routing
        assert c.post("/v1/completions", json={"prompt": [1], "max_tokens": 1, "data_parallel_rank": 1}).status_code == 200
        assert c.post("/v1/completions", json={"prompt": [1], "max_tokens": 1, "data_parallel_rank": 5}).status_code == 400
    finally:
        eng.shutdown()


def test_partition_count_mismatch_fails_startup():
    eng = make_sim_engine(SimConfig(), partitions=1)
    try:
        with pytest.raises(RuntimeError, match="declared 2 engines but the launched engine exposes 1 schedulers"):
            Frontend(eng, IdTokenizer(), "sim", declared_engines=2)
    finally:
        eng.shutdown()


def test_stop_string_and_stop_token_and_logprob_shapes():
    eng, c = make(SimConfig(script=[10, 11, 12, 13]))
    try:
        r = c.post("/v1/completions", json={"prompt": [1], "max_tokens": 8, "stop": ["<12>"]}).json()
        assert r["choices"][0]["text"] == "<10><11>" and r["choices"][0]["finish_reason"] == "stop"
        r = c.post("/v1/completions", json={"prompt": [1], "max_tokens": 8, "stop_token_ids": [12]}).json()
        assert r["choices"][0]["text"] == "<10><11>" and r["choices"][0]["finish_reason"] == "stop"
        r = c.post("/v1/completions", json={"prompt": [[1, 2], [3]], "max_tokens": 2}).json()
        assert [ch["index"] for ch in r["choices"]] == [0, 1]
    finally:
        eng.shutdown()


def test_tool_call_roundtrip_stream_and_non_stream():
    call = '<tool_call>\n{"name": "get_weather", "arguments": {"city": "Paris"}}\n</tool_call>'
    tok = IdTokenizer()

    class CharTok(IdTokenizer):
        def decode(self, ids):
            return "".join(chr(i) for i in ids)

        def encode(self, text):
            return [ord(ch) for ch in text]

    script = [ord(ch) for ch in call]
    eng = make_sim_engine(SimConfig(script=script, eos_token_ids=()), model_name="sim-model")
    fe = Frontend(eng, CharTok(), "sim-model")
    c = TestClient(create_app(fe))
    try:
        tools = [{"type": "function", "function": {"name": "get_weather", "parameters": {}}}]
        body = {"messages": [{"role": "user", "content": "weather?"}], "tools": tools, "max_tokens": len(script)}
        r = c.post("/v1/chat/completions", json=body).json()
        tc = r["choices"][0]["message"]["tool_calls"]
        assert tc[0]["function"]["name"] == "get_weather" and json.loads(tc[0]["function"]["arguments"]) == {"city": "Paris"}
        rs = c.post("/v1/chat/completions", json={**body, "stream": True})
        chunks = [json.loads(e) for e in sse_events(rs.text)[:-1]]
        calls = [x["choices"][0]["delta"]["tool_calls"][0] for x in chunks if x["choices"] and x["choices"][0]["delta"].get("tool_calls")]
        assert len(calls) == 1 and calls[0]["function"]["name"] == "get_weather"
        assert not any("<tool_call>" in (x["choices"][0]["delta"].get("content") or "") for x in chunks if x["choices"])
    finally:
        eng.shutdown()


def test_fatal_step_fails_requests_instead_of_hanging():
    eng, c = make(SimConfig(base_ttft_s=0.2))
    try:
        eng.sim_schedulers[0].fatal_next_step = True
        r = c.post("/v1/completions", json={"prompt": [1], "max_tokens": 2})
        assert r.status_code == 500
        assert c.get("/health").status_code == 503
    finally:
        eng.shutdown()


def test_serving_bench_harness_against_sim_engine(tmp_path):
    """The HTTP load generator reports every request and sane latency percentiles."""
    import json
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench_serving

    assert bench_serving.percentiles([1.0, 2.0, 3.0, 4.0])["p50"] in (2.0, 3.0)
    out = tmp_path / "r.json"
    rc = bench_serving.main(["--spawn", "sim", "--num-prompts", "12", "--input-len", "24", "--output-len", "6", "--concurrency", "3", "--warmup", "1", "--json", str(out)])
    assert rc == 0
    r = json.loads(out.read_text())
    assert r["completed"] == 12 and r["failed"] == 0
    assert r["output_tokens"] == 12 * 6 and r["input_tokens"] == 12 * 24
    assert r["ttft_ms"]["p50"] > 0 and r["e2el_ms"]["p99"] >= r["ttft_ms"]["p50"]


def test_waiting_updates_fold_into_one_event():
    """A connection that fell behind gets everything that is waiting as one update: tokens in
    order, logprobs aligned to them, the terminal last."""
    import asyncio

    from pegainfer_b200.engine.contract import FinishReason, RequestUpdate, Terminal, TokenLogprob
    from pegainfer_b200.server.openai import _merge_updates

    async def go():
        q = asyncio.Queue()
        q.put_nowait(RequestUpdate(id=7, tokens=[3], logprobs=[TokenLogprob(token=3, logprob=-0.5, top=[])]))
        q.put_nowait(RequestUpdate(id=7, tokens=[4, 5], cached_tokens=16))
        q.put_nowait(RequestUpdate(id=7, tokens=[6], terminal=Terminal.finished(FinishReason.LENGTH)))
        q.put_nowait(RequestUpdate(id=7, tokens=[99]))  # never merged: it follows the terminal
        first = RequestUpdate(id=7, tokens=[1, 2])
        return _merge_updates(first, q), q.qsize()

    m, left = asyncio.run(go())
    assert m.tokens == [1, 2, 3, 4, 5, 6] and left == 1
    assert [None if l is None else l.token for l in m.logprobs] == [None, None, 3, None, None, None]
    assert m.cached_tokens == 16 and m.terminal.finish_reason == FinishReason.LENGTH
