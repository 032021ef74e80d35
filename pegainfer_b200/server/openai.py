"""OpenAI-compatible HTTP frontend over the step-contract engine.

Routes: ``/health``, ``/v1/models``, ``/v1/completions`` (+SSE), ``/v1/chat/completions``
(+SSE, tool calls), ``/metrics``, ``/v1/load_lora_adapter``, ``/v1/unload_lora_adapter``.
The server binds only after the engine is ready, so "port reachable" means "engine
ready".  Unsupported sampling parameters are rejected with a 400, never ignored.
A client disconnect aborts the request in the scheduler.

Reference parity: pegainfer-frontend/src/vllm/mod.rs:62-414 (serve paths),
src/vllm/wire.rs:14-163 (parameter conversion, honor-or-reject),
src/vllm/request_contract.rs:16-90, src/vllm/lora.rs:72-200 (LoRA routes),
pegainfer-sim/tests/frontend_e2e.rs:194-866 (observable HTTP behaviour).
"""
from __future__ import annotations

import asyncio
import json
import time
import uuid
from typing import Any, AsyncIterator, Optional

from fastapi import FastAPI
from fastapi import Request as HttpRequest
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..engine.contract import FinishReason, Request, RequestUpdate, SamplingParams
from .metrics import ServerMetrics
from .tokenizer import IncrementalDetokenizer, extract_tool_calls

LORA_XARG = "pegainfer_lora_adapter"


class BadRequest(Exception):
    def __init__(self, message: str, status: int = 400):
        super().__init__(message)
        self.status = status
        self.message = message


def convert_sampling(body: dict, eos_known: bool) -> SamplingParams:
    """OpenAI/vLLM request fields -> SamplingParams (honor-or-reject)."""
    for name in ("frequency_penalty", "presence_penalty"):
        if body.get(name) not in (None, 0, 0.0):
            raise BadRequest(f"{name} is not supported")
    if body.get("repetition_penalty") not in (None, 1, 1.0):
        raise BadRequest("repetition_penalty is not supported")
    if body.get("ec_transfer_params") is not None:
        raise BadRequest("ec_transfer_params is not supported")
    if body.get("n") not in (None, 1) or body.get("best_of") not in (None, 1):
        raise BadRequest("n / best_of other than 1 are not supported")
    if body.get("logit_bias"):
        raise BadRequest("logit_bias is not supported")
    temp = body.get("temperature")
    temp = 1.0 if temp is None else float(temp)
    min_p = float(body.get("min_p") or 0.0)
    if not (0.0 <= min_p < 1.0):
        raise BadRequest("min_p must be in [0, 1)")
    top_p = float(body.get("top_p") if body.get("top_p") is not None else 1.0)
    if not (0.0 < top_p <= 1.0):
        raise BadRequest("top_p must be in (0, 1]")
    top_k = int(body.get("top_k") if body.get("top_k") is not None else -1)
    if top_k == 0:
        top_k = -1
    seed = body.get("seed")
    stop_ids = tuple(int(t) for t in (body.get("stop_token_ids") or ()))
    ignore_eos = bool(body.get("ignore_eos", False))
    if temp <= 0:
        temp = 0.0
    return SamplingParams(temperature=temp, top_k=top_k, top_p=top_p, min_p=min_p, seed=int(seed) if seed is not None else None, ignore_eos=ignore_eos, stop_token_ids=stop_ids)


def _stops(body: dict) -> list:
    s = body.get("stop")
    if s is None:
        return []
    if isinstance(s, str):
        return [s]
    return [x for x in s if x]


class _LoopBridge:
    """Scheduler thread -> event loop hand-off.  A decode step produces one update per running
    request; waking the loop once per update (a lock and a socket write each) costs the
    scheduler thread about a millisecond per step at 64 streams, so updates are queued here and
    the loop is woken once per burst."""

    def __init__(self, loop):
        import threading

        self.loop = loop
        self._lock = threading.Lock()
        self._pending: list = []
        self._scheduled = False

    def push(self, q, upd) -> None:
        with self._lock:
            self._pending.append((q, upd))
            if self._scheduled:
                return
            self._scheduled = True
        self.loop.call_soon_threadsafe(self._drain)

    def _drain(self) -> None:
        with self._lock:
            items, self._pending = self._pending, []
            self._scheduled = False
        for q, upd in items:
            q.put_nowait(upd)


def _merge_updates(first: RequestUpdate, q) -> RequestUpdate:
    """``first`` followed by every update already waiting in ``q``, as one update."""
    out = RequestUpdate(
        id=first.id, scheduled=first.scheduled, tokens=list(first.tokens), logprobs=list(first.logprobs or []), cached_tokens=first.cached_tokens,
        prompt_echo=first.prompt_echo, kv_transfer=first.kv_transfer, terminal=first.terminal,
    )
    while out.terminal is None:
        try:
            nxt = q.get_nowait()
        except asyncio.QueueEmpty:
            break
        if nxt.logprobs or out.logprobs:  # keep the per-token alignment
            out.logprobs = (out.logprobs or [None] * len(out.tokens)) + list(nxt.logprobs or [None] * len(nxt.tokens))
        out.tokens.extend(nxt.tokens)
        if out.cached_tokens is None:
            out.cached_tokens = nxt.cached_tokens
        if out.prompt_echo is None:
            out.prompt_echo = nxt.prompt_echo
        if nxt.kv_transfer is not None:
            out.kv_transfer = nxt.kv_transfer
        out.terminal = nxt.terminal
    return out


class Frontend:
    """Protocol logic independent of the web framework (unit-testable)."""

    def __init__(self, engine, tokenizer, model_name: str, declared_engines: Optional[int] = None, lora_manager=None):
        if declared_engines is not None and declared_engines != engine.num_partitions:
            raise RuntimeError(f"declared {declared_engines} engines but the launched engine exposes {engine.num_partitions} schedulers")
        self.engine = engine
        self.tok = tokenizer
        self.model_name = model_name
        self.metrics = ServerMetrics(model_name)
        self.lora = lora_manager
        self.created = int(time.time())
        self._bridges: dict = {}  # event loop id -> _LoopBridge

    # -- request construction ---------------------------------------------------
    def _prompt_ids(self, prompt) -> list:
        if isinstance(prompt, str):
            return [self.tok.encode(prompt)]
        if isinstance(prompt, list):
            if not prompt:
                raise BadRequest("prompt is empty")
            if all(isinstance(x, int) for x in prompt):
                return [list(prompt)]
            if all(isinstance(x, str) for x in prompt):
                return [self.tok.encode(x) for x in prompt]
            if all(isinstance(x, list) and all(isinstance(t, int) for t in x) for x in prompt):
                return [list(x) for x in prompt]
        raise BadRequest("prompt must be a string, a list of strings, a list of token ids or a list of token-id lists")

    def build_request(self, body: dict, prompt_ids: list) -> Request:
        params = convert_sampling(body, True)
        max_tokens = body.get("max_tokens", body.get("max_completion_tokens"))
        max_tokens = 16 if max_tokens is None else int(max_tokens)
        if max_tokens < 0:
            raise BadRequest("max_tokens must be >= 0")
        lp = body.get("logprobs")
        if isinstance(lp, bool):
            lp = int(body.get("top_logprobs") or 0) if lp else 0
            lp = max(lp, 1) if body.get("logprobs") else 0
        lp = int(lp or 0)
        if lp > 20:
            raise BadRequest("logprobs must be <= 20")
        xargs = body.get("vllm_xargs") or {}
        lora = xargs.get(LORA_XARG)
        if lora is not None and not isinstance(lora, str):
            raise BadRequest(f"vllm_xargs.{LORA_XARG} must be a string")
        if lora is None and body.get("model") not in (None, self.model_name) and self.lora is not None and self.lora.has(body.get("model")):
            lora = body.get("model")
        kvp = xargs.get("kv_transfer_params", body.get("kv_transfer_params"))
        dp = body.get("data_parallel_rank", xargs.get("data_parallel_rank"))
        return Request(
            prompt_tokens=prompt_ids,
            params=params,
            max_tokens=max(max_tokens, 1),
            lora_adapter=lora,
            kv_transfer_params=kvp,
            logprobs=lp,
            echo=bool(body.get("echo", False)),
            cache_salt=body.get("cache_salt"),
            data_parallel_rank=int(dp) if dp is not None else None,
            client_label=body.get("request_id"),
        )

    # -- streaming core ----------------------------------------------------------------
    def _bridge_for(self, loop) -> "_LoopBridge":
        b = self._bridges.get(id(loop))
        if b is None or b.loop is not loop:
            b = _LoopBridge(loop)
            self._bridges[id(loop)] = b
        return b

    async def run_request(self, req: Request, stops: list, disconnected=None) -> AsyncIterator[dict]:
        """Yields events: {"text", "token_ids", "logprobs", "finish_reason", "usage", ...}."""
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        t_start = time.monotonic()
        bridge = self._bridge_for(loop)
        try:
            stream = self.engine.submit(req, listener=lambda upd: bridge.push(q, upd))
        except ValueError as e:
            raise BadRequest(str(e))
        detok = IncrementalDetokenizer(self.tok)
        n_out = 0
        cached = 0
        t_last = None
        first = True
        text_all = ""
        watch = None
        if disconnected is not None:
            # client-gone detection runs beside the token path instead of as a timeout around
            # every queue read (a timer and a task per token add up at a few thousand tokens/s)
            async def _watch():
                while not stream.closed:
                    await asyncio.sleep(0.25)
                    if await disconnected():
                        stream.abort()
                        return

            watch = asyncio.create_task(_watch())
        try:
            while True:
                upd: RequestUpdate = await q.get()
                if not stops and not q.empty():
                    # the engine ran ahead of this connection: fold everything that is waiting into one
                    # event, so a frontend that falls behind sends fewer, larger chunks instead of lagging
                    # (with stop strings every update is looked at on its own: token counts end at the hit)
                    upd = _merge_updates(upd, q)
                ev: dict = {}
                now = time.monotonic()
                if upd.cached_tokens is not None:
                    cached = upd.cached_tokens
                if upd.prompt_echo is not None:
                    ev["echo_text"] = self.tok.decode(upd.prompt_echo.tokens)
                    ev["echo_tokens"] = upd.prompt_echo.tokens
                if upd.tokens:
                    if first:
                        queue_s = 0.0
                        self.metrics.observe_first_token(now - t_start, queue_s, len(req.prompt_tokens), cached)
                        first = False
                        self.metrics.observe_tokens(len(upd.tokens), None)
                    else:
                        self.metrics.observe_tokens(len(upd.tokens), now - t_last)
                    t_last = now
                    n_out += len(upd.tokens)
                    delta = detok.push(upd.tokens)
                    ev["token_ids"] = list(upd.tokens)
                    ev["logprobs"] = upd.logprobs
                    hit = None
                    if stops and delta:
                        text_all_new = text_all + delta
                        for s in stops:
                            i = text_all_new.find(s, max(0, len(text_all) - len(s)))
                            if i >= 0 and (hit is None or i < hit):
                                hit = i
                        if hit is not None:
                            delta = text_all_new[:hit][len(text_all) :]
                    text_all += delta
                    ev["text"] = delta
                    if hit is not None and upd.terminal is None:
                        stream.abort()
                        ev["finish_reason"] = "stop"
                        ev["usage"] = self._usage(req, n_out, cached)
                        self.metrics.observe_finish("stop", now - t_start)
                        yield ev
                        return
                if upd.kv_transfer is not None:
                    ev["kv_transfer_params"] = upd.kv_transfer
                if upd.terminal is not None:
                    term = upd.terminal
                    if term.kind == "finished":
                        reason = {FinishReason.STOP: "stop", FinishReason.LENGTH: "length", FinishReason.ABORT: "abort"}[term.finish_reason]
                        ev["finish_reason"] = reason
                        ev["usage"] = self._usage(req, n_out, cached)
                        self.metrics.observe_finish(reason, now - t_start)
                        yield ev
                        return
                    if term.kind == "rejected":
                        raise BadRequest(f"request rejected ({term.reject_reason.value}): {term.message}")
                    raise BadRequest(f"request failed: {term.message}", status=500)
                if ev:
                    yield ev
        finally:
            if watch is not None:
                watch.cancel()
            if not stream.closed:
                stream.abort()

    def _usage(self, req: Request, n_out: int, cached: int) -> dict:
        n_in = len(req.prompt_tokens)
        return {"prompt_tokens": n_in, "completion_tokens": n_out, "total_tokens": n_in + n_out, "prompt_tokens_details": {"cached_tokens": cached}}

    @staticmethod
    def _lp_completion(lps, tok) -> Optional[dict]:
        lps = [l for l in (lps or []) if l is not None]
        if not lps:
            return None
        return {
            "tokens": [tok.decode([l.token]) for l in lps],
            "token_logprobs": [l.logprob for l in lps],
            "top_logprobs": [{tok.decode([t]): v for t, v in l.top} for l in lps],
        }


def create_app(fe: Frontend):
    app = FastAPI(title="pegainfer-b200")

    def err(message: str, status: int = 400):
        return JSONResponse({"error": {"message": message, "type": "invalid_request_error" if status < 500 else "internal_error", "code": status}}, status_code=status)

    @app.get("/health")
    async def health():
        if not fe.engine.healthy():
            return PlainTextResponse("engine down", status_code=503)
        return PlainTextResponse("ok")

    @app.get("/v1/models")
    async def models():
        data = [{"id": fe.model_name, "object": "model", "created": fe.created, "owned_by": "pegainfer-b200", "max_model_len": fe.engine.info.max_model_len}]
        if fe.lora is not None:
            data += [{"id": n, "object": "model", "created": fe.created, "owned_by": "pegainfer-b200", "parent": fe.model_name} for n in fe.lora.names()]
        return {"object": "list", "data": data}

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse(fe.metrics.render(fe.engine.metrics()), media_type="text/plain; version=0.0.4")

    def sse(obj) -> bytes:
        return ("data: " + (obj if isinstance(obj, str) else json.dumps(obj)) + "\n\n").encode()

    async def _body(http: HttpRequest) -> dict:
        try:
            body = await http.json()
        except Exception:
            raise BadRequest("request body is not valid JSON")
        if not isinstance(body, dict):
            raise BadRequest("request body must be a JSON object")
        return body

    # ---------------------------------------------------------------- completions
    @app.post("/v1/completions")
    async def completions(http: HttpRequest):
        try:
            body = await _body(http)
            prompts = fe._prompt_ids(body.get("prompt"))
            reqs = [fe.build_request(body, p) for p in prompts]
        except BadRequest as e:
            return err(e.message, e.status)
        rid = "cmpl-" + uuid.uuid4().hex
        created = int(time.time())
        stops = _stops(body)
        include_usage = bool((body.get("stream_options") or {}).get("include_usage"))

        if body.get("stream"):
            async def gen():
                usage_total = {"prompt_tokens": 0, "completion_tokens": 0, "total_tokens": 0}
                try:
                    for idx, req in enumerate(reqs):
                        async for ev in fe.run_request(req, stops, http.is_disconnected):
                            text = ev.get("echo_text", "") + ev.get("text", "")
                            choice = {"index": idx, "text": text, "logprobs": fe._lp_completion(ev.get("logprobs"), fe.tok), "finish_reason": ev.get("finish_reason")}
                            if text or choice["finish_reason"]:
                                yield sse({"id": rid, "object": "text_completion", "created": created, "model": fe.model_name, "choices": [choice]})
                            if "usage" in ev:
                                for k in usage_total:
                                    usage_total[k] += ev["usage"][k]
                    if include_usage:
                        yield sse({"id": rid, "object": "text_completion", "created": created, "model": fe.model_name, "choices": [], "usage": usage_total})
                except BadRequest as e:
                    yield sse({"error": {"message": e.message, "code": e.status}})
                yield sse("[DONE]")

            return StreamingResponse(gen(), media_type="text/event-stream")

        async def one(idx, req):
            text, lps, finish, usage, kvt = "", [], None, None, None
            async for ev in fe.run_request(req, stops, http.is_disconnected):
                text += ev.get("echo_text", "") + ev.get("text", "")
                lps += ev.get("logprobs") or []
                finish = ev.get("finish_reason", finish)
                usage = ev.get("usage", usage)
                kvt = ev.get("kv_transfer_params", kvt)
            return {"index": idx, "text": text, "logprobs": fe._lp_completion(lps, fe.tok), "finish_reason": finish}, usage, kvt

        try:
            results = await asyncio.gather(*[one(i, r) for i, r in enumerate(reqs)])
        except BadRequest as e:
            return err(e.message, e.status)
        usage = {k: sum(u[k] for _, u, _ in results) for k in ("prompt_tokens", "completion_tokens", "total_tokens")}
        usage["prompt_tokens_details"] = {"cached_tokens": sum(u["prompt_tokens_details"]["cached_tokens"] for _, u, _ in results)}
        out = {"id": rid, "object": "text_completion", "created": created, "model": fe.model_name, "choices": [c for c, _, _ in results], "usage": usage}
        kvts = [k for _, _, k in results if k is not None]
        if kvts:
            out["kv_transfer_params"] = kvts[0]
        return out

    # ---------------------------------------------------------------- chat
    @app.post("/v1/chat/completions")
    async def chat(http: HttpRequest):
        try:
            body = await _body(http)
            msgs = body.get("messages")
            if not isinstance(msgs, list) or not msgs:
                raise BadRequest("messages must be a non-empty list")
            tools = body.get("tools")
            ids = fe.tok.apply_chat_template(msgs, tools=tools, add_generation_prompt=True)
            req = fe.build_request(body, ids)
        except BadRequest as e:
            return err(e.message, e.status)
        rid = "chatcmpl-" + uuid.uuid4().hex
        created = int(time.time())
        stops = _stops(body)
        include_usage = bool((body.get("stream_options") or {}).get("include_usage"))

        def chunk(delta, finish=None, usage=None, choices=True):
            c = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": fe.model_name, "choices": [{"index": 0, "delta": delta, "finish_reason": finish}] if choices else []}
            if usage is not None:
                c["usage"] = usage
            return c

        if body.get("stream"):
            async def gen():
                try:
                    yield sse(chunk({"role": "assistant", "content": ""}))
                    usage = None
                    held = ""  # text held back while it may be part of a tool call
                    n_calls = 0
                    async for ev in fe.run_request(req, stops, http.is_disconnected):
                        text = ev.get("text", "")
                        if tools:
                            held += text
                            text = ""
                            if "<tool_call>" not in held and not any(held.endswith("<tool_call>"[:k]) for k in range(1, 11)):
                                text, held = held, ""
                            elif "</tool_call>" in held:
                                content, calls = extract_tool_calls(held)
                                for cl in calls:
                                    cl = dict(cl, index=n_calls)
                                    n_calls += 1
                                    yield sse(chunk({"tool_calls": [cl]}))
                                text, held = content, ""
                        if text:
                            yield sse(chunk({"content": text}))
                        if ev.get("finish_reason"):
                            if held:
                                yield sse(chunk({"content": held}))
                            usage = ev.get("usage")
                            fr = "tool_calls" if n_calls and ev["finish_reason"] == "stop" else ev["finish_reason"]
                            yield sse(chunk({}, finish=fr))
                    if include_usage and usage is not None:
                        yield sse(chunk({}, usage=usage, choices=False))
                except BadRequest as e:
                    yield sse({"error": {"message": e.message, "code": e.status}})
                yield sse("[DONE]")

            return StreamingResponse(gen(), media_type="text/event-stream")
        text, finish, usage, lps = "", None, None, []
        try:
            async for ev in fe.run_request(req, stops, http.is_disconnected):
                text += ev.get("text", "")
                lps += ev.get("logprobs") or []
                finish = ev.get("finish_reason", finish)
                usage = ev.get("usage", usage)
        except BadRequest as e:
            return err(e.message, e.status)
        message: dict = {"role": "assistant", "content": text}
        if tools:
            content, calls = extract_tool_calls(text)
            if calls:
                message = {"role": "assistant", "content": content or None, "tool_calls": calls}
                if finish == "stop":
                    finish = "tool_calls"
        choice = {"index": 0, "message": message, "finish_reason": finish}
        lp = [l for l in lps if l is not None]
        if lp:
            choice["logprobs"] = {"content": [{"token": fe.tok.decode([l.token]), "logprob": l.logprob, "top_logprobs": [{"token": fe.tok.decode([t]), "logprob": v} for t, v in l.top]} for l in lp]}
        return {"id": rid, "object": "chat.completion", "created": created, "model": fe.model_name, "choices": [choice], "usage": usage}

    # ---------------------------------------------------------------- LoRA control
    @app.post("/v1/load_lora_adapter")
    async def load_lora(http: HttpRequest):
        try:
            body = await _body(http)
        except BadRequest as e:
            return err(e.message, e.status)
        if fe.lora is None:
            return err("LoRA is not enabled (start the server with --enable-lora)")
        name, path = body.get("lora_name"), body.get("lora_path")
        if not isinstance(name, str) or not isinstance(path, str):
            return err("lora_name and lora_path are required strings")
        try:
            await asyncio.get_running_loop().run_in_executor(None, fe.lora.load, name, path)
        except Exception as e:  # noqa: BLE001 - surfaced to the client
            return err(f"failed to load adapter: {e}")
        return PlainTextResponse(f"Success: LoRA adapter '{name}' added successfully.")

    @app.post("/v1/unload_lora_adapter")
    async def unload_lora(http: HttpRequest):
        try:
            body = await _body(http)
        except BadRequest as e:
            return err(e.message, e.status)
        if fe.lora is None:
            return err("LoRA is not enabled (start the server with --enable-lora)")
        name = body.get("lora_name")
        if not isinstance(name, str) or not fe.lora.has(name):
            return err(f"LoRA adapter {name!r} is not loaded", 404)
        await asyncio.get_running_loop().run_in_executor(None, fe.lora.unload, name)
        return PlainTextResponse(f"Success: LoRA adapter '{name}' removed successfully.")

    return app


def serve(engine, tokenizer, model_name: str, host: str = "127.0.0.1", port: int = 8000, declared_engines=None, lora_manager=None, log_level="warning"):
    import sys

    # The scheduler thread and the event loop share the interpreter lock; the default 5 ms switch
    # interval lets a busy event loop hold a decode step up for longer than the step itself.
    sys.setswitchinterval(2e-4)
    """Blocking: run the HTTP server until interrupted (the engine is already up)."""
    import uvicorn

    fe = Frontend(engine, tokenizer, model_name, declared_engines, lora_manager)
    uvicorn.run(create_app(fe), host=host, port=port, log_level=log_level)
