"""OpenAI-compatible HTTP API (FastAPI).

Routes: ``/v1/models``, ``/v1/chat/completions`` (+SSE), ``/v1/completions`` (+SSE), ``/tokenize``,
``/detokenize``, ``/health``, ``/healthz``, ``/version``, ``/metrics`` (Prometheus, vLLM-compatible
names), ``/v1/metrics`` (JSON), ``/trace``, ``/v1/placement`` and the admin group
``/v1/models/{load,unload,status,available}``.  Errors use the OpenAI envelope
``{"error": {message, type, code}}``; a failure in the middle of a stream is its own SSE frame
with no ``[DONE]`` after it; unsupported parameters are refused, never silently dropped.

Reference counterparts: crates/plowrt/src/serve/mod.rs:1495-1538 (router), chat.rs:36,
openai.rs:176-1067 (types), stream.rs:141-309 (SSE), docs/serving-openai-compat.md.
"""
from __future__ import annotations

import asyncio
import json
import queue
import time
import uuid

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from .. import __version__
from ..obs import prometheus
from ..runtime.engine import EngineHealth
from ..runtime.scheduler import GenParams
from . import tools as tools_mod
from .template import ChatTemplateError

REFUSED_PARAMS = ("echo", "best_of", "suffix", "functions", "function_call")


class ApiError(Exception):
    def __init__(self, status, message, typ="invalid_request_error", code=None):
        self.status, self.message, self.typ, self.code = status, message, typ, code


def _envelope(e: ApiError) -> JSONResponse:
    headers = {"Retry-After": str(getattr(e, "retry_after", 1))} if e.status == 429 else None
    return JSONResponse(status_code=e.status, content={"error": {"message": e.message, "type": e.typ, "code": e.code}}, headers=headers)


def _gen_params(body: dict, default_max: int) -> GenParams:
    for k in REFUSED_PARAMS:
        if body.get(k) is not None:
            raise ApiError(400, f"parameter '{k}' is not supported", code="unsupported_parameter")
    n = body.get("n", 1)
    if not isinstance(n, int) or isinstance(n, bool) or not 1 <= n <= 8:
        raise ApiError(400, "n must be an integer in [1, 8]", code="invalid_value")
    if n > 1 and body.get("stream"):
        raise ApiError(400, "n > 1 is not supported with stream", code="unsupported_parameter")
    rf = body.get("response_format")
    json_mode = False
    if rf is not None:
        kind = rf.get("type") if isinstance(rf, dict) else rf
        if kind == "json_object":
            json_mode = True
        elif kind != "text":
            raise ApiError(400, f"response_format '{kind}' is not supported (text, json_object)", code="unsupported_parameter")
    bias = body.get("logit_bias")
    if bias is not None:
        try:
            bias = {int(k): float(v) for k, v in dict(bias).items()}
        except (TypeError, ValueError):
            raise ApiError(400, "logit_bias maps token ids to numbers", code="invalid_value")
        if len(bias) > 300 or any(not -100.0 <= v <= 100.0 for v in bias.values()):
            raise ApiError(400, "logit_bias takes at most 300 entries with values in [-100, 100]", code="invalid_value")
    t = body.get("temperature")
    temperature = 1.0 if t is None else float(t)
    if temperature < 0 or temperature > 2:
        raise ApiError(400, "temperature must be in [0, 2]", code="invalid_value")
    top_p = float(body.get("top_p", 1.0) if body.get("top_p") is not None else 1.0)
    if not 0 < top_p <= 1:
        raise ApiError(400, "top_p must be in (0, 1]", code="invalid_value")
    stop = body.get("stop") or []
    if isinstance(stop, str):
        stop = [stop]
    if len(stop) > 4:
        raise ApiError(400, "at most 4 stop sequences", code="invalid_value")
    mt = body.get("max_completion_tokens") or body.get("max_tokens") or default_max
    if int(mt) < 1:
        raise ApiError(400, "max_tokens must be >= 1", code="invalid_value")
    lp = body.get("top_logprobs") if body.get("logprobs") else None
    if body.get("logprobs") is True and lp is None:
        lp = 0
    if isinstance(body.get("logprobs"), int) and not isinstance(body.get("logprobs"), bool):
        lp = int(body["logprobs"])
    return GenParams(max_tokens=int(mt), temperature=temperature, top_p=top_p, top_k=int(body.get("top_k") or 0),
                     min_p=float(body.get("min_p") or 0.0), presence_penalty=float(body.get("presence_penalty") or 0.0),
                     frequency_penalty=float(body.get("frequency_penalty") or 0.0),
                     repetition_penalty=float(body.get("repetition_penalty") or 1.0), seed=body.get("seed"),
                     stop=list(stop), stop_token_ids=list(body.get("stop_token_ids") or []),
                     ignore_eos=bool(body.get("ignore_eos", False)), min_tokens=int(body.get("min_tokens") or 0),
                     logprobs=lp, logit_bias=bias or None, deadline_ms=(float(body["deadline_ms"]) if body.get("deadline_ms") else None),
                     json_mode=json_mode)


def _finish(reason: str) -> tuple:
    """(finish_reason, x_plow_finish_reason)"""
    if reason in ("stop", "length"):
        return reason, None
    if reason in ("preempted", "cancelled", "deadline"):
        return "length", reason
    return "stop", reason


class ModelEntry:
    def __init__(self, name, mux, tokenizer, template, created=None, tool_family=None, reasoning=False):
        self.name, self.mux, self.tok, self.template = name, mux, tokenizer, template
        self.created = created or int(time.time())
        self.tool_family = tool_family        # serve.tools parser family (None = detect from the text)
        self.reasoning = reasoning            # split <think>…</think> into reasoning_content


class AppState:
    def __init__(self, api_keys=None, timeline=None, loader=None):
        self.models: dict[str, ModelEntry] = {}
        self.api_keys = set(api_keys or [])
        self.timeline = timeline
        self.loader = loader          # callable(name, path) -> ModelEntry for the admin routes
        self.manager = None           # serve.manager.ModelManager: residency within a memory budget (optional)
        self.fingerprint = f"plow-b200-{__version__}"
        self.router = None            # data-parallel router (optional)

    def add(self, entry: ModelEntry):
        self.models[entry.name] = entry

    def get(self, name):
        if name in self.models:
            return self.models[name]
        if len(self.models) == 1 and not name:
            return next(iter(self.models.values()))
        raise ApiError(404, f"model '{name}' not found", code="model_not_found")


def create_app(state: AppState) -> FastAPI:
    app = FastAPI(title="plowrt", version=__version__)
    app.state.plow = state

    @app.exception_handler(ApiError)
    async def _api_err(_req, exc: ApiError):
        return _envelope(exc)

    @app.middleware("http")
    async def _auth(request: Request, call_next):
        if state.api_keys and request.url.path.startswith("/v1"):
            auth = request.headers.get("authorization", "")
            if not (auth.startswith("Bearer ") and auth[7:] in state.api_keys):
                return _envelope(ApiError(401, "invalid API key", "authentication_error", "invalid_api_key"))
        return await call_next(request)

    # ---- meta ----------------------------------------------------------------------------------
    @app.get("/health")
    @app.get("/healthz")
    async def health():
        states = [m.mux.engine.health for m in state.models.values()]
        if states and all(s == EngineHealth.DEAD for s in states):
            return JSONResponse(status_code=503, content={"status": "dead"})
        return {"status": "degraded" if any(s != EngineHealth.HEALTHY for s in states) else "ok"}

    @app.get("/version")
    async def version():
        return {"version": __version__, "system_fingerprint": state.fingerprint}

    @app.get("/models")
    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [
            {"id": m.name, "object": "model", "created": m.created, "owned_by": "plow",
             "max_model_len": m.mux.engine.max_ctx, "x_plow_modalities": ["text"]} for m in state.models.values()]}

    @app.get("/metrics")
    async def metrics():
        return PlainTextResponse("".join(prometheus.render(m.name, m.mux) for m in state.models.values()))

    @app.get("/v1/metrics")
    async def metrics_json():
        return {m.name: m.mux.metrics.snapshot() for m in state.models.values()}

    @app.get("/trace")
    async def trace():
        if not state.timeline or not state.timeline.enabled:
            raise ApiError(404, "tracing is off (start with --trace)", code="trace_disabled")
        return PlainTextResponse(state.timeline.to_json(), media_type="application/json")

    @app.get("/v1/load")
    async def load_estimate():
        return {m.name: m.mux.load_estimate() for m in state.models.values()}

    @app.get("/v1/placement")
    async def placement():
        return {m.name: {"slots": m.mux.engine.max_slots, "live": len(m.mux.live),
                         "kv_pages": m.mux.engine.pool.n_pages, "kv_pages_free": m.mux.engine.pool.available(),
                         "health": m.mux.engine.health} for m in state.models.values()}

    @app.post("/v1/tokenize")
    @app.post("/tokenize")
    async def tokenize(body: dict):
        m = state.get(body.get("model", ""))
        if "messages" in body:
            text = m.template.render(body["messages"], add_generation_prompt=body.get("add_generation_prompt", True))
        else:
            text = body.get("prompt", "")
        ids = m.tok.encode(text)
        return {"tokens": ids, "count": len(ids), "max_model_len": m.mux.engine.max_ctx}

    @app.post("/v1/detokenize")
    @app.post("/detokenize")
    async def detokenize(body: dict):
        m = state.get(body.get("model", ""))
        return {"prompt": m.tok.decode(body.get("tokens", []))}

    # ---- admin ---------------------------------------------------------------------------------
    @app.get("/v1/models/status")
    async def models_status():
        return {m.name: {"state": "resident", "health": m.mux.engine.health, "live": len(m.mux.live)} for m in state.models.values()}

    @app.get("/v1/models/available")
    async def models_available():
        if state.manager is not None:
            return {"models": state.manager.available(), "status": state.manager.status()}
        return {"models": sorted(state.models)}

    @app.post("/v1/models/load")
    async def models_load(body: dict):
        if state.manager is not None:
            from .manager import ResidencyError
            try:
                entry = await asyncio.get_running_loop().run_in_executor(None, state.manager.acquire, body.get("model"), body.get("path"))
            except ResidencyError as e:
                raise ApiError(409, str(e), code="residency")
            state.add(entry)
            for gone in [n for n in state.models if n not in state.manager.resident]:
                state.models.pop(gone, None)
            return {"model": body.get("model"), "state": "resident", "evictions": state.manager.evictions}
        if state.loader is None:
            raise ApiError(400, "this server was started without a model loader", code="admin_disabled")
        name, path = body.get("model"), body.get("path")
        if not name or not path:
            raise ApiError(400, "model and path are required")
        entry = await asyncio.get_running_loop().run_in_executor(None, state.loader, name, path)
        state.add(entry)
        return {"model": name, "state": "resident"}

    @app.post("/v1/models/unload")
    async def models_unload(body: dict):
        m = state.get(body.get("model", ""))
        await asyncio.get_running_loop().run_in_executor(None, m.mux.drain, float(body.get("timeout_s", 30)))
        m.mux.stop()
        state.models.pop(m.name, None)
        return {"model": m.name, "state": "unloaded"}

    # ---- generation ----------------------------------------------------------------------------
    async def _next_chunk(req):
        loop = asyncio.get_running_loop()
        while True:
            try:
                return req.out.get_nowait()
            except queue.Empty:
                await asyncio.sleep(0.001)
                _ = loop

    def _submit(m: ModelEntry, ids: list, params: GenParams):
        if len(ids) + 1 > m.mux.engine.max_ctx:
            raise ApiError(400, f"prompt of {len(ids)} tokens exceeds the model's context length {m.mux.engine.max_ctx}",
                           code="context_length_exceeded")
        params.max_tokens = min(params.max_tokens, m.mux.engine.max_ctx - len(ids))
        mux = state.router.route(m, ids) if state.router else m.mux
        return mux.submit(ids, params)

    def _fan_out(m: ModelEntry, ids: list, params: GenParams, n: int) -> list:
        """n - 1 further samples of the same prompt (the prefix cache shares its KV pages); each gets a seed of its own."""
        import dataclasses
        out = []
        for i in range(1, n):
            p = dataclasses.replace(params, seed=(params.seed + i) if params.seed is not None else None, session_id=None, session_end=False)
            out.append(_submit(m, ids, p))
        return out

    def _sum_usage(usages: list) -> dict:
        u = dict(usages[0] or {})
        u["completion_tokens"] = sum((x or {}).get("completion_tokens", 0) for x in usages)
        u["total_tokens"] = u.get("prompt_tokens", 0) + u["completion_tokens"]
        return u

    async def _collect(req):
        text, toks, lps = [], [], []
        while True:
            ch = await _next_chunk(req)
            if ch.kind == "token":
                text.append(ch.text)
                toks.append(ch.token_id)
                if ch.logprob is not None:
                    lps.append((ch.token_id, ch.logprob, ch.top_logprobs))
            elif ch.kind == "done":
                text.append(ch.text)
                return "".join(text), toks, lps, ch.finish_reason, ch.usage
            else:
                if ch.error == "overloaded" or ch.finish_reason == "overloaded":
                    e = ApiError(429, "server is overloaded", "rate_limit_error", "overloaded")
                    e.retry_after = int((ch.usage or {}).get("retry_after_s", 1))
                    raise e
                if ch.error == "context_length_exceeded":
                    raise ApiError(400, "context length exceeded", code="context_length_exceeded")
                raise ApiError(503 if "dead" in (ch.error or "") else 500, ch.error or "generation failed", "server_error", "engine_error")

    def _lp_block(m, lps):
        if not lps:
            return None
        return {"content": [{"token": m.tok.decode([t]), "logprob": lp,
                             "top_logprobs": [{"token": m.tok.decode([a]), "logprob": b} for a, b in (top or [])]}
                            for (t, lp, top) in lps]}

    @app.post("/v1/chat/completions")
    async def chat(body: dict, request: Request):
        m = state.get(body.get("model", ""))
        msgs = body.get("messages")
        if not isinstance(msgs, list) or not msgs:
            raise ApiError(400, "messages must be a non-empty list")
        params = _gen_params(body, default_max=256)
        params.session_id = request.headers.get("x-session-id")
        params.session_end = request.headers.get("x-session-end", "") in ("1", "true")
        try:
            prompt = m.template.render([dict(x) for x in msgs], tools=body.get("tools"))
        except ChatTemplateError as e:
            raise ApiError(400, f"chat template error: {e}", code="template_error")
        ids = m.tok.encode(prompt)
        req = _submit(m, ids, params)
        rid, created = f"chatcmpl-{uuid.uuid4().hex[:24]}", int(time.time())
        base = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": m.name,
                "system_fingerprint": state.fingerprint}
        want_reasoning = bool(getattr(m, "reasoning", False)) or bool(body.get("separate_reasoning"))
        want_tools = bool(body.get("tools")) and body.get("tool_choice") != "none"
        if body.get("stream"):
            include_usage = bool((body.get("stream_options") or {}).get("include_usage"))
            splitter = tools_mod.StreamSplitter() if want_reasoning else None

            def _delta(text, final=False):
                if splitter is None:
                    return {"content": text} if text else {}
                r, c = splitter.feed(text, final)
                d = {}
                if r:
                    d["reasoning_content"] = r
                if c:
                    d["content"] = c
                return d

            async def sse():
                yield "data: " + json.dumps({**base, "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]}) + "\n\n"
                acc = []
                while True:
                    if await request.is_disconnected():
                        req.cancelled = True
                        return
                    ch = await _next_chunk(req)
                    if ch.kind == "token":
                        acc.append(ch.text)
                        if want_tools:
                            continue          # tool calls are parsed from the whole message and sent with the last chunk
                        d = _delta(ch.text)
                        if d:
                            yield "data: " + json.dumps({**base, "choices": [{"index": 0, "delta": d, "finish_reason": None}]}) + "\n\n"
                    elif ch.kind == "done":
                        fr, xfr = _finish(ch.finish_reason)
                        acc.append(ch.text)
                        if want_tools:
                            full = "".join(acc)
                            reasoning, rest = tools_mod.split_reasoning(full) if want_reasoning else (None, full)
                            content, calls = tools_mod.extract_tool_calls(rest, getattr(m, "tool_family", None))
                            d = {"content": content} if content else {}
                            if reasoning:
                                d["reasoning_content"] = reasoning
                            if calls:
                                d["tool_calls"] = [dict(c, index=i) for i, c in enumerate(calls)]
                                fr = "tool_calls"
                        else:
                            d = _delta(ch.text, final=True)
                        last = {**base, "choices": [{"index": 0, "delta": d, "finish_reason": fr}]}
                        if xfr:
                            last["x_plow_finish_reason"] = xfr
                        yield "data: " + json.dumps(last) + "\n\n"
                        if include_usage:
                            yield "data: " + json.dumps({**base, "choices": [], "usage": ch.usage}) + "\n\n"
                        yield "data: [DONE]\n\n"
                        return
                    else:
                        yield "data: " + json.dumps({"error": {"message": ch.error, "type": "server_error", "code": "engine_error"}}) + "\n\n"
                        return   # no [DONE] after an error frame
            return StreamingResponse(sse(), media_type="text/event-stream")
        others = _fan_out(m, ids, params, int(body.get("n") or 1))
        results = [await _collect(req)] + [await _collect(r) for r in others]
        choices, xfr = [], None
        for i, (text, toks, lps, reason, _u) in enumerate(results):
            fr, x = _finish(reason)
            xfr = xfr or x
            message = {"role": "assistant", "content": text}
            if want_reasoning:
                reasoning, text = tools_mod.split_reasoning(text)
                message["content"] = text
                if reasoning is not None:
                    message["reasoning_content"] = reasoning
            if want_tools:
                content, calls = tools_mod.extract_tool_calls(text, getattr(m, "tool_family", None))
                if calls:
                    message["content"] = content or None
                    message["tool_calls"] = calls
                    fr = "tool_calls"
            choices.append({"index": i, "message": message, "finish_reason": fr, "logprobs": _lp_block(m, lps)})
        out = {"id": rid, "object": "chat.completion", "created": created, "model": m.name,
               "system_fingerprint": state.fingerprint, "choices": choices, "usage": _sum_usage([r[4] for r in results])}
        if xfr:
            out["x_plow_finish_reason"] = xfr
        return out

    @app.post("/v1/completions")
    async def completions(body: dict, request: Request):
        m = state.get(body.get("model", ""))
        prompt = body.get("prompt")
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            ids = list(prompt)
        elif isinstance(prompt, str):
            ids = m.tok.encode(prompt)
        else:
            raise ApiError(400, "prompt must be a string or a list of token ids")
        if not ids:
            raise ApiError(400, "prompt is empty")
        params = _gen_params(body, default_max=16)
        req = _submit(m, ids, params)
        rid, created = f"cmpl-{uuid.uuid4().hex[:24]}", int(time.time())
        if body.get("stream"):
            async def sse():
                while True:
                    if await request.is_disconnected():
                        req.cancelled = True
                        return
                    ch = await _next_chunk(req)
                    if ch.kind == "token":
                        yield "data: " + json.dumps({"id": rid, "object": "text_completion", "created": created, "model": m.name,
                                                     "choices": [{"index": 0, "text": ch.text, "finish_reason": None}]}) + "\n\n"
                    elif ch.kind == "done":
                        fr, _x = _finish(ch.finish_reason)
                        yield "data: " + json.dumps({"id": rid, "object": "text_completion", "created": created, "model": m.name,
                                                     "choices": [{"index": 0, "text": ch.text, "finish_reason": fr}], "usage": ch.usage}) + "\n\n"
                        yield "data: [DONE]\n\n"
                        return
                    else:
                        yield "data: " + json.dumps({"error": {"message": ch.error, "type": "server_error", "code": "engine_error"}}) + "\n\n"
                        return
            return StreamingResponse(sse(), media_type="text/event-stream")
        others = _fan_out(m, ids, params, int(body.get("n") or 1))
        results = [await _collect(req)] + [await _collect(r) for r in others]
        return {"id": rid, "object": "text_completion", "created": created, "model": m.name,
                "system_fingerprint": state.fingerprint,
                "choices": [{"index": i, "text": text, "finish_reason": _finish(reason)[0], "token_ids": toks, "logprobs": _lp_block(m, lps)}
                            for i, (text, toks, lps, reason, _u) in enumerate(results)],
                "usage": _sum_usage([r[4] for r in results])}

    return app
