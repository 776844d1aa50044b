"""OpenAI-compatible HTTP server (FastAPI): chat completions with SSE, completions, models, embeddings, health, metrics, admin.

Reference: the axum router (crates/oxibonsai-runtime/src/server.rs:203-243), ChatML prompt builder (:514-551), SSE framing
``role chunk -> content chunks -> finish chunk -> [DONE]`` with UTF-8-safe incremental decoding (:391-512), ``x-request-id``
echo (:36-60), bearer auth that skips ``/health`` and ``/metrics`` (crates/oxibonsai-serve/src/main.rs:159-170,338-370),
admin endpoints (admin.rs:45-302), embeddings (embeddings.rs), extended request fields - tools, logprobs / top_logprobs
(per-token log-probabilities from the step's logits), n <= 4, response_format (json_object / json_schema: a grammar
constraint whose vocabulary mask the GPU sampler applies at every step), stop, seed (api_types.rs:13-345).  The reference serialises requests on one mutex and ignores the
request's temperature; here requests run concurrently through the continuous-batching scheduler and per-request
sampling parameters are applied.
"""
from __future__ import annotations

import asyncio
import hashlib
import json
import math
import os
import threading
import time
import uuid
from dataclasses import replace
from typing import Any, Callable, Protocol, Sequence

from fastapi import FastAPI, Request
from fastapi.responses import HTMLResponse, JSONResponse, PlainTextResponse, StreamingResponse

from ..runtime.kv_policy import KvCachePolicy
from ..runtime.metrics import InferenceMetrics, RequestRateTracker
from ..runtime.presets import SamplingParams
from ..runtime.resilience import CircuitBreaker, CircuitOpenError, RateLimiter, check_health
from ..runtime.streaming import CorsConfig, RequestContext, RequestLogger
from ..tokenizer import StreamingDecoder, chat_prompt
from .config import ServerConfig


class Backend(Protocol):
    """What the server needs from an engine."""

    model_name: str
    max_seq_len: int

    def submit(self, prompt: Sequence[int], params: SamplingParams, max_tokens: int, on_token: Callable[[int], None] | None,
               request_id: str): ...   # returns an object with wait(), tokens, finish_reason, cancel()

    def kv_utilization(self) -> float: ...


class SchedulerBackend:
    """Backend over a :class:`BatchScheduler` (GPU)."""

    supports_on_done = True            # ``submit(..., on_done=callback)``: called on the scheduler's thread when the request ends

    def __init__(self, scheduler, model_name: str):
        self.s = scheduler
        self.model_name = model_name
        self.max_seq_len = scheduler.engine.max_seq_len

    def submit(self, prompt, params, max_tokens, on_token, request_id, **extra):
        # extra: constraint (TokenConstraint) and logprobs (int) of the request, when it asked for them
        return self.s.submit(prompt, params, max_tokens, on_token=on_token, request_id=request_id, **extra)

    def kv_utilization(self) -> float:
        e = self.s.engine
        return e.kv_utilization() if hasattr(e, "kv_utilization") else e.kv.utilization

    def set_after_step(self, fn) -> None:
        self.s.after_step = fn


class ReplicaBackend:
    """Backend over several :class:`BatchScheduler` s, one per GPU (data-parallel replicas of the whole model): a request goes
    to the replica that its session key hashes to while that replica is healthy and not overloaded, else to the least loaded
    one (``runtime.distributed.ReplicaPool``), so a conversation keeps hitting the replica that holds its prefix cache."""

    supports_on_done = True

    def __init__(self, schedulers: list, model_name: str):
        from ..runtime.distributed import ReplicaPool
        self.schedulers = {f"gpu{i}": s for i, s in enumerate(schedulers)}
        cap = max(1, schedulers[0].engine.max_batch)
        self.pool = ReplicaPool(self.schedulers, capacity=cap)
        self.model_name = model_name
        self.max_seq_len = schedulers[0].engine.max_seq_len

    def submit(self, prompt, params, max_tokens, on_token, request_id, session_key: str | None = None, **extra):
        nid, req = self.pool.submit(session_key or request_id, prompt, params, max_tokens, on_token=on_token, request_id=request_id, **extra)
        req.replica = nid
        threading.Thread(target=lambda: (req.done.wait(), self.pool.finished(nid)), name=f"replica-done-{request_id[:8]}", daemon=True).start()
        return req

    def kv_utilization(self) -> float:
        return max(s.engine.kv_utilization() for s in self.schedulers.values())

    def set_after_step(self, fn) -> None:
        for s in self.schedulers.values():
            s.after_step = fn

    def replica_loads(self) -> dict:
        return {k: {"live": s.active, "queued": len(s.queue)} for k, s in self.schedulers.items()}


class SerialBackend:
    """Backend over an engine that serves one request at a time (``runtime.engine.GenericFormatEngine``, or anything with a
    ``generate_stream(prompt, max_tokens, params, stop_at_eos)`` generator): every request gets a worker thread and the
    engine's own lock serialises them, which is how the reference serves all requests (one engine behind a mutex,
    crates/oxibonsai-runtime/src/server.rs).  Returns the scheduler's ``Request`` object, so the routes treat both backends alike."""

    def __init__(self, engine, model_name: str):
        self.engine = engine
        self.model_name = model_name
        self.max_seq_len = engine.max_seq_len

    def submit(self, prompt, params, max_tokens, on_token, request_id):
        from ..runtime.scheduler import Request as Job
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if len(prompt) + 1 > self.max_seq_len:
            raise ValueError(f"prompt of {len(prompt)} tokens does not fit max_seq_len {self.max_seq_len}")
        r = Job(list(prompt), params.validate(), max_tokens, on_token=on_token, request_id=request_id, t_submit=time.perf_counter())

        def run():
            try:
                for tok in self.engine.generate_stream(r.prompt, r.max_tokens, r.params, r.stop_at_eos):
                    now = time.perf_counter()
                    if r.t_first_token is None:
                        r.t_first_token = now
                    r.tokens.append(tok)
                    r.token_times.append(now)
                    if r.on_token is not None:
                        r.on_token(tok)
                    if r.cancelled:
                        r.finish_reason = "cancelled"
                        break
                if r.finish_reason is None:
                    r.finish_reason = "length" if len(r.tokens) >= r.max_tokens else "stop"
            except Exception as e:          # surfaced by Request.wait()
                r.error = e
                r.finish_reason = "error"
            finally:
                r.t_done = time.perf_counter()
                r.done.set()

        threading.Thread(target=run, name=f"serial-{request_id[:8]}", daemon=True).start()
        return r

    def kv_utilization(self) -> float:
        return 0.0


_END = object()      # queue sentinel: the request is done (or timed out)


def new_request_id() -> str:
    return uuid.uuid4().hex


def _hash_embed(text: str, dim: int = 512) -> list[float]:
    """Deterministic bag-of-hashed-tokens embedding (the reference serves TF-IDF / identity embedders of dimension 512)."""
    v = [0.0] * dim
    for w in text.lower().split():
        h = int.from_bytes(hashlib.blake2b(w.encode(), digest_size=8).digest(), "little")
        v[h % dim] += 1.0 if (h >> 63) & 1 == 0 else -1.0
    n = math.sqrt(sum(x * x for x in v)) or 1.0
    return [x / n for x in v]


def create_app(backend: Backend, tokenizer, config: ServerConfig | None = None, metrics: InferenceMetrics | None = None,
               kv_policy: KvCachePolicy | None = None):
    cfg = config or ServerConfig()
    metrics = metrics or InferenceMetrics()
    breaker = CircuitBreaker()
    limiter = RateLimiter(global_rate=1e6, global_burst=1e6, client_rate=1e5, client_burst=1e5)
    app = FastAPI(title="oxibonsai-b200")
    app.state.metrics, app.state.backend, app.state.config, app.state.breaker = metrics, backend, cfg, breaker
    # KV-pressure controller (FP16 -> Q8 -> Q4 with hysteresis): fed with the page utilisation after every request; its
    # level is exported as a gauge and as the page format recommended for newly admitted sequences
    kv_policy = app.state.kv_policy = kv_policy or KvCachePolicy()
    cors = app.state.cors = CorsConfig()
    http_log = RequestLogger()
    started = time.time()
    sem = asyncio.Semaphore(cfg.max_concurrent * max(1, getattr(cfg, "replicas", 1)))      # max_concurrent is per engine

    def error(status: int, message: str, typ: str = "invalid_request_error", rid: str | None = None):
        r = JSONResponse({"error": {"message": message, "type": typ, "code": status}}, status_code=status)
        if rid:
            r.headers["x-request-id"] = rid
        return r

    @app.middleware("http")
    async def auth_and_ids(request: Request, call_next):
        rid = request.headers.get("x-request-id") or new_request_id()
        request.state.request_id = rid
        path = request.url.path
        ctx = RequestContext(rid, request.method, path)
        http_log.log_request(ctx)
        origin = request.headers.get("origin")
        if request.method == "OPTIONS" and origin:      # CORS preflight: answered here, never reaches a route
            pre = PlainTextResponse("", status_code=204 if cors.is_origin_allowed(origin) else 403)
            pre.headers.update(cors.access_control_headers(origin))
            pre.headers["x-request-id"] = rid
            http_log.log_response(ctx, pre.status_code)
            return pre
        if cfg.bearer_token and path not in ("/health", cfg.metrics_path):
            if request.headers.get("authorization", "") != f"Bearer {cfg.bearer_token}":
                return error(401, "missing or invalid bearer token", "authentication_error", rid)
        client = request.client.host if request.client else "unknown"
        if not limiter.allow(client):
            return error(429, "rate limit exceeded", "rate_limit_error", rid)
        resp = await call_next(request)
        resp.headers["x-request-id"] = rid
        if origin:
            resp.headers.update(cors.access_control_headers(origin))
        http_log.log_response(ctx, resp.status_code)
        return resp

    def sampling_from(body: dict) -> tuple[SamplingParams, int]:
        p = SamplingParams(temperature=cfg.temperature, top_k=cfg.top_k, top_p=cfg.top_p, repetition_penalty=cfg.repetition_penalty,
                           max_tokens=cfg.max_tokens, seed=cfg.seed)
        upd = {}
        for k in ("temperature", "top_p", "top_k", "seed", "repetition_penalty"):
            if body.get(k) is not None:
                upd[k] = body[k]
        p = replace(p, **upd).validate()
        mt = body.get("max_tokens") or body.get("max_completion_tokens") or cfg.max_tokens
        return p, max(1, min(int(mt), 8192))

    def apply_stop(text: str, stops: list[str]) -> tuple[str, bool]:
        cut = min((text.find(s) for s in stops if s and s in text), default=-1)
        return (text[:cut], True) if cut >= 0 else (text, False)

    _table: list = []

    def token_table():
        """Byte strings of the vocabulary for the constraint engines (built once, on the first constrained request)."""
        if not _table:
            from ..runtime.constrained import TokenTable
            _table.append(TokenTable.from_tokenizer(tokenizer))
        return _table[0]

    def constraint_from(body: dict):
        """The request's token constraint.  ``tool_choice`` "required" / a named function (with ``tools``) -> a call of one of
        those tools with arguments of the tool's schema; ``response_format`` ``{"type": "json_object"}`` -> any JSON value,
        ``{"type": "json_schema", "json_schema": {"schema": {...}}}`` -> JSON of that shape; None for plain text."""
        eos = getattr(tokenizer, "eos_token_id", None)
        if body.get("tools") and body.get("tool_choice") not in (None, "auto", "none"):
            # a forced tool call: the sampler may only write <tool_call>{"name":...,"arguments":<the tool's schema>}</tool_call>
            from ..runtime.tools import ToolCallError, build_tool_constraint, tool_choice_names
            try:
                names = tool_choice_names(body["tool_choice"], body["tools"])
                if names is not None:
                    return build_tool_constraint(token_table(), body["tools"], names, eos)
            except ToolCallError as e:
                raise ValueError(str(e)) from e
        rf = body.get("response_format")
        if not isinstance(rf, dict) or rf.get("type") in (None, "text"):
            return None
        from ..runtime.constrained import json_constraint, json_schema_constraint
        if rf["type"] == "json_object":
            return json_constraint(token_table(), eos)
        if rf["type"] == "json_schema":
            spec = rf.get("json_schema") or {}
            schema = spec.get("schema", spec)
            return json_schema_constraint(token_table(), schema, eos)
        raise ValueError(f"unsupported response_format type {rf['type']!r}")

    def logprobs_from(body: dict, chat: bool):
        """Number of alternatives to report per token, or None: chat uses ``logprobs: true`` + ``top_logprobs: n``,
        completions ``logprobs: n``."""
        lp = body.get("logprobs")
        if lp is None or lp is False:
            return None
        n = int(body.get("top_logprobs") or 0) if chat else (0 if lp is True else int(lp))
        if not 0 <= n <= 20:
            raise ValueError("'top_logprobs' must be between 0 and 20")
        return n

    async def run_generation(prompt_ids: list[int], params: SamplingParams, max_tokens: int, rid: str, stops: list[str],
                             extra: dict | None = None, sink: dict | None = None):
        """Async generator of (text_delta, finish_reason | None).  ``extra``: constraint / logprobs of the request, handed to
        the backend; ``sink``: receives the backend's request object under "req" (for the recorded log-probabilities)."""
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        tracker = RequestRateTracker()

        def on_token(tok: int):
            loop.call_soon_threadsafe(q.put_nowait, tok)

        # Breaker accounting happens here and only here, once per request: a rejection by the open breaker touches
        # nothing (it must not restart the recovery timer), a failed submit or a failed / timed-out generation counts one
        # failure, a generation that ran to its end counts one success.
        if not breaker.allow():
            raise CircuitOpenError("circuit open")
        completed = False
        t0 = time.perf_counter()
        try:
            req = backend.submit(prompt_ids, params, max_tokens, on_token, rid, **(extra or {}))
            if sink is not None:
                sink["req"] = req
        except Exception:
            breaker.record_failure()
            raise
        metrics.prompt_tokens.inc(len(prompt_ids))
        waiter = loop.run_in_executor(None, lambda: req.done.wait(cfg.request_timeout_ms / 1000.0))
        dec = StreamingDecoder()
        n_tok, first = 0, True
        text, sent = "", 0

        def feed(piece: str) -> tuple[str, bool]:
            """Appends decoded text; returns (delta safe to send, stop sequence hit).  Text that could still turn
            into a stop sequence is held back until it is disambiguated."""
            nonlocal text, sent
            text += piece
            cut, hit = apply_stop(text, stops)
            if hit:
                delta, sent = cut[sent:], len(cut)
                text = cut
                return delta, True
            hold = 0
            for st in stops:
                for L in range(min(len(st) - 1, len(text)), 0, -1):
                    if text.endswith(st[:L]):
                        hold = max(hold, L)
                        break
            safe = max(sent, len(text) - hold)
            delta, sent = text[sent:safe], safe
            return delta, False

        # the end of the request arrives through the same queue as its tokens (after them: both are queued on the loop in
        # order), so the hot loop is one ``await q.get()`` per wake-up and drains whatever else is already there
        waiter.add_done_callback(lambda _f: q.put_nowait(_END))
        try:
            while True:
                item = await q.get()
                toks, finished = [], False
                while True:
                    if item is _END:
                        finished = True
                        break
                    toks.append(item)
                    if q.empty():
                        break
                    item = q.get_nowait()
                # tokens that piled up while this coroutine waited for its turn go out as one delta: under load the number of
                # SSE events per stream falls instead of the event loop falling further behind
                piece = ""
                for tok in toks:
                    tracker.on_token()
                    n_tok += 1
                    if first:
                        metrics.prefill_seconds.observe(time.perf_counter() - t0)
                        first = False
                    piece += dec.push(tokenizer.token_bytes(tok))
                if piece:
                    delta, hit = feed(piece)
                    if delta:
                        yield delta, None
                    if hit:
                        req.cancel()
                        completed = True
                        yield "", "stop"
                        return
                if finished:
                    if not waiter.result():
                        req.cancel()
                        raise TimeoutError("request timed out")
                    if getattr(req, "error", None) is not None:
                        raise req.error
                    tail = dec.flush()
                    delta, hit = feed(tail) if tail else ("", False)
                    rest = delta + ("" if hit else text[sent:])
                    if rest:
                        yield rest, None
                    completed = True
                    yield "", ("stop" if hit else (req.finish_reason or "stop"))
                    return
        except (GeneratorExit, asyncio.CancelledError):
            completed = None          # the consumer went away: neither a success nor a failure of the engine
            raise
        except Exception:
            breaker.record_failure()
            raise
        finally:
            dt = time.perf_counter() - t0
            metrics.tokens_generated.inc(n_tok)
            metrics.request_seconds.observe(dt)
            if n_tok and dt > 0:
                metrics.tokens_per_second.observe(n_tok / dt)
            metrics.aggregator.record(tracker)
            util = backend.kv_utilization()
            metrics.kv_utilization.set(util)
            kv_policy.observe(util)
            metrics.kv_level.set(kv_policy.metric_value())
            if completed:
                breaker.record_success()

    async def native_stream(handle, chat: bool, prompt_ids, params, max_tokens, rid, stops, extra, obj_id, created, model, echo: str = ""):
        loop = asyncio.get_running_loop()
        await sem.acquire()
        if not breaker.allow():
            sem.release()
            metrics.errors.inc()
            return error(503, "circuit open", "server_error", rid)
        kind = "chat.completion.chunk" if chat else "text_completion"
        head = (f'{{"id": {json.dumps(obj_id)}, "object": "{kind}", "created": {created}, "model": {json.dumps(model)}, '
                f'"choices": [{{"index": 0, ')
        first = ""
        if chat:
            first = "data: " + json.dumps({"id": obj_id, "object": kind, "created": created, "model": model,
                                           "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]}) + "\n\n"
        elif echo:
            first = f'data: {head}"text": {json.dumps(echo)}, "finish_reason": null}}]}}\n\n'
        try:
            stream = handle.open_stream(head, chat, stops, first, cfg.request_timeout_ms)
        except ConnectionError:
            sem.release()
            return error(499, "client closed the connection", "server_error", rid)
        t0 = time.perf_counter()
        metrics.active_requests.inc()

        def on_done(req):                      # the scheduler's thread
            try:
                err = None if req.error is None else (str(req.error) or type(req.error).__name__)
                if stream.state == 3:
                    err = "request timed out"
                n_tok = stream.finish(req.finish_reason, err)
                dt = time.perf_counter() - t0
                tracker = RequestRateTracker()
                tracker.t_admit = t0
                for t in req.token_times:
                    tracker.on_token(t)
                if req.t_first_token is not None:
                    metrics.prefill_seconds.observe(req.t_first_token - t0)
                metrics.tokens_generated.inc(max(0, n_tok))
                metrics.request_seconds.observe(dt)
                if n_tok > 0 and dt > 0:
                    metrics.tokens_per_second.observe(n_tok / dt)
                metrics.aggregator.record(tracker)
                util = backend.kv_utilization()
                metrics.kv_utilization.set(util)
                kv_policy.observe(util)
                metrics.kv_level.set(kv_policy.metric_value())
                if err is not None:
                    metrics.errors.inc()
                    breaker.record_failure()
                elif stream.state != 2:        # a client that went away is neither a success nor a failure of the engine
                    breaker.record_success()
            finally:
                metrics.active_requests.dec()
                loop.call_soon_threadsafe(sem.release)

        try:
            backend.submit(prompt_ids, params, max_tokens, stream.push, rid, on_done=on_done, **extra)
        except Exception as e:  # noqa: BLE001
            breaker.record_failure()
            metrics.errors.inc()
            metrics.active_requests.dec()
            sem.release()
            stream.abandon()
            handle.stream = None
            status = 503 if isinstance(e, CircuitOpenError) or type(e).__name__ in ("QueueFull", "Unavailable", "SchedulerStopped", "MemoryError") else 500
            return error(status, str(e), "server_error", rid)
        metrics.prompt_tokens.inc(len(prompt_ids))
        from .native_front import NATIVE_STREAM_HEADER
        return PlainTextResponse("", headers={NATIVE_STREAM_HEADER.decode(): "1", "content-type": "text/event-stream", "x-request-id": rid,
                                              "cache-control": "no-cache"})

    template = getattr(cfg, "chat_template", "auto")
    if template == "auto":                    # the family the model's name points at (Llama-3, Mistral, Gemma, Qwen), else ChatML
        from ..tokenizer.toolkit import ChatTemplateKind
        kind = ChatTemplateKind.infer_from_name(str(getattr(backend, "model_name", "")))
        template = kind.value if kind is not None else "chatml"
    app.state.chat_template = template

    def encode_chat(messages: list[dict]) -> list[int]:
        return tokenizer.encode(chat_prompt(messages, template))

    # ---- routes -----------------------------------------------------------------------------------
    @app.get("/health")
    async def health():
        return PlainTextResponse("ok")

    @app.get("/health/detail")
    async def health_detail():
        return check_health(True, backend.kv_utilization(), breaker=breaker)

    @app.get(cfg.metrics_path)
    async def metrics_route():
        if not cfg.metrics_enabled:
            return error(404, "metrics disabled")
        return PlainTextResponse(metrics.render_prometheus(), media_type="text/plain; version=0.0.4")

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": backend.model_name, "object": "model", "created": int(started), "owned_by": "oxibonsai"}]}

    async def completion_common(request: Request, chat: bool):
        rid = request.state.request_id
        metrics.requests.inc()
        try:
            body = await request.json()
        except Exception:
            metrics.errors.inc()
            return error(400, "request body is not valid JSON", rid=rid)
        try:
            if chat:
                msgs = body.get("messages")
                if not isinstance(msgs, list) or not msgs:
                    raise ValueError("'messages' must be a non-empty list")
                if body.get("tools"):
                    from ..runtime.tools import tools_system_prompt
                    msgs = [{"role": "system", "content": tools_system_prompt(body["tools"])}] + list(msgs)
                prompt_ids = encode_chat(msgs)
            else:
                prompt = body.get("prompt")
                if isinstance(prompt, list):
                    prompt = prompt[0] if prompt else ""
                if not isinstance(prompt, str) or prompt == "":
                    raise ValueError("'prompt' must be a non-empty string")
                prompt_ids = tokenizer.encode(prompt)
            if len(prompt_ids) > cfg.max_input_tokens or len(prompt_ids) + 1 >= backend.max_seq_len:
                raise ValueError(f"prompt of {len(prompt_ids)} tokens exceeds the input limit")
            params, max_tokens = sampling_from(body)
            n = int(body.get("n") or 1)
            if not 1 <= n <= 4:
                raise ValueError("'n' must be between 1 and 4")
            stops = body.get("stop") or []
            stops = [stops] if isinstance(stops, str) else list(stops)
            top_lp = logprobs_from(body, chat)
            constraint_from(body)          # validated here (a 400 for a bad schema); built again per choice below: it is stateful
        except (ValueError, TypeError) as e:
            metrics.errors.inc()
            return error(400, str(e), rid=rid)

        # completions only: the prompt comes back in front of the generated text (reference: ``echo``, completions.rs:88)
        echo = prompt if (not chat and body.get("echo")) else ""
        created = int(time.time())
        obj_id = ("chatcmpl-" if chat else "cmpl-") + rid[:24]
        model = body.get("model") or backend.model_name

        def extras() -> dict:
            ex: dict[str, Any] = {}
            c = constraint_from(body)
            if c is not None:
                ex["constraint"] = c
            if top_lp is not None:
                ex["logprobs"] = top_lp
            return ex

        def logprobs_json(req) -> dict | None:
            """OpenAI shape: one entry per generated token with its log-probability and the requested alternatives."""
            if top_lp is None or req is None:
                return None
            piece = lambda t: tokenizer.token_bytes(t).decode("utf-8", errors="replace")
            content = [{"token": piece(tok), "logprob": lp, "bytes": list(tokenizer.token_bytes(tok)),
                        "top_logprobs": [{"token": piece(t), "logprob": l} for t, l in top]}
                       for tok, (lp, top) in zip(req.tokens, getattr(req, "token_logprobs", []))]
            return {"content": content}

        front = request.scope.get("extensions", {}).get("oxibonsai.front")
        if body.get("stream") and front is not None and front.front.has_vocab and getattr(backend, "supports_on_done", False):
            # Behind the native front the stream never comes back through this coroutine: sampled token ids go from the
            # scheduler's thread straight into the front, which detokenises, holds back stop sequences, frames and writes.
            return await native_stream(front, chat, prompt_ids, params, max_tokens, rid, stops, extras(), obj_id, created, model, echo)

        if body.get("stream"):
            async def sse():
                metrics.active_requests.inc()
                try:
                    async with sem:
                        if chat:
                            first = {"id": obj_id, "object": "chat.completion.chunk", "created": created, "model": model,
                                     "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]}
                            yield f"data: {json.dumps(first)}\n\n"
                        # the fixed part of every chunk is serialised once; per token only the text is encoded
                        head_json = (f'data: {{"id": {json.dumps(obj_id)}, "object": "{"chat.completion.chunk" if chat else "text_completion"}", '
                                     f'"created": {created}, "model": {json.dumps(model)}, "choices": [{{"index": 0, ')
                        if echo:
                            yield f'{head_json}"text": {json.dumps(echo)}, "finish_reason": null}}]}}\n\n'
                        async for delta, fin in run_generation(prompt_ids, params, max_tokens, rid, stops, extras()):
                            if not (delta or fin):
                                continue
                            if chat:
                                body_json = f'"delta": {{"content": {json.dumps(delta)}}}' if delta else '"delta": {}'
                            else:
                                body_json = f'"text": {json.dumps(delta)}'
                            yield f'{head_json}{body_json}, "finish_reason": {json.dumps(fin)}}}]}}\n\n'
                        yield "data: [DONE]\n\n"
                except Exception as e:  # noqa: BLE001
                    metrics.errors.inc()
                    yield f"data: {json.dumps({'error': {'message': str(e), 'type': 'server_error'}})}\n\n"
                finally:
                    metrics.active_requests.dec()
            return StreamingResponse(sse(), media_type="text/event-stream", headers={"x-request-id": rid, "cache-control": "no-cache"})

        metrics.active_requests.inc()
        try:
            async with sem:
                choices, completion_tokens = [], 0
                for i in range(n):
                    text, fin = "", "stop"
                    sink: dict = {}
                    async for delta, f in run_generation(prompt_ids, replace(params, seed=params.seed + i), max_tokens, rid, stops, extras(), sink):
                        text += delta
                        fin = f or fin
                    lpj = logprobs_json(sink.get("req"))
                    completion_tokens += len(tokenizer.encode(text)) if text else 0
                    if chat:
                        msg: dict[str, Any] = {"role": "assistant", "content": text}
                        if body.get("tools"):
                            from ..runtime.tools import parse_tool_calls
                            calls = parse_tool_calls(text)
                            if calls:
                                msg = {"role": "assistant", "content": None, "tool_calls": calls}
                                fin = "tool_calls"
                        choices.append({"index": i, "message": msg, "finish_reason": fin, **({"logprobs": lpj} if lpj else {})})
                    else:
                        choices.append({"index": i, "text": echo + text, "finish_reason": fin, **({"logprobs": lpj} if lpj else {})})
        except TimeoutError as e:
            metrics.errors.inc()
            return error(504, str(e), "timeout", rid)
        except Exception as e:  # noqa: BLE001
            metrics.errors.inc()
            status = 503 if isinstance(e, CircuitOpenError) or type(e).__name__ in ("QueueFull", "Unavailable", "SchedulerStopped", "MemoryError") else 500
            return error(status, str(e), "server_error", rid)
        finally:
            metrics.active_requests.dec()
        usage = {"prompt_tokens": len(prompt_ids), "completion_tokens": completion_tokens, "total_tokens": len(prompt_ids) + completion_tokens}
        return {"id": obj_id, "object": "chat.completion" if chat else "text_completion", "created": created, "model": model,
                "choices": choices, "usage": usage}

    @app.post("/v1/chat/completions")
    async def chat_completions(request: Request):
        return await completion_common(request, True)

    @app.post("/v1/chat/completions/extended")
    async def chat_completions_extended(request: Request):
        return await completion_common(request, True)

    @app.post("/v1/completions")
    async def completions(request: Request):
        return await completion_common(request, False)

    @app.post("/v1/embeddings")
    async def embeddings(request: Request):
        body = await request.json()
        inp = body.get("input")
        texts = [inp] if isinstance(inp, str) else list(inp or [])
        if not texts:
            return error(400, "'input' must be a string or a list of strings")
        data = [{"object": "embedding", "index": i, "embedding": _hash_embed(t)} for i, t in enumerate(texts)]
        ntok = sum(len(tokenizer.encode(t)) for t in texts)
        return {"object": "list", "data": data, "model": body.get("model") or backend.model_name, "usage": {"prompt_tokens": ntok, "total_tokens": ntok}}

    @app.get("/admin/status")
    async def admin_status():
        return {"uptime_seconds": time.time() - started, "model": backend.model_name, "active_requests": metrics.active_requests.get(),
                "requests_total": metrics.requests.get(), "errors_total": metrics.errors.get(), "circuit": breaker.state.value,
                "kv_utilization": backend.kv_utilization(), "kv_level": kv_policy.level.name,
                "kv_page_format_for_new_sequences": kv_policy.page_format()}

    @app.get("/admin/config")
    async def admin_config():
        d = {k: v for k, v in vars(cfg).items()}
        if d.get("bearer_token"):
            d["bearer_token"] = "***"
        return d

    @app.post("/admin/reset-metrics")
    async def admin_reset():
        metrics.reset()
        return {"status": "ok"}

    @app.get("/admin/cache-stats")
    async def admin_cache():
        return {"kv_utilization": backend.kv_utilization()}

    @app.get("/admin/workload-stats")
    async def admin_workload():
        """Sliding-window request telemetry and the KV-cache policy state in one document (admin.rs:223-260)."""
        snap = metrics.aggregator.snapshot()
        lvl = kv_policy.level
        return {"request_rate": {"completed_requests": snap["completed_requests"], "mean_tokens_per_second": snap["tokens_per_second"],
                                 "tbt_p50_seconds": snap["itl_p50"], "tbt_p95_seconds": snap["itl_p95"],
                                 "mean_queue_wait_seconds": snap["queue_wait"]},
                "kv_cache": {"level": lvl.name.lower(), "memory_factor": lvl.bytes_per_element / 2.0, "pressure_ewma": kv_policy.smoothed_pressure,
                             "samples": kv_policy.observations, "upgrades": kv_policy.upgrades, "downgrades": kv_policy.downgrades,
                             "page_format_for_new_sequences": kv_policy.page_format()},
                "status": "ok"}

    @app.get("/ui")
    async def ui():
        p = os.path.join(os.path.dirname(__file__), "chat.html")
        return HTMLResponse(open(p, encoding="utf-8").read())

    # ---- retrieval endpoints (reference: crates/oxibonsai-runtime/src/rag_server.rs:484-492) ----
    from ..rag import RagPipeline
    app.state.rag = RagPipeline()

    @app.post("/rag/index")
    async def rag_index(request: Request):
        body = await request.json()
        docs = body.get("documents") or ([body["text"]] if "text" in body else [])
        if not docs:
            return error(400, "expected 'text' or 'documents'", "invalid_request_error", request.state.request_id)
        n = sum(app.state.rag.index_document(d if isinstance(d, str) else d["text"], (body.get("metadata") if isinstance(d, str) else d.get("metadata")))
                for d in docs)
        return {"indexed_chunks": n, **app.state.rag.stats()}

    @app.delete("/rag/index")
    async def rag_clear():
        # a fresh pipeline rather than an emptied one, so that a fitted embedder starts over too (rag_server.rs:456-474)
        app.state.rag = RagPipeline()
        return {"status": "cleared"}

    @app.post("/rag/query")
    async def rag_query(request: Request):
        body = await request.json()
        q = body.get("query")
        if not q:
            return error(400, "expected 'query'", "invalid_request_error", request.state.request_id)
        hits = app.state.rag.query(q, body.get("top_k"))
        out = {"hits": [{"text": h.text, "score": h.score, "metadata": h.metadata} for h in hits], "prompt": app.state.rag.build_prompt(q, body.get("top_k"))}
        if body.get("generate"):
            p, mt = sampling_from(body)
            text, _, n_prompt, n_tok = await _collect(out["prompt"], p, mt, request.state.request_id)
            out["answer"], out["usage"] = text, {"prompt_tokens": n_prompt, "completion_tokens": n_tok}
        return out

    @app.get("/rag/stats")
    async def rag_stats():
        return app.state.rag.stats()

    async def _collect(prompt_text: str, p: SamplingParams, max_tokens: int, rid: str):
        ids = tokenizer.encode(prompt_text)
        parts, reason, n = [], "stop", 0
        async for delta, fin in run_generation(ids, p, max_tokens, rid, []):
            if delta:
                parts.append(delta)
                n += 1
            if fin:
                reason = fin
        return "".join(parts), reason, len(ids), n

    return app


def generate_json(engine_generate, tokenizer, request_json: str) -> str:
    """String-in / string-out JSON API for embedding the engine in another host (the reference exposes the same shape
    for its WASM build, crates/oxibonsai-runtime/src/wasm_api.rs:140): ``{"prompt": ..., "max_tokens": ...}`` ->
    ``{"text": ..., "tokens": ..., "error": null}``."""
    import json as _json
    try:
        req = _json.loads(request_json)
        ids = tokenizer.encode(req["prompt"])
        out = engine_generate(ids, int(req.get("max_tokens", 128)))
        return _json.dumps({"text": tokenizer.decode(out), "tokens": len(out), "error": None})
    except Exception as e:  # the caller gets a JSON error, never an exception
        return _json.dumps({"text": "", "tokens": 0, "error": str(e)})


def serve(app, host: str, port: int, log_level: str = "info", tokenizer=None, native: bool = True, vocab_size: int | None = None) -> None:
    """Serves the application: through the native front (``csrc/runtime/http_front.cpp``; with ``tokenizer`` it also streams
    completions without the interpreter) or, with ``native=False``, through uvicorn."""
    if native:
        from .native_front import serve as serve_native

        def ready(front) -> None:
            # the schedulers tell the front when a step's tokens are all in: one wake-up of its I/O thread per step
            backend = getattr(app.state, "backend", None)
            if hasattr(backend, "set_after_step"):
                backend.set_after_step(front.kick)
                front.set_lazy(True)
        serve_native(app, host, port, tokenizer=tokenizer, vocab_size=vocab_size, on_ready=ready)
        return
    import uvicorn
    uvicorn.run(app, host=host, port=port, log_level=log_level if log_level in ("debug", "info", "warning", "error") else "info")
