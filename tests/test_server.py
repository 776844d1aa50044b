"""HTTP surface against a fake backend (no GPU): routing, SSE framing, auth, errors, metrics, config layering."""
import json
import threading

import pytest

from oxibonsai_b200.runtime.presets import SamplingParams
from oxibonsai_b200.server.config import ServerConfig, load_config
from oxibonsai_b200.tokenizer import ByteTokenizer


class _Req:
    def __init__(self):
        self.done = threading.Event()
        self.tokens, self.finish_reason, self.error, self.cancelled = [], None, None, False

    def cancel(self):
        self.cancelled = True


class FakeBackend:
    """Echoes a fixed reply byte by byte; records the sampling parameters it was given."""

    model_name, max_seq_len = "fake-bonsai", 4096

    def __init__(self, reply="héllo wörld", fail=False):
        self.reply, self.fail, self.seen = reply.encode("utf-8"), fail, []

    def submit(self, prompt, params, max_tokens, on_token, request_id):
        if self.fail:
            raise RuntimeError("engine exploded")
        self.seen.append((list(prompt), params, max_tokens, request_id))
        r = _Req()

        def run():
            for b in self.reply[:max_tokens]:
                if r.cancelled:
                    break
                r.tokens.append(b)
                if on_token:
                    on_token(b)
            r.finish_reason = "length" if len(self.reply) > max_tokens else "stop"
            r.done.set()

        threading.Thread(target=run, daemon=True).start()
        return r

    def kv_utilization(self):
        return 0.25


@pytest.fixture()
def client():
    from fastapi.testclient import TestClient
    from oxibonsai_b200.server.app import create_app
    be = FakeBackend()
    app = create_app(be, ByteTokenizer(), ServerConfig())
    c = TestClient(app)
    c.backend = be
    return c


def test_health_models_and_request_id(client):
    r = client.get("/health")
    assert r.status_code == 200 and r.text == "ok" and r.headers["x-request-id"]
    r = client.get("/v1/models", headers={"x-request-id": "abc123"})
    assert r.headers["x-request-id"] == "abc123"
    assert r.json()["data"][0]["id"] == "fake-bonsai"
    assert client.get("/health/detail").json()["status"] == "healthy"


def test_chat_completion_applies_request_sampling(client):
    body = {"messages": [{"role": "user", "content": "hi"}], "temperature": 0.2, "top_p": 0.5, "seed": 7, "max_tokens": 100}
    j = client.post("/v1/chat/completions", json=body).json()
    assert j["object"] == "chat.completion" and j["choices"][0]["message"] == {"role": "assistant", "content": "héllo wörld"}
    assert j["choices"][0]["finish_reason"] == "stop" and j["usage"]["prompt_tokens"] > 0
    prompt, params, mt, _ = client.backend.seen[-1]
    assert bytes(prompt).decode().startswith("<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n")
    assert (params.temperature, params.top_p, params.seed, mt) == (0.2, 0.5, 7, 100)


def test_streaming_sse_framing_is_utf8_safe(client):
    with client.stream("POST", "/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "stream": True}) as r:
        assert r.headers["content-type"].startswith("text/event-stream")
        events = [l[6:] for l in r.iter_lines() if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert chunks[0]["choices"][0]["delta"] == {"role": "assistant"}
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks[1:])
    assert text == "héllo wörld" and "�" not in text
    assert chunks[-1]["choices"][0]["finish_reason"] == "stop"
    assert all(c["object"] == "chat.completion.chunk" for c in chunks)


def test_completions_stop_sequences_and_length(client):
    j = client.post("/v1/completions", json={"prompt": "abc", "stop": [" w"]}).json()
    assert j["choices"][0]["text"] == "héllo" and j["choices"][0]["finish_reason"] == "stop"
    j = client.post("/v1/completions", json={"prompt": "abc", "max_tokens": 3}).json()
    assert j["choices"][0]["finish_reason"] == "length"
    j = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "q"}], "n": 2}).json()
    assert len(j["choices"]) == 2


def test_error_envelope(client):
    r = client.post("/v1/chat/completions", json={"messages": []})
    assert r.status_code == 400 and r.json()["error"]["type"] == "invalid_request_error"
    r = client.post("/v1/chat/completions", content=b"{not json", headers={"content-type": "application/json"})
    assert r.status_code == 400
    assert client.post("/v1/completions", json={"prompt": "x", "temperature": -1}).status_code == 400
    assert client.post("/v1/completions", json={"prompt": "x", "n": 9}).status_code == 400


def test_backend_failure_maps_to_5xx_and_counts():
    from fastapi.testclient import TestClient
    from oxibonsai_b200.server.app import create_app
    app = create_app(FakeBackend(fail=True), ByteTokenizer(), ServerConfig())
    c = TestClient(app)
    r = c.post("/v1/completions", json={"prompt": "x"})
    assert r.status_code == 500 and "exploded" in r.json()["error"]["message"]
    assert app.state.metrics.errors.get() == 1


def test_bearer_auth_skips_health_and_metrics():
    from fastapi.testclient import TestClient
    from oxibonsai_b200.server.app import create_app
    app = create_app(FakeBackend(), ByteTokenizer(), ServerConfig(bearer_token="s3cret-token-0123456789"))
    c = TestClient(app)
    assert c.get("/health").status_code == 200 and c.get("/metrics").status_code == 200
    assert c.get("/v1/models").status_code == 401
    assert c.get("/v1/models", headers={"authorization": "Bearer s3cret-token-0123456789"}).status_code == 200


def test_metrics_embeddings_admin(client):
    client.post("/v1/completions", json={"prompt": "abc"})
    text = client.get("/metrics").text
    for name in ("oxibonsai_requests_total 1", "oxibonsai_tokens_generated_total", "oxibonsai_prefill_duration_seconds_bucket",
                 "oxibonsai_kv_cache_utilization 0.25", "oxibonsai_inter_token_latency_p95_seconds", "oxibonsai_kv_cache_compression_level"):
        assert name in text
    e = client.post("/v1/embeddings", json={"input": ["a b c", "a b d"]}).json()
    assert len(e["data"]) == 2 and len(e["data"][0]["embedding"]) == 512
    st = client.get("/admin/status").json()
    assert st["model"] == "fake-bonsai" and st["circuit"] == "closed"
    ws = client.get("/admin/workload-stats").json()
    assert ws["status"] == "ok" and ws["request_rate"]["completed_requests"] == 1 and ws["request_rate"]["tbt_p95_seconds"] >= 0.0
    assert ws["kv_cache"]["level"] == "fp16" and ws["kv_cache"]["memory_factor"] == 1.0 and ws["kv_cache"]["samples"] == 1
    assert client.post("/admin/reset-metrics").json() == {"status": "ok"}
    assert "oxibonsai_requests_total 0" in client.get("/metrics").text
    ui = client.get("/ui").text
    assert "<html" in ui and "/v1/chat/completions" in ui and "getReader" in ui          # the page streams from the chat route


def test_config_layering_and_validation(tmp_path):
    toml = tmp_path / "s.toml"
    toml.write_text('[server]\nport = 9000\nhost = "127.0.0.1"\n[sampling]\ntemperature = 0.3\nmax_tokens = 64\n')
    cfg = load_config(["--config", str(toml), "--port", "9100"], env={"OXIBONSAI_TEMPERATURE": "0.5", "OXIBONSAI_PORT": "9050"})
    assert (cfg.port, cfg.host, cfg.temperature, cfg.max_tokens) == (9100, "127.0.0.1", 0.5, 64)   # CLI > env > TOML > defaults
    with pytest.raises(ValueError):
        ServerConfig(port=0).validate()
    with pytest.raises(ValueError):
        ServerConfig(bearer_token="short").validate()
    with pytest.raises(ValueError):
        ServerConfig(model_path="/nonexistent/model.gguf").validate()
    with pytest.raises(ValueError):
        ServerConfig(temperature=3.0).validate()


def test_rag_routes_and_json_api(client):
    r = client.post("/rag/index", json={"documents": ["Bonsai trees need careful watering.", {"text": "Pines like full sun.", "metadata": {"k": 1}}]})
    assert r.status_code == 200 and r.json()["documents"] == 2 and r.json()["indexed_chunks"] == 2
    q = client.post("/rag/query", json={"query": "what do pines like?", "top_k": 1}).json()
    assert q["hits"][0]["text"] == "Pines like full sun." and "Question: what do pines like?" in q["prompt"]
    a = client.post("/rag/query", json={"query": "pines?", "generate": True, "max_tokens": 50}).json()
    assert a["answer"] == "héllo wörld" and a["usage"]["completion_tokens"] > 0
    assert client.get("/rag/stats").json()["chunks"] == 2 and client.post("/rag/query", json={}).status_code == 400
    assert client.delete("/rag/index").json() == {"status": "cleared"} and client.get("/rag/stats").json()["chunks"] == 0
    assert client.post("/rag/index", json={"text": "Maples turn red in autumn."}).json()["documents"] == 1
    from oxibonsai_b200.server.app import generate_json
    tok = ByteTokenizer()
    out = json.loads(generate_json(lambda ids, n: ids[:n], tok, json.dumps({"prompt": "abcdef", "max_tokens": 3})))
    assert out == {"text": "abc", "tokens": 3, "error": None}
    assert json.loads(generate_json(lambda ids, n: ids, tok, "{broken"))["error"]


def test_tool_call_parsing():
    from oxibonsai_b200.runtime.tools import parse_tool_calls, tools_system_prompt
    calls = parse_tool_calls('sure <tool_call>{"name": "get_weather", "arguments": {"city": "Kyoto"}}</tool_call>')
    assert calls[0]["function"]["name"] == "get_weather" and json.loads(calls[0]["function"]["arguments"]) == {"city": "Kyoto"}
    assert parse_tool_calls("no json here") == []
    assert "get_weather" in tools_system_prompt([{"type": "function", "function": {"name": "get_weather", "description": "d"}}])


def test_cors_preflight_kv_policy_and_request_log(client, caplog):
    import logging
    with caplog.at_level(logging.INFO, logger="oxibonsai.http"):
        r = client.options("/v1/chat/completions", headers={"origin": "https://app.example", "access-control-request-method": "POST"})
        assert r.status_code == 204 and r.headers["access-control-allow-origin"] == "*" and "POST" in r.headers["access-control-allow-methods"]
        r = client.post("/v1/completions", json={"prompt": "abc"}, headers={"origin": "https://app.example"})
        assert r.headers["access-control-allow-origin"] == "*"
    lines = [rec.getMessage() for rec in caplog.records]
    assert any(l.startswith("--> POST /v1/completions") for l in lines) and any(l.startswith("<-- 200 POST /v1/completions") for l in lines)
    # the fake backend reports 25 % page utilisation: the controller stays at FP16 and says so
    st = client.get("/admin/status").json()
    assert st["kv_level"] == "FP16" and st["kv_page_format_for_new_sequences"] == "f16"
    assert "oxibonsai_kv_cache_compression_level 0" in client.get("/metrics").text
    client.app.state.cors.allowed_origins = ("https://only.example",)
    r = client.options("/v1/models", headers={"origin": "https://evil.example"})
    assert r.status_code == 403 and "access-control-allow-origin" not in r.headers


class _OneAtATimeEngine:
    """A ``generate_stream`` engine that fails if two requests ever overlap (what the serial backend has to prevent)."""

    max_seq_len = 64

    def __init__(self, reply=b"serial ok"):
        self.reply, self.lock, self.busy, self.overlaps, self.calls = reply, threading.Lock(), 0, 0, []

    def generate_stream(self, prompt, max_tokens, params, stop_at_eos=True):
        with self.lock:
            self.busy += 1
            self.overlaps += self.busy > 1
            self.calls.append((list(prompt), max_tokens, params.temperature))
            try:
                for b in self.reply[:max_tokens]:
                    yield b
            finally:
                self.busy -= 1


def test_serial_backend_serves_single_request_engines():
    from fastapi.testclient import TestClient
    from oxibonsai_b200.server.app import SerialBackend, create_app
    eng = _OneAtATimeEngine()
    be = SerialBackend(eng, "generic-q8")
    assert be.max_seq_len == 64 and be.kv_utilization() == 0.0
    # direct: tokens, finish reasons, cancellation, argument checks
    r = be.submit([1, 2, 3], SamplingParams(temperature=0.0), 4, None, "a" * 32)
    assert bytes(r.wait(5)) == b"seri" and r.finish_reason == "length" and r.ttft is not None
    r = be.submit([1], SamplingParams(), 50, None, "b" * 32)
    assert bytes(r.wait(5)) == b"serial ok" and r.finish_reason == "stop"
    seen, box, ready = [], {}, threading.Event()

    def cancel_after_first(t):
        seen.append(t)
        ready.wait(5)                 # the request object exists only once submit() has returned
        box["r"].cancel()
    box["r"] = r = be.submit([1], SamplingParams(), 50, cancel_after_first, "c" * 32)
    ready.set()
    r.wait(5)
    assert r.finish_reason == "cancelled" and len(seen) == 1
    with pytest.raises(ValueError):
        be.submit([], SamplingParams(), 4, None, "d" * 32)
    with pytest.raises(ValueError):
        be.submit(list(range(64)), SamplingParams(), 4, None, "e" * 32)
    # an engine error reaches the waiter
    class Broken(_OneAtATimeEngine):
        def generate_stream(self, *a, **k):
            raise RuntimeError("boom")
            yield 0
    bad = SerialBackend(Broken(), "x").submit([1], SamplingParams(), 4, None, "f" * 32)
    with pytest.raises(RuntimeError):
        bad.wait(5)
    # through the HTTP routes, several requests at once: all answered, never two inside the engine
    c = TestClient(create_app(be, ByteTokenizer(), ServerConfig()))
    out = []
    def ask():
        out.append(c.post("/v1/completions", json={"prompt": "hi", "max_tokens": 32}).json()["choices"][0]["text"])
    ts = [threading.Thread(target=ask) for _ in range(4)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert out == ["serial ok"] * 4 and eng.overlaps == 0
    assert c.get("/v1/models").json()["data"][0]["id"] == "generic-q8"


class _FailingGeneration(FakeBackend):
    """Accepts the request and then fails inside the generation (the engine raised while decoding)."""

    def __init__(self):
        super().__init__()
        self.broken = True

    def submit(self, prompt, params, max_tokens, on_token, request_id):
        if not self.broken:
            return super().submit(prompt, params, max_tokens, on_token, request_id)
        r = _Req()
        r.error, r.finish_reason = RuntimeError("kernel reported status 2"), "error"
        r.done.set()
        return r


def test_breaker_opens_on_generation_errors_and_recovers_under_steady_traffic():
    from fastapi.testclient import TestClient
    from oxibonsai_b200.runtime.resilience import CircuitState
    from oxibonsai_b200.server.app import create_app
    be = _FailingGeneration()
    app = create_app(be, ByteTokenizer(), ServerConfig())
    br = app.state.breaker
    now = [1000.0]
    br._clock = lambda: now[0]
    c = TestClient(app)
    body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4}
    for i in range(br.config.failure_threshold):
        assert br.state == CircuitState.CLOSED
        assert c.post("/v1/chat/completions", json=body).status_code == 500
        assert br.failures == i + 1 or br.state == CircuitState.OPEN      # failures accumulate: nothing zeroes them in between
    assert br.state == CircuitState.OPEN
    opened_at = br._opened_at
    # rejected requests keep arriving: they are answered 503 and leave the breaker (and its recovery timer) alone
    for _ in range(4):
        now[0] += 5.0
        assert c.post("/v1/chat/completions", json=body).status_code == 503
    assert br.state == CircuitState.OPEN and br._opened_at == opened_at and br.total_rejected == 4
    # after the recovery time the next request is let through as a probe; the engine is healthy again
    now[0] = opened_at + br.config.recovery_seconds + 0.1
    be.broken = False
    assert c.post("/v1/chat/completions", json=body).status_code == 200
    assert br.state == CircuitState.HALF_OPEN
    assert c.post("/v1/chat/completions", json=body).status_code == 200
    assert br.state == CircuitState.CLOSED and br.failures == 0


def test_breaker_counts_a_failed_submit_once():
    from fastapi.testclient import TestClient
    from oxibonsai_b200.server.app import create_app
    app = create_app(FakeBackend(fail=True), ByteTokenizer(), ServerConfig())
    c = TestClient(app)
    assert c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}]}).status_code == 500
    assert app.state.breaker.failures == 1


class _ExtrasBackend(FakeBackend):
    """Records the constraint / logprobs a request carried and answers with recorded log-probabilities."""

    def submit(self, prompt, params, max_tokens, on_token, request_id, **extra):
        self.extra = extra
        r = super().submit(prompt, params, max_tokens, on_token, request_id)
        r.done.wait(5)
        n = extra.get("logprobs")
        r.token_logprobs = [(-0.5 - i, [(65 + i, -0.5 - i), (66 + i, -2.0)][: n or 0]) for i in range(len(r.tokens))] if n is not None else []
        return r


def _client_with(backend):
    from fastapi.testclient import TestClient
    from oxibonsai_b200.server.app import create_app
    return TestClient(create_app(backend, ByteTokenizer(), ServerConfig()))


def test_response_format_becomes_a_token_constraint_and_logprobs_are_returned():
    from oxibonsai_b200.runtime.constrained import GrammarConstraint
    be = _ExtrasBackend(reply="{}")
    c = _client_with(be)
    body = {"messages": [{"role": "user", "content": "json please"}], "response_format": {"type": "json_object"},
            "logprobs": True, "top_logprobs": 2, "max_tokens": 8}
    j = c.post("/v1/chat/completions", json=body).json()
    assert isinstance(be.extra["constraint"], GrammarConstraint) and be.extra["logprobs"] == 2
    mask = be.extra["constraint"].allowed_mask()            # a JSON value may start with '{' but not with '}'
    assert (mask[ord("{") >> 5] >> (ord("{") & 31)) & 1 and not (mask[ord("}") >> 5] >> (ord("}") & 31)) & 1
    lp = j["choices"][0]["logprobs"]["content"]
    assert [e["token"] for e in lp] == ["{", "}"] and lp[0]["logprob"] == -0.5 and len(lp[0]["top_logprobs"]) == 2
    # a schema is compiled too; plain text carries neither field
    body = {"messages": [{"role": "user", "content": "x"}], "max_tokens": 4,
            "response_format": {"type": "json_schema", "json_schema": {"schema": {"type": "object", "properties": {"a": {"type": "integer"}}, "required": ["a"]}}}}
    assert c.post("/v1/chat/completions", json=body).status_code == 200 and isinstance(be.extra["constraint"], GrammarConstraint)
    j = c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "max_tokens": 4}).json()
    assert be.extra == {} and "logprobs" not in j["choices"][0]
    assert c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "response_format": {"type": "yaml"}}).status_code == 400
    assert c.post("/v1/completions", json={"prompt": "x", "logprobs": 3, "max_tokens": 4}).json()["choices"][0]["logprobs"]["content"]


def test_forced_tool_choice_constrains_the_generation():
    """``tool_choice`` with ``tools``: the backend receives a constraint that only admits a call of the named tool; the
    response carries it as ``tool_calls``.  A tool that is not defined is a 400."""
    import numpy as np
    from fastapi.testclient import TestClient
    from oxibonsai_b200.runtime.constrained import mask_to_bool
    from oxibonsai_b200.server.app import create_app

    class ConstraintFollower(FakeBackend):
        def submit(self, prompt, params, max_tokens, on_token, request_id, constraint=None, **extra):
            r = _Req()
            self.seen.append(constraint)

            def run():
                for _ in range(max_tokens):
                    if constraint is None or constraint.finished():
                        break
                    ok = np.flatnonzero(mask_to_bool(constraint.allowed_mask(), 256))
                    pick = next((int(t) for t in ok if 97 <= t < 123 or t in b'"{}<>/_:,'), int(ok[0]))
                    constraint.advance(pick)
                    r.tokens.append(pick)
                    if on_token:
                        on_token(pick)
                r.finish_reason = "stop"
                r.done.set()
            threading.Thread(target=run, daemon=True).start()
            return r

    be = ConstraintFollower()
    c = TestClient(create_app(be, ByteTokenizer(), ServerConfig()))
    tools = [{"type": "function", "function": {"name": "get_time", "parameters": {"type": "object", "required": ["tz"], "properties": {"tz": {"enum": ["utc", "jst"]}}}}},
             {"type": "function", "function": {"name": "get_weather", "parameters": {"type": "object", "properties": {"city": {"type": "string"}}}}}]
    body = {"messages": [{"role": "user", "content": "what time is it"}], "tools": tools, "max_tokens": 200,
            "tool_choice": {"type": "function", "function": {"name": "get_time"}}}
    r = c.post("/v1/chat/completions", json=body)
    assert r.status_code == 200, r.text
    choice = r.json()["choices"][0]
    assert choice["finish_reason"] == "tool_calls" and choice["message"]["content"] is None
    call = choice["message"]["tool_calls"][0]
    assert call["function"]["name"] == "get_time" and json.loads(call["function"]["arguments"])["tz"] in ("utc", "jst")
    assert be.seen[-1] is not None
    body["tool_choice"] = "auto"
    c.post("/v1/chat/completions", json=body)
    assert be.seen[-1] is None                                   # free text: no constraint
    body["tool_choice"] = {"type": "function", "function": {"name": "launch_rocket"}}
    r = c.post("/v1/chat/completions", json=body)
    assert r.status_code == 400 and "unknown tool" in r.json()["error"]["message"]


def test_chat_template_follows_the_model_name_or_the_configuration():
    from fastapi.testclient import TestClient
    from oxibonsai_b200.server.app import create_app

    class Named(FakeBackend):
        def __init__(self, name):
            super().__init__()
            self.model_name = name

    def prompt_of(backend, cfg):
        c = TestClient(create_app(backend, ByteTokenizer(), cfg))
        assert c.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "hi"}], "max_tokens": 2}).status_code == 200
        return bytes(backend.seen[-1][0]).decode()
    assert prompt_of(Named("Ternary-Bonsai-8B"), ServerConfig()).startswith("<|im_start|>user\nhi<|im_end|>")
    assert prompt_of(Named("Meta-Llama-3-8B-Instruct"), ServerConfig()).startswith("<|begin_of_text|><|start_header_id|>user")
    assert "[INST] hi [/INST]" in prompt_of(Named("whatever"), ServerConfig(chat_template="mistral"))
    with pytest.raises(ValueError, match="chat_template"):
        ServerConfig(chat_template="jinja").validate(check_paths=False)


def test_echo_returns_the_prompt_in_front_of_the_completion(client):
    r = client.post("/v1/completions", json={"prompt": "Say: ", "max_tokens": 5, "echo": True}).json()
    assert r["choices"][0]["text"] == "Say: héllo"[:5 + 5] or r["choices"][0]["text"].startswith("Say: ")
    plain = client.post("/v1/completions", json={"prompt": "Say: ", "max_tokens": 5}).json()
    assert r["choices"][0]["text"] == "Say: " + plain["choices"][0]["text"]
    with client.stream("POST", "/v1/completions", json={"prompt": "Say: ", "max_tokens": 5, "echo": True, "stream": True}) as s:
        events = [json.loads(l[6:]) for l in s.iter_lines() if l.startswith("data: ") and l != "data: [DONE]"]
    assert events[0]["choices"][0]["text"] == "Say: " and "".join(e["choices"][0]["text"] for e in events) == r["choices"][0]["text"]
    chat = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": "x"}], "max_tokens": 3, "echo": True}).json()
    assert not chat["choices"][0]["message"]["content"].startswith("<|im_start|>")          # echo is a completions field only


def test_rate_limiter_buckets_and_refund():
    from oxibonsai_b200.runtime.resilience import RateLimiter, TokenBucket
    now = [0.0]
    clock = lambda: now[0]
    b = TokenBucket(rate=2.0, burst=3.0, clock=clock)
    assert [b.try_acquire() for _ in range(4)] == [True, True, True, False]
    now[0] += 1.0                                                       # two tokens back
    assert b.try_acquire() and b.try_acquire() and not b.try_acquire()
    # the global bucket refuses: the client's allowance is untouched, so it can use all of it once the global one refills
    rl = RateLimiter(global_rate=1.0, global_burst=2.0, client_rate=1.0, client_burst=4.0, max_clients=2, clock=clock)
    assert rl.allow("a") and rl.allow("a") and not rl.allow("a") and not rl.allow("a") and rl.rejected == 2
    now[0] += 2.0                                                       # global: two tokens again; "a" took only two of its four so far
    assert rl.allow("a") and rl.allow("a") and not rl.allow("b")
    # the table of clients is bounded: the least recently seen one goes
    rl.allow("c")
    assert list(rl._clients) == ["b", "c"]
