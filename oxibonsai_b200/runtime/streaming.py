"""Server-sent-event helpers and request middleware pieces shared by the HTTP front ends.

Reference: crates/oxibonsai-runtime/src/streaming.rs:19-267 (``SseFormatter``: first chunk with the role, one chunk per
text delta, final chunk with the finish reason and optional usage, the ``[DONE]`` sentinel, error events; ``TokenStream``
holding back incomplete UTF-8; ``StreamStats``) and middleware.rs (``RequestContext``, ``RequestIdGen``,
``RequestLogger`` request / response lines, ``CorsConfig``).
"""
from __future__ import annotations

import json
import time
from dataclasses import dataclass, field

from ..tokenizer import StreamingDecoder


class SseFormatter:
    def __init__(self, request_id: str, model: str, created: int | None = None, include_usage: bool = False, object_name: str = "chat.completion.chunk"):
        self.id, self.model, self.created, self.include_usage, self.object = request_id, model, created or int(time.time()), include_usage, object_name

    def _chunk(self, delta: dict, finish_reason: str | None = None, usage: dict | None = None) -> dict:
        c = {"id": self.id, "object": self.object, "created": self.created, "model": self.model,
             "choices": [{"index": 0, "delta": delta, "finish_reason": finish_reason}]}
        if usage is not None:
            c["usage"] = usage
        return c

    @staticmethod
    def format_event(payload: dict | str, event: str | None = None) -> str:
        data = payload if isinstance(payload, str) else json.dumps(payload, ensure_ascii=False, separators=(",", ":"))
        head = f"event: {event}\n" if event else ""
        return head + "".join(f"data: {line}\n" for line in data.split("\n")) + "\n"

    def first_chunk(self) -> str:
        return self.format_event(self._chunk({"role": "assistant"}))

    def token_chunk(self, text: str) -> str:
        return self.format_event(self._chunk({"content": text}))

    def final_chunk(self, finish_reason: str = "stop", usage: dict | None = None) -> str:
        return self.format_event(self._chunk({}, finish_reason, usage if self.include_usage else None))

    @staticmethod
    def done_sentinel() -> str:
        return "data: [DONE]\n\n"

    def error_event(self, message: str, kind: str = "server_error") -> str:
        return self.format_event({"error": {"message": message, "type": kind}}, event="error")


class TokenStream:
    """Accumulates token bytes and releases only complete UTF-8 text."""

    def __init__(self):
        self._dec = StreamingDecoder()
        self.emitted = ""

    def push_token_bytes(self, data: bytes) -> str:
        out = self._dec.push(data)
        self.emitted += out
        return out

    def flush(self) -> str:
        out = self._dec.flush()
        self.emitted += out
        return out

    def is_empty(self) -> bool:
        return not self.emitted


@dataclass
class StreamStats:
    prompt_tokens: int = 0
    completion_tokens: int = 0
    started: float = field(default_factory=time.perf_counter)
    first_token_at: float | None = None
    finished_at: float | None = None

    def on_token(self) -> None:
        if self.first_token_at is None:
            self.first_token_at = time.perf_counter()
        self.completion_tokens += 1

    def finish(self) -> None:
        self.finished_at = time.perf_counter()

    def throughput(self) -> float:
        end = self.finished_at or time.perf_counter()
        return self.completion_tokens / (end - self.started) if end > self.started else 0.0

    def ttft(self) -> float | None:
        return None if self.first_token_at is None else self.first_token_at - self.started

    def to_usage_chunk(self) -> dict:
        return {"prompt_tokens": self.prompt_tokens, "completion_tokens": self.completion_tokens, "total_tokens": self.prompt_tokens + self.completion_tokens}


# ---- middleware pieces -----------------------------------------------------------------------------------------------------------
@dataclass
class RequestContext:
    request_id: str
    method: str = ""
    path: str = ""
    started: float = field(default_factory=time.perf_counter)

    def elapsed_ms(self) -> float:
        return (time.perf_counter() - self.started) * 1e3


class RequestIdGen:
    """Monotonic ids with a process-unique prefix (cheap alternative to random ids for logs)."""

    def __init__(self, prefix: str = "req"):
        self.prefix, self._n = prefix, 0

    def next(self) -> str:
        self._n += 1
        return f"{self.prefix}-{self._n:08d}"


class RequestLogger:
    def __init__(self, logger=None, log_bodies: bool = False, max_body: int = 512):
        import logging
        self.log, self.log_bodies, self.max_body = logger or logging.getLogger("oxibonsai.http"), log_bodies, max_body

    @staticmethod
    def format_request_line(ctx: RequestContext) -> str:
        return f"--> {ctx.method} {ctx.path} [{ctx.request_id}]"

    @staticmethod
    def format_response_line(ctx: RequestContext, status: int) -> str:
        return f"<-- {status} {ctx.method} {ctx.path} [{ctx.request_id}] {ctx.elapsed_ms():.1f} ms"

    def log_request(self, ctx: RequestContext, body: bytes | None = None) -> None:
        line = self.format_request_line(ctx)
        if self.log_bodies and body:
            line += " " + body[: self.max_body].decode("utf-8", errors="replace")
        self.log.info(line)

    def log_response(self, ctx: RequestContext, status: int) -> None:
        (self.log.warning if status >= 500 else self.log.info)(self.format_response_line(ctx, status))


@dataclass
class CorsConfig:
    allowed_origins: tuple[str, ...] = ("*",)
    allowed_methods: tuple[str, ...] = ("GET", "POST", "OPTIONS")
    allowed_headers: tuple[str, ...] = ("authorization", "content-type", "x-request-id")
    max_age: int = 600

    def is_origin_allowed(self, origin: str) -> bool:
        return "*" in self.allowed_origins or origin in self.allowed_origins

    def access_control_headers(self, origin: str) -> dict[str, str]:
        if not self.is_origin_allowed(origin):
            return {}
        return {"access-control-allow-origin": "*" if "*" in self.allowed_origins else origin,
                "access-control-allow-methods": ", ".join(self.allowed_methods), "access-control-allow-headers": ", ".join(self.allowed_headers),
                "access-control-max-age": str(self.max_age)}
