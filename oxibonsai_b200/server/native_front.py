"""The native HTTP / SSE front: C++ sockets and token streaming, the ASGI application behind it.

Reference: the axum server (crates/oxibonsai-runtime/src/server.rs:203-243) and its SSE framing with UTF-8-safe incremental
decoding (:391-512).  ``csrc/runtime/http_front.cpp`` owns the listening socket, parses requests and writes responses on an
epoll thread; this module hands every parsed request to the ASGI application (the same FastAPI routes that any other ASGI
server would run) and writes its answer back through the C ABI.  A streamed completion does not go through the
application's response at all: the route opens a :class:`NativeStream`, the scheduler thread pushes sampled token ids into it
(one short foreign call per token), and detokenisation, stop-sequence hold-back, JSON
escaping, SSE and chunked framing and the socket writes happen in C++.
"""
from __future__ import annotations

import asyncio
import ctypes as C
import struct
import threading
from typing import Iterable
from urllib.parse import unquote

from .. import _native

NATIVE_STREAM_HEADER = b"x-oxibonsai-native-stream"
_STATES = {0: "live", 1: "stop", 2: "client_gone", 3: "timed_out", 4: "finished", -1: "unknown"}


def _lib():
    lib = _native.host()
    if not getattr(lib, "_bfront_ready", False):
        lib.bfront_create.restype = C.c_void_p
        lib.bfront_create.argtypes = [C.c_char_p, C.c_int, C.c_int]
        lib.bfront_port.argtypes = [C.c_void_p]
        lib.bfront_start.argtypes = [C.c_void_p]
        lib.bfront_stop.argtypes = [C.c_void_p]
        lib.bfront_stop.restype = None
        lib.bfront_destroy.argtypes = [C.c_void_p]
        lib.bfront_destroy.restype = None
        lib.bfront_set_vocab.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_uint32]
        lib.bfront_set_vocab.restype = None
        lib.bfront_next_event.restype = C.c_void_p
        lib.bfront_next_event.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int)]
        lib.bfront_free.argtypes = [C.c_void_p]
        lib.bfront_free.restype = None
        lib.bfront_respond.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_char_p, C.c_char_p, C.c_uint64]
        lib.bfront_respond_start.argtypes = [C.c_void_p, C.c_int64, C.c_int, C.c_char_p]
        lib.bfront_respond_chunk.argtypes = [C.c_void_p, C.c_int64, C.c_char_p, C.c_uint64]
        lib.bfront_respond_end.argtypes = [C.c_void_p, C.c_int64]
        lib.bfront_stream_open.restype = C.c_int64
        lib.bfront_stream_open.argtypes = [C.c_void_p, C.c_int64, C.c_char_p, C.c_int, C.c_char_p, C.c_char_p, C.c_int]
        lib.bfront_stream_begin.argtypes = [C.c_void_p, C.c_int64, C.c_char_p]
        lib.bfront_stream_push.argtypes = [C.c_void_p, C.c_int64, C.c_int32]
        lib.bfront_stream_finish.restype = C.c_int64
        lib.bfront_stream_finish.argtypes = [C.c_void_p, C.c_int64, C.c_char_p, C.c_char_p]
        lib.bfront_stream_abandon.argtypes = [C.c_void_p, C.c_int64]
        lib.bfront_stream_abandon.restype = None
        lib.bfront_set_lazy.argtypes = [C.c_void_p, C.c_int]
        lib.bfront_set_lazy.restype = None
        lib.bfront_kick.argtypes = [C.c_void_p]
        lib.bfront_kick.restype = None
        lib.bfront_set_idle_timeout.argtypes = [C.c_void_p, C.c_int]
        lib.bfront_set_idle_timeout.restype = None
        lib.bfront_stats.argtypes = [C.c_void_p, C.POINTER(C.c_uint64)]
        lib.bfront_stats.restype = None
        # The per-token call is a few hundred nanoseconds of work under a mutex: it keeps the interpreter lock (``PyDLL``).
        # Releasing it would let another Python thread take it, and the sampling thread would wait a switch interval
        # (milliseconds) to get it back - once per token.
        held = C.PyDLL(lib._name)
        held.bfront_stream_push.argtypes = [C.c_void_p, C.c_int64, C.c_int32]
        held.bfront_kick.argtypes = [C.c_void_p]
        held.bfront_kick.restype = None
        lib._bfront_push_held = held.bfront_stream_push
        lib._bfront_kick_held = held.bfront_kick
        lib._bfront_ready = True
    return lib


class StreamClosed(RuntimeError):
    """The stream takes no more tokens: a stop sequence was hit, the client left or the request's time is up."""

    def __init__(self, state: int):
        super().__init__(f"stream closed: {_STATES.get(state, state)}")
        self.state = state


def _header_block(headers: Iterable[tuple[bytes, bytes]], skip: tuple[bytes, ...] = ()) -> bytes:
    out = bytearray()
    for k, v in headers:
        lk = k.lower()
        if lk in skip or lk in (b"content-length", b"transfer-encoding", b"connection"):
            continue
        out += k + b": " + v + b"\r\n"
    return bytes(out)


class NativeStream:
    """A token stream on one connection.  ``push`` is called from the thread that samples tokens."""

    def __init__(self, front: "NativeFront", sid: int):
        self.front, self.sid = front, sid
        self.state = 0
        self._push = front._lib._bfront_push_held
        self._h = front._h

    def push(self, token: int) -> None:
        st = self._push(self._h, self.sid, token)
        if st:
            self.state = st
            raise StreamClosed(st)

    def begin(self, headers: Iterable[tuple[bytes, bytes]]) -> bool:
        block = _header_block(headers, skip=(NATIVE_STREAM_HEADER,))
        return self.front._lib.bfront_stream_begin(self._h, self.sid, block) == 0

    def finish(self, finish_reason: str | None = None, error: str | None = None) -> int:
        return int(self.front._lib.bfront_stream_finish(self._h, self.sid, (finish_reason or "").encode(), error.encode() if error else None))

    def abandon(self) -> None:
        self.front._lib.bfront_stream_abandon(self._h, self.sid)


class NativeFront:
    """The listening socket and its I/O thread."""

    def __init__(self, host: str = "127.0.0.1", port: int = 0, backlog: int = 1024):
        self._lib = _lib()
        self._h = self._lib.bfront_create(host.encode(), int(port), int(backlog))
        if not self._h:
            raise OSError(f"cannot listen on {host}:{port}")
        self.host, self.port = host, int(self._lib.bfront_port(self._h))
        self._stopped = False
        self._closed = False
        self.has_vocab = False

    def start(self) -> "NativeFront":
        self._lib.bfront_start(self._h)
        return self

    def stop(self) -> None:
        if not self._stopped:
            self._stopped = True
            self._lib.bfront_stop(self._h)

    def close(self) -> None:
        """Stops the I/O thread and closes every socket.  The native object stays valid for the rest of the process, so a
        thread that still holds a stream or waits for an event gets "gone" / end-of-events instead of a dangling pointer."""
        if not self._closed:
            self._closed = True
            self.stop()
            self._lib.bfront_destroy(self._h)

    def set_vocab(self, tokenizer, vocab_size: int | None = None) -> None:
        """Token id -> bytes for every id, so that streams detokenise without the interpreter."""
        n = max(int(vocab_size or 0), int(getattr(tokenizer, "vocab_size", 0) or 0))

        def piece(i: int) -> bytes:
            try:
                return tokenizer.token_bytes(i)
            except Exception:  # noqa: BLE001 - an id the tokenizer does not know prints nothing
                return b""
        pieces = [piece(i) for i in range(n)]
        offsets = (C.c_uint32 * (n + 1))()
        total = 0
        for i, p in enumerate(pieces):
            offsets[i] = total
            total += len(p)
        offsets[n] = total
        self._lib.bfront_set_vocab(self._h, b"".join(pieces), offsets, n)
        self.has_vocab = True

    def next_event(self, timeout_ms: int = 200):
        """(kind, conn, method, target, raw headers, body, peer) or None on time-out; raises EOFError once stopped and drained."""
        stopped = C.c_int(0)
        p = self._lib.bfront_next_event(self._h, timeout_ms, C.byref(stopped))
        if not p:
            if stopped.value:
                raise EOFError("front stopped")
            return None
        try:
            kind, conn = struct.unpack("<iq", C.string_at(p, 12))
            lens = struct.unpack("<5I", C.string_at(p + 12, 20))
            blob = C.string_at(p + 32, sum(lens))
        finally:
            self._lib.bfront_free(p)
        parts, off = [], 0
        for n in lens:
            parts.append(blob[off:off + n])
            off += n
        return (kind, conn, parts[0].decode("latin-1"), parts[1].decode("latin-1"), parts[2], parts[3], parts[4].decode())

    def respond(self, conn: int, status: int, headers: Iterable[tuple[bytes, bytes]], body: bytes) -> bool:
        return self._lib.bfront_respond(self._h, conn, status, _header_block(headers), body, len(body)) == 0

    def respond_start(self, conn: int, status: int, headers: Iterable[tuple[bytes, bytes]]) -> bool:
        return self._lib.bfront_respond_start(self._h, conn, status, _header_block(headers)) == 0

    def respond_chunk(self, conn: int, data: bytes) -> bool:
        return self._lib.bfront_respond_chunk(self._h, conn, data, len(data)) == 0

    def respond_end(self, conn: int) -> bool:
        return self._lib.bfront_respond_end(self._h, conn) == 0

    def open_stream(self, conn: int, chunk_head: str, chat: bool, stops: list[str], first_event: str = "", timeout_ms: int = 0) -> NativeStream:
        blob = struct.pack("<I", len(stops))
        for s in stops:
            b = s.encode("utf-8")
            blob += struct.pack("<I", len(b)) + b
        sid = self._lib.bfront_stream_open(self._h, conn, chunk_head.encode("utf-8"), 1 if chat else 0, blob, first_event.encode("utf-8"), int(timeout_ms))
        if sid <= 0:
            raise ConnectionError("the connection is gone")
        return NativeStream(self, sid)

    def set_lazy(self, on: bool) -> None:
        """Lazy wake-ups: pushed tokens are written when :meth:`kick` is called (the producer does that once per decode
        step) or, failing that, within a few milliseconds."""
        self._lib.bfront_set_lazy(self._h, 1 if on else 0)

    def kick(self) -> None:
        self._lib._bfront_kick_held(self._h)

    def set_idle_timeout(self, seconds: float) -> None:
        """Keep-alive connections that wait for a request and move no byte for this long are closed (default 75 s; 0: never)."""
        self._lib.bfront_set_idle_timeout(self._h, int(seconds * 1000))

    def stats(self) -> dict:
        out = (C.c_uint64 * 8)()
        self._lib.bfront_stats(self._h, out)
        keys = ("connections_accepted", "requests", "stream_tokens", "stream_events", "bytes_out", "open_connections", "open_streams", "idle_closed")
        return dict(zip(keys, (int(v) for v in out)))


class FrontHandle:
    """What a route finds under ``request.scope["extensions"]["oxibonsai.front"]``: the front and the request's connection."""

    def __init__(self, front: NativeFront, conn: int):
        self.front, self.conn = front, conn
        self.stream: NativeStream | None = None

    def open_stream(self, chunk_head: str, chat: bool, stops: list[str], first_event: str = "", timeout_ms: int = 0) -> NativeStream:
        self.stream = self.front.open_stream(self.conn, chunk_head, chat, stops, first_event, timeout_ms)
        return self.stream


def _parse_headers(raw: bytes) -> list[tuple[bytes, bytes]]:
    out = []
    for line in raw.split(b"\r\n"):
        if not line:
            continue
        k, _, v = line.partition(b":")
        out.append((k.strip().lower(), v.strip()))
    return out


class AsgiBridge:
    """Runs an ASGI application behind a :class:`NativeFront`: one task per request on this thread's event loop."""

    def __init__(self, app, front: NativeFront):
        self.app, self.front = app, front
        self._gone: dict[int, asyncio.Event] = {}
        self._tasks: set[asyncio.Task] = set()
        self.requests = 0

    async def _lifespan(self, phase: str, state: dict) -> None:
        """Runs the application's startup / shutdown handlers (ASGI lifespan protocol); applications without them are fine."""
        q_in: asyncio.Queue = asyncio.Queue()
        q_out: asyncio.Queue = asyncio.Queue()
        if phase == "startup":
            async def run():
                try:
                    await self.app({"type": "lifespan", "asgi": {"version": "3.0", "spec_version": "2.0"}, "state": state}, q_in.get, q_out.put)
                except Exception:  # noqa: BLE001 - an application without lifespan support
                    pass
                # raised, or returned without taking part in the protocol: whoever still waits for an answer gets this one
                await q_out.put({"type": "lifespan.startup.failed.unsupported"})
            self._life = (asyncio.ensure_future(run()), q_in, q_out)
            await q_in.put({"type": "lifespan.startup"})
            msg = await q_out.get()
            if msg["type"] == "lifespan.startup.failed":
                raise RuntimeError(f"application startup failed: {msg.get('message', '')}")
        else:
            task, q_in, q_out = self._life
            if not task.done():
                await q_in.put({"type": "lifespan.shutdown"})
                try:
                    await asyncio.wait_for(q_out.get(), 10)
                except asyncio.TimeoutError:
                    task.cancel()

    async def _handle(self, conn: int, method: str, target: str, raw_headers: bytes, body: bytes, peer: str, state: dict) -> None:
        front = self.front
        path, _, query = target.partition("?")
        host, _, port = peer.rpartition(":")
        handle = FrontHandle(front, conn)
        gone = self._gone.setdefault(conn, asyncio.Event())
        scope = {"type": "http", "asgi": {"version": "3.0", "spec_version": "2.3"}, "http_version": "1.1", "method": method.upper(), "scheme": "http",
                 "path": unquote(path), "raw_path": path.encode("latin-1"), "query_string": query.encode("latin-1"), "root_path": "",
                 "headers": _parse_headers(raw_headers), "client": (host, int(port or 0)), "server": (front.host, front.port),
                 "extensions": {"oxibonsai.front": handle}, "state": dict(state)}
        sent_body = False
        started: dict = {}

        async def receive():
            nonlocal sent_body
            if not sent_body:
                sent_body = True
                return {"type": "http.request", "body": body, "more_body": False}
            await gone.wait()
            return {"type": "http.disconnect"}

        async def send(msg):
            t = msg["type"]
            if t == "http.response.start":
                started.update(status=msg["status"], headers=list(msg.get("headers", [])), mode=None)
                if handle.stream is not None and any(k.lower() == NATIVE_STREAM_HEADER for k, _ in started["headers"]):
                    started["mode"] = "native"
                    handle.stream.begin(started["headers"])
                return
            if t != "http.response.body" or started.get("mode") == "native":
                return
            data, more = msg.get("body", b""), msg.get("more_body", False)
            if started["mode"] is None:
                if not more:
                    started["mode"] = "done"
                    if not front.respond(conn, started["status"], started["headers"], data):
                        raise OSError("client disconnected")
                    return
                started["mode"] = "chunked"
                if not front.respond_start(conn, started["status"], started["headers"]):
                    raise OSError("client disconnected")
            if started["mode"] == "chunked":
                if data and not front.respond_chunk(conn, data):
                    raise OSError("client disconnected")
                if not more:
                    started["mode"] = "done"
                    front.respond_end(conn)

        try:
            await self.app(scope, receive, send)
        except Exception as e:  # noqa: BLE001 - the application's own error handling has already had its chance
            if not started:
                front.respond(conn, 500, [(b"content-type", b"text/plain")], f"internal error: {type(e).__name__}".encode())
            elif started.get("mode") == "chunked":
                front.respond_end(conn)
        finally:
            if handle.stream is not None and started.get("mode") != "native":
                handle.stream.abandon()               # a stream was opened but the route answered in another way
            self._gone.pop(conn, None)

    async def serve(self, stop: threading.Event | None = None, grace_seconds: float = 5.0) -> None:
        """Dispatches requests until ``stop`` is set; requests that are being answered then get ``grace_seconds`` to finish."""
        loop = asyncio.get_running_loop()
        state: dict = {}
        await self._lifespan("startup", state)
        try:
            while stop is None or not stop.is_set():
                try:
                    ev = await loop.run_in_executor(None, self.front.next_event, 200)
                except EOFError:
                    break
                if ev is None:
                    continue
                kind, conn = ev[0], ev[1]
                if kind == 2:
                    g = self._gone.pop(conn, None)
                    if g is not None:
                        g.set()
                    continue
                self.requests += 1
                task = asyncio.ensure_future(self._handle(conn, *ev[2:], state))
                self._tasks.add(task)
                task.add_done_callback(self._tasks.discard)
        finally:
            if self._tasks and grace_seconds > 0:
                await asyncio.wait(list(self._tasks), timeout=grace_seconds)
            for t in list(self._tasks):
                t.cancel()
            await self._lifespan("shutdown", state)


def serve(app, host: str, port: int, tokenizer=None, stop: threading.Event | None = None, on_ready=None, vocab_size: int | None = None,
          grace_seconds: float = 5.0) -> None:
    """Serves ``app`` until ``stop`` is set or the process receives SIGINT / SIGTERM, then shuts down gracefully: no new
    requests are dispatched, requests being answered and token streams being produced get ``grace_seconds`` to finish, then
    every socket is closed.  With ``tokenizer`` the front detokenises streamed completions itself; ``vocab_size``: the
    model's vocabulary when it is larger than the tokenizer's."""
    import signal
    import time
    front = NativeFront(host, port)
    if tokenizer is not None:
        front.set_vocab(tokenizer, vocab_size)
    front.start()
    if on_ready is not None:
        on_ready(front)
    stop = stop or threading.Event()
    previous = {}
    if threading.current_thread() is threading.main_thread():
        for sig in (signal.SIGINT, signal.SIGTERM):
            previous[sig] = signal.signal(sig, lambda *_: stop.set())
    bridge = AsgiBridge(app, front)
    try:
        asyncio.run(bridge.serve(stop, grace_seconds))
        deadline = time.monotonic() + grace_seconds
        while front.stats()["open_streams"] and time.monotonic() < deadline:      # streams are fed by the scheduler, not by a task
            time.sleep(0.02)
    except KeyboardInterrupt:
        pass
    finally:
        for sig, handler in previous.items():
            signal.signal(sig, handler)
        front.close()
