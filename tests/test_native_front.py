"""The C++ HTTP / SSE front on CPU: request parsing and keep-alive, the token stream (UTF-8 boundaries, stop-sequence
hold-back, JSON escaping, chunked SSE framing) against a Python restatement, and the whole application behind it against
the same application driven through its own Python streaming path."""
import http.client
import json
import random
import socket
import threading
import time

import pytest

from oxibonsai_b200.runtime.presets import SamplingParams
from oxibonsai_b200.server.native_front import AsgiBridge, NativeFront, StreamClosed
from oxibonsai_b200.tokenizer import ByteTokenizer, StreamingDecoder

HEAD = '{"id": "x", "choices": [{"index": 0, '


class _Echo(threading.Thread):
    """Answers every request with a JSON description of it; "/stream" runs ``self.script(front, conn)``."""

    def __init__(self, front, script=None):
        super().__init__(daemon=True)
        self.front, self.script, self.closed = front, script, []

    def run(self):
        f = self.front
        while True:
            try:
                ev = f.next_event(100)
            except EOFError:
                return
            if ev is None:
                continue
            kind, conn, method, target, hdrs, body, peer = ev
            if kind == 2:
                self.closed.append(conn)
            elif target.startswith("/stream") and self.script:
                self.script(f, conn)
            else:
                f.respond(conn, 200, [(b"content-type", b"application/json")],
                          json.dumps({"method": method, "target": target, "body": len(body), "headers": hdrs.decode("latin-1")}).encode())


@pytest.fixture()
def front():
    f = NativeFront("127.0.0.1", 0)
    f.set_vocab(ByteTokenizer())
    f.start()
    yield f
    f.close()


def _events(raw: str) -> list:
    out = []
    for block in raw.split("\n\n"):
        if block.startswith("data: "):
            out.append(block[6:] if block[6:] == "[DONE]" else json.loads(block[6:]))
    return out


def test_requests_keep_alive_pipelining_and_errors(front):
    _Echo(front).start()
    c = http.client.HTTPConnection("127.0.0.1", front.port, timeout=10)
    c.request("GET", "/a/b?x=1", headers={"X-Thing": "v"})
    r = c.getresponse()
    d = json.loads(r.read())
    assert r.status == 200 and d["method"] == "GET" and d["target"] == "/a/b?x=1" and "X-Thing: v" in d["headers"]
    c.request("POST", "/p", body=b"z" * 300000)                          # larger than one read; same connection
    assert json.loads(c.getresponse().read())["body"] == 300000
    c.request("HEAD", "/h")                                              # headers as for GET, no body; the connection stays usable
    r = c.getresponse()
    assert r.status == 200 and int(r.getheader("content-length")) > 0 and r.read() == b""
    c.request("GET", "/after-head")
    assert json.loads(c.getresponse().read())["target"] == "/after-head"
    # two requests in one write, answered in order on one connection
    s = socket.create_connection(("127.0.0.1", front.port))
    s.sendall(b"GET /one HTTP/1.1\r\nHost: x\r\n\r\nPOST /two HTTP/1.1\r\nHost: x\r\nContent-Length: 3\r\nConnection: close\r\n\r\nabc")
    data = b""
    while chunk := s.recv(65536):
        data += chunk
    assert data.count(b"HTTP/1.1 200 OK") == 2 and data.index(b"/one") < data.index(b"/two") and b"connection: close" in data
    # a chunked request body (with a chunk extension and a trailer), sent in two pieces, then a second request on the same connection
    s = socket.create_connection(("127.0.0.1", front.port))
    s.sendall(b"POST /chunked HTTP/1.1\r\nHost: x\r\nTransfer-Encoding: chunked\r\n\r\n5;ext=1\r\nhello\r\n")
    time.sleep(0.05)
    s.sendall(b"6\r\n world\r\n0\r\nX-Trailer: v\r\n\r\nGET /after-chunked HTTP/1.1\r\nConnection: close\r\n\r\n")
    data = b""
    while chunk := s.recv(65536):
        data += chunk
    assert b'"target": "/chunked", "body": 11' in data and b'"target": "/after-chunked"' in data
    # Expect: 100-continue is answered before the body is sent
    s = socket.create_connection(("127.0.0.1", front.port))
    s.sendall(b"POST /e HTTP/1.1\r\nHost: x\r\nContent-Length: 4\r\nExpect: 100-continue\r\n\r\n")
    assert s.recv(100).startswith(b"HTTP/1.1 100 Continue")
    s.sendall(b"data")
    assert b'"body": 4' in s.recv(65536)
    s.close()
    for bad, status in ((b"NONSENSE\r\n\r\n", b"400"), (b"GET / HTTP/1.1\r\nContent-Length: x\r\n\r\n", b"400"),
                        (b"POST / HTTP/1.1\r\nTransfer-Encoding: chunked\r\n\r\nzz\r\nabc\r\n0\r\n\r\n", b"400"),
                        (b"POST / HTTP/1.1\r\nTransfer-Encoding: chunked\r\n\r\n3\r\nabcXX0\r\n\r\n", b"400"),
                        (b"POST / HTTP/1.1\r\nContent-Length: 3\r\nContent-Length: 5\r\n\r\nabcde", b"400"), (b"GET / HTTP/1.1\r\nA: " + b"a" * 70000 + b"\r\n\r\n", b"431")):
        s = socket.create_connection(("127.0.0.1", front.port))
        s.sendall(bad)
        assert s.recv(200).split(b" ")[1] == status
        s.close()
    st = front.stats()
    assert st["requests"] == 9 and st["connections_accepted"] == 10


def _reference_stream(tokens, stops):
    """The Python streaming path's text logic (StreamingDecoder + stop hold-back): returns (text sent, stop hit)."""
    dec, text, sent = StreamingDecoder(), "", ""
    tb = ByteTokenizer().token_bytes
    for t in tokens:
        text += dec.push(tb(t))
        cut = min((text.find(s) for s in stops if s and s in text), default=-1)
        if cut >= 0:
            return text[:cut], True
    text += dec.flush()
    return text, False


@pytest.mark.parametrize("seed", range(6))
def test_token_stream_matches_the_python_text_logic(front, seed):
    rng = random.Random(seed)
    alphabet = ["a", "b", "é", "ü", "\n", '"', "\\", "日本", "🙂", "\t", "<", "END", "</s>", "\x01"]
    stops = [["END"], ["</s>", "b\n"], [], ["日本"], ["🙂a"], ["ab", "ba"]][seed]
    text = "".join(rng.choice(alphabet) for _ in range(60))
    tokens = list(text.encode("utf-8"))
    if seed == 2:
        tokens += [0xE6, 0x97]                       # the generation ends inside a character
    got = {}

    def script(f, conn):
        s = f.open_stream(conn, HEAD, True, stops, "", 0)
        s.begin([(b"content-type", b"text/event-stream")])
        hit = False
        for t in tokens:
            try:
                s.push(t)
            except StreamClosed as e:
                hit = e.state == 1
                break
        got["hit"], got["n"] = hit, s.finish("length")

    _Echo(front, script).start()
    c = http.client.HTTPConnection("127.0.0.1", front.port, timeout=10)
    c.request("GET", "/stream")
    r = c.getresponse()
    evs = _events(r.read().decode("utf-8"))
    assert r.status == 200 and r.getheader("transfer-encoding") == "chunked" and evs[-1] == "[DONE]"
    want_text, want_hit = _reference_stream(tokens, stops)
    deadline = time.monotonic() + 5
    while "n" not in got and time.monotonic() < deadline:      # the producer returns from finish() after the client has the bytes
        time.sleep(0.005)
    sent = "".join(e["choices"][0]["delta"].get("content", "") for e in evs[:-1])
    assert sent == want_text and got["hit"] == want_hit
    assert evs[-2]["choices"][0]["finish_reason"] == ("stop" if want_hit else "length") and evs[-2]["choices"][0]["delta"] == {}
    # nothing that could still become a stop sequence was sent early: every prefix of the deltas is stop-free
    acc = ""
    for e in evs[:-2]:
        acc += e["choices"][0]["delta"]["content"]
        assert not any(s in acc for s in stops)
    c.request("GET", "/next")                          # the connection is reusable after a stream
    assert c.getresponse().status == 200


def test_stream_before_the_head_client_loss_and_deadline(front):
    state = {}

    def script(f, conn):
        s = f.open_stream(conn, HEAD, False, [], "", 150 if state.get("deadline") else 0)
        if state.get("early"):                        # the generation is over before the response head is written
            for t in b"hi":
                s.push(t)
            s.finish("stop")
            s.begin([(b"content-type", b"text/event-stream")])
            return
        s.begin([(b"content-type", b"text/event-stream")])
        try:
            for i in range(400):
                s.push(ord("a"))
                time.sleep(0.005)
            state["result"] = "ran to the end"
        except StreamClosed as e:
            state["result"] = e.state
        s.finish("length")

    echo = _Echo(front, script)
    echo.start()
    state["early"] = True
    c = http.client.HTTPConnection("127.0.0.1", front.port, timeout=10)
    c.request("GET", "/stream")
    evs = _events(c.getresponse().read().decode())
    assert [e["choices"][0]["text"] for e in evs[:-1]] == ["h", "i", ""] and evs[-2]["choices"][0]["finish_reason"] == "stop"
    state.clear()
    s = socket.create_connection(("127.0.0.1", front.port))
    s.sendall(b"GET /stream HTTP/1.1\r\nHost: x\r\n\r\n")
    s.recv(200)
    s.close()                                          # the client goes away in mid-stream
    deadline = time.monotonic() + 5
    while "result" not in state and time.monotonic() < deadline:
        time.sleep(0.01)
    assert state["result"] == 2 and echo.closed
    state.clear()
    state["deadline"] = True
    c = http.client.HTTPConnection("127.0.0.1", front.port, timeout=10)
    c.request("GET", "/stream")
    c.getresponse().read()
    deadline = time.monotonic() + 5
    while "result" not in state and time.monotonic() < deadline:
        time.sleep(0.005)
    assert state["result"] == 3                        # the request's time ran out: the producer is told to stop
    assert front.stats()["open_streams"] == 0


# ---- the application behind the front ----------------------------------------------------------------------------------
def _serve_app(app, tokenizer):
    import asyncio
    front = NativeFront("127.0.0.1", 0)
    front.set_vocab(tokenizer)
    front.start()
    stop = threading.Event()
    bridge = AsgiBridge(app, front)
    t = threading.Thread(target=lambda: asyncio.run(bridge.serve(stop)), daemon=True)
    t.start()
    return front, stop, t


def test_application_behind_the_front_streams_like_the_python_path():
    from fastapi.testclient import TestClient
    from test_scheduler_cpu import FakeEngine
    from oxibonsai_b200.runtime.scheduler import BatchScheduler
    from oxibonsai_b200.server.app import SchedulerBackend, create_app
    from oxibonsai_b200.server.config import ServerConfig

    class ByteEngine(FakeEngine):                      # tokens stay below 256 so that the byte tokenizer can print them
        def finish_sequence(self, prompt, slot):
            return 97 + super().finish_sequence(prompt, slot) % 26

        def step_batch(self, positions):
            return [97 + t % 26 for t in super().step_batch(positions)]

        def kv_utilization(self):
            return 0.1

    class Named:
        name = "fake"

    eng = ByteEngine()
    eng.config = Named()
    sched = BatchScheduler(eng, prefill_chunk_tokens=16, eos_token=-1).start()
    tok = ByteTokenizer()
    app = create_app(SchedulerBackend(sched, "fake-bonsai"), tok, ServerConfig(bearer_token="t" * 16))
    front, stop, thread = _serve_app(app, tok)
    try:
        auth = {"Authorization": "Bearer " + "t" * 16, "Content-Type": "application/json"}
        c = http.client.HTTPConnection("127.0.0.1", front.port, timeout=20)
        c.request("GET", "/health")
        r = c.getresponse()
        assert r.status == 200 and r.read() == b"ok"
        c.request("POST", "/v1/chat/completions", body=b"{}", headers={"Content-Type": "application/json"})
        r = c.getresponse()
        assert r.status == 401 and r.read()
        req = {"messages": [{"role": "user", "content": "hello there"}], "max_tokens": 40, "stream": True, "stop": ["xyz"]}
        c.request("POST", "/v1/chat/completions", body=json.dumps(req), headers=auth)
        r = c.getresponse()
        native = _events(r.read().decode())
        assert r.status == 200 and r.getheader("content-type").startswith("text/event-stream") and r.getheader("x-request-id")
        assert r.getheader("x-oxibonsai-native-stream") is None
        with TestClient(app) as tc:                    # the same application without the front: its own streaming path
            py = _events(tc.post("/v1/chat/completions", json=req, headers=auth).text)
        text = lambda evs: "".join(e["choices"][0]["delta"].get("content", "") for e in evs if e != "[DONE]")
        assert native[0]["choices"][0]["delta"] == {"role": "assistant"} and native[-1] == "[DONE]" and py[-1] == "[DONE]"
        assert text(native) == text(py) == "bcdefghijklmnopqrstuvw"          # the stop sequence "xyz" follows and is not sent
        assert native[-2]["choices"][0]["finish_reason"] == py[-2]["choices"][0]["finish_reason"] == "stop"
        del req["stop"]
        c.request("POST", "/v1/chat/completions", body=json.dumps(req), headers=auth)
        plain = _events(c.getresponse().read().decode())
        assert len(text(plain)) == 40 and plain[-2]["choices"][0]["finish_reason"] == "length"
        assert native[1]["object"] == "chat.completion.chunk" and native[1]["model"] == "fake-bonsai"
        # completions endpoint, not streamed: goes through the application's ordinary response
        c.request("POST", "/v1/completions", body=json.dumps({"prompt": "abc", "max_tokens": 5}), headers=auth)
        r = c.getresponse()
        d = json.loads(r.read())
        assert r.status == 200 and len(d["choices"][0]["text"]) == 5
        # 16 streams at once over the front
        results = {}

        def one(i):
            cc = http.client.HTTPConnection("127.0.0.1", front.port, timeout=30)
            cc.request("POST", "/v1/completions", body=json.dumps({"prompt": "p" * (i + 1), "max_tokens": 30, "stream": True}), headers=auth)
            results[i] = _events(cc.getresponse().read().decode())

        ts = [threading.Thread(target=one, args=(i,)) for i in range(16)]
        [t.start() for t in ts]
        [t.join(30) for t in ts]
        assert len(results) == 16 and all(r[-1] == "[DONE]" and sum(len(e["choices"][0]["text"]) for e in r[:-1]) == 30 for r in results.values())
        m = app.state.metrics
        assert m.tokens_generated.get() >= 40 + 16 * 30 and m.active_requests.get() == 0 and m.aggregator.snapshot()["completed_requests"] >= 18
        c.request("GET", "/metrics")
        assert b"oxibonsai_tokens_generated_total" in c.getresponse().read()
        st = front.stats()
        assert st["stream_tokens"] >= 40 + 16 * 30 and st["open_streams"] == 0
    finally:
        stop.set()
        thread.join(5)
        front.close()
        sched.stop()


def test_front_is_race_free_under_thread_sanitizer(tmp_path):
    """The front's C++ compiled with -fsanitize=thread together with a driver that runs clients, a dispatcher and a token
    producer concurrently (tests/front_tsan_driver.cpp): no data race may be reported."""
    import os
    import subprocess
    here = os.path.dirname(os.path.abspath(__file__))
    src = os.path.join(os.path.dirname(here), "oxibonsai_b200", "csrc", "runtime", "http_front.cpp")
    exe = str(tmp_path / "front_tsan")
    probe = subprocess.run(["g++", "-fsanitize=thread", "-x", "c++", "-", "-o", str(tmp_path / "probe")], input="int main(){return 0;}", capture_output=True, text=True)
    if probe.returncode != 0:
        pytest.skip("the host compiler has no ThreadSanitizer runtime")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-pthread", "-fsanitize=thread", src, os.path.join(here, "front_tsan_driver.cpp"), "-o", exe],
                           capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-3000:]
    for _ in range(2):
        run = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=dict(os.environ, TSAN_OPTIONS="halt_on_error=0"))
        assert run.returncode == 0 and "tsan driver ok" in run.stdout, run.stdout[-1000:] + run.stderr[-3000:]
        assert "WARNING: ThreadSanitizer" not in run.stderr, run.stderr[-4000:]


def test_client_that_leaves_frees_its_slot_and_failed_submits_answer_503():
    """Behind the front a stream whose client goes away is cancelled at its next token (the scheduler frees the slot), and a
    backend that refuses a request (queue full) answers 503 on the same connection instead of opening a stream."""
    import socket
    from test_scheduler_cpu import FakeEngine
    from oxibonsai_b200.runtime.scheduler import BatchScheduler
    from oxibonsai_b200.server.app import SchedulerBackend, create_app
    from oxibonsai_b200.server.config import ServerConfig

    class SlowBytes(FakeEngine):
        def finish_sequence(self, prompt, slot):
            return 97 + super().finish_sequence(prompt, slot) % 26

        def step_batch(self, positions):
            return [97 + t % 26 for t in super().step_batch(positions)]

        def kv_utilization(self):
            return 0.0

    eng = SlowBytes(step_delay=0.01)
    eng.config = type("C", (), {"name": "fake"})()
    sched = BatchScheduler(eng, prefill_chunk_tokens=16, eos_token=-1, queue_capacity=1).start()
    tok = ByteTokenizer()
    app = create_app(SchedulerBackend(sched, "fake"), tok, ServerConfig())
    front, stop, thread = _serve_app(app, tok)
    app.state.backend.set_after_step(front.kick)
    front.set_lazy(True)
    try:
        body = json.dumps({"prompt": "abcdefgh", "max_tokens": 2000, "stream": True}).encode()
        s = socket.create_connection(("127.0.0.1", front.port))
        s.sendall(b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: " + str(len(body)).encode() + b"\r\n\r\n" + body)
        got = b""
        while got.count(b"data: ") < 5:
            got += s.recv(65536)
        assert sched.active == 1
        s.close()                                              # the client leaves after a few tokens
        deadline = time.monotonic() + 5
        while sched.active and time.monotonic() < deadline:
            time.sleep(0.01)
        assert sched.active == 0 and sched.tokens_generated < 1500        # cancelled long before max_tokens
        assert front.stats()["open_streams"] == 0 and app.state.metrics.active_requests.get() == 0
        # the admission queue holds one request: a burst of eight is partly refused with 503 (how many depends on timing), not hung
        conns = []
        for _ in range(8):
            c = http.client.HTTPConnection("127.0.0.1", front.port, timeout=20)
            c.request("POST", "/v1/completions", body=json.dumps({"prompt": "abcdefgh", "max_tokens": 40, "stream": True}), headers={"Content-Type": "application/json"})
            conns.append(c)
        statuses = []
        for c in conns:
            r = c.getresponse()
            statuses.append(r.status)
            data = r.read()
            assert (b"[DONE]" in data) if r.status == 200 else (b"error" in data)
        assert statuses.count(200) >= 1 and statuses.count(503) >= 1 and set(statuses) <= {200, 503}
        assert app.state.metrics.active_requests.get() == 0
    finally:
        stop.set()
        thread.join(5)
        front.close()
        sched.stop()


def test_idle_connections_are_closed_but_streams_are_not(front):
    """A connection that waits for a request (or sits on half of one) without moving a byte is closed after the idle
    time-out; a connection whose stream is being produced slowly is not."""
    front.set_idle_timeout(0.3)

    def script(f, conn):
        s = f.open_stream(conn, HEAD, False, [], "", 0)
        s.begin([(b"content-type", b"text/event-stream")])
        time.sleep(0.8)                                    # longer than the idle time-out, no byte in between
        s.push(ord("z"))
        s.finish("stop")

    _Echo(front, script).start()
    idle = socket.create_connection(("127.0.0.1", front.port))
    half = socket.create_connection(("127.0.0.1", front.port))
    half.sendall(b"POST /x HTTP/1.1\r\nContent-Length: 100\r\n\r\npartial")
    c = http.client.HTTPConnection("127.0.0.1", front.port, timeout=10)
    c.request("GET", "/stream")
    evs = _events(c.getresponse().read().decode())
    assert [e["choices"][0]["text"] for e in evs[:-1]] == ["z", ""] and evs[-1] == "[DONE]"
    for sk in (idle, half):
        sk.settimeout(3)
        assert sk.recv(100) == b""                         # closed by the server
        sk.close()
    assert front.stats()["idle_closed"] == 2


def test_sigterm_shuts_the_server_down_gracefully(tmp_path):
    """``serve()`` in a child process: SIGTERM while a stream is being produced lets that stream finish ("[DONE]" arrives),
    then the process exits with status 0."""
    import os
    import signal
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = f"""
import sys
sys.path.insert(0, {root!r}); sys.path.insert(0, {os.path.join(root, 'benchmarks')!r})
from front_overhead import run_server
run_server("native", int(sys.argv[1]), 4, 20.0)
"""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    child = subprocess.Popen([sys.executable, "-c", code, str(port)], env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    try:
        for _ in range(200):
            try:
                socket.create_connection(("127.0.0.1", port), timeout=0.2).close()
                break
            except OSError:
                time.sleep(0.1)
        body = json.dumps({"prompt": "abc", "max_tokens": 40, "stream": True}).encode()
        s = socket.create_connection(("127.0.0.1", port))
        s.sendall(b"POST /v1/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: " + str(len(body)).encode() + b"\r\n\r\n" + body)
        got = b""
        while got.count(b"data: ") < 3:
            got += s.recv(65536)
        child.send_signal(signal.SIGTERM)                  # 40 tokens at 20 ms per step: the stream still has ~0.7 s to go
        s.settimeout(10)
        while True:
            chunk = s.recv(65536)
            if not chunk:
                break
            got += chunk
        assert b"data: [DONE]" in got and got.count(b"data: ") == 40 + 2      # 40 tokens, the finish chunk, [DONE]
        assert child.wait(15) == 0
    finally:
        if child.poll() is None:
            child.kill()


def test_python_driven_streams_and_errors_pass_through_the_bridge():
    """A backend without completion callbacks streams through the application's own SSE generator: the bridge forwards its
    chunks with chunked framing; an application error before the response starts becomes a 500; the connection survives."""
    from test_server import FakeBackend
    from oxibonsai_b200.server.app import create_app
    from oxibonsai_b200.server.config import ServerConfig
    tok = ByteTokenizer()
    app = create_app(FakeBackend("héllo wörld"), tok, ServerConfig())

    @app.get("/boom")
    async def boom():
        raise RuntimeError("kaput")

    front, stop, thread = _serve_app(app, tok)
    try:
        c = http.client.HTTPConnection("127.0.0.1", front.port, timeout=20)
        c.request("POST", "/v1/chat/completions", body=json.dumps({"messages": [{"role": "user", "content": "x"}], "stream": True, "max_tokens": 64}),
                  headers={"Content-Type": "application/json"})
        r = c.getresponse()
        evs = _events(r.read().decode())
        assert r.status == 200 and r.getheader("transfer-encoding") == "chunked" and evs[-1] == "[DONE]"
        assert "".join(e["choices"][0]["delta"].get("content", "") for e in evs[:-1]) == "héllo wörld"
        assert front.stats()["stream_tokens"] == 0                      # not a native stream: the application produced the events
        c.request("GET", "/boom")
        r = c.getresponse()
        assert r.status == 500 and r.read()
        c.request("GET", "/v1/models")
        assert json.loads(c.getresponse().read())["data"][0]["id"] == "fake-bonsai"
        c.request("GET", "/nowhere")
        assert c.getresponse().status == 404
    finally:
        stop.set()
        thread.join(5)
        front.close()


def test_http10_clients_get_unframed_streams_that_end_with_the_connection(front):
    def script(f, conn):
        s = f.open_stream(conn, HEAD, False, [], "", 0)
        s.begin([(b"content-type", b"text/event-stream")])
        for t in b"ok":
            s.push(t)
        s.finish("stop")

    _Echo(front, script).start()
    s = socket.create_connection(("127.0.0.1", front.port))
    s.sendall(b"GET /stream HTTP/1.0\r\nHost: x\r\n\r\n")
    data = b""
    while chunk := s.recv(65536):
        data += chunk
    head, _, body = data.partition(b"\r\n\r\n")
    assert b"transfer-encoding" not in head.lower() and b"connection: close" in head
    evs = _events(body.decode())                               # no chunk sizes between the events
    assert [e["choices"][0]["text"] for e in evs[:-1]] == ["o", "k", ""] and evs[-1] == "[DONE]" and body.startswith(b"data: ")
    s = socket.create_connection(("127.0.0.1", front.port))
    s.sendall(b"GET /plain HTTP/1.0\r\n\r\n")
    data = b""
    while chunk := s.recv(65536):
        data += chunk
    assert data.startswith(b"HTTP/1.1 200 OK") and b"content-length" in data and b'"target": "/plain"' in data


def test_listen_address_may_be_a_name_or_an_ipv6_address():
    """"::" listens on both families and names the client by its own family's address; a name resolves; a bad one is refused."""
    import asyncio

    async def app(scope, receive, send):
        if scope["type"] != "http":
            return
        body = json.dumps({"client": scope["client"][0]}).encode()
        await send({"type": "http.response.start", "status": 200, "headers": [(b"content-type", b"application/json"), (b"content-length", str(len(body)).encode())]})
        await send({"type": "http.response.body", "body": body})

    try:
        front = NativeFront("::", 0)
    except OSError:
        pytest.skip("no IPv6 on this host")
    front.start()
    stop = threading.Event()
    t = threading.Thread(target=lambda: asyncio.run(AsgiBridge(app, front).serve(stop)), daemon=True)
    t.start()
    try:
        seen = {}
        for host in ("127.0.0.1", "::1"):
            c = http.client.HTTPConnection(host, front.port, timeout=10)
            c.request("GET", "/whoami")
            r = c.getresponse()
            assert r.status == 200
            seen[host] = json.loads(r.read())["client"]
            c.close()
        assert seen == {"127.0.0.1": "127.0.0.1", "::1": "::1"}
    finally:
        stop.set()
        t.join(5)
        front.close()
    named = NativeFront("localhost", 0)
    assert named.port > 0
    named.close()
    with pytest.raises(OSError):
        NativeFront("no.such.host.invalid", 0)
