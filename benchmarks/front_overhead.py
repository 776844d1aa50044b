"""Cost of the serving front without a GPU: N concurrent SSE streams against the real application and scheduler over a
synthetic engine whose decode step takes a fixed time.

    python benchmarks/front_overhead.py --front native --streams 64 --tokens 256 --step-ms 0
    python benchmarks/front_overhead.py --front uvicorn --streams 64 --tokens 256 --step-ms 0

With ``--step-ms 0`` the engine is free and the figure is the ceiling that the front (HTTP, SSE framing, detokenisation,
the scheduler's own bookkeeping) puts on tokens per second; with the step time of a real model it shows how much of that
step's rate survives.  The server runs in a child process, the clients (raw sockets on an asyncio loop, they only count
events) in this one.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class SyntheticEngine:
    """The scheduler's engine interface with no model behind it: token i of a stream is a letter; a step sleeps."""

    max_seq_len, prefill_min_tokens = 1 << 20, 16

    class config:
        name = "synthetic"

    def __init__(self, max_batch: int, step_ms: float):
        self.max_batch, self.step_s, self.n = max_batch, step_ms / 1e3, 0
        self.exact = True

    def bind_thread(self):
        pass

    def begin_sequence(self, prompt, max_total, slot, params):
        return 0

    def prefill(self, part, slot, pos0):
        pass

    def finish_sequence(self, prompt, slot):
        return 97

    def step_batch(self, positions):
        if self.step_s:
            time.sleep(self.step_s)
        self.n += 1
        return [97 + (self.n + b) % 26 for b in range(len(positions))]

    # the split step: the "GPU" is busy for step_ms from the launch on, whatever the host does meanwhile
    supports_overlap = True

    def launch_batch(self, positions):
        self._ready = time.perf_counter() + self.step_s
        self._batch = len(positions)

    def collect_batch(self, batch):
        wait = self._ready - time.perf_counter()
        if wait > 0:
            time.sleep(wait)
        self.n += 1
        return [97 + (self.n + b) % 26 for b in range(batch)]

    def move_slot(self, src, dst):
        pass

    def close_sequence(self, slot):
        pass

    def kv_utilization(self):
        return 0.0


def run_server(front: str, port: int, streams: int, step_ms: float, overlap: bool = False) -> None:
    from oxibonsai_b200.runtime.scheduler import BatchScheduler
    from oxibonsai_b200.server.app import SchedulerBackend, create_app, serve
    from oxibonsai_b200.server.config import ServerConfig
    from oxibonsai_b200.tokenizer import ByteTokenizer
    sched = BatchScheduler(SyntheticEngine(streams, step_ms), eos_token=-1, overlap=overlap).start()
    tok = ByteTokenizer()
    app = create_app(SchedulerBackend(sched, "synthetic"), tok, ServerConfig(max_concurrent=streams))
    serve(app, "127.0.0.1", port, "error", tokenizer=tok, native=(front == "native"))


async def one_stream(port: int, tokens: int, out: dict, i: int) -> None:
    body = json.dumps({"prompt": "x" * 32, "max_tokens": tokens, "stream": True}).encode()
    reader, writer = await asyncio.open_connection("127.0.0.1", port)
    writer.write(b"POST /v1/completions HTTP/1.1\r\nHost: b\r\nContent-Type: application/json\r\nConnection: close\r\nContent-Length: "
                 + str(len(body)).encode() + b"\r\n\r\n" + body)
    t0 = time.perf_counter()
    first, events, last = None, 0, t0
    while True:
        data = await reader.read(65536)
        if not data:
            break
        n = data.count(b"data: ")
        if n:
            last = time.perf_counter()
            if first is None:
                first = last
            events += n
    writer.close()
    out[i] = (first, last, events)


async def drive(port: int, streams: int, tokens: int) -> dict:
    out: dict = {}
    t0 = time.perf_counter()
    await asyncio.gather(*(one_stream(port, tokens, out, i) for i in range(streams)))
    t1 = time.perf_counter()
    firsts = [v[0] for v in out.values() if v[0] is not None]
    return {"wall_s": t1 - t0, "all_live_s": max(v[1] for v in out.values()) - max(firsts), "events": sum(v[2] for v in out.values()),
            "t_all_started": max(firsts) - t0}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--front", choices=("native", "uvicorn"), default="native")
    ap.add_argument("--streams", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--step-ms", type=float, default=0.0)
    ap.add_argument("--port", type=int, default=18431)
    ap.add_argument("--overlap", action="store_true", help="overlapped decode steps in the scheduler")
    ap.add_argument("--serve", action="store_true", help=argparse.SUPPRESS)
    a = ap.parse_args()
    if a.serve:
        run_server(a.front, a.port, a.streams, a.step_ms, a.overlap)
        return 0
    child = subprocess.Popen([sys.executable, os.path.abspath(__file__), "--serve", "--front", a.front, "--port", str(a.port),
                              "--streams", str(a.streams), "--step-ms", str(a.step_ms)] + (["--overlap"] if a.overlap else []), env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    try:
        import socket
        for _ in range(200):
            try:
                socket.create_connection(("127.0.0.1", a.port), timeout=0.2).close()
                break
            except OSError:
                time.sleep(0.1)
        asyncio.run(drive(a.port, 4, 16))                       # warm-up
        r = asyncio.run(drive(a.port, a.streams, a.tokens))
    finally:
        child.terminate()
        child.wait(10)
    total = a.streams * a.tokens
    print(json.dumps({"front": a.front, "overlap": a.overlap, "streams": a.streams, "tokens_per_stream": a.tokens, "engine_step_ms": a.step_ms,
                      "tokens_per_s": round(total / r["wall_s"], 1), "wall_s": round(r["wall_s"], 3), "sse_events": r["events"],
                      "engine_ceiling_tokens_per_s": round(a.streams / (a.step_ms / 1e3), 1) if a.step_ms else None}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
