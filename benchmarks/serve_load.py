#!/usr/bin/env python
"""Load generator for the OpenAI-compatible server: N concurrent SSE chat streams, aggregate tok/s, TTFT and inter-token latency.

The serving configuration of the reference's own deployment shape (one router, streaming chat completions;
crates/oxibonsai-runtime/src/server.rs:203-243,391-512) scaled to a multi-GPU box: a Ternary-Bonsai-4B-shaped TQ2_0_g128
checkpoint (36 layers, hidden 2560, 32 Q / 8 KV heads, head_dim 128, intermediate 9728, tied embeddings), Q8 KV cache, the
Balanced preset (T = 0.7, top-k 40, top-p 0.9), 64 concurrent streams with prompts of 128..2048 tokens and 256 output tokens.

    python benchmarks/serve_load.py --replicas 1                      # one GPU
    python benchmarks/serve_load.py --replicas 8                      # one engine per GPU behind one HTTP front
    python benchmarks/serve_load.py --tensor-parallel 8               # one engine over eight GPUs (torchrun under the hood)

The script writes the synthetic checkpoint (no tokenizer file: the server falls back to the byte tokenizer, so a prompt of n
ASCII characters is n tokens), starts ``python -m oxibonsai_b200.server`` as a child process, waits for /health, drives the
streams with aiohttp and prints one JSON line.  Times are wall-clock on the client; a token's time is the arrival of its SSE
chunk.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import os
import random
import socket
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SHAPES = {
    "4b": dict(hidden=2560, inter=9728, layers=36, heads=32, kv_heads=8, head_dim=128, vocab=151936, name="Ternary-Bonsai-4B-shaped"),
    "8b": dict(hidden=4096, inter=12288, layers=36, heads=32, kv_heads=8, head_dim=128, vocab=151936, name="Ternary-Bonsai-8B-shaped"),
    "tiny": dict(hidden=512, inter=1024, layers=2, heads=4, kv_heads=2, head_dim=128, vocab=4096, name="tiny"),
}


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


async def one_stream(session, url: str, prompt: str, max_tokens: int, seed: int) -> dict:
    body = {"messages": [{"role": "user", "content": prompt}], "stream": True, "max_tokens": max_tokens, "temperature": 0.7, "top_k": 40,
            "top_p": 0.9, "seed": seed}
    t0 = time.perf_counter()
    times: list[float] = []
    out = {"t0": t0, "times": times, "status": None, "finish": None, "error": None}
    try:
        async with session.post(url, json=body) as resp:
            out["status"] = resp.status
            if resp.status != 200:
                out["error"] = (await resp.text())[:300]
                return out
            async for raw in resp.content:
                line = raw.decode("utf-8", errors="replace").strip()
                if not line.startswith("data:") or line.endswith("[DONE]"):
                    continue
                try:
                    j = json.loads(line[5:])
                    if "error" in j:
                        out["error"] = json.dumps(j["error"])[:300]
                        continue
                    ch = j["choices"][0]
                except Exception:
                    continue
                if (ch.get("delta") or {}).get("content"):
                    times.append(time.perf_counter())
                if ch.get("finish_reason"):
                    out["finish"] = ch["finish_reason"]
    except Exception as e:  # noqa: BLE001 - a failed stream is part of the result
        out["error"] = f"{type(e).__name__}: {e}"[:300]
    return out


async def drive(url: str, prompts: list[str], max_tokens: int) -> list[dict]:
    import aiohttp
    timeout = aiohttp.ClientTimeout(total=3600)
    async with aiohttp.ClientSession(timeout=timeout, connector=aiohttp.TCPConnector(limit=0)) as session:
        return await asyncio.gather(*[one_stream(session, url, p, max_tokens, 42 + i) for i, p in enumerate(prompts)])


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="4b", choices=list(SHAPES))
    ap.add_argument("--streams", type=int, default=64)
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=2048)
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--kv", default="q8")
    ap.add_argument("--replicas", type=int, default=1)
    ap.add_argument("--tensor-parallel", type=int, default=1)
    ap.add_argument("--kv-policy", default="off")
    ap.add_argument("--prefill-chunk-boost", type=int, default=4)
    ap.add_argument("--front", choices=("native", "uvicorn"), default="native", help="the server's HTTP front")
    ap.add_argument("--overlap", action="store_true", help="the server launches decode step k + 1 before delivering the tokens of step k")
    ap.add_argument("--model-dir", default=os.environ.get("BONSAI_BENCH_DIR", "/tmp/oxibonsai_b200_bench"))
    a = ap.parse_args()

    from oxibonsai_b200.core import Qwen3Config, write_synthetic_gguf
    os.makedirs(a.model_dir, exist_ok=True)
    path = os.path.join(a.model_dir, f"{a.model}_tq2_seed42.gguf")
    if not os.path.exists(path):
        write_synthetic_gguf(path + ".tmp", Qwen3Config(context=65536, **SHAPES[a.model]), tied=a.model != "8b", seed=42)
        os.replace(path + ".tmp", path)

    port = free_port()
    per_engine = -(-a.streams // max(1, a.replicas))
    args = ["--model-path", path, "--host", "127.0.0.1", "--port", str(port), "--kv-cache", a.kv, "--max-seq-len", str(a.prompt_max + a.max_tokens + 64),
            "--max-concurrent", str(per_engine), "--max-input-tokens", str(a.prompt_max + 64), "--log-level", "warning", "--kv-policy", a.kv_policy,
            "--replicas", str(a.replicas), "--tensor-parallel", str(a.tensor_parallel), "--prefill-chunk-boost", str(a.prefill_chunk_boost),
            "--native-front" if a.front == "native" else "--no-native-front", "--overlap-steps" if a.overlap else "--no-overlap-steps"]
    if a.tensor_parallel > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.tensor_parallel}", "--master-addr", "127.0.0.1",
               "--master-port", str(free_port()), "-m", "oxibonsai_b200.server", *args]
    else:
        cmd = [sys.executable, "-m", "oxibonsai_b200.server", *args]
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    server = subprocess.Popen(cmd, env=env, stdout=subprocess.DEVNULL, stderr=sys.stderr)
    try:
        import urllib.request
        t_end = time.time() + 900
        while True:
            if server.poll() is not None:
                raise SystemExit(f"server exited with code {server.returncode}")
            try:
                if urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2).status == 200:
                    break
            except Exception:
                pass
            if time.time() > t_end:
                raise SystemExit("server did not come up")
            time.sleep(0.5)
        rnd = random.Random(42)
        # the chat template adds ~30 tokens around the content
        prompts = ["".join(rnd.choice("abcdefghijklmnopqrstuvwxyz ") for _ in range(max(1, rnd.randint(a.prompt_min, a.prompt_max) - 30))) for _ in range(a.streams)]
        url = f"http://127.0.0.1:{port}/v1/chat/completions"
        asyncio.run(drive(url, prompts[:2], 8))                       # warm-up: graph capture, tokenizer tables
        def server_tokens() -> float:
            for line in urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=10).read().decode().splitlines():
                if line.startswith("oxibonsai_tokens_generated_total"):
                    return float(line.split()[-1])
            return 0.0
        n0 = server_tokens()
        t0 = time.perf_counter()
        res = asyncio.run(drive(url, prompts, a.max_tokens))
        wall = time.perf_counter() - t0
        generated = server_tokens() - n0          # the server's own count: every sampled token, whatever text it decodes to
    finally:
        server.terminate()          # this exact child process (torchrun forwards the signal to its ranks)
        try:
            server.wait(timeout=30)
        except subprocess.TimeoutExpired:
            server.kill()
    chunks = sum(len(r["times"]) for r in res)
    ttft = sorted(r["times"][0] - r["t0"] for r in res if r["times"])
    itl = sorted(b - x for r in res for x, b in zip(r["times"], r["times"][1:]))
    # all streams live: from the last first-token to the first last-token
    live = [r for r in res if r["times"]]
    lo, hi = (max(r["times"][0] for r in live), min(r["times"][-1] for r in live)) if live else (0.0, 0.0)
    finishes: dict = {}
    for r in res:
        finishes[str(r["finish"])] = finishes.get(str(r["finish"]), 0) + 1
    errors = [r["error"] for r in res if r["error"]]
    steady = sum(1 for r in res for x in r["times"] if lo < x <= hi)
    pct = lambda v, q: None if not v else round(v[min(len(v) - 1, int(q * len(v)))], 4)
    print(json.dumps({
        "metric": f"aggregate decode tok/s over {a.streams} concurrent SSE streams", "model": SHAPES[a.model]["name"], "kv_cache": a.kv,
        "parallelism": f"tp{a.tensor_parallel}" if a.tensor_parallel > 1 else f"{a.replicas} replica(s)",
        "front": a.front, "overlap_steps": a.overlap, "prefill_chunk_boost": a.prefill_chunk_boost, "prompt_tokens": [a.prompt_min, a.prompt_max], "max_tokens": a.max_tokens, "preset": "balanced (T 0.7, top-k 40, top-p 0.9)",
        "streams_ok": sum(1 for r in res if r["status"] == 200 and not r["error"]), "finish_reasons": finishes, "errors": errors[:3],
        "generated_tokens_server_count": int(generated), "content_chunks": chunks, "wall_s": round(wall, 3),
        "tokens_per_s_overall": round(generated / wall, 1), "chunks_per_s_overall": round(chunks / wall, 1),
        "tokens_per_s_all_streams_live": None if hi <= lo else round(steady / (hi - lo), 1),
        "p50_ttft_s": pct(ttft, 0.5), "p95_ttft_s": pct(ttft, 0.95), "p50_itl_s": pct(itl, 0.5), "p95_itl_s": pct(itl, 0.95),
        "note": "a content chunk is one SSE delta: usually one token (the byte tokenizer may hold back incomplete UTF-8)"}))


if __name__ == "__main__":
    main()
