#!/usr/bin/env python
"""Headline benchmark: decode tokens/s of a Ternary-Bonsai-8B-shaped checkpoint, batch 1 and 64 concurrent streams.

Workload (the reference's headline metric on the shape its README quotes for Ternary-Bonsai-8B): a seeded random-init
TQ2_0_g128 GGUF with 36 layers, hidden 4096, 32 Q / 8 KV heads, head_dim 128, intermediate 12288, vocab 151936 and an
f16 LM head; a random-token prompt is prefilled and then decoded greedily one token per step.  A "step" is one decode
token: embed, 36 layers over the live KV context, LM head, sampler.

With N > 1 GPUs the headline ``value`` is the tensor-parallel engine at TP = N decoding ONE stream (strong scaling: the
total work is fixed, ``global_batch`` 1): column-parallel QKV / gate-up, row-parallel attention-output / down projections
whose all-reduce + residual add is the epilogue of the GEMV kernel itself (8-byte {value, tag} stores into the peers'
memory over NVLink), vocab-parallel LM head.  Reported beside it, under their own keys:
  ``streams``           - 64 concurrent streams on the same engine (TP = N at N > 1);
  ``nccl_tp_baseline``  - the same TP engine with ``torch.distributed.all_reduce`` (NCCL) in place of the fused epilogues;
  ``replicas``          - N independent single-GPU engines, one stream (and 64 / N streams) each: the arrangement the
                          single-GPU reference would be deployed in on a multi-GPU box;
  ``exact_f32``         - the exact-f32 mode (f32 activations end to end, the mode that passes the token gate) and the
                          largest logit difference between it and the timed fast mode on the same 8B-shaped prompt;
  ``gate``              - the correctness gate: the 1.7B-shaped checkpoint of the reference's CPU-path configuration
                          (28 layers, hidden 2048, vocab 151936, seed 42), 16-token prompt, 32 greedy tokens in exact mode
                          at TP = N, compared with the stream the C++ restatement of the reference's CPU scalar path
                          produced (``benchmarks/golden_config1.json``, with the top-1/top-2 logit gap of every step).

Timing: W untimed warm-up steps, then K steps between CUDA events on the launching stream, bracketed by a barrier +
synchronize; the max over ranks is reported.  Every step streams ~3.1 GB / N of packed weights + LM head per GPU, far more
than the 126 MB L2, so no explicit L2 flush is needed.  The ``e2e`` value is measured through the public API
(``EngineBuilder().model_path(..).build().generate_stream``): each step uploads (token, position) from pinned host
memory, replays the step and reads the sampled token and the step's status word back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

PUBLISHED_BASELINE_TOK_S = 21.9  # Ternary-Bonsai-1.7B, native CUDA, RTX 3060 (reference README.md:287)
WATCHDOG_S = 900                 # a rank that never comes back from a collective may not hold the result line back longer
HERE = os.path.dirname(os.path.abspath(__file__))


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="8b", choices=["8b", "4b", "1.7b", "tiny"])
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--kv", default="f16")
    ap.add_argument("--streams", type=int, default=64, help="concurrent sequences of the aggregate-throughput measurement (0 = skip)")
    ap.add_argument("--stream-prompt-len", type=int, default=1024)
    ap.add_argument("--no-replicas", action="store_true", help="skip the independent-replica measurement at N > 1")
    ap.add_argument("--no-gate", action="store_true", help="skip the correctness gate")
    ap.add_argument("--no-extras", action="store_true", help="skip the exact-f32 and NCCL-baseline measurements")
    ap.add_argument("--model-dir", default=os.environ.get("BONSAI_BENCH_DIR", "/tmp/oxibonsai_b200_bench"))
    return ap.parse_args()


SHAPES = {
    "8b": dict(hidden=4096, inter=12288, layers=36, heads=32, kv_heads=8, head_dim=128, vocab=151936, name="Ternary-Bonsai-8B-shaped", tied=False),
    "4b": dict(hidden=2560, inter=9728, layers=36, heads=32, kv_heads=8, head_dim=128, vocab=151936, name="Ternary-Bonsai-4B-shaped", tied=True),
    "1.7b": dict(hidden=2048, inter=6144, layers=28, heads=16, kv_heads=8, head_dim=128, vocab=151936, name="Ternary-Bonsai-1.7B-shaped", tied=True),
    "tiny": dict(hidden=512, inter=1024, layers=2, heads=4, kv_heads=2, head_dim=128, vocab=4096, name="tiny", tied=True),
}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows: list[list[str]] = []
        self._stop = threading.Event()
        self._t: threading.Thread | None = None

    def _run(self):
        # one long-running nvidia-smi in loop mode (a row every 100 ms); reading the settings changes nothing on the GPU
        try:
            cmd = ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"]
            if self.gpu >= 0:
                cmd += ["-i", str(self.gpu)]       # gpu < 0: every GPU of the node (rows carry the index)
            self._proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self._proc.stdout:
                if line.strip():
                    self.rows.append([c.strip() for c in line.split(",")])
                if self._stop.is_set():
                    break
        except Exception:
            pass

    def start(self):
        self._proc = None
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        t_end = time.time() + 10.0   # the first row arrives before the timed region starts (nvidia-smi can take seconds on 8 GPUs)
        while not self.rows and time.time() < t_end:
            time.sleep(0.05)

    def stop(self) -> dict:
        self._stop.set()
        if getattr(self, "_proc", None) is not None:
            self._proc.terminate()      # this exact child process
        if self._t:
            self._t.join(timeout=6)
        sm = sorted(float(r[1]) for r in self.rows if len(r) > 2 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in self.rows if len(r) > 2 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for i, n in enumerate(names):
                if len(r) > 5 + i and r[5 + i].lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(self.rows)}


def reference_arm(args) -> None:
    """The reference is a Rust workspace; this image has no cargo/rustc and pip cannot install it."""
    print(json.dumps({"impl": "reference", "unavailable": "reference is a Rust/Cargo workspace: no setup.py/pyproject.toml for pip and no cargo/rustc "
                      "in the image, so baseline/_ref cannot be built offline"}))


def measure(eng, args, cfg, prompt, n_streams: int, barrier, dev, gen, e2e: bool, sched_e2e: bool, clocks_gpu: int | None) -> dict:
    """Batch-1 device-timed decode, end-to-end decode through the public API, and the aggregate of ``n_streams``
    sequences decoded together - all on ``eng``.  Returns raw times; the caller reduces over ranks."""
    import torch
    from oxibonsai_b200.ops import cuda_ops as K
    r = eng.runner
    prompt_len = len(prompt)
    total_steps = args.warmup + args.steps
    out = {"e2e_s": float("nan"), "e2e_steps": 0, "st_ms": float("nan"), "st_e2e_s": float("nan"), "st_e2e_tokens": 0, "clocks": None,
           "ttfts": [], "itl_p95": None}
    eng._bind_slot(0, prompt_len + 2 * total_steps + 16)
    eng._set_sampling(0, eng.sampling)
    barrier()
    t0 = time.time()
    eng.prefill(prompt, 0)
    K.sample(r.logits[:1], out=r.tokens[:1])
    r.positions[:1].fill_(prompt_len)
    torch.cuda.synchronize(dev)
    out["ttft"] = time.time() - t0
    clocks = ClockSampler(clocks_gpu) if clocks_gpu is not None else None
    if clocks:
        clocks.start()            # before the warm-up, so that waiting for its first row does not idle the GPU before the timed steps
    for _ in range(args.warmup):
        r.step(1, sample=True)
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        r.step(1, sample=True)
    ev1.record()
    barrier()
    out["dev_ms"] = ev0.elapsed_time(ev1)
    if clocks:
        out["clocks"] = clocks.stop()
    r.check_status()
    eng._release_slot(0)
    out["launches"] = r.kernel_launches(1, sample=True) * args.steps

    if e2e:
        it = eng.generate_stream(prompt, max_tokens=args.warmup + args.steps, stop_at_eos=False)
        times = []
        barrier()
        for _tok in it:
            times.append(time.perf_counter())
        barrier()
        # token i is available at times[i]; steps after the warm-up tokens are the timed ones
        if len(times) > args.warmup:
            out["e2e_s"], out["e2e_steps"] = times[-1] - times[args.warmup - 1], len(times) - args.warmup

    S = n_streams
    sp_len = min(args.stream_prompt_len, prompt_len)
    if S >= 2:
        for s_ in range(S):
            eng._bind_slot(s_, sp_len + 2 * total_steps + 16)
            eng._set_sampling(s_, eng.sampling)
            eng.prefill(torch.randint(0, cfg.vocab, (sp_len,), generator=gen).tolist(), s_)
        K.sample(r.logits[:S], out=r.tokens[:S])
        r.positions[:S].fill_(sp_len)
        for _ in range(args.warmup):
            r.step(S, sample=True)
        barrier()
        ev0.record()
        for _ in range(args.steps):
            r.step(S, sample=True)
        ev1.record()
        barrier()
        out["st_ms"] = ev0.elapsed_time(ev1)
        r.check_status()
        for s_ in range(S):
            eng._release_slot(s_)
        if sched_e2e:
            # end to end through the continuous-batching scheduler: per step the positions go up from pinned memory
            # and the S sampled tokens come back to the host
            from oxibonsai_b200.runtime.scheduler import BatchScheduler
            sched = BatchScheduler(eng, eos_token=-1)
            # Prompts are admitted one chunk per decode step, so the first streams are many tokens ahead when the last one
            # starts: every stream gets enough tokens to be still running then, and the timed window is the stretch in
            # which all S streams are live (from the last stream's first token to the first stream's last one).
            n_out = args.warmup + args.steps + 3 * S
            reqs = [sched.submit(torch.randint(0, cfg.vocab, (sp_len,), generator=gen).tolist(), eng.sampling, n_out) for _ in range(S)]
            sched.start()
            for q_ in reqs:
                q_.wait(timeout=1800)
            sched.stop()
            t_start = max(q_.token_times[0] for q_ in reqs)
            t_end = min(q_.token_times[-1] for q_ in reqs)
            out["st_e2e_tokens"] = sum(sum(1 for x in q_.token_times if t_start < x <= t_end) for q_ in reqs)
            out["st_e2e_s"] = t_end - t_start
            out["ttfts"] = sorted(q_.t_first_token - q_.t_submit for q_ in reqs if q_.t_first_token is not None)
            out["itl_p95"] = sorted(b_ - a_ for q_ in reqs for a_, b_ in zip(q_.token_times, q_.token_times[1:]))[int(0.95 * sum(len(q_.token_times) - 1 for q_ in reqs))]
    return out


def run_gate(args, world: int, rank: int, local_rank: int) -> dict:
    """Correctness gate on the reference's CPU-path configuration: the 1.7B-shaped TQ2_0_g128 checkpoint (seed 42, tied f16
    embedding), a 16-token random prompt, 32 greedy tokens in exact mode at TP = world, against the committed stream of the
    C++ restatement of the reference's CPU scalar path."""
    import torch
    import torch.distributed as dist
    from oxibonsai_b200.core import Qwen3Config, write_synthetic_gguf
    from oxibonsai_b200.runtime import EngineBuilder
    with open(os.path.join(HERE, "benchmarks", "golden_config1.json")) as f:
        gold = json.load(f)
    shape = dict(SHAPES["1.7b"])
    tied = shape.pop("tied")
    cfg = Qwen3Config(context=65536, **shape)
    path = os.path.join(args.model_dir, "1.7b_tq2_seed42.gguf")
    if rank == 0 and not os.path.exists(path):
        write_synthetic_gguf(path + ".tmp", cfg, tied=tied, seed=42)
        os.replace(path + ".tmp", path)
    if world > 1:
        dist.barrier()
    prompt = torch.randint(0, cfg.vocab, (16,), generator=torch.Generator().manual_seed(42)).tolist()
    assert prompt == gold["prompt"], "the gate's prompt generator no longer reproduces the committed prompt"
    b = EngineBuilder().model_path(path).preset("greedy").max_seq_len(64).kv_cache("f32").device(f"cuda:{local_rank}")
    if world > 1:
        b = b.tensor_parallel(rank, world)
    eng = b.build()
    got = eng.generate(prompt, 32, stop_at_eos=False)
    want = gold["tokens"]
    first_bad = next((i for i, (a_, b_) in enumerate(zip(got, want)) if a_ != b_), None)
    res = {"config": "Ternary-Bonsai-1.7B-shaped TQ2_0_g128, seed 42, 16-token prompt, 32 greedy tokens, exact-f32 mode", "tp": world,
           "match": got == want, "distinct_tokens": len(set(want)), "min_top2_gap": round(min(gold["top2_gaps"][: len(want)]), 6),
           "first_mismatch": first_bad, "tokens_head": got[:8]}
    del eng
    torch.cuda.empty_cache()
    return res


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from oxibonsai_b200.core import Qwen3Config, write_synthetic_gguf
    from oxibonsai_b200.runtime import EngineBuilder

    shape = dict(SHAPES[args.model])
    tied = shape.pop("tied")
    prompt_len = args.prompt_len if args.prompt_len is not None else (4096 if args.model != "tiny" else 32)
    max_seq = prompt_len + 2 * (args.warmup + args.steps) + 16
    cfg = Qwen3Config(context=65536, **shape)
    os.makedirs(args.model_dir, exist_ok=True)
    path = os.path.join(args.model_dir, f"{args.model}_tq2_seed42.gguf")
    if rank == 0 and not os.path.exists(path):
        t0 = time.time()
        write_synthetic_gguf(path + ".tmp", cfg, tied=tied, seed=42)
        os.replace(path + ".tmp", path)
        print(f"[bench] wrote {path} in {time.time() - t0:.1f}s", file=sys.stderr)
    if world > 1:
        dist.barrier()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def reduce_max(vals):
        t = torch.tensor(vals, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    S = args.streams if args.streams >= 2 else 0
    prompt = torch.randint(0, cfg.vocab, (prompt_len,), generator=torch.Generator().manual_seed(42)).tolist()
    extra: dict = {"gate": None, "exact_f32": None, "nccl_tp_baseline": None, "replicas": None}
    head: dict = {}
    emitted: list = []

    def emit():
        """Rank 0 prints the result line (once)."""
        if rank != 0 or emitted or not head:
            return
        emitted.append(True)
        print(json.dumps({**head, **extra, "impl": "ours"}))
        sys.stdout.flush()

    if world > 1:
        def bail():
            if head:
                extra["watchdog"] = f"a later measurement gave no answer within {WATCHDOG_S} s"
                emit()
            os._exit(0 if head else 3)
        dog = threading.Timer(WATCHDOG_S, bail)
        dog.daemon = True
        dog.start()

    # ---------------- correctness gate (cheap, before anything is timed) ----------------
    if not args.no_gate:
        try:
            extra["gate"] = run_gate(args, world, rank, local_rank)
        except Exception as e:   # noqa: BLE001 - reported in the result line
            extra["gate"] = {"tp": world, "match": False, "error": f"{type(e).__name__}: {e}"[:300]}
        print(f"[bench] rank {rank}: gate {extra['gate']}", file=sys.stderr)

    # ---------------- headline: one engine over all N GPUs (tensor parallel at N > 1) ----------------
    t0 = time.time()
    b = (EngineBuilder().model_path(path).preset("greedy").max_seq_len(max_seq).max_batch(max(1, S)).kv_cache(args.kv)
         .device(f"cuda:{local_rank}"))
    if world > 1:
        b = b.tensor_parallel(rank, world)
    eng = b.build()
    bytes_step = eng.weights.packed_bytes
    print(f"[bench] rank {rank}: engine (tp{world}) ready in {time.time() - t0:.1f}s; packed bytes/step/GPU {bytes_step / 1e9:.3f} GB; "
          f"switch multicast {getattr(getattr(eng.runner, 'tp', None), 'multicast', None)}", file=sys.stderr)
    # rank 0 samples the clocks of every GPU of the job (one nvidia-smi for the node), the other ranks none
    m = measure(eng, args, cfg, prompt, S, barrier, dev, torch.Generator().manual_seed(7), e2e=True, sched_e2e=(world == 1),
                clocks_gpu=(0 if world == 1 else -1) if rank == 0 else None)
    dev_ms, e2e_s, st_ms, st_e2e_s, ttft = reduce_max([m["dev_ms"], m["e2e_s"], m["st_ms"], m["st_e2e_s"], m["ttft"]])
    ms_per_step = dev_ms / args.steps
    value = 1000.0 / ms_per_step                               # one stream, one token per step
    e2e_value = m["e2e_steps"] / e2e_s if e2e_s == e2e_s and e2e_s > 0 else None
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(HERE, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm = peaks.get("hbm_gbs", 6650.0)
    sp_len = min(args.stream_prompt_len, prompt_len)
    ttfts = m["ttfts"]
    head.update({
        "metric": "decode tok/s (batch 1), Ternary-Bonsai-8B-shaped TQ2_0_g128" if args.model == "8b" else f"decode tok/s (batch 1), {cfg.name}",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": round(value / PUBLISHED_BASELINE_TOK_S, 2),
        "dtype": "int8x2 activations per 128-input group (16 bits of the group maximum), exact integer products and sums (mma.sync u8 x s8 -> s32), f32 scales and residual stream; 2-bit weights as stored; f16 KV and f16 tensor-core attention",
        "data": "synthetic (seeded random-init GGUF, random prompt tokens)",
        "config": {"model": cfg.name, "global_batch": 1, "seq_len": prompt_len, "decode_tokens": args.steps, "kv_cache": args.kv,
                   "parallelism": "single GPU" if world == 1 else f"tp{world} (one stream over all GPUs; fused GEMV->all-reduce epilogues over NVLink peer memory)",
                   "l2": "inputs larger than L2 (each step streams the packed weights + LM head)", "weights_bytes_per_step_per_gpu": bytes_step,
                   "nvlink_switch_multicast": bool(world > 1 and getattr(eng.runner.tp, "multicast", False))},
        "clocks": m["clocks"],
        "e2e": {"value": None if e2e_value is None else round(e2e_value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 8 * world,
                "d2h_bytes_per_step": 8 * world, "ttft_s": round(ttft, 3)},
        "p50_ttft_s": round(ttft, 3),
        "gpu_launches": m["launches"] * world,
        "streams": None if S < 2 else {
            "metric": f"aggregate decode tok/s, {S} concurrent streams" + (f" at tp{world}" if world > 1 else ""),
            "n_streams": S, "prompt_len": sp_len, "value": round(S * args.steps / (st_ms * 1e-3), 1),
            "ms_per_step": round(st_ms / args.steps, 4), "unit": "tokens/s",
            "e2e_value": None if not m["st_e2e_tokens"] else round(m["st_e2e_tokens"] / st_e2e_s, 1),
            "e2e_h2d_bytes_per_step": 4 * S, "e2e_d2h_bytes_per_step": 4 * S + 4,
            "p50_ttft_s": None if not ttfts else round(ttfts[len(ttfts) // 2], 3),
            "p95_itl_s": None if m.get("itl_p95") is None else round(m["itl_p95"], 4),
            "note": "scheduler run: all streams are submitted at once and admitted one 512-token prompt chunk per decode step, so TTFT "
                    "includes queueing behind the other prompts; e2e_value counts the stretch in which all streams are live"},
        "hbm_roofline_frac_of_measured" if peaks else "hbm_roofline_frac_of_fallback": round(bytes_step / (ms_per_step * 1e-3) / (hbm * 1e9), 4),
    })

    # ---------------- the same TP engine with NCCL all-reduce in place of the fused epilogues ----------------
    if world > 1 and not args.no_extras:
        try:
            from oxibonsai_b200.ops import cuda_ops as K
            from oxibonsai_b200.parallel.nccl_baseline import NcclTpDecoder
            r = eng.runner
            eng._bind_slot(0, prompt_len + 2 * (args.warmup + args.steps) + 16)
            eng._set_sampling(0, eng.sampling)
            eng.prefill(prompt, 0)
            K.sample(r.logits[:1], out=r.tokens[:1])
            r.positions[:1].fill_(prompt_len)
            nd = NcclTpDecoder(eng)
            for _ in range(args.warmup):
                nd.step()
            barrier()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for _ in range(args.steps):
                nd.step()
            ev1.record()
            barrier()
            (n_ms,) = reduce_max([ev0.elapsed_time(ev1)])
            eng._release_slot(0)
            extra["nccl_tp_baseline"] = {"parallelism": f"tp{world}", "what": "same engine and kernels; row-parallel partial sums reduced by "
                                         "torch.distributed.all_reduce (NCCL) + residual add, logits by all_gather_into_tensor; one CUDA graph per step",
                                         "tokens_per_s": round(1000.0 * args.steps / n_ms, 2), "ms_per_token": round(n_ms / args.steps, 4),
                                         "fused_speedup": round(n_ms / dev_ms, 3)}
            del nd
        except Exception as e:   # noqa: BLE001
            extra["nccl_tp_baseline"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    del eng
    torch.cuda.empty_cache()

    # ---------------- exact-f32 mode on the same shape, and how far the fast mode's logits are from it ----------------
    if not args.no_extras:
        try:
            from oxibonsai_b200.ops import cuda_ops as K
            short = prompt[:128]
            x_steps = min(args.steps, 32)

            def build(kv, exact):
                bb = (EngineBuilder().model_path(path).preset("greedy").max_seq_len(128 + 2 * x_steps + 24).max_batch(1).kv_cache(kv)
                      .device(f"cuda:{local_rank}").exact(exact))
                return (bb.tensor_parallel(rank, world) if world > 1 else bb).build()

            def last_logits(e):
                e._bind_slot(0, 128 + 2 * x_steps + 16)
                e._set_sampling(0, e.sampling)
                rr = e.runner
                toks = torch.tensor(short, dtype=torch.int32, device=dev)
                pos = torch.arange(128, dtype=torch.int32, device=dev)
                for i in range(128):          # token by token through the decode path in both modes: same code path, same context
                    rr.tokens[:1].copy_(toks[i: i + 1])
                    rr.positions[:1].copy_(pos[i: i + 1])
                    rr.step_eager(1, sample=False, lm_head=(i == 127))
                torch.cuda.synchronize(dev)
                return rr.logits[0, : cfg.vocab].clone()

            ex = build("f32", True)
            lg_exact = last_logits(ex)
            rr = ex.runner
            K.sample(rr.logits[:1], out=rr.tokens[:1])
            rr.positions[:1].fill_(128)
            for _ in range(3):
                rr.step(1, sample=True)
            barrier()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            for _ in range(x_steps):
                rr.step(1, sample=True)
            ev1.record()
            barrier()
            (x_ms,) = reduce_max([ev0.elapsed_time(ev1)])
            del ex, rr
            torch.cuda.empty_cache()
            fa = build("f16", False)
            lg_fast = last_logits(fa)
            del fa
            torch.cuda.empty_cache()
            diff = (lg_fast - lg_exact).abs()
            top2 = torch.topk(lg_exact, 2).values
            extra["exact_f32"] = {"tokens_per_s": round(1000.0 * x_steps / x_ms, 2), "ms_per_token": round(x_ms / x_steps, 4), "context": 128,
                                  "steps": x_steps, "kv_cache": "f32",
                                  "fast_vs_exact_logits": {"prompt_tokens": 128, "max_abs_diff": round(float(diff.max()), 5),
                                                           "mean_abs_diff": round(float(diff.mean()), 6), "logit_std": round(float(lg_exact.std()), 4),
                                                           "top1_top2_gap": round(float(top2[0] - top2[1]), 5),
                                                           "same_argmax": bool(int(lg_fast.argmax()) == int(lg_exact.argmax()))}}
        except Exception as e:   # noqa: BLE001
            extra["exact_f32"] = {"error": f"{type(e).__name__}: {e}"[:300]}

    # ---------------- N independent replicas (how the single-GPU reference would be deployed on this box) ----------------
    if world > 1 and not args.no_replicas:
        try:
            per_replica = -(-S // world) if S >= 2 else 0
            reng = (EngineBuilder().model_path(path).preset("greedy").max_seq_len(max_seq).max_batch(max(1, per_replica)).kv_cache(args.kv)
                    .device(f"cuda:{local_rank}").build())
            rm = measure(reng, args, cfg, prompt, per_replica, barrier, dev, torch.Generator().manual_seed(42 + rank), e2e=False, sched_e2e=False,
                         clocks_gpu=None)
            r_dev, r_st = reduce_max([rm["dev_ms"], rm["st_ms"]])
            extra["replicas"] = {"parallelism": f"dp{world} (one engine per GPU, no communication)", "batch1_tokens_per_s_aggregate": round(world * 1000.0 * args.steps / r_dev, 2),
                                 "batch1_ms_per_token_per_replica": round(r_dev / args.steps, 4),
                                 "streams_total": per_replica * world,
                                 "streams_tokens_per_s": None if per_replica < 2 else round(per_replica * world * args.steps / (r_st * 1e-3), 1)}
            del reng
        except Exception as e:   # noqa: BLE001
            extra["replicas"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    emit()
    if world > 1:
        dog.cancel()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
