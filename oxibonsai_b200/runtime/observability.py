"""Profiler with analytic FLOP counters and CUDA-event timers, memory profiler, log setup, request ids, streaming
metrics, generation quality metrics, the hardware auto-tuner and formatting helpers.

Reference: crates/oxibonsai-runtime/src/profiler.rs:30-561 (scoped events, traces, per-prefix aggregation, GFLOP/s,
``flop_counter``), memory.rs:42-244 (RSS sampling), tracing_setup.rs:14-98, request_id.rs:39-, stream_metrics.rs:37-243
(TTFT / time-between-tokens aggregator), quality_metrics.rs, auto_tuner.rs (CPU features + memory budget there; GPU
properties and the 180 GB HBM budget here) and convenience.rs.
"""
from __future__ import annotations

import json
import logging
import math
import os
import re
import threading
import time
from collections import Counter, defaultdict
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any, Callable, Sequence


# ---- FLOP counters -----------------------------------------------------------------------------------------------------------
class flop_counter:
    @staticmethod
    def matmul(m: int, n: int, k: int) -> int:
        return 2 * m * n * k

    @staticmethod
    def linear(tokens: int, in_features: int, out_features: int) -> int:
        return 2 * tokens * in_features * out_features

    @staticmethod
    def attention(tokens: int, context: int, heads: int, head_dim: int) -> int:
        return 4 * tokens * context * heads * head_dim

    @staticmethod
    def rms_norm(tokens: int, hidden: int) -> int:
        return 4 * tokens * hidden

    @staticmethod
    def swiglu_ffn(tokens: int, hidden: int, inter: int) -> int:
        return 6 * tokens * hidden * inter + 4 * tokens * inter

    @staticmethod
    def decoder_step(cfg, context: int, tokens: int = 1) -> int:
        """FLOPs of ``tokens`` new tokens through a Qwen3-shaped decoder at the given context length."""
        q, kv = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
        per_layer = (flop_counter.linear(tokens, cfg.hidden, q + 2 * kv) + flop_counter.attention(tokens, context, cfg.heads, cfg.head_dim)
                     + flop_counter.linear(tokens, q, cfg.hidden) + flop_counter.swiglu_ffn(tokens, cfg.hidden, cfg.inter)
                     + 2 * flop_counter.rms_norm(tokens, cfg.hidden))
        return cfg.layers * per_layer + flop_counter.linear(tokens, cfg.hidden, cfg.vocab)


@dataclass
class ProfileEvent:
    name: str
    start: float
    end: float = 0.0
    flops: int = 0
    metadata: dict = field(default_factory=dict)

    def duration_ms(self) -> float:
        return (self.end - self.start) * 1e3

    def gflops_per_second(self) -> float:
        d = self.end - self.start
        return self.flops / d / 1e9 if d > 0 and self.flops else 0.0


@dataclass
class ProfileTrace:
    name: str
    events: list[ProfileEvent] = field(default_factory=list)

    def top_events(self, n: int = 5) -> list[ProfileEvent]:
        return sorted(self.events, key=lambda e: e.duration_ms(), reverse=True)[:n]

    def duration_for_prefix(self, prefix: str) -> float:
        return sum(e.duration_ms() for e in self.events if e.name.startswith(prefix))

    def avg_duration_for_prefix(self, prefix: str) -> float:
        ev = [e.duration_ms() for e in self.events if e.name.startswith(prefix)]
        return sum(ev) / len(ev) if ev else 0.0

    def aggregate_gflops(self) -> float:
        t = sum(e.end - e.start for e in self.events if e.flops)
        return sum(e.flops for e in self.events) / t / 1e9 if t > 0 else 0.0

    def layer_breakdown(self) -> dict[str, float]:
        out: dict[str, float] = defaultdict(float)
        for e in self.events:
            out[e.name.split(".", 1)[0]] += e.duration_ms()
        return dict(out)

    def summary(self) -> str:
        total = sum(e.duration_ms() for e in self.events)
        lines = [f"trace {self.name}: {len(self.events)} events, {total:.3f} ms, {self.aggregate_gflops():.1f} GFLOP/s"]
        lines += [f"  {e.name:<32} {e.duration_ms():9.3f} ms" for e in self.top_events()]
        return "\n".join(lines)


class Profiler:
    """Scoped wall-clock events grouped into traces.  ``cuda=True`` brackets each event with a device synchronise so the
    time covers the kernels launched inside it (for per-kernel device times use ``cuda_timer``)."""

    def __init__(self, enabled: bool = True, cuda: bool = False):
        self._enabled, self._cuda = enabled, cuda
        self._traces: list[ProfileTrace] = []
        self._current: ProfileTrace | None = None
        self._lock = threading.Lock()

    def is_enabled(self) -> bool:
        return self._enabled

    def begin_trace(self, name: str) -> None:
        self._current = ProfileTrace(name)

    def end_trace(self) -> ProfileTrace | None:
        t, self._current = self._current, None
        if t is not None:
            with self._lock:
                self._traces.append(t)
        return t

    def _sync(self) -> None:
        if self._cuda:
            import torch
            torch.cuda.synchronize()

    @contextmanager
    def scoped(self, name: str, flops: int = 0, **metadata):
        if not self._enabled:
            yield None
            return
        self._sync()
        ev = ProfileEvent(name, time.perf_counter(), flops=flops, metadata=metadata)
        try:
            yield ev
        finally:
            self._sync()
            ev.end = time.perf_counter()
            if self._current is None:
                self._current = ProfileTrace("default")
            self._current.events.append(ev)

    def profile(self, name: str, fn: Callable[[], Any], flops: int = 0) -> Any:
        with self.scoped(name, flops):
            return fn()

    def traces(self) -> list[ProfileTrace]:
        return list(self._traces)

    def last_trace(self) -> ProfileTrace | None:
        return self._traces[-1] if self._traces else self._current

    def aggregate_stats(self) -> dict[str, dict]:
        agg: dict[str, list[float]] = defaultdict(list)
        for t in self._traces + ([self._current] if self._current else []):
            for e in t.events:
                agg[e.name].append(e.duration_ms())
        return {k: {"count": len(v), "total_ms": sum(v), "mean_ms": sum(v) / len(v), "max_ms": max(v)} for k, v in agg.items()}


@contextmanager
def cuda_timer(result: dict, key: str):
    """Times the enclosed launches on the device with CUDA events; ``result[key]`` receives milliseconds."""
    import torch
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    try:
        yield
    finally:
        b.record()
        b.synchronize()
        result[key] = a.elapsed_time(b)


# ---- memory --------------------------------------------------------------------------------------------------------------------
def kernel_histogram(run, iterations: int = 3, warmup: int = 1) -> dict[str, dict]:
    """Per-kernel device-time table of ``run()`` (a callable that launches GPU work, e.g. ``lambda: runner.step(1)``): kernel
    name -> {"count", "total_us", "mean_us", "max_us"} over ``iterations`` calls after ``warmup`` unrecorded ones, from the
    CUDA activity records of ``torch.profiler`` (kernels replayed from a CUDA graph are recorded like any other).  A
    diagnostic view of where a step's device time goes - the counterpart of the reference profiler's per-operation table
    (crates/oxibonsai-runtime/src/profiler.rs); figures taken this way carry the profiler's overhead and are not benchmark
    numbers, and a kernel launched with programmatic dependent launch is on the device while it still waits for its
    predecessor, so the durations of a chained step overlap and add up to more than the step's wall time."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    for _ in range(max(0, warmup)):
        run()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(max(1, iterations)):
            run()
        torch.cuda.synchronize()
    table: dict[str, dict] = {}
    for ev in prof.events():
        if str(getattr(ev, "device_type", "")).endswith("CUDA") and ev.name and not ev.name.startswith(("Memcpy", "Memset")):
            dur = float(getattr(ev, "device_time", 0.0) or getattr(ev, "cuda_time", 0.0) or 0.0)
            row = table.setdefault(ev.name, {"count": 0, "total_us": 0.0, "max_us": 0.0})
            row["count"] += 1
            row["total_us"] += dur
            row["max_us"] = max(row["max_us"], dur)
    for row in table.values():
        row["mean_us"] = row["total_us"] / row["count"]
    return dict(sorted(table.items(), key=lambda kv: -kv[1]["total_us"]))


def get_rss_bytes() -> int:
    try:
        with open("/proc/self/statm") as f:
            return int(f.read().split()[1]) * os.sysconf("SC_PAGE_SIZE")
    except (OSError, ValueError, IndexError):
        return 0


@dataclass
class MemorySnapshot:
    timestamp: float
    rss_bytes: int
    device_allocated: int = 0
    device_reserved: int = 0
    label: str = ""


class MemoryProfiler:
    def __init__(self):
        self._start = get_rss_bytes()
        self._peak = self._start
        self._samples = 0
        self.snapshots: list[MemorySnapshot] = []

    def sample(self) -> int:
        rss = get_rss_bytes()
        self._peak = max(self._peak, rss)
        self._samples += 1
        return rss

    def peak_rss_bytes(self) -> int:
        return self._peak

    def start_rss_bytes(self) -> int:
        return self._start

    def delta_bytes(self) -> int:
        return get_rss_bytes() - self._start

    def sample_count(self) -> int:
        return self._samples

    def current_rss_bytes(self) -> int:
        return get_rss_bytes()

    def take_snapshot(self, label: str = "") -> MemorySnapshot:
        alloc = reserved = 0
        try:
            import torch
            if torch.cuda.is_available():
                alloc, reserved = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
        except Exception:
            pass
        s = MemorySnapshot(time.time(), self.sample(), alloc, reserved, label)
        self.snapshots.append(s)
        return s


# ---- logging -------------------------------------------------------------------------------------------------------------------
class _JsonFormatter(logging.Formatter):
    def format(self, record: logging.LogRecord) -> str:
        d = {"ts": self.formatTime(record), "level": record.levelname.lower(), "target": record.name, "message": record.getMessage()}
        for k in ("request_id", "tokens", "duration_ms"):
            if hasattr(record, k):
                d[k] = getattr(record, k)
        return json.dumps(d)


def init_tracing(log_level: str = "info", json_logs: bool = False, stream=None) -> logging.Logger:
    """Configures the ``oxibonsai`` logger (text or JSON lines).  ``OXIBONSAI_LOG`` overrides the level."""
    level = os.environ.get("OXIBONSAI_LOG", log_level).upper()
    logger = logging.getLogger("oxibonsai")
    logger.setLevel(getattr(logging, level, logging.INFO))
    for h in list(logger.handlers):
        logger.removeHandler(h)
    h = logging.StreamHandler(stream)
    h.setFormatter(_JsonFormatter() if json_logs else logging.Formatter("%(asctime)s %(levelname)-5s %(name)s: %(message)s"))
    logger.addHandler(h)
    logger.propagate = False
    return logger


# ---- request ids ---------------------------------------------------------------------------------------------------------------
class RequestId:
    """128-bit id rendered as 32 hex digits or in UUID form (version 4, variant 1 bits set)."""
    _lock = threading.Lock()
    _state = (time.time_ns() ^ (os.getpid() << 32)) & ((1 << 64) - 1)

    def __init__(self, high: int, low: int):
        self.high, self.low = high & ((1 << 64) - 1), low & ((1 << 64) - 1)

    @classmethod
    def _next64(cls) -> int:
        with cls._lock:   # SplitMix64
            cls._state = (cls._state + 0x9E3779B97F4A7C15) & ((1 << 64) - 1)
            z = cls._state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & ((1 << 64) - 1)
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & ((1 << 64) - 1)
        return z ^ (z >> 31)

    @classmethod
    def new(cls) -> "RequestId":
        hi, lo = cls._next64(), cls._next64()
        hi = (hi & ~(0xF << 12)) | (0x4 << 12)
        lo = (lo & ~(0x3 << 62)) | (0x2 << 62)
        return cls(hi, lo)

    @classmethod
    def from_pair(cls, high: int, low: int) -> "RequestId":
        return cls(high, low)

    def as_hex(self) -> str:
        return f"{self.high:016x}{self.low:016x}"

    def as_uuid(self) -> str:
        h = self.as_hex()
        return f"{h[:8]}-{h[8:12]}-{h[12:16]}-{h[16:20]}-{h[20:]}"

    @classmethod
    def from_hex(cls, s: str) -> "RequestId":
        if len(s) != 32 or not re.fullmatch(r"[0-9a-fA-F]{32}", s):
            raise ValueError("expected 32 hex digits")
        return cls(int(s[:16], 16), int(s[16:], 16))

    @classmethod
    def from_uuid(cls, s: str) -> "RequestId":
        return cls.from_hex(s.replace("-", ""))

    def as_bytes(self) -> bytes:
        return self.high.to_bytes(8, "big") + self.low.to_bytes(8, "big")

    @classmethod
    def from_bytes(cls, b: bytes) -> "RequestId":
        if len(b) != 16:
            raise ValueError("expected 16 bytes")
        return cls(int.from_bytes(b[:8], "big"), int.from_bytes(b[8:], "big"))

    def __eq__(self, other) -> bool:
        return isinstance(other, RequestId) and (self.high, self.low) == (other.high, other.low)

    def __hash__(self) -> int:
        return hash((self.high, self.low))

    def __str__(self) -> str:
        return self.as_uuid()


# ---- streaming metrics -------------------------------------------------------------------------------------------------------------
def _pct(v: Sequence[float], q: float) -> float:
    if not v:
        return 0.0
    s = sorted(v)
    return s[min(len(s) - 1, int(math.ceil(q * len(s))) - 1 if q > 0 else 0)]


class RequestStreamMetrics:
    def __init__(self, prompt_tokens: int = 0):
        self.prompt_tokens, self.t0 = prompt_tokens, time.perf_counter()
        self.t_first: float | None = None
        self.t_last: float | None = None
        self.t_end: float | None = None
        self.gaps: list[float] = []
        self.tokens = 0

    def record_token(self, now: float | None = None) -> None:
        now = time.perf_counter() if now is None else now
        if self.t_first is None:
            self.t_first = now
        else:
            self.gaps.append(now - self.t_last)
        self.t_last = now
        self.tokens += 1

    record_first_token = record_token

    def finish(self, now: float | None = None) -> None:
        self.t_end = time.perf_counter() if now is None else now

    def ttft(self) -> float | None:
        return None if self.t_first is None else self.t_first - self.t0

    def median_tbt(self) -> float:
        return _pct(self.gaps, 0.5)

    def p99_tbt(self) -> float:
        return _pct(self.gaps, 0.99)

    def mean_tbt(self) -> float:
        return sum(self.gaps) / len(self.gaps) if self.gaps else 0.0

    def e2e_latency(self) -> float:
        return (self.t_end or self.t_last or self.t0) - self.t0

    def tokens_per_second(self) -> float:
        d = self.e2e_latency()
        return self.tokens / d if d > 0 else 0.0

    def completion_tokens(self) -> int:
        return self.tokens

    def snapshot(self) -> dict:
        return {"ttft_ms": None if self.ttft() is None else self.ttft() * 1e3, "median_tbt_ms": self.median_tbt() * 1e3,
                "p99_tbt_ms": self.p99_tbt() * 1e3, "tokens": self.tokens, "tokens_per_second": self.tokens_per_second(),
                "e2e_ms": self.e2e_latency() * 1e3}


class StreamingMetricsAggregator:
    def __init__(self):
        self._snaps: list[dict] = []
        self._lock = threading.Lock()

    def record(self, m: RequestStreamMetrics) -> None:
        with self._lock:
            self._snaps.append(m.snapshot())

    def num_requests(self) -> int:
        return len(self._snaps)

    def avg_ttft_ms(self) -> float:
        v = [s["ttft_ms"] for s in self._snaps if s["ttft_ms"] is not None]
        return sum(v) / len(v) if v else 0.0

    def p50_ttft_ms(self) -> float:
        return _pct([s["ttft_ms"] for s in self._snaps if s["ttft_ms"] is not None], 0.5)

    def avg_tokens_per_second(self) -> float:
        v = [s["tokens_per_second"] for s in self._snaps]
        return sum(v) / len(v) if v else 0.0

    def p99_e2e_ms(self) -> float:
        return _pct([s["e2e_ms"] for s in self._snaps], 0.99)

    def p95_tbt_ms(self) -> float:
        return _pct([s["p99_tbt_ms"] for s in self._snaps], 0.95)

    def total_completion_tokens(self) -> int:
        return sum(s["tokens"] for s in self._snaps)

    def report(self) -> dict:
        return {"requests": self.num_requests(), "avg_ttft_ms": self.avg_ttft_ms(), "p50_ttft_ms": self.p50_ttft_ms(),
                "avg_tokens_per_second": self.avg_tokens_per_second(), "p99_e2e_ms": self.p99_e2e_ms(), "completion_tokens": self.total_completion_tokens()}


# ---- generation quality --------------------------------------------------------------------------------------------------------------
def extract_ngrams(tokens: Sequence, n: int) -> list[tuple]:
    return [tuple(tokens[i:i + n]) for i in range(len(tokens) - n + 1)] if n > 0 else []


@dataclass
class RepetitionMetrics:
    unigram_repetition: float
    bigram_repetition: float
    trigram_repetition: float
    longest_repeat: int

    @classmethod
    def compute(cls, tokens: Sequence) -> "RepetitionMetrics":
        def rep(n):
            g = extract_ngrams(tokens, n)
            return 1.0 - len(set(g)) / len(g) if g else 0.0
        longest, run = 0, 1
        for a, b in zip(tokens, tokens[1:]):
            run = run + 1 if a == b else 1
            longest = max(longest, run)
        return cls(rep(1), rep(2), rep(3), longest if len(tokens) > 1 else len(tokens))

    def is_degenerate(self, threshold: float = 0.5) -> bool:
        return self.trigram_repetition > threshold or self.longest_repeat >= 8

    def summary(self) -> str:
        return f"rep1={self.unigram_repetition:.2f} rep2={self.bigram_repetition:.2f} rep3={self.trigram_repetition:.2f} run={self.longest_repeat}"


@dataclass
class DiversityMetrics:
    distinct_1: float
    distinct_2: float
    entropy: float

    @classmethod
    def compute(cls, tokens: Sequence) -> "DiversityMetrics":
        def distinct(n):
            g = extract_ngrams(tokens, n)
            return len(set(g)) / len(g) if g else 0.0
        return cls(distinct(1), distinct(2), token_entropy(tokens))

    def overall_diversity(self) -> float:
        return (self.distinct_1 + self.distinct_2) / 2

    def summary(self) -> str:
        return f"distinct-1={self.distinct_1:.2f} distinct-2={self.distinct_2:.2f} entropy={self.entropy:.2f}"


def token_entropy(tokens: Sequence) -> float:
    c = Counter(tokens)
    n = sum(c.values())
    return -sum(v / n * math.log(v / n) for v in c.values()) if n else 0.0


def perplexity_from_logprobs(log_probs: Sequence[float]) -> float:
    return math.exp(-sum(log_probs) / len(log_probs)) if log_probs else 1.0


def bleu(candidate: Sequence, references: Sequence[Sequence], max_n: int = 4) -> float:
    """Sentence BLEU with brevity penalty and +1 smoothing above unigrams."""
    if not candidate:
        return 0.0
    logs = 0.0
    for n in range(1, max_n + 1):
        cg = Counter(extract_ngrams(candidate, n))
        best: Counter = Counter()
        for r in references:
            for g, c in Counter(extract_ngrams(r, n)).items():
                best[g] = max(best[g], c)
        match = sum(min(c, best[g]) for g, c in cg.items())
        total = sum(cg.values())
        if n == 1:
            if match == 0:
                return 0.0
            p = match / total
        else:
            p = (match + 1) / (total + 1)
        logs += math.log(p) / max_n
    ref_len = min((abs(len(r) - len(candidate)), len(r)) for r in references)[1]
    bp = 1.0 if len(candidate) >= ref_len else math.exp(1 - ref_len / len(candidate))
    return bp * math.exp(logs)


def self_bleu(generations: Sequence[Sequence]) -> float:
    if len(generations) < 2:
        return 0.0
    return sum(bleu(g, [h for j, h in enumerate(generations) if j != i]) for i, g in enumerate(generations)) / len(generations)


@dataclass
class GenerationQualityReport:
    repetition: RepetitionMetrics
    diversity: DiversityMetrics
    length: int

    @classmethod
    def compute(cls, tokens: Sequence) -> "GenerationQualityReport":
        return cls(RepetitionMetrics.compute(tokens), DiversityMetrics.compute(tokens), len(tokens))

    def quality_score(self) -> float:
        return max(0.0, min(1.0, self.diversity.overall_diversity() * (1.0 - self.repetition.trigram_repetition)))

    def summary(self) -> str:
        return f"len={self.length} {self.repetition.summary()} {self.diversity.summary()} score={self.quality_score():.2f}"


class BatchQualityAnalyzer:
    def __init__(self):
        self.reports: list[GenerationQualityReport] = []
        self.generations: list[Sequence] = []

    def add_generation(self, tokens: Sequence) -> None:
        self.generations.append(list(tokens))
        self.reports.append(GenerationQualityReport.compute(tokens))

    def mean_quality_score(self) -> float:
        return sum(r.quality_score() for r in self.reports) / len(self.reports) if self.reports else 0.0

    def mean_diversity(self) -> float:
        return sum(r.diversity.overall_diversity() for r in self.reports) / len(self.reports) if self.reports else 0.0

    def degenerate_fraction(self) -> float:
        return sum(r.repetition.is_degenerate() for r in self.reports) / len(self.reports) if self.reports else 0.0

    def self_bleu_score(self) -> float:
        return self_bleu(self.generations)

    def num_reports(self) -> int:
        return len(self.reports)

    def report(self) -> dict:
        return {"n": self.num_reports(), "quality": self.mean_quality_score(), "diversity": self.mean_diversity(),
                "degenerate": self.degenerate_fraction(), "self_bleu": self.self_bleu_score()}


# ---- auto tuner ---------------------------------------------------------------------------------------------------------------------
KV_BYTES = {"f32": 4.0, "f16": 2.0, "q8": 1.0 + 4.0 / 128, "q4": 0.5 + 4.0 / 128}


@dataclass
class MemoryBudget:
    weight_bytes: int
    kv_bytes_per_token: float
    activation_bytes: int
    total_bytes: int

    @classmethod
    def estimate(cls, cfg, kv: str = "f16", tp: int = 1, total_bytes: int = 180 * 10 ** 9, bits_per_weight: float = 2.125, max_batch: int = 64,
                 prefill_chunk: int = 1024) -> "MemoryBudget":
        q, kvd = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
        per_layer = cfg.hidden * (q + 2 * kvd) + q * cfg.hidden + 3 * cfg.hidden * cfg.inter
        weights = int(cfg.layers * per_layer * bits_per_weight / 8 / tp + 2 * cfg.vocab * cfg.hidden * 2 / tp)
        kv_tok = cfg.layers * 2 * kvd * KV_BYTES[kv] / tp
        act = int(prefill_chunk * (cfg.hidden * 10 + cfg.inter * 2 / tp + (q + 2 * kvd) * 4 / tp) + max_batch * cfg.vocab * 4)
        return cls(weights, kv_tok, act, total_bytes)

    def max_context_length(self, batch: int = 1, reserve: float = 0.08) -> int:
        free = self.total_bytes * (1 - reserve) - self.weight_bytes - self.activation_bytes
        return max(0, int(free / (self.kv_bytes_per_token * batch)))

    def fits_context(self, context: int, batch: int = 1) -> bool:
        return self.max_context_length(batch) >= context

    def summary(self) -> str:
        return (f"weights {format_bytes(self.weight_bytes)}, KV {self.kv_bytes_per_token / 1024:.1f} KiB/token, activations "
                f"{format_bytes(self.activation_bytes)}, max context (batch 1) {self.max_context_length():,} tokens")


@dataclass
class TuningRecommendation:
    kv_cache: str
    max_batch: int
    prefill_chunk: int
    attention_splits: int
    tensor_parallel: int
    notes: list[str] = field(default_factory=list)

    def summary(self) -> str:
        return (f"kv={self.kv_cache} max_batch={self.max_batch} prefill_chunk={self.prefill_chunk} attention_splits={self.attention_splits} "
                f"tp={self.tensor_parallel}" + ("; " + "; ".join(self.notes) if self.notes else ""))


class AutoTuner:
    """Picks serving parameters from the device properties and the model shape."""

    def __init__(self, sm_count: int = 148, memory_bytes: int = 180 * 10 ** 9, n_gpus: int = 1):
        self.sm_count, self.memory_bytes, self.n_gpus = sm_count, memory_bytes, n_gpus

    @classmethod
    def detect(cls) -> "AutoTuner":
        try:
            import torch
            if torch.cuda.is_available():
                p = torch.cuda.get_device_properties(0)
                return cls(p.multi_processor_count, p.total_memory, torch.cuda.device_count())
        except Exception:
            pass
        return cls()

    def with_memory_mb(self, mb: int) -> "AutoTuner":
        self.memory_bytes = mb << 20
        return self

    def recommend(self, cfg, target_context: int = 4096, target_batch: int = 64) -> TuningRecommendation:
        notes = []
        for kv in ("f16", "q8", "q4"):
            b = MemoryBudget.estimate(cfg, kv, 1, self.memory_bytes, max_batch=target_batch)
            if b.fits_context(target_context, target_batch):
                break
            notes.append(f"{kv} KV does not hold {target_batch} x {target_context} tokens")
        tp = 1
        while tp < self.n_gpus and cfg.kv_heads % (tp * 2) == 0 and not MemoryBudget.estimate(cfg, kv, tp, self.memory_bytes, max_batch=target_batch).fits_context(target_context, target_batch):
            tp *= 2
        splits = max(1, min(64, 2 * self.sm_count // max(1, cfg.kv_heads // tp)))
        return TuningRecommendation(kv, target_batch, 1024, splits, tp, notes)

    def benchmark_kernel(self, name: str, fn: Callable[[], None], iters: int = 20) -> dict:
        fn()
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        dt = (time.perf_counter() - t0) / iters
        return {"kernel": name, "mean_us": dt * 1e6, "iters": iters}

    def report(self, cfg) -> str:
        return f"{self.sm_count} SMs, {format_bytes(self.memory_bytes)} x {self.n_gpus} GPU(s): {self.recommend(cfg).summary()}"


# ---- formatting helpers ------------------------------------------------------------------------------------------------------------------
def format_token_count(n: int) -> str:
    return f"{n / 1e6:.1f}M" if n >= 1_000_000 else (f"{n / 1e3:.1f}K" if n >= 1000 else str(n))


def format_bytes(n: float) -> str:
    for unit in ("B", "KiB", "MiB", "GiB", "TiB"):
        if abs(n) < 1024 or unit == "TiB":
            return f"{n:.1f} {unit}" if unit != "B" else f"{int(n)} B"
        n /= 1024
    return f"{n:.1f} TiB"


def format_duration(seconds: float) -> str:
    if seconds < 1e-3:
        return f"{seconds * 1e6:.0f} us"
    if seconds < 1:
        return f"{seconds * 1e3:.1f} ms"
    if seconds < 60:
        return f"{seconds:.2f} s"
    m, s = divmod(int(seconds), 60)
    return f"{m}m{s:02d}s" if m < 60 else f"{m // 60}h{m % 60:02d}m"


def format_tokens_per_second(tps: float) -> str:
    return f"{tps:,.1f} tok/s"


def validate_model_file(path: str) -> dict:
    """Cheap sanity check of a GGUF file: exists, magic, version, tensor count."""
    import struct
    info = {"path": path, "exists": os.path.exists(path), "valid": False}
    if not info["exists"]:
        return info
    info["size_bytes"] = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(24)
    if len(head) >= 24 and head[:4] == b"GGUF":
        ver, nt, nkv = struct.unpack("<IQQ", head[4:24])
        info.update(valid=ver in (2, 3), version=ver, tensors=nt, metadata_entries=nkv)
    return info


def estimate_memory_requirements(cfg, context: int = 4096, batch: int = 1, kv: str = "f16") -> dict:
    b = MemoryBudget.estimate(cfg, kv)
    kvb = int(b.kv_bytes_per_token * context * batch)
    return {"weights": b.weight_bytes, "kv_cache": kvb, "activations": b.activation_bytes, "total": b.weight_bytes + kvb + b.activation_bytes}
