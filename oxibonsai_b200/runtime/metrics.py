"""Metrics: counters, gauges, histograms, Prometheus text exposition and per-request rate trackers.

Reference: hand-rolled Counter / Gauge / Histogram and the 16 ``oxibonsai_*`` series (crates/oxibonsai-runtime/src/metrics.rs:28-436),
``RequestRateTracker`` (time-between-tokens ring of 128, EWMA tokens/s with alpha 0.2, queue wait = admission to first token)
and ``RequestRateAggregator`` with a window of 256 (request_metrics.rs:74-240), ``StreamingMetricsAggregator``
(stream_metrics.rs:37-243).  Series names are kept so dashboards built for the reference keep working.
"""
from __future__ import annotations

import bisect
import threading
import time
from collections import deque


class Counter:
    def __init__(self, name: str, help_: str):
        self.name, self.help = name, help_
        self._v = 0.0
        self._lock = threading.Lock()

    def inc(self, n: float = 1.0) -> None:
        with self._lock:
            self._v += n

    def get(self) -> float:
        return self._v

    def reset(self) -> None:
        with self._lock:
            self._v = 0.0

    def render(self) -> str:
        return f"# HELP {self.name} {self.help}\n# TYPE {self.name} counter\n{self.name} {_num(self._v)}\n"


class Gauge(Counter):
    def set(self, v: float) -> None:
        with self._lock:
            self._v = float(v)

    def dec(self, n: float = 1.0) -> None:
        self.inc(-n)

    def render(self) -> str:
        return f"# HELP {self.name} {self.help}\n# TYPE {self.name} gauge\n{self.name} {_num(self._v)}\n"


class Histogram:
    DEFAULT_BUCKETS = (0.001, 0.0025, 0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0, 30.0, 60.0)

    def __init__(self, name: str, help_: str, buckets=DEFAULT_BUCKETS):
        self.name, self.help = name, help_
        self.buckets = tuple(sorted(buckets))
        self.counts = [0] * (len(self.buckets) + 1)
        self.sum = 0.0
        self.count = 0
        self._lock = threading.Lock()

    def observe(self, v: float) -> None:
        with self._lock:
            self.counts[bisect.bisect_left(self.buckets, v)] += 1
            self.sum += v
            self.count += 1

    def reset(self) -> None:
        with self._lock:
            self.counts = [0] * (len(self.buckets) + 1)
            self.sum, self.count = 0.0, 0

    def quantile(self, q: float) -> float:
        """Upper bound of the bucket that contains the q-quantile (inf for the overflow bucket)."""
        if self.count == 0:
            return 0.0
        target, cum = q * self.count, 0
        for b, c in zip(self.buckets + (float("inf"),), self.counts):
            cum += c
            if cum >= target:
                return b
        return float("inf")

    def render(self) -> str:
        out = [f"# HELP {self.name} {self.help}", f"# TYPE {self.name} histogram"]
        cum = 0
        for b, c in zip(self.buckets, self.counts):
            cum += c
            out.append(f'{self.name}_bucket{{le="{_num(b)}"}} {cum}')
        out.append(f'{self.name}_bucket{{le="+Inf"}} {self.count}')
        out.append(f"{self.name}_sum {_num(self.sum)}")
        out.append(f"{self.name}_count {self.count}")
        return "\n".join(out) + "\n"


def _num(v: float) -> str:
    return str(int(v)) if float(v).is_integer() and abs(v) < 1e15 else repr(float(v))


class RequestRateTracker:
    """Per-request token timing: time between tokens, smoothed tokens/s, queue wait."""

    def __init__(self, ring: int = 128, alpha: float = 0.2):
        self.t_admit = time.perf_counter()
        self.t_first: float | None = None
        self.t_last: float | None = None
        self.tbt: deque[float] = deque(maxlen=ring)
        self.alpha = alpha
        self.ewma_tps = 0.0
        self.tokens = 0

    def on_token(self, now: float | None = None) -> None:
        now = time.perf_counter() if now is None else now
        if self.t_first is None:
            self.t_first = now
        elif self.t_last is not None:
            dt = now - self.t_last
            self.tbt.append(dt)
            if dt > 0:
                inst = 1.0 / dt
                self.ewma_tps = inst if self.ewma_tps == 0.0 else self.alpha * inst + (1 - self.alpha) * self.ewma_tps
        self.t_last = now
        self.tokens += 1

    @property
    def queue_wait(self) -> float:
        return 0.0 if self.t_first is None else self.t_first - self.t_admit

    def percentile_tbt(self, q: float) -> float:
        if not self.tbt:
            return 0.0
        v = sorted(self.tbt)
        return v[min(len(v) - 1, int(q * len(v)))]


class RequestRateAggregator:
    """Rolling window over finished requests."""

    def __init__(self, window: int = 256):
        self.tps: deque[float] = deque(maxlen=window)
        self.waits: deque[float] = deque(maxlen=window)
        self.tbts: deque[float] = deque(maxlen=window * 8)
        self.completed = 0
        self._lock = threading.Lock()

    def record(self, tr: RequestRateTracker) -> None:
        with self._lock:
            if tr.ewma_tps > 0:
                self.tps.append(tr.ewma_tps)
            self.waits.append(tr.queue_wait)
            self.tbts.extend(tr.tbt)
            self.completed += 1

    def snapshot(self) -> dict:
        with self._lock:
            def pct(v, q):
                v = sorted(v)
                return v[min(len(v) - 1, int(q * len(v)))] if v else 0.0
            return {"completed_requests": self.completed,
                    "tokens_per_second": sum(self.tps) / len(self.tps) if self.tps else 0.0,
                    "itl_p50": pct(self.tbts, 0.5), "itl_p95": pct(self.tbts, 0.95),
                    "queue_wait": sum(self.waits) / len(self.waits) if self.waits else 0.0}


class InferenceMetrics:
    """The engine/server metric set, rendered at ``/metrics``."""

    def __init__(self):
        c, g, h = Counter, Gauge, Histogram
        self.tokens_generated = c("oxibonsai_tokens_generated_total", "Tokens generated")
        self.requests = c("oxibonsai_requests_total", "Requests received")
        self.errors = c("oxibonsai_errors_total", "Requests that failed")
        self.prompt_tokens = c("oxibonsai_prompt_tokens_total", "Prompt tokens processed")
        self.prefill_seconds = h("oxibonsai_prefill_duration_seconds", "Prefill (time to first token) duration")
        self.decode_token_seconds = h("oxibonsai_decode_token_duration_seconds", "Per-token decode duration",
                                      (0.0002, 0.0005, 0.001, 0.002, 0.005, 0.01, 0.02, 0.05, 0.1, 0.5, 1.0))
        self.request_seconds = h("oxibonsai_request_duration_seconds", "End-to-end request duration")
        self.tokens_per_second = h("oxibonsai_tokens_per_second", "Per-request decode throughput",
                                   (1, 5, 10, 20, 50, 100, 200, 500, 1000, 2000, 5000))
        self.active_requests = g("oxibonsai_active_requests", "Requests in flight")
        self.kv_utilization = g("oxibonsai_kv_cache_utilization", "Fraction of KV pages in use")
        self.model_memory = g("oxibonsai_model_memory_bytes", "Bytes of device memory held by weights")
        self.request_tps = g("oxibonsai_request_tokens_per_second", "Smoothed per-request tokens per second")
        self.itl_p50 = g("oxibonsai_inter_token_latency_p50_seconds", "Median inter-token latency")
        self.itl_p95 = g("oxibonsai_inter_token_latency_p95_seconds", "95th percentile inter-token latency")
        self.queue_wait = g("oxibonsai_queue_wait_seconds", "Mean admission-to-first-token wait")
        self.kv_level = g("oxibonsai_kv_cache_compression_level", "KV cache format: 0 FP16, 1 Q8, 2 Q4")
        self.aggregator = RequestRateAggregator()

    def all(self):
        return [v for v in vars(self).values() if isinstance(v, (Counter, Histogram))]

    def update_request_rate(self) -> None:
        s = self.aggregator.snapshot()
        self.request_tps.set(s["tokens_per_second"])
        self.itl_p50.set(s["itl_p50"])
        self.itl_p95.set(s["itl_p95"])
        self.queue_wait.set(s["queue_wait"])

    def reset(self) -> None:
        for m in self.all():
            m.reset()

    def render_prometheus(self) -> str:
        self.update_request_rate()
        return "".join(m.render() for m in self.all())
