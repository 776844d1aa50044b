"""Failure handling on the host: circuit breaker, retries, time-outs, rate limiting, idempotency, health.

Reference: ``CircuitBreaker`` closed -> open -> half-open with threshold 5 failures, 30 s recovery, 3 probe requests and
2 successes to close (crates/oxibonsai-runtime/src/circuit_breaker.rs:13-246); ``retry_with_backoff`` / ``with_timeout`` /
error classification (recovery.rs:12-199); token-bucket rate limiter per client and global (rate_limiter.rs:97-326);
idempotency cache (middleware.rs:294-366); health checks with RSS < 80 % healthy / < 95 % degraded and KV
utilisation < 0.75 / < 0.90 (health.rs:10-245).  Nothing here touches a GPU: failures are detected and injected on
the host (exceptions, time-outs, dropped heartbeats).
"""
from __future__ import annotations

import threading
import time
from collections import OrderedDict
from dataclasses import dataclass
from enum import Enum
from typing import Callable, TypeVar

T = TypeVar("T")


class CircuitState(Enum):
    CLOSED = "closed"
    OPEN = "open"
    HALF_OPEN = "half_open"


class CircuitOpenError(RuntimeError):
    pass


@dataclass
class CircuitBreakerConfig:
    failure_threshold: int = 5
    recovery_seconds: float = 30.0
    half_open_max_requests: int = 3
    success_threshold: int = 2


class CircuitBreaker:
    def __init__(self, config: CircuitBreakerConfig | None = None, clock: Callable[[], float] = time.monotonic):
        self.config = config or CircuitBreakerConfig()
        self._clock = clock
        self._lock = threading.Lock()
        self.state = CircuitState.CLOSED
        self.failures = 0
        self.successes = 0
        self._opened_at = 0.0
        self._probes = 0
        self.total_rejected = 0

    def allow(self) -> bool:
        with self._lock:
            if self.state == CircuitState.OPEN:
                if self._clock() - self._opened_at >= self.config.recovery_seconds:
                    self.state = CircuitState.HALF_OPEN
                    self._probes = 0
                    self.successes = 0
                else:
                    self.total_rejected += 1
                    return False
            if self.state == CircuitState.HALF_OPEN:
                if self._probes >= self.config.half_open_max_requests:
                    self.total_rejected += 1
                    return False
                self._probes += 1
            return True

    def record_success(self) -> None:
        with self._lock:
            if self.state == CircuitState.HALF_OPEN:
                self.successes += 1
                if self.successes >= self.config.success_threshold:
                    self.state = CircuitState.CLOSED
                    self.failures = 0
            else:
                self.failures = 0

    def record_failure(self) -> None:
        with self._lock:
            if self.state == CircuitState.OPEN:
                return                      # already open: a late failure must not restart the recovery timer
            if self.state == CircuitState.HALF_OPEN:
                self._open()
            else:
                self.failures += 1
                if self.failures >= self.config.failure_threshold:
                    self._open()

    def _open(self) -> None:
        self.state = CircuitState.OPEN
        self._opened_at = self._clock()

    def call(self, fn: Callable[[], T]) -> T:
        if not self.allow():
            raise CircuitOpenError("circuit open")
        try:
            r = fn()
        except Exception:
            self.record_failure()
            raise
        self.record_success()
        return r


def is_retryable(e: Exception) -> bool:
    if getattr(e, "retryable", False):
        return True
    return isinstance(e, (TimeoutError, ConnectionError, MemoryError))


def retry_with_backoff(fn: Callable[[], T], attempts: int = 3, base_delay: float = 0.05, factor: float = 2.0, max_delay: float = 2.0,
                       sleep: Callable[[float], None] = time.sleep) -> T:
    delay = base_delay
    for i in range(attempts):
        try:
            return fn()
        except Exception as e:
            if i == attempts - 1 or not is_retryable(e):
                raise
            sleep(min(delay, max_delay))
            delay *= factor
    raise RuntimeError("unreachable")


def with_timeout(fn: Callable[[], T], seconds: float) -> T:
    """Runs ``fn`` on a worker thread and raises TimeoutError if it does not finish in time."""
    box: dict = {}

    def run():
        try:
            box["v"] = fn()
        except Exception as e:  # noqa: BLE001
            box["e"] = e

    t = threading.Thread(target=run, daemon=True)
    t.start()
    t.join(seconds)
    if t.is_alive():
        raise TimeoutError(f"operation exceeded {seconds}s")
    if "e" in box:
        raise box["e"]
    return box["v"]


def memory_aware_batch_size(requested: int, bytes_per_item: int, free_bytes: int, safety: float = 0.8) -> int:
    if bytes_per_item <= 0:
        return requested
    return max(1, min(requested, int(free_bytes * safety) // bytes_per_item))


class TokenBucket:
    def __init__(self, rate: float, burst: float, clock: Callable[[], float] = time.monotonic):
        self.rate, self.burst = rate, burst
        self._tokens = burst
        self._clock = clock
        self._t = clock()
        self._lock = threading.Lock()

    def try_acquire(self, n: float = 1.0) -> bool:
        with self._lock:
            now = self._clock()
            self._tokens = min(self.burst, self._tokens + (now - self._t) * self.rate)
            self._t = now
            if self._tokens >= n:
                self._tokens -= n
                return True
            return False

    def give_back(self, n: float = 1.0) -> None:
        """Returns tokens taken for work that was then refused elsewhere."""
        with self._lock:
            self._tokens = min(self.burst, self._tokens + n)


class RateLimiter:
    """Global bucket plus one bucket per client id (LRU-bounded)."""

    def __init__(self, global_rate: float = 100.0, global_burst: float = 200.0, client_rate: float = 10.0, client_burst: float = 20.0,
                 max_clients: int = 10000, clock: Callable[[], float] = time.monotonic):
        self._clock = clock
        self._global = TokenBucket(global_rate, global_burst, clock)
        self._client_rate, self._client_burst = client_rate, client_burst
        self._clients: OrderedDict[str, TokenBucket] = OrderedDict()
        self._max = max_clients
        self._lock = threading.Lock()
        self.rejected = 0

    def allow(self, client: str) -> bool:
        with self._lock:
            b = self._clients.get(client)
            if b is None:
                b = TokenBucket(self._client_rate, self._client_burst, self._clock)
                self._clients[client] = b
                if len(self._clients) > self._max:
                    self._clients.popitem(last=False)
            else:
                self._clients.move_to_end(client)
        ok = b.try_acquire()
        if ok and not self._global.try_acquire():
            b.give_back()                      # refused for everybody: the client's own allowance is not spent on it
            ok = False
        if not ok:
            self.rejected += 1
        return ok


class IdempotencyCache:
    def __init__(self, capacity: int = 1024, ttl: float = 300.0, clock: Callable[[], float] = time.monotonic):
        self._d: OrderedDict[str, tuple[float, object]] = OrderedDict()
        self.capacity, self.ttl, self._clock = capacity, ttl, clock
        self._lock = threading.Lock()

    def get(self, key: str):
        with self._lock:
            v = self._d.get(key)
            if v is None:
                return None
            if self._clock() - v[0] > self.ttl:
                del self._d[key]
                return None
            self._d.move_to_end(key)
            return v[1]

    def put(self, key: str, value) -> None:
        with self._lock:
            self._d[key] = (self._clock(), value)
            self._d.move_to_end(key)
            while len(self._d) > self.capacity:
                self._d.popitem(last=False)


class HealthStatus(Enum):
    HEALTHY = "healthy"
    DEGRADED = "degraded"
    UNHEALTHY = "unhealthy"


def rss_fraction() -> float:
    try:
        with open("/proc/self/statm") as f:
            rss_pages = int(f.read().split()[1])
        with open("/proc/meminfo") as f:
            total_kb = int(next(l for l in f if l.startswith("MemTotal")).split()[1])
        import os
        return rss_pages * os.sysconf("SC_PAGE_SIZE") / (total_kb * 1024)
    except Exception:
        return 0.0


def check_health(model_loaded: bool, kv_utilization: float, rss: float | None = None, breaker: CircuitBreaker | None = None) -> dict:
    rss = rss_fraction() if rss is None else rss
    checks = {
        "model": HealthStatus.HEALTHY if model_loaded else HealthStatus.UNHEALTHY,
        "memory": HealthStatus.HEALTHY if rss < 0.80 else (HealthStatus.DEGRADED if rss < 0.95 else HealthStatus.UNHEALTHY),
        "kv_cache": HealthStatus.HEALTHY if kv_utilization < 0.75 else (HealthStatus.DEGRADED if kv_utilization < 0.90 else HealthStatus.UNHEALTHY),
    }
    if breaker is not None:
        checks["circuit"] = {CircuitState.CLOSED: HealthStatus.HEALTHY, CircuitState.HALF_OPEN: HealthStatus.DEGRADED,
                             CircuitState.OPEN: HealthStatus.UNHEALTHY}[breaker.state]
    order = [HealthStatus.HEALTHY, HealthStatus.DEGRADED, HealthStatus.UNHEALTHY]
    worst = max(checks.values(), key=order.index)
    return {"status": worst.value, "checks": {k: v.value for k, v in checks.items()}}
