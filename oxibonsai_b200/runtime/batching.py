"""Queues and front ends over the engine and the continuous-batching scheduler: a bounded queue with back-pressure, a work
queue whose items carry their own result slot, one-call batch generation, an ``asyncio`` front, and a scheduler that is
stepped by the caller instead of by a thread.

Reference: crates/oxibonsai-runtime/src - request_queue.rs (``BoundedQueue``: ``try_push`` fails at once when full so the
caller can answer 503, ``push_timeout`` / ``pop_timeout``, statistics; ``InferenceWorkItem`` with waiting time and expiry;
``InferenceQueue``), batch_engine.rs (``batch_generate`` / ``batch_generate_with_timeout``, ``BatchResult`` with a finish
reason, ``RequestQueue.drain_batch``), async_engine.rs (``AsyncInferenceEngine``: ``generate`` / ``generate_streaming``
under a concurrency limit; the thread-per-call form of that name lives in ``runtime/distributed.py``, the form here,
``AsyncSchedulerFront``, feeds the batched scheduler), continuous_batch.rs (``ContinuousBatchScheduler``: ``submit_with_priority``, ``step``,
``run_to_completion``, ``get_result``, ``drain_completed``, throughput statistics).  The reference's batch engine loops over
the requests one after another; here every front end feeds the same batched decode step.
"""
from __future__ import annotations

import asyncio
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, AsyncIterator, Callable, Generic, Sequence, TypeVar

from .presets import SamplingParams
from .scheduler import BatchScheduler, QueueFull, Request

T = TypeVar("T")


# ---- bounded queue ------------------------------------------------------------------------------------------------------------
@dataclass
class QueueStats:
    pushed: int = 0
    popped: int = 0
    rejected: int = 0
    timed_out: int = 0
    peak_depth: int = 0


class BoundedQueue(Generic[T]):
    """FIFO with a fixed capacity.  A full queue refuses (``try_push``) or makes the producer wait (``push_timeout``)."""

    def __init__(self, capacity: int):
        if capacity < 1:
            raise ValueError("capacity must be positive")
        self._cap, self._items = capacity, deque()
        self._lock = threading.Lock()
        self._not_full, self._not_empty = threading.Condition(self._lock), threading.Condition(self._lock)
        self._stats = QueueStats()

    def try_push(self, item: T) -> bool:
        with self._lock:
            if len(self._items) >= self._cap:
                self._stats.rejected += 1
                return False
            self._push(item)
            return True

    def push_timeout(self, item: T, timeout: float) -> bool:
        deadline = time.monotonic() + timeout
        with self._not_full:
            while len(self._items) >= self._cap:
                left = deadline - time.monotonic()
                if left <= 0 or not self._not_full.wait(left):
                    if len(self._items) >= self._cap:
                        self._stats.timed_out += 1
                        return False
            self._push(item)
            return True

    def _push(self, item: T) -> None:
        self._items.append(item)
        self._stats.pushed += 1
        self._stats.peak_depth = max(self._stats.peak_depth, len(self._items))
        self._not_empty.notify()

    def pop(self) -> T | None:
        with self._lock:
            return self._pop()

    def pop_timeout(self, timeout: float) -> T | None:
        deadline = time.monotonic() + timeout
        with self._not_empty:
            while not self._items:
                left = deadline - time.monotonic()
                if left <= 0 or not self._not_empty.wait(left):
                    if not self._items:
                        return None
            return self._pop()

    def _pop(self) -> T | None:
        if not self._items:
            return None
        self._stats.popped += 1
        item = self._items.popleft()
        self._not_full.notify()
        return item

    def drain(self, limit: int | None = None) -> list[T]:
        with self._lock:
            n = len(self._items) if limit is None else min(limit, len(self._items))
            out = [self._items.popleft() for _ in range(n)]
            self._stats.popped += n
            self._not_full.notify_all()
            return out

    def __len__(self) -> int:
        with self._lock:
            return len(self._items)

    def is_empty(self) -> bool:
        return len(self) == 0

    def is_full(self) -> bool:
        return len(self) >= self._cap

    def capacity(self) -> int:
        return self._cap

    def utilization(self) -> float:
        return len(self) / self._cap

    def stats(self) -> QueueStats:
        with self._lock:
            return QueueStats(**vars(self._stats))


@dataclass
class InferenceWorkItem:
    prompt: Sequence[int]
    max_tokens: int
    params: SamplingParams
    deadline: float | None = None                 # monotonic time after which nobody waits for the answer any more
    enqueued_at: float = field(default_factory=time.monotonic)
    done: threading.Event = field(default_factory=threading.Event)
    tokens: list[int] | None = None
    error: Exception | None = None

    def wait_time(self) -> float:
        return time.monotonic() - self.enqueued_at

    def is_expired(self) -> bool:
        return self.deadline is not None and time.monotonic() > self.deadline

    def result(self, timeout: float | None = None) -> list[int]:
        if not self.done.wait(timeout):
            raise TimeoutError("no result in time")
        if self.error is not None:
            raise self.error
        return self.tokens or []


class InferenceQueue:
    """Producers ``submit`` work items and wait on them; a worker thread takes them off the queue (dropping the expired
    ones) and runs ``generate(prompt, max_tokens, params) -> tokens``."""

    def __init__(self, generate: Callable[[Sequence[int], int, SamplingParams], list[int]], capacity: int = 64):
        self._generate, self._q = generate, BoundedQueue(capacity)
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self.expired = 0

    def start(self) -> "InferenceQueue":
        self._thread = threading.Thread(target=self._run, name="bonsai-inference-queue", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def submit(self, prompt: Sequence[int], max_tokens: int, params: SamplingParams | None = None, ttl: float | None = None) -> InferenceWorkItem:
        item = InferenceWorkItem(list(prompt), max_tokens, params or SamplingParams(), None if ttl is None else time.monotonic() + ttl)
        if not self._q.try_push(item):
            raise QueueFull(f"inference queue is full ({self._q.capacity()} items)")
        return item

    def queue_depth(self) -> int:
        return len(self._q)

    def is_full(self) -> bool:
        return self._q.is_full()

    def stats(self) -> QueueStats:
        return self._q.stats()

    def _run(self) -> None:
        while not self._stop.is_set():
            item = self._q.pop_timeout(0.05)
            if item is None:
                continue
            if item.is_expired():
                self.expired += 1
                item.error = TimeoutError(f"expired after {item.wait_time():.3f} s in the queue")
            else:
                try:
                    item.tokens = self._generate(item.prompt, item.max_tokens, item.params)
                except Exception as e:  # noqa: BLE001 - handed to whoever waits on the item
                    item.error = e
            item.done.set()


# ---- one-call batches ---------------------------------------------------------------------------------------------------------
class FinishReason(Enum):
    MAX_TOKENS = "length"
    STOP = "stop"
    TIMEOUT = "timeout"
    CANCELLED = "cancelled"
    ERROR = "error"


@dataclass
class BatchConfig:
    max_batch_size: int = 64
    timeout: float | None = None


@dataclass
class BatchResult:
    tokens: list[int]
    finish_reason: FinishReason
    seconds: float
    ttft: float | None = None
    error: str | None = None


def _finish(r: Request, timed_out: bool) -> FinishReason:
    if r.error is not None:
        return FinishReason.ERROR
    if timed_out:
        return FinishReason.TIMEOUT
    return {"length": FinishReason.MAX_TOKENS, "stop": FinishReason.STOP, "cancelled": FinishReason.CANCELLED}.get(r.finish_reason or "stop", FinishReason.STOP)


def batch_generate_with_timeout(scheduler: BatchScheduler, prompts: Sequence[Sequence[int]], max_tokens: int, params: SamplingParams | None = None,
                                timeout: float | None = None) -> list[BatchResult]:
    """Submits every prompt to a running scheduler (they decode together, as many at a time as the engine has slots) and
    waits for all of them; after ``timeout`` seconds the unfinished ones are cancelled and reported with what they have."""
    p = params or SamplingParams()
    t0 = time.perf_counter()
    reqs = [scheduler.submit(pr, p, max_tokens) for pr in prompts]
    deadline = None if timeout is None else time.monotonic() + timeout
    out = []
    for r in reqs:
        left = None if deadline is None else max(0.0, deadline - time.monotonic())
        finished = r.done.wait(left)
        if not finished:
            r.cancel()
            r.done.wait(5.0)
        out.append(BatchResult(list(r.tokens), _finish(r, not finished), (r.t_done or time.perf_counter()) - t0, r.ttft, None if r.error is None else str(r.error)))
    return out


def batch_generate(scheduler: BatchScheduler, prompts: Sequence[Sequence[int]], max_tokens: int, params: SamplingParams | None = None,
                   config: BatchConfig | None = None) -> list[BatchResult]:
    cfg = config or BatchConfig()
    out: list[BatchResult] = []
    for i in range(0, len(prompts), cfg.max_batch_size):
        out += batch_generate_with_timeout(scheduler, prompts[i:i + cfg.max_batch_size], max_tokens, params, cfg.timeout)
    return out


@dataclass
class BatchRequest:
    prompt: Sequence[int]
    max_tokens: int
    params: SamplingParams = field(default_factory=SamplingParams)


class RequestQueue:
    """Collects requests and hands them out in batches of at most ``batch_size``."""

    def __init__(self, capacity: int = 256):
        self._q: BoundedQueue[BatchRequest] = BoundedQueue(capacity)

    def push(self, request: BatchRequest) -> bool:
        return self._q.try_push(request)

    def drain_batch(self, batch_size: int) -> list[BatchRequest]:
        return self._q.drain(batch_size)

    def __len__(self) -> int:
        return len(self._q)

    def is_empty(self) -> bool:
        return self._q.is_empty()

    def is_full(self) -> bool:
        return self._q.is_full()

    def capacity(self) -> int:
        return self._q.capacity()


# ---- asyncio front ------------------------------------------------------------------------------------------------------------
class AsyncSchedulerFront:
    """``await engine.generate(...)`` / ``async for token in engine.generate_streaming(...)`` over a running scheduler, with
    at most ``max_concurrent`` requests in flight from this front (further callers wait their turn)."""

    def __init__(self, scheduler: BatchScheduler, max_concurrent: int = 64, metrics=None):
        self.scheduler, self._max, self.metrics = scheduler, max_concurrent, metrics
        self._active = 0
        self._sem: asyncio.Semaphore | None = None

    def with_metrics(self, metrics) -> "AsyncSchedulerFront":
        self.metrics = metrics
        return self

    def engine(self):
        return self.scheduler.engine

    def active_requests(self) -> int:
        return self._active

    def max_concurrent(self) -> int:
        return self._max

    def has_capacity(self) -> bool:
        return self._active < self._max

    def _semaphore(self) -> asyncio.Semaphore:
        if self._sem is None:
            self._sem = asyncio.Semaphore(self._max)
        return self._sem

    async def generate(self, prompt: Sequence[int], max_tokens: int, params: SamplingParams | None = None) -> list[int]:
        return [t async for t in self.generate_streaming(prompt, max_tokens, params)]

    async def generate_streaming(self, prompt: Sequence[int], max_tokens: int, params: SamplingParams | None = None) -> AsyncIterator[int]:
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        end = object()
        async with self._semaphore():
            self._active += 1
            req = None
            try:
                req = self.scheduler.submit(prompt, params or SamplingParams(), max_tokens, on_token=lambda t: loop.call_soon_threadsafe(q.put_nowait, t),
                                            on_done=lambda r: loop.call_soon_threadsafe(q.put_nowait, end))
                n = 0
                while True:
                    item = await q.get()
                    if item is end:
                        break
                    n += 1
                    yield item
                if req.error is not None:
                    raise req.error
                if self.metrics is not None:
                    self.metrics.tokens_generated.inc(n)
            finally:
                if req is not None and not req.done.is_set():
                    req.cancel()                      # the consumer stopped iterating: free the slot
                self._active -= 1


# ---- a scheduler stepped by its caller ----------------------------------------------------------------------------------------
class RequestPriority(Enum):
    LOW = 2
    NORMAL = 1
    HIGH = 0                                          # served first


class RequestState(Enum):
    QUEUED = "queued"
    RUNNING = "running"
    FINISHED = "finished"
    FAILED = "failed"


@dataclass
class SchedulerStats:
    steps: int
    tokens_generated: int
    prompt_tokens: int
    completed: int
    seconds: float

    def tokens_per_second(self) -> float:
        return self.tokens_generated / self.seconds if self.seconds > 0 else 0.0


class ContinuousBatchScheduler:
    """The continuous-batching scheduler without its thread: the caller submits requests and calls ``step`` (one admission
    step and one decode step of everything that is running) or ``run_to_completion``."""

    def __init__(self, engine, eos_token: int | None = -1, **scheduler_options):
        self._s = BatchScheduler(engine, eos_token=eos_token, **scheduler_options)
        engine.bind_thread()
        self._by_id: dict[int, Request] = {}
        self._next_id = 0
        self._completed: list[int] = []
        self._t0 = time.perf_counter()

    def submit(self, prompt: Sequence[int], max_tokens: int, params: SamplingParams | None = None) -> int:
        return self.submit_with_priority(prompt, max_tokens, RequestPriority.NORMAL, params)

    def submit_with_priority(self, prompt: Sequence[int], max_tokens: int, priority: RequestPriority, params: SamplingParams | None = None) -> int:
        rid = self._next_id
        self._next_id += 1
        self._by_id[rid] = self._s.submit(prompt, params or SamplingParams(), max_tokens, priority=priority.value,
                                          on_done=lambda r, rid=rid: self._completed.append(rid))
        return rid

    def step(self) -> int:
        """One scheduling step; returns the number of tokens it produced."""
        before = self._s.tokens_generated
        self._s._admit()
        if self._s.live:
            self._s._step()
        return self._s.tokens_generated - before

    def run_to_completion(self, max_steps: int = 1_000_000) -> int:
        steps = 0
        while not self.is_idle() and steps < max_steps:
            self.step()
            steps += 1
        return steps

    def state(self, rid: int) -> RequestState:
        r = self._by_id[rid]
        if r.done.is_set():
            return RequestState.FAILED if r.error is not None else RequestState.FINISHED
        return RequestState.RUNNING if r in self._s.live or (self._s._pending is not None and self._s._pending["r"] is r) else RequestState.QUEUED

    def get_result(self, rid: int) -> list[int] | None:
        r = self._by_id.get(rid)
        return list(r.tokens) if r is not None and r.done.is_set() and r.error is None else None

    def request(self, rid: int) -> Request:
        return self._by_id[rid]

    def queue_depth(self) -> int:
        return len(self._s.queue)

    def active_count(self) -> int:
        return self._s.active + (1 if self._s._pending is not None else 0)

    def completed_count(self) -> int:
        return sum(1 for r in self._by_id.values() if r.done.is_set())

    def is_idle(self) -> bool:
        return self.queue_depth() == 0 and self.active_count() == 0

    def drain_completed(self) -> list[tuple[int, list[int]]]:
        """(id, tokens) of the requests that finished since the last call, in the order they finished; they are forgotten."""
        done, self._completed = self._completed, []
        return [(rid, list(self._by_id.pop(rid).tokens)) for rid in done]

    def throughput_stats(self) -> SchedulerStats:
        return SchedulerStats(self._s.steps, self._s.tokens_generated, self._s.prompt_tokens, self.completed_count(), time.perf_counter() - self._t0)


# ---- token healing around a generation loop -----------------------------------------------------------------------------------
class HealingDecoder:
    """Heals the end of the prompt once (a prompt that stops inside a word is re-cut at a boundary the model knows), then
    draws ``max_tokens`` tokens with the caller's ``sample``."""

    def __init__(self, config=None):
        from .context import TokenHealer
        self.healer = TokenHealer(config)

    def generate(self, prompt_tokens: Sequence[int], max_tokens: int, token_bytes: Callable[[int], bytes], vocab_size: int,
                 get_logits: Callable[[list[int]], Any], sample: Callable[[Any], int]):
        """Returns (healing result, generated tokens).  ``get_logits(tokens)`` gives the next-token logits after
        ``tokens``; ``sample(logits)`` picks a token id."""
        healed = self.healer.heal(prompt_tokens, token_bytes, vocab_size, get_logits)
        seq, out = list(healed.tokens), []
        for _ in range(max_tokens):
            tok = int(sample(get_logits(seq)))
            out.append(tok)
            seq.append(tok)
        return healed, out
