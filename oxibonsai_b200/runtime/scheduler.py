"""Continuous batching: a background loop that admits requests into engine slots and steps all live sequences together.

Reference: ``ContinuousBatchScheduler`` (crates/oxibonsai-runtime/src/continuous_batch.rs:28-380: priority queues, admission,
per-step bookkeeping - but every step re-runs a whole single-sequence generate per request), ``BoundedQueue`` /
``InferenceQueue`` with back-pressure (request_queue.rs:52-357) and ``AsyncInferenceEngine`` (async_engine.rs:26-154).
Here one decode step advances every live sequence through the batched tcgen05 path, prompts are prefilled into a
free slot between steps, and finished sequences free their KV pages immediately.  Live sequences always occupy
slots 0..n-1: when a sequence ends, the last live slot is moved into the hole (only its block-table row and
sampler state move; KV pages are referenced, never copied).
"""
from __future__ import annotations

import itertools
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Sequence

from .presets import SamplingParams


class QueueFull(RuntimeError):
    """Raised when the admission queue is at capacity (maps to HTTP 503)."""


@dataclass(order=True)
class _Queued:
    priority: int
    seq: int
    request: "Request" = field(compare=False)


@dataclass
class Request:
    prompt: Sequence[int]
    params: SamplingParams
    max_tokens: int
    stop_at_eos: bool = True
    priority: int = 0                      # lower value = served first
    on_token: Callable[[int], None] | None = None
    request_id: str = ""
    # filled by the scheduler
    tokens: list[int] = field(default_factory=list)
    finish_reason: str | None = None
    error: Exception | None = None
    t_submit: float = 0.0
    t_first_token: float | None = None
    t_done: float | None = None
    token_times: list[float] = field(default_factory=list)
    done: threading.Event = field(default_factory=threading.Event)
    cancelled: bool = False

    def wait(self, timeout: float | None = None) -> list[int]:
        if not self.done.wait(timeout):
            raise TimeoutError("generation did not finish in time")
        if self.error is not None:
            raise self.error
        return self.tokens

    def cancel(self) -> None:
        self.cancelled = True

    @property
    def ttft(self) -> float | None:
        return None if self.t_first_token is None else self.t_first_token - self.t_submit


class BoundedPriorityQueue:
    """Priority queue with a hard capacity; ``put`` raises :class:`QueueFull` instead of blocking."""

    def __init__(self, capacity: int):
        self.capacity = capacity
        self._q: queue.PriorityQueue = queue.PriorityQueue()
        self._seq = itertools.count()
        self._lock = threading.Lock()
        self.rejected = 0

    def put(self, r: Request) -> None:
        with self._lock:
            if self._q.qsize() >= self.capacity:
                self.rejected += 1
                raise QueueFull(f"admission queue full ({self.capacity})")
            self._q.put(_Queued(r.priority, next(self._seq), r))

    def get_nowait(self) -> Request | None:
        try:
            return self._q.get_nowait().request
        except queue.Empty:
            return None

    def __len__(self) -> int:
        return self._q.qsize()


class BatchScheduler:
    """Owns an ``InferenceEngine`` (max_batch > 1) and serves requests with continuous batching."""

    def __init__(self, engine, queue_capacity: int = 1024, eos_token: int | None = None, idle_sleep: float = 0.0005):
        from ..core.oracle import EOS_TOKEN
        self.engine = engine
        self.eos = EOS_TOKEN if eos_token is None else eos_token
        self.queue = BoundedPriorityQueue(queue_capacity)
        self.idle_sleep = idle_sleep
        self.live: list[Request] = []          # live[i] occupies slot i
        self._pos: list[int] = []              # next position of slot i
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self.steps = 0
        self.tokens_generated = 0
        self.prompt_tokens = 0
        self.lock = threading.Lock()

    # ---- public API ------------------------------------------------------------------------------
    def start(self) -> "BatchScheduler":
        if self._thread is None:
            self._thread = threading.Thread(target=self._loop, name="bonsai-scheduler", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
            self._thread = None

    def submit(self, prompt: Sequence[int], params: SamplingParams, max_tokens: int, **kw) -> Request:
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if len(prompt) + 1 > self.engine.max_seq_len:
            raise ValueError(f"prompt of {len(prompt)} tokens does not fit max_seq_len {self.engine.max_seq_len}")
        r = Request(list(prompt), params.validate(), max_tokens, t_submit=time.perf_counter(), **kw)
        self.queue.put(r)
        return r

    @property
    def active(self) -> int:
        return len(self.live)

    # ---- loop ------------------------------------------------------------------------------------
    def _loop(self) -> None:
        import torch
        eng = self.engine
        torch.cuda.set_device(eng.device)
        while not self._stop.is_set():
            try:
                admitted = self._admit()
                if not self.live:
                    if not admitted:
                        time.sleep(self.idle_sleep)
                    continue
                self._step()
            except Exception as e:  # a failing step must not wedge the waiting clients
                for r in self.live:
                    r.error = e
                    r.done.set()
                for s in range(len(self.live)):
                    eng._release_slot(s)
                self.live, self._pos = [], []

    def _admit(self) -> bool:
        eng = self.engine
        any_new = False
        while len(self.live) < eng.max_batch:
            r = self.queue.get_nowait()
            if r is None:
                break
            if r.cancelled:
                r.finish_reason = "cancelled"
                r.done.set()
                continue
            slot = len(self.live)
            total = min(eng.max_seq_len, len(r.prompt) + r.max_tokens)
            try:
                first = eng.open_sequence(r.prompt, total, slot, r.params)
            except MemoryError:
                # KV pool exhausted: put the request back and wait for a sequence to finish
                eng._release_slot(slot)
                self.queue.put(r)
                break
            except Exception as e:
                eng._release_slot(slot)
                r.error = e
                r.done.set()
                continue
            self.prompt_tokens += len(r.prompt)
            self.live.append(r)
            self._pos.append(len(r.prompt))
            any_new = True
            if self._emit(slot, first):
                self._retire(slot)
        return any_new

    def _emit(self, slot: int, tok: int) -> bool:
        """Delivers a sampled token; returns True when the sequence is finished."""
        r = self.live[slot]
        now = time.perf_counter()
        if r.cancelled:
            r.finish_reason = "cancelled"
            return True
        if r.stop_at_eos and tok == self.eos:
            r.finish_reason = "stop"
            return True
        r.tokens.append(tok)
        r.token_times.append(now)
        if r.t_first_token is None:
            r.t_first_token = now
        self.tokens_generated += 1
        if r.on_token is not None:
            try:
                r.on_token(tok)
            except Exception:
                r.cancelled = True
        if len(r.tokens) >= r.max_tokens or self._pos[slot] + 1 >= self.engine.max_seq_len:
            r.finish_reason = "length"
            return True
        return False

    def _retire(self, slot: int) -> None:
        eng = self.engine
        r = self.live[slot]
        r.t_done = time.perf_counter()
        r.done.set()
        last = len(self.live) - 1
        eng._release_slot(slot)
        if slot != last:
            eng.move_slot(last, slot)
            self.live[slot] = self.live[last]
            self._pos[slot] = self._pos[last]
        self.live.pop()
        self._pos.pop()

    def _step(self) -> None:
        import torch
        eng, r = self.engine, self.engine.runner
        B = len(self.live)
        # the device holds each slot's last token; positions are set from the host's view
        pos = torch.tensor(self._pos, dtype=torch.int32).pin_memory()
        r.positions[:B].copy_(pos, non_blocking=True)
        r.step(B, sample=True)
        toks = eng._read_tokens(B)      # tokens + the step's status word in one copy; raises on an expired wait
        self.steps += 1
        for s in range(B):
            self._pos[s] += 1
        # retire from the highest slot down so that moves never touch an unprocessed slot
        for s in range(B - 1, -1, -1):
            if self._emit(s, toks[s]):
                self._retire(s)
