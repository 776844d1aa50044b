"""Continuous batching: a background loop that admits requests into engine slots and steps all live sequences together.

Reference: ``ContinuousBatchScheduler`` (crates/oxibonsai-runtime/src/continuous_batch.rs:28-380: priority queues, admission,
per-step bookkeeping - but every step re-runs a whole single-sequence generate per request), ``BoundedQueue`` /
``InferenceQueue`` with back-pressure (request_queue.rs:52-357) and ``AsyncInferenceEngine`` (async_engine.rs:26-154).
Here one decode step advances every live sequence through the batched tcgen05 path, and finished sequences free their KV
pages immediately.  A new prompt is prefilled into the first free slot in chunks of ``prefill_chunk_tokens``, one chunk per
scheduler iteration, with a decode step of the live batch after every chunk - so a 2048-token newcomer delays the tokens of
the running streams by one chunk's time per step instead of the whole prompt's (the reference's ``ChunkedPrefill`` plans the
chunks, crates/oxibonsai-model/src/chunked_prefill.rs:9-320, but runs them back to back).  Live sequences always occupy
slots 0..n-1: when a sequence ends, the last live slot is moved into the hole (only its block-table row and sampler state
move; KV pages are referenced, never copied).
"""
from __future__ import annotations

import itertools
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Sequence

from .presets import SamplingParams


class _Cancelled(Exception):
    pass


class SchedulerStopped(RuntimeError):
    """The scheduler's loop has ended on a fatal error (its engine is being torn down): it takes no more requests."""


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
    kv_format: str | None = None           # page format the sequence was admitted in (set when a KV policy is active)
    constraint: object | None = None       # TokenConstraint: the sampler only picks tokens it allows; ends the request when complete
    logprobs: int | None = None            # not None: record the log-probability of every token and of the top `logprobs` ones
    token_logprobs: list = field(default_factory=list)   # [(logprob, [(token, logprob), ...]), ...] when `logprobs` is set
    on_done: Callable[["Request"], None] | None = None   # called once, on the scheduler's thread, when the request has ended (any way)

    def finish(self) -> None:
        """Marks the request as ended and tells its owner (once)."""
        cb, self.on_done = self.on_done, None
        self.done.set()
        if cb is not None:
            try:
                cb(self)
            except Exception:  # noqa: BLE001 - the owner's bookkeeping must not stop the scheduler
                pass

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

    def __init__(self, engine, queue_capacity: int = 1024, eos_token: int | None = None, idle_sleep: float = 0.0005,
                 prefill_chunk_tokens: int = 512, kv_policy=None, prefill_chunk_boost: int = 1,
                 before_launch: Callable[[], None] | None = None, on_fatal: Callable[[Exception], bool] | None = None,
                 idle_hook: Callable[[], None] | None = None, idle_hook_seconds: float = 30.0, overlap: bool = False, admit_tokens_per_step: int = 0):
        """``kv_policy``: a :class:`~oxibonsai_b200.runtime.kv_policy.KvCachePolicy`; when given, the scheduler feeds it the
        engine's KV utilisation after every admission and retirement, and every newly admitted sequence gets its pages in the
        format of the policy's current level (FP16 / Q8 / Q4, as far as the engine has pools for them)."""
        self.kv_policy = kv_policy
        # ``before_launch`` runs at the top of every loop iteration that has work (a watchdog's check: it raises before
        # kernels that need a lost peer are launched).  ``on_fatal(error)`` sees every exception that failed the live
        # requests; when it returns True the loop ends (the owner rebuilds the engine and starts a new scheduler).
        # ``idle_hook`` runs every ``idle_hook_seconds`` while nothing is live (a tensor-parallel leader's keep-alive).
        self.before_launch, self.on_fatal, self.idle_hook, self.idle_hook_seconds = before_launch, on_fatal, idle_hook, idle_hook_seconds
        self.fatal: Exception | None = None
        # ``overlap``: launch decode step k + 1 as soon as the tokens of step k are on the host, and deliver those tokens
        # (callbacks, bookkeeping, the front's writes) while the GPU runs it.  Taken only when the batch cannot change under
        # the step in flight: no constrained or log-probability request, nobody at a length limit or an end-of-sequence
        # token.  A request that ends unpredictably (its client left, a stop sequence) has one token too many computed; that
        # token is dropped and the slot is freed after the step.  Needs ``launch_batch`` / ``collect_batch`` on the engine.
        self.overlap = bool(overlap) and bool(getattr(engine, "supports_overlap", False))
        self._inflight: int | None = None      # number of slots of the decode step that has been launched and not collected
        self._zombies: set[int] = set()        # slots of requests that ended while that step was in flight
        self.overlapped_steps = 0
        self.after_step: Callable[[], None] | None = None     # called once after the tokens of a decode step (or of an admission)
                                                               # have been delivered: a front that batches its writes per step
        from ..core.oracle import EOS_TOKEN
        self.engine = engine
        self.prefill_chunk_tokens = max(16, int(prefill_chunk_tokens))
        # While fewer than a quarter of the slots decode, prompt chunks are ``prefill_chunk_boost`` times as long: few streams
        # wait behind the chunk then, and long chunks fill the GPU better (1 = always the same chunk length).
        self.prefill_chunk_boost = max(1, int(prefill_chunk_boost))
        self._pending: dict | None = None      # the request being prefilled: {"r", "slot", "done"} (slot >= len(live))
        # One decode step admits one prompt chunk by default, so a workload of short generations never fills the batch
        # (requests that live n steps keep ~n slots busy).  With ``admit_tokens_per_step`` > 0 further queued prompts are
        # admitted before the step while their cost stays within that many prompt tokens, a prompt counting for at least
        # ``admit_floor_tokens`` (the fixed cost of a prefill pass: one read of the weights and its launches).
        self.admit_tokens_per_step = max(0, int(admit_tokens_per_step))
        self.admit_floor_tokens = 128
        self._admit_cost = 0                   # prompt tokens the last _admit() call put through the engine
        self._deferred: Request | None = None  # popped from the queue, waiting for KV pages
        self.admissions = 0
        self.prefill_chunks = 0
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
        with self.lock:                      # against the fatal path, which closes the scheduler and then empties the queue
            if self.fatal is not None:
                raise SchedulerStopped(f"the scheduler stopped: {self.fatal}")
            self.queue.put(r)
        return r

    @property
    def active(self) -> int:
        return len(self.live)

    # ---- loop ------------------------------------------------------------------------------------
    def _loop(self) -> None:
        eng = self.engine
        eng.bind_thread()
        last_idle = time.monotonic()
        while not self._stop.is_set():
            try:
                if self.before_launch is not None and (self.live or self._pending is not None or self._deferred is not None or len(self.queue)):
                    self.before_launch()
                admitted = self._admit()
                if admitted and self.admit_tokens_per_step and not self.overlap:
                    spent = max(self._admit_cost, self.admit_floor_tokens)
                    while (spent < self.admit_tokens_per_step and self._pending is None and len(self.live) < eng.max_batch
                           and len(self.queue) and self._admit()):
                        spent += max(self._admit_cost, self.admit_floor_tokens)
                if not self.live:
                    if not admitted:
                        if self.idle_hook is not None and time.monotonic() - last_idle >= self.idle_hook_seconds:
                            last_idle = time.monotonic()
                            self.idle_hook()
                        time.sleep(self.idle_sleep)
                    continue
                last_idle = time.monotonic()
                if self.overlap:
                    self._step_overlapped()
                else:
                    self._step()
            except Exception as e:  # a failing step must not wedge the waiting clients
                fatal = False
                if self.on_fatal is not None:
                    try:
                        fatal = bool(self.on_fatal(e))
                    except Exception:  # noqa: BLE001 - the hook must not keep the clients waiting
                        fatal = False
                for r in self.live:
                    r.error = e
                    r.finish()
                if self._pending is not None:
                    self._pending["r"].error = e
                    self._pending["r"].finish()
                slots = list(range(len(self.live))) + ([self._pending["slot"]] if self._pending is not None else [])
                self.live, self._pos, self._pending = [], [], None
                self._inflight, self._zombies = None, set()
                if fatal:                          # the engine is about to be torn down: its slots go with it
                    with self.lock:
                        self.fatal = e             # from here on submit() refuses, so the queue emptied below stays empty
                    if self._deferred is not None:
                        self._deferred.error = e
                        self._deferred.finish()
                        self._deferred = None
                    while (r := self.queue.get_nowait()) is not None:
                        r.error = e
                        r.finish()
                    return
                for s in slots:
                    try:
                        eng.close_sequence(s)
                    except Exception:  # noqa: BLE001 - a second failure while cleaning up changes nothing for the clients
                        pass

    def _speculation_safe(self, B: int, toks: Sequence[int]) -> bool:
        """True when delivering ``toks`` cannot end or alter any of the B sequences in a way the scheduler can foresee."""
        limit = self.engine.max_seq_len
        for s in range(B):
            r = self.live[s]
            if r.cancelled or r.constraint is not None or r.logprobs is not None or (r.stop_at_eos and toks[s] == self.eos):
                return False
            if len(r.tokens) + 2 > r.max_tokens or self._pos[s] + 2 >= limit:      # this token or the next one is the last
                return False
        return True

    def _step_overlapped(self) -> None:
        eng = self.engine
        if self._inflight is None:
            if any(r.constraint is not None for r in self.live):                   # masks depend on the token before: plain step
                self._step()
                return
            self._inflight = len(self.live)
            eng.launch_batch(self._pos[:self._inflight])
        B = self._inflight
        toks = eng.collect_batch(B)                                                # raises on an expired wait, like step_batch
        self._inflight = None
        self.steps += 1
        for s in range(B):
            self._pos[s] += 1
        zombies, self._zombies = self._zombies, set()
        # (a sequence admitted while the step was in flight joins at the next launch: no speculation past it)
        if not zombies and B == len(self.live) and not self._stop.is_set() and self._speculation_safe(B, toks):
            eng.launch_batch(self._pos[:B])                                        # step k + 1 runs while step k's tokens go out
            self._inflight = B
            self.overlapped_steps += 1
        ended = []
        for s in range(B - 1, -1, -1):
            if s in zombies:                       # computed for a request that had already ended: dropped
                ended.append(s)
            elif self._emit(s, toks[s]):
                ended.append(s)
        if self._inflight is not None:
            for s in ended:                        # the step in flight still uses these slots: end the requests now, free the slots after it
                r = self.live[s]
                r.t_done = time.perf_counter()
                r.finish()
            self._zombies = set(ended)
        else:
            for s in ended:                        # highest slot first, so moves never touch an unprocessed slot
                self._retire(s)
        if self.after_step is not None:
            self.after_step()

    def _admit(self) -> bool:
        """Makes progress on admission: at most one prompt chunk per call.  Returns True when something was done."""
        eng = self.engine
        self._admit_cost = 0
        if self._pending is None:
            if len(self.live) >= eng.max_batch:
                return False
            r, self._deferred = self._deferred, None
            while True:
                if r is None:
                    r = self.queue.get_nowait()
                    if r is None:
                        return False
                if not r.cancelled:
                    break
                r.finish_reason = "cancelled"
                r.finish()
                r = None
            slot = len(self.live)
            total = min(eng.max_seq_len, len(r.prompt) + r.max_tokens)
            try:
                if self.kv_policy is not None:
                    r.kv_format = self.kv_policy.page_format()
                    covered = eng.begin_sequence(r.prompt, total, slot, r.params, r.kv_format)
                    self.kv_policy.observe(eng.kv_utilization())
                else:
                    covered = eng.begin_sequence(r.prompt, total, slot, r.params)
            except MemoryError as e:
                eng.close_sequence(slot)
                if not self.live:
                    # nothing left to retire: the pool cannot hold this request at all
                    r.error = e
                    r.finish()
                    return True
                # KV pool exhausted: the request keeps its place at the head and is tried again once a sequence has finished
                # (outside the queue, whose capacity a concurrent submit may have used up meanwhile)
                self._deferred = r
                return False
            except Exception as e:
                eng.close_sequence(slot)
                r.error = e
                r.finish()
                return True
            self._pending = {"r": r, "slot": slot, "done": covered}
        p = self._pending
        r, slot = p["r"], p["slot"]
        try:
            if r.cancelled:
                raise _Cancelled()
            n = len(r.prompt)
            # short remainders go in one piece; never leave a tail shorter than the engine's batched-prefill threshold
            chunk = self.prefill_chunk_tokens * (self.prefill_chunk_boost if 4 * len(self.live) < eng.max_batch else 1)
            end = n if n - p["done"] <= chunk + eng.prefill_min_tokens else p["done"] + chunk
            eng.prefill(r.prompt[p["done"]:end], slot, p["done"])
            self.prefill_chunks += 1
            self._admit_cost = end - p["done"]
            p["done"] = end
            if end < n:
                return True
            if r.constraint is not None:
                r.constraint.reset()
                first = eng.finish_sequence(r.prompt, slot, r.constraint.allowed_mask())
            else:
                first = eng.finish_sequence(r.prompt, slot)
        except _Cancelled:
            eng.close_sequence(slot)
            r.finish_reason = "cancelled"
            r.finish()
            self._pending = None
            return True
        except Exception as e:
            eng.close_sequence(slot)
            r.error = e
            r.finish()
            self._pending = None
            return True
        self._pending = None
        if r.logprobs is not None:               # from the prefill logits, which stay with the prefill slot
            r.token_logprobs.append(eng.token_logprobs(slot, first, r.logprobs))
        dst = len(self.live)
        if slot != dst:                          # sequences retired while this one was prefilling: close the gap
            eng.move_slot(slot, dst)
        self.prompt_tokens += len(r.prompt)
        self.admissions += 1
        self.live.append(r)
        self._pos.append(len(r.prompt))
        if self._emit(dst, first):
            self._retire(dst)
        if self.after_step is not None:
            self.after_step()
        return True

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
        if r.logprobs is not None and len(r.token_logprobs) < len(r.tokens):   # (the first token's was taken at admission)
            r.token_logprobs.append(self.engine.token_logprobs(slot, tok, r.logprobs))
        if r.constraint is not None:
            r.constraint.advance(tok)
            if r.constraint.finished():
                r.finish_reason = "stop"
        if r.t_first_token is None:
            r.t_first_token = now
        self.tokens_generated += 1
        if r.on_token is not None:
            try:
                r.on_token(tok)
            except Exception:
                r.cancelled = True
        if r.finish_reason == "stop":
            return True
        if len(r.tokens) >= r.max_tokens or self._pos[slot] + 1 >= self.engine.max_seq_len:
            r.finish_reason = "length"
            return True
        return False

    def _retire(self, slot: int) -> None:
        r = self.live[slot]
        if not r.done.is_set():
            r.t_done = time.perf_counter()
            r.finish()
        self._free_slot(slot)

    def _free_slot(self, slot: int) -> None:
        eng = self.engine
        last = len(self.live) - 1
        eng.close_sequence(slot)
        if self.kv_policy is not None:
            self.kv_policy.observe(eng.kv_utilization())
        if slot != last:
            eng.move_slot(last, slot)
            self.live[slot] = self.live[last]
            self._pos[slot] = self._pos[last]
        self.live.pop()
        self._pos.pop()

    def _step(self) -> None:
        eng = self.engine
        B = len(self.live)
        # the device holds each slot's last token; positions are set from the host's view
        masks = {s: r.constraint.allowed_mask() for s, r in enumerate(self.live) if r.constraint is not None}
        # raises when a kernel of the step recorded an expired wait
        toks = eng.step_batch(self._pos, masks) if masks else eng.step_batch(self._pos)
        self.steps += 1
        for s in range(B):
            self._pos[s] += 1
        # retire from the highest slot down so that moves never touch an unprocessed slot
        for s in range(B - 1, -1, -1):
            if self._emit(s, toks[s]):
                self._retire(s)
        if self.after_step is not None:
            self.after_step()
