"""Queues and front ends over the scheduler (fake engine, no GPU): bounded queue, inference queue, one-call batches, asyncio
front, caller-stepped scheduler, healing decoder."""
import asyncio
import threading
import time

import numpy as np
import pytest

from oxibonsai_b200.runtime import batching as B
from oxibonsai_b200.runtime.presets import SamplingParams
from oxibonsai_b200.runtime.scheduler import BatchScheduler, QueueFull
from test_scheduler_cpu import FakeEngine, _expected


def test_bounded_queue_backpressure_and_stats():
    q = B.BoundedQueue(2)
    assert q.try_push("a") and q.try_push("b") and not q.try_push("c") and q.is_full() and q.utilization() == 1.0 and q.capacity() == 2
    t0 = time.monotonic()
    assert not q.push_timeout("c", 0.05) and time.monotonic() - t0 >= 0.04
    threading.Timer(0.05, q.pop).start()
    assert q.push_timeout("c", 2.0)                      # a slot opened while waiting
    assert q.drain(1) == ["b"] and q.pop() == "c" and q.pop() is None and q.is_empty()
    assert q.pop_timeout(0.02) is None
    threading.Timer(0.03, lambda: q.try_push("late")).start()
    assert q.pop_timeout(2.0) == "late"
    st = q.stats()
    assert (st.pushed, st.popped, st.rejected, st.timed_out, st.peak_depth) == (4, 4, 1, 1, 2)
    with pytest.raises(ValueError):
        B.BoundedQueue(0)


def test_inference_queue_runs_items_and_drops_expired_ones():
    calls = []

    def gen(prompt, n, params):
        calls.append(list(prompt))
        time.sleep(0.05)
        if prompt[0] == 99:
            raise RuntimeError("boom")
        return [prompt[0]] * n

    iq = B.InferenceQueue(gen, capacity=3).start()
    try:
        a = iq.submit([1], 2)
        b = iq.submit([99], 2)
        c = iq.submit([3], 1, ttl=0.01)                   # waits behind two 50 ms jobs: expired when its turn comes
        with pytest.raises(QueueFull):
            for _ in range(5):
                iq.submit([4], 1)
        assert a.result(5) == [1, 1]
        with pytest.raises(RuntimeError, match="boom"):
            b.result(5)
        with pytest.raises(TimeoutError, match="expired"):
            c.result(5)
        assert iq.expired == 1 and [3] not in calls and a.wait_time() > 0
    finally:
        iq.stop()


def test_batch_generate_and_timeout():
    eng = FakeEngine(step_delay=0.002)
    sched = BatchScheduler(eng, eos_token=-1, prefill_chunk_tokens=32).start()
    try:
        prompts = [list(range(10 + i, 30 + 2 * i)) for i in range(6)]
        res = B.batch_generate(sched, prompts, 7, config=B.BatchConfig(max_batch_size=4))
        assert [r.tokens for r in res] == [_expected(p, 7) for p in prompts]
        assert all(r.finish_reason is B.FinishReason.MAX_TOKENS and r.error is None and r.ttft is not None and r.seconds > 0 for r in res)
        slow = B.batch_generate_with_timeout(sched, [list(range(5, 40))], 5000, timeout=0.1)[0]
        assert slow.finish_reason is B.FinishReason.TIMEOUT and 0 < len(slow.tokens) < 5000
        eng.fail_next_step = True
        bad = B.batch_generate_with_timeout(sched, [list(range(3, 25))], 6)[0]
        assert bad.finish_reason is B.FinishReason.ERROR and "status 2" in bad.error
    finally:
        sched.stop()
    rq = B.RequestQueue(3)
    assert all(rq.push(B.BatchRequest([i], 4)) for i in range(3)) and not rq.push(B.BatchRequest([9], 4)) and rq.is_full() and rq.capacity() == 3
    assert [r.prompt for r in rq.drain_batch(2)] == [[0], [1]] and len(rq) == 1 and not rq.is_empty()


def test_async_front_limits_concurrency_and_streams():
    eng = FakeEngine(step_delay=0.001)
    sched = BatchScheduler(eng, eos_token=-1).start()
    front = B.AsyncSchedulerFront(sched, max_concurrent=2)
    seen_active = []

    async def one(i):
        out = []
        async for tok in front.generate_streaming(list(range(i, i + 20)), 9):
            seen_active.append(front.active_requests())
            out.append(tok)
        return out

    async def main():
        results = await asyncio.gather(*(one(i) for i in range(5)))
        whole = await front.generate(list(range(7, 27)), 4)
        # a consumer that stops early frees its slot: the request is cancelled
        agen = front.generate_streaming(list(range(40, 70)), 1000)
        first = [await agen.__anext__() for _ in range(3)]
        await agen.aclose()
        return results, whole, first

    try:
        results, whole, first = asyncio.run(main())
        assert results == [_expected(list(range(i, i + 20)), 9) for i in range(5)] and whole == _expected(list(range(7, 27)), 4)
        assert first == _expected(list(range(40, 70)), 3) and max(seen_active) <= 2 and front.active_requests() == 0
        assert front.has_capacity() and front.max_concurrent() == 2 and front.engine() is eng
        deadline = time.monotonic() + 5
        while sched.active and time.monotonic() < deadline:
            time.sleep(0.01)
        assert sched.active == 0
    finally:
        sched.stop()


def test_caller_stepped_scheduler():
    eng = FakeEngine()
    s = B.ContinuousBatchScheduler(eng, prefill_chunk_tokens=64)
    assert s.is_idle() and s.step() == 0
    prompts = {name: list(range(a, b)) for name, (a, b) in {"low": (5, 30), "normal": (40, 60), "high": (70, 95)}.items()}
    eng.max_batch = 1                                     # one slot: the order of service is the order of priority
    low = s.submit_with_priority(prompts["low"], 3, B.RequestPriority.LOW)
    normal = s.submit(prompts["normal"], 3)
    high = s.submit_with_priority(prompts["high"], 3, B.RequestPriority.HIGH)
    assert s.queue_depth() == 3 and s.state(high) is B.RequestState.QUEUED and s.get_result(high) is None
    steps = s.run_to_completion()
    assert s.is_idle() and steps >= 6 and s.completed_count() == 3
    done = s.drain_completed()
    assert [rid for rid, _ in done] == [high, normal, low] and dict(done)[low] == _expected(prompts["low"], 3)
    assert s.drain_completed() == [] and s.queue_depth() == 0 and s.active_count() == 0
    st = s.throughput_stats()
    assert st.tokens_generated == 9 and st.completed == 0 and st.prompt_tokens == sum(len(p) for p in prompts.values()) and st.tokens_per_second() > 0
    eng.max_batch = 4
    a, b = s.submit(list(range(3, 20)), 5), s.submit(list(range(8, 30)), 2)
    produced = 0
    while not s.is_idle():
        produced += s.step()
        if s.state(a) is B.RequestState.RUNNING:
            assert s.active_count() >= 1
    assert produced == 7 and s.state(a) is B.RequestState.FINISHED and s.get_result(b) == _expected(list(range(8, 30)), 2) and s.request(a).finish_reason == "length"


def test_healing_decoder_recuts_the_prompt_then_generates():
    vocab = [b"", b"hel", b"hello", b" wor", b" world", b"!", b"x"]
    tb = lambda i: vocab[i]

    def logits(seq):
        z = np.full(len(vocab), -5.0)
        z[{(): 1, (1,): 4, (2,): 4, (2, 4): 5}.get(tuple(seq), 6)] = 3.0       # after "hello": " world"; after "hel": also " world" (a bad cut)
        if tuple(seq) == ():
            z[2] = 4.0                                      # at the start the model prefers "hello" to "hel"
        return z

    dec = B.HealingDecoder()
    healed, out = dec.generate([1], 2, tb, len(vocab), logits, lambda z: int(np.argmax(z)))
    assert healed.tokens == [1] and not healed.was_healed() and len(out) == 2     # a single token: nothing to look back to
    healed, out = dec.generate([5, 1], 2, tb, len(vocab), lambda seq: logits(seq[1:]), lambda z: int(np.argmax(z)))
    assert healed.was_healed() and healed.removed == [1] and healed.tokens == [5, 2] and out == [4, 5]   # "hel" -> "hello", then " world", "!"
