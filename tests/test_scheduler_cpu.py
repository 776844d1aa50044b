"""Continuous-batching scheduler against a fake engine (no GPU): chunked admission interleaved with decode steps, slot
compaction while a prompt is still prefilling, error and cancellation paths."""
import threading
import time

from oxibonsai_b200.runtime.presets import SamplingParams
from oxibonsai_b200.runtime.scheduler import BatchScheduler


class FakeEngine:
    """Token i of a sequence is (sum of its prompt + i) % 1000; records every call so that orderings can be asserted."""

    max_batch, max_seq_len, prefill_min_tokens = 4, 100000, 16

    def __init__(self, step_delay=0.0):
        self.log = []
        self.slots = {}            # slot -> {"seed", "n", "prefilled"}
        self.step_delay = step_delay
        self.fail_next_step = False

    def bind_thread(self):
        pass

    def begin_sequence(self, prompt, max_total, slot, params):
        assert slot not in self.slots
        self.slots[slot] = {"seed": sum(prompt), "n": 0, "prefilled": 0, "len": len(prompt)}
        self.log.append(("begin", slot, len(prompt)))
        return 0

    def prefill(self, part, slot, pos0):
        s = self.slots[slot]
        assert pos0 == s["prefilled"]
        s["prefilled"] += len(part)
        self.log.append(("prefill", slot, pos0, len(part)))

    def finish_sequence(self, prompt, slot):
        s = self.slots[slot]
        assert s["prefilled"] == len(prompt)
        self.log.append(("finish", slot))
        s["n"] = 1
        return s["seed"] % 1000

    def step_batch(self, positions):
        if self.fail_next_step:
            self.fail_next_step = False
            raise RuntimeError("decode step reported status 2")
        time.sleep(self.step_delay)
        B = len(positions)
        self.log.append(("step", B))
        out = []
        for b in range(B):
            s = self.slots[b]
            assert positions[b] == s["len"] + s["n"] - 1
            out.append((s["seed"] + s["n"]) % 1000)
            s["n"] += 1
        return out

    def move_slot(self, src, dst):
        self.log.append(("move", src, dst))
        self.slots[dst] = self.slots.pop(src)

    def close_sequence(self, slot):
        self.slots.pop(slot, None)


def _expected(prompt, n):
    return [(sum(prompt) + i) % 1000 for i in range(n)]


def test_prompt_chunks_interleave_with_decode_steps():
    eng = FakeEngine()
    sched = BatchScheduler(eng, eos_token=-1, prefill_chunk_tokens=64)
    a = sched.submit(list(range(1, 21)), SamplingParams(), 40)
    sched.start()
    while not a.tokens:
        time.sleep(0.001)
    b = sched.submit(list(range(330)), SamplingParams(), 5)     # 330 tokens = 4 x 64 + 74: a tail of 10 would be shorter than the
    #                                                             engine's batched-prefill threshold, so it joins the last chunk
    assert b.wait(10) == _expected(list(range(330)), 5) and a.wait(10) == _expected(list(range(1, 21)), 40)
    sched.stop()
    chunks = [e for e in eng.log if e[0] == "prefill" and e[1] == 1]
    assert [c[3] for c in chunks] == [64, 64, 64, 64, 74]
    # between two chunks of the newcomer the running stream got a decode step
    idx = [eng.log.index(c) for c in chunks]
    for i0, i1 in zip(idx, idx[1:]):
        assert ("step", 1) in eng.log[i0:i1]
    assert sched.prefill_chunks >= 5


def test_slot_gap_is_closed_when_a_stream_ends_during_a_prefill():
    eng = FakeEngine(step_delay=0.02)
    sched = BatchScheduler(eng, eos_token=-1, prefill_chunk_tokens=32)
    a = sched.submit([5] * 20, SamplingParams(), 3)             # ends after three tokens (two slow decode steps) ...
    sched.start()
    while not a.tokens:
        time.sleep(0.001)
    b = sched.submit([7] * 400, SamplingParams(), 6)            # ... while this one is still being prefilled into slot 1
    assert a.wait(10) == _expected([5] * 20, 3)
    assert b.wait(10) == _expected([7] * 400, 6)
    sched.stop()
    assert ("move", 1, 0) in eng.log and not eng.slots


def test_failed_step_fails_live_and_pending_requests_and_the_loop_survives():
    eng = FakeEngine(step_delay=0.002)
    sched = BatchScheduler(eng, eos_token=-1, prefill_chunk_tokens=32).start()
    a = sched.submit([1] * 20, SamplingParams(), 1000)
    while not a.tokens:
        time.sleep(0.001)
    b = sched.submit([2] * 4000, SamplingParams(), 4)
    while not any(e[0] == "prefill" and e[1] == 1 for e in eng.log):
        time.sleep(0.001)
    eng.fail_next_step = True
    for r in (a, b):
        try:
            r.wait(10)
            raise AssertionError("expected the step failure to surface")
        except RuntimeError as e:
            assert "status 2" in str(e)
    c = sched.submit([3] * 20, SamplingParams(), 4)
    assert c.wait(10) == _expected([3] * 20, 4)
    sched.stop()


def test_cancel_while_prefilling_frees_the_slot():
    eng = FakeEngine(step_delay=0.001)
    sched = BatchScheduler(eng, eos_token=-1, prefill_chunk_tokens=16).start()
    a = sched.submit([1] * 20, SamplingParams(), 200)
    while not a.tokens:
        time.sleep(0.001)
    b = sched.submit([2] * 5000, SamplingParams(), 4)
    while not any(e[0] == "prefill" and e[1] == 1 for e in eng.log):
        time.sleep(0.001)
    b.cancel()
    assert b.done.wait(10) and b.finish_reason == "cancelled"
    a.cancel()
    assert a.done.wait(10)
    sched.stop()
    assert not eng.slots


def test_policy_level_sets_the_page_format_of_the_next_sequence():
    """The scheduler asks the KV policy for a format at every admission and feeds it the engine's utilisation: once the
    pressure crosses the policy's thresholds, sequences admitted from then on get Q8 and then Q4 pages."""
    from oxibonsai_b200.runtime.kv_policy import KvCachePolicy, KvPolicyConfig

    class Eng(FakeEngine):
        util = 0.1
        formats = []

        def begin_sequence(self, prompt, max_total, slot, params, kv_format=None):
            self.formats.append(kv_format)
            return super().begin_sequence(prompt, max_total, slot, params)

        def kv_utilization(self):
            return self.util

    eng = Eng()
    pol = KvCachePolicy(KvPolicyConfig(alpha=1.0))
    sched = BatchScheduler(eng, eos_token=-1, kv_policy=pol).start()
    a = sched.submit([1] * 20, SamplingParams(), 2)
    a.wait(10)
    eng.util = 0.85                                   # moderate pressure is observed when the next one is admitted ...
    b = sched.submit([2] * 20, SamplingParams(), 2)
    b.wait(10)
    c = sched.submit([3] * 20, SamplingParams(), 2)   # ... so this one is the first to get the denser format
    c.wait(10)
    eng.util = 0.97
    d = sched.submit([4] * 20, SamplingParams(), 2)
    d.wait(10)
    e = sched.submit([5] * 20, SamplingParams(), 2)
    e.wait(10)
    sched.stop()
    assert eng.formats == ["f16", "f16", "q8", "q8", "q4"] and [r.kv_format for r in (a, c, e)] == ["f16", "q8", "q4"]
    assert pol.upgrades == 2


def test_constrained_request_sends_masks_and_ends_when_the_constraint_is_complete():
    import numpy as np

    class Exactly(object):
        """Allows exactly the token sequence ``seq``; complete after the last one."""

        def __init__(self, seq):
            self.seq, self.i = seq, 0

        def reset(self):
            self.i = 0

        def allowed_mask(self):
            m = np.zeros(32, dtype=np.uint32)
            t = self.seq[self.i]
            m[t >> 5] |= np.uint32(1 << (t & 31))
            return m

        def advance(self, tok):
            self.i += 1
            return True

        def is_complete(self):
            return self.i >= len(self.seq)

        def finished(self):
            return self.i >= len(self.seq)

    class Eng(FakeEngine):
        seen_masks = []

        def finish_sequence(self, prompt, slot, mask=None):
            super().finish_sequence(prompt, slot)
            return self._pick(slot, mask)

        def step_batch(self, positions, masks=None):
            out = super().step_batch(positions)
            for s, m in (masks or {}).items():
                out[s] = self._pick(s, m)
            return out

        def _pick(self, slot, mask):
            if mask is None:
                return self.slots[slot]["seed"] % 1000
            self.seen_masks.append(mask.copy())
            return int(np.flatnonzero(np.unpackbits(mask.view(np.uint8), bitorder="little"))[0])

        def token_logprobs(self, slot, tok, n):
            return (-1.0, [(tok, -1.0)][:n])

    eng = Eng()
    sched = BatchScheduler(eng, eos_token=-1).start()
    free = sched.submit([9] * 20, SamplingParams(), 6)
    tied = sched.submit([1] * 20, SamplingParams(), 50, constraint=Exactly([7, 300, 12]), logprobs=1)
    assert tied.wait(10) == [7, 300, 12] and tied.finish_reason == "stop"
    assert len(tied.token_logprobs) == 3 and tied.token_logprobs[0] == (-1.0, [(7, -1.0)])
    assert len(free.wait(10)) == 6
    sched.stop()
    assert len(eng.seen_masks) == 3


def test_prompt_chunks_are_longer_while_few_streams_decode():
    eng = FakeEngine()                                         # four slots: "few" means none is decoding
    sched = BatchScheduler(eng, eos_token=-1, prefill_chunk_tokens=64, prefill_chunk_boost=4)
    a = sched.submit(list(range(600)), SamplingParams(), 3)
    sched.start()
    assert a.wait(10) == _expected(list(range(600)), 3)
    sched.stop()
    assert [e[3] for e in eng.log if e[0] == "prefill"] == [256, 256, 88]


def test_watchdog_hook_stops_launches_and_a_fatal_error_ends_the_loop():
    """``before_launch`` runs before work is launched (not while idle); an error that ``on_fatal`` claims fails the live and
    the queued requests and ends the loop with ``fatal`` set, so the owner can rebuild the engine; ``idle_hook`` fires while
    nothing is live."""
    eng = FakeEngine(step_delay=0.002)
    state = {"checks": 0, "lost": False, "idle": 0}

    class Lost(RuntimeError):
        pass

    def check():
        state["checks"] += 1
        if state["lost"]:
            raise Lost("rank 1 lost")

    sched = BatchScheduler(eng, prefill_chunk_tokens=16, before_launch=check, on_fatal=lambda e: isinstance(e, Lost),
                           idle_hook=lambda: state.__setitem__("idle", state["idle"] + 1), idle_hook_seconds=0.02).start()
    time.sleep(0.15)
    assert state["checks"] == 0 and state["idle"] >= 2                  # idle: the keep-alive runs, the watchdog is not asked
    a = sched.submit(list(range(20)), SamplingParams(), 400)
    while len(a.tokens) < 5:
        time.sleep(0.005)
    assert state["checks"] >= 5
    steps_before = sum(1 for e in eng.log if e[0] == "step")
    state["lost"] = True
    b = sched.submit(list(range(30)), SamplingParams(), 5)             # may or may not be picked up before the loss is seen
    assert a.done.wait(5) and b.done.wait(5)
    assert isinstance(a.error, Lost) and isinstance(b.error, Lost) and isinstance(sched.fatal, Lost)
    assert sum(1 for e in eng.log if e[0] == "step") <= steps_before + 1   # nothing was launched after the check raised
    sched._thread.join(2)
    assert not sched._thread.is_alive()
    assert not any(e[0] == "close" for e in eng.log[-2:])              # the slots are left to the engine that is torn down
    sched.stop()


class OverlapEngine(FakeEngine):
    """FakeEngine with the split step: ``launch_batch`` computes the step, ``collect_batch`` hands it out.  Checks the rules
    of a step in flight: its slots are neither closed nor moved nor stepped again before it is collected."""
    supports_overlap = True

    def __init__(self, step_delay=0.0):
        super().__init__(step_delay)
        self.inflight = None

    def launch_batch(self, positions):
        assert self.inflight is None, "a second step was launched before the first was collected"
        self.inflight = (len(positions), super().step_batch(list(positions)))
        self.log.append(("launch", len(positions)))

    def collect_batch(self, batch):
        assert self.inflight is not None and self.inflight[0] == batch
        toks, self.inflight = self.inflight[1], None
        return toks

    def step_batch(self, positions, masks=None):
        assert self.inflight is None, "a plain step while another one is in flight"
        return super().step_batch(positions)

    def finish_sequence(self, prompt, slot, mask=None):
        return super().finish_sequence(prompt, slot)

    def close_sequence(self, slot):
        assert self.inflight is None or slot >= self.inflight[0], "a slot of the step in flight was closed"
        super().close_sequence(slot)

    def move_slot(self, src, dst):
        assert self.inflight is None or (src >= self.inflight[0] and dst >= self.inflight[0]), "a slot of the step in flight was moved"
        super().move_slot(src, dst)


def test_overlapped_steps_give_the_same_streams_and_respect_the_step_in_flight():
    """With ``overlap`` the next decode step is launched before the tokens of the last one are delivered.  The streams are
    the same as without it, natural endings never cost an extra token, and a request that ends unpredictably (a callback
    that raises) is dropped after the step that was already running."""
    def run(overlap):
        eng = OverlapEngine()
        sched = BatchScheduler(eng, eos_token=-1, prefill_chunk_tokens=32, overlap=overlap)
        assert sched.overlap == overlap
        seen = []

        def bail(tok):
            seen.append(tok)
            if len(seen) == 7:
                raise RuntimeError("client went away")
        reqs = [sched.submit(list(range(10 + i, 40 + 3 * i)), SamplingParams(), 20 + 9 * i) for i in range(3)]
        reqs.append(sched.submit(list(range(5, 25)), SamplingParams(), 100, on_token=bail))
        sched.start()
        late = sched.submit(list(range(50, 90)), SamplingParams(), 15)          # admitted while the others decode
        for r in reqs + [late]:
            assert r.done.wait(10)
        sched.stop()
        assert eng.inflight is None and not eng.slots and sched.active == 0
        return [list(r.tokens) for r in reqs + [late]], [r.finish_reason for r in reqs + [late]], eng, sched

    plain, why_plain, _, _ = run(False)
    over, why_over, eng, sched = run(True)
    assert over == plain and why_over == why_plain == ["length", "length", "length", "cancelled", "length"]
    assert [len(t) for t in over] == [20, 29, 38, 7, 15]
    assert sched.overlapped_steps > 20 and sum(1 for e in eng.log if e[0] == "launch") >= sched.overlapped_steps
    # with nothing but predictable endings every launched step is used: tokens computed == tokens delivered
    eng2 = OverlapEngine()
    s2 = BatchScheduler(eng2, eos_token=-1, overlap=True)
    rs = [s2.submit(list(range(3, 30)), SamplingParams(), n) for n in (5, 9, 9, 30)]
    s2.start()
    for r in rs:
        assert r.done.wait(10)
    s2.stop()
    computed = sum(e[1] for e in eng2.log if e[0] == "step")
    assert computed == sum(len(r.tokens) - 1 for r in rs)                      # (the first token of a stream comes from its prefill)


def test_overlap_is_off_for_constrained_requests_and_unsupported_engines():
    eng = FakeEngine()
    assert BatchScheduler(eng, eos_token=-1, overlap=True).overlap is False     # no launch / collect on this engine

    class Until3:
        def __init__(self):
            self.n = 0

        def reset(self):
            self.n = 0

        def allowed_mask(self):
            return None

        def advance(self, tok):
            self.n += 1
            return True

        def finished(self):
            return self.n >= 3

    eng = OverlapEngine()
    sched = BatchScheduler(eng, eos_token=-1, overlap=True).start()
    a = sched.submit(list(range(20)), SamplingParams(), 50, constraint=Until3())
    b = sched.submit(list(range(20, 45)), SamplingParams(), 12)
    assert a.done.wait(10) and b.done.wait(10)
    sched.stop()
    assert len(a.tokens) == 3 and a.finish_reason == "stop" and len(b.tokens) == 12
    first_launch = next(i for i, e in enumerate(eng.log) if e[0] == "launch")
    steps_before = [e for e in eng.log[:first_launch] if e[0] == "step"]
    assert steps_before                                                         # while the constrained request lived, plain steps were taken


def test_budgeted_admission_fills_the_batch_on_short_generations():
    """One admission per decode step keeps about as many slots busy as a request lives steps; with a token budget several
    queued prompts join before each step, within the budget, and a long prompt still goes in one chunk per step."""
    class Wide(FakeEngine):
        max_batch = 16

    def run(budget):
        eng = Wide()
        sched = BatchScheduler(eng, eos_token=-1, queue_capacity=256, prefill_chunk_tokens=64, admit_tokens_per_step=budget)
        sched.admit_floor_tokens = 16
        prompts = [[i + 1] * 10 for i in range(100)]
        reqs = [sched.submit(p, SamplingParams(), 6) for p in prompts]
        long = sched.submit([3] * 300, SamplingParams(), 6)               # 300 tokens: chunks of 64, one per step
        sched.start()
        try:
            for r, p in zip(reqs, prompts):
                assert r.wait(timeout=30) == _expected(p, 6)
            assert long.wait(timeout=30) == _expected([3] * 300, 6)
        finally:
            sched.stop()
        assert sched.active == 0 and sched.admissions == 101 and not eng.slots
        sizes = [e[1] for e in eng.log if e[0] == "step"]
        # admissions between two decode steps
        between, run_ = [], 0
        for e in eng.log:
            if e[0] == "finish":
                run_ += 1
            elif e[0] == "step":
                between.append(run_)
                run_ = 0
        return sizes, between, eng.log

    sizes1, between1, _ = run(0)
    assert max(between1) == 1 and max(sizes1) <= 6                        # a request lives 5 steps after its admission
    sizes4, between4, log = run(64)                                       # 64 tokens at a floor of 16: up to four prompts per step
    assert max(between4) == 4 and max(sizes4) == 16 and len(sizes4) < 0.5 * len(sizes1)
    # the long prompt never shared a step's budget with another admission once it was pending, and took one chunk per step
    chunks = [i for i, e in enumerate(log) if e[0] == "prefill" and e[3] == 64]
    assert len(chunks) >= 3
    for a, b in zip(chunks, chunks[1:]):
        assert any(e[0] == "step" for e in log[a:b])


def test_a_request_without_kv_pages_keeps_its_place_and_does_not_need_queue_room():
    """When the pool cannot take the next request it waits at the head, outside the queue: a submit that fills the queue
    meanwhile cannot make the wait fail, later requests do not overtake it, and a request that no retirement can ever make room
    for fails by itself."""
    class Tight(FakeEngine):
        max_batch = 4

        def begin_sequence(self, prompt, max_total, slot, params):
            if len(prompt) > 50:
                raise MemoryError("KV cache exhausted: the prompt alone needs more pages than the pool has")
            if len(self.slots) >= 2:                                     # pages for two sequences
                raise MemoryError("KV cache exhausted")
            return super().begin_sequence(prompt, max_total, slot, params)

    eng = Tight(step_delay=0.002)
    sched = BatchScheduler(eng, eos_token=-1, queue_capacity=2)
    order = []
    mk = lambda i, n: sched.submit([i + 1] * 5, SamplingParams(), n, on_done=lambda r, i=i: order.append(i))
    a, b = mk(0, 30), mk(1, 30)
    sched.start()
    try:
        while sched.active < 2:
            time.sleep(0.001)
        c = mk(2, 4)                                                     # popped, finds no pages, waits at the head
        while len(sched.queue):
            time.sleep(0.001)
        d, e = mk(3, 4), mk(4, 4)                                        # the queue is full again while c waits
        for r in (a, b, c, d, e):
            r.wait(timeout=30)
        assert all(r.error is None for r in (a, b, c, d, e))
        assert [len(r.tokens) for r in (a, b, c, d, e)] == [30, 30, 4, 4, 4]
        assert order.index(2) < order.index(3) < order.index(4)
        big = sched.submit([7] * 60, SamplingParams(), 4)
        big.done.wait(30)
        assert isinstance(big.error, MemoryError)
        assert mk(5, 3).wait(timeout=30) == _expected([6] * 5, 3)        # and the scheduler carries on
    finally:
        sched.stop()
    assert sched.active == 0 and not eng.slots
