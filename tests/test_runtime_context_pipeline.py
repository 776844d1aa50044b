"""Context windows, budgets, token healing, chunked-prefill planning, the prefix-cache trie and the pipeline API (CPU)."""
import numpy as np
import pytest

from oxibonsai_b200.runtime import context as CX


def test_context_window_strategies():
    w = CX.ContextWindow(10, CX.TruncationStrategy.KEEP_LAST)
    w.set_system_prompt([100, 101])
    assert w.append(range(6)) == 0 and w.remaining_capacity() == 2 and not w.is_at_limit()
    assert w.append([6, 7, 8, 9]) == 2 and w.tokens() == [100, 101] + list(range(2, 10)) and w.is_at_limit()
    assert w.utilization() == 1.0
    f = CX.ContextWindow(4, CX.TruncationStrategy.KEEP_FIRST)
    f.append(range(7))
    assert f.tokens() == [0, 1, 2, 3]
    b = CX.ContextWindow(4, CX.TruncationStrategy.KEEP_BOTH_ENDS)
    b.append(range(8))
    assert b.tokens() == [0, 1, 6, 7]
    e = CX.ContextWindow(3, CX.TruncationStrategy.ERROR)
    with pytest.raises(CX.ContextError):
        e.append(range(5))
    with pytest.raises(CX.ContextError):
        CX.ContextWindow(2).set_system_prompt([1, 2, 3])
    w.clear_conversation()
    assert len(w) == 2


def test_conversation_context_evicts_whole_turns_but_keeps_system():
    c = CX.ConversationContext(10)
    c.add_turn("system", "s", [1, 2])
    c.add_turn("user", "a", [3, 4, 5])
    c.add_turn("assistant", "b", [6, 7, 8])
    c.add_turn("user", "c", [9, 10, 11, 12])
    assert [t.role for t in c.turns] == ["system", "assistant", "user"] and c.total_tokens() == 9 and not c.is_full()
    assert c.build_tokens()[:2] == [1, 2] and c.last_turn().content == "c" and c.turn_count() == 3
    c.clear()
    assert c.utilization() == 0.0


def test_budgets():
    b = CX.RequestBudget(CX.BudgetConfig().with_max_completion(3), 10)
    assert b.record_token() and b.record_token() and not b.record_token() and b.is_exhausted() and b.remaining_completion_tokens() == 0
    t = CX.RequestBudget(CX.BudgetConfig().with_max_total(12), 10)
    assert t.remaining_completion_tokens() == 2 and t.total_tokens() == 10
    h = CX.RequestBudget(CX.BudgetConfig(max_completion=1, policy=CX.BudgetPolicy.HARD_STOP), 1)
    h.record_token()
    with pytest.raises(CX.BudgetError):
        h.record_token()
    with pytest.raises(CX.BudgetError):
        CX.RequestBudget(CX.BudgetConfig(max_total=5, policy=CX.BudgetPolicy.HARD_STOP), 9)
    w = CX.RequestBudget(CX.BudgetConfig(max_completion=1, policy=CX.BudgetPolicy.WARN), 0)
    assert w.record_tokens(3) and w.overrun == 2
    assert CX.RequestBudget(CX.BudgetConfig.unlimited(), 5).remaining_completion_tokens() is None
    g = CX.GlobalTokenBudget(100)
    g.record(40)
    assert g.remaining() == 60 and g.utilization() == 0.4 and not g.is_exhausted()
    assert CX.GlobalTokenBudget.unlimited().remaining() is None
    est = CX.TokenCostEstimate.compute(1000, 100, 10000.0, 100.0)
    assert est.total_seconds == pytest.approx(1.1) and "1000 prompt" in est.summary()


def test_token_healing_replaces_a_split_word():
    vocab = [b"hel", b"hello", b" wor", b" world", b"x", b"!"]
    tb = lambda i: vocab[i]
    # after "hello" the model strongly prefers " world" (3) over " wor" (2)
    def logits(tokens):
        x = np.full(len(vocab), -5.0)
        x[3] = 5.0 if tokens[-1] == 1 else -5.0
        return x
    res = CX.TokenHealer.with_lookback(1).heal([1, 2], tb, len(vocab), logits)
    assert res.was_healed() and res.tokens == [1, 3] and res.removed == [2] and res.replacement == [3]
    same = CX.TokenHealer().heal([1, 5], tb, len(vocab), logits)
    assert not same.was_healed() and same.tokens == [1, 5]
    assert CX.TokenHealer.is_continuation_token("hel", "lo") and not CX.TokenHealer.is_continuation_token("hello", " world")
    assert CX.TokenHealer.token_prob(np.array([0.0, 0.0]), 1) == pytest.approx(0.5)


def test_chunked_prefill_planner():
    cfg = CX.ChunkedPrefillConfig(chunk_size=4).with_overlap(1)
    chunks = CX.create_prefill_chunks(10, cfg)
    assert [(c.start, c.end) for c in chunks] == [(0, 4), (3, 7), (6, 10)] and chunks[-1].is_last and len(chunks[0]) == 4
    s = CX.PrefillScheduler(10, CX.ChunkedPrefillConfig(4))
    kinds = []
    while not s.is_complete():
        kinds.append(s.next_action().kind)
    assert kinds == ["prefill", "decode", "prefill", "decode", "prefill"] and s.next_action().kind == "done" and s.total_chunks() == 3
    assert s.progress() == 1.0 and s.memory_savings(4096) == pytest.approx(0.6)
    pf = CX.PrefillScheduler(10, CX.ChunkedPrefillConfig(4).with_priority(CX.PrefillPriority.PREFILL_FIRST))
    assert [pf.next_action().kind for _ in range(4)] == ["prefill"] * 3 + ["done"]
    with pytest.raises(ValueError):
        CX.create_prefill_chunks(5, CX.ChunkedPrefillConfig(2, overlap=2))
    est = CX.peak_memory_estimate(32768, 1024, 4096, 12288, 36, 8, 128, 151936)
    assert est.kv_bytes == 32768 * 36 * 2 * 8 * 128 * 2 and "KV" in est.summary() and est.total_bytes > est.kv_bytes


def test_prefix_cache_trie():
    from oxibonsai_b200.runtime.prefix_cache import PrefixCache
    ref = {}

    def retain(p):
        for x in p:
            ref[x] = ref.get(x, 0) + 1

    def release(p):
        for x in p:
            ref[x] -= 1
    pc = PrefixCache(4, 3, retain, release)
    assert pc.insert(list(range(10)), [10, 11, 12]) == 2 and pc.size == 2
    assert pc.lookup(list(range(10))) == [10, 11] and pc.lookup(list(range(8)), max_tokens=7) == [10]
    assert pc.lookup([9, 9, 9, 9]) == [] and pc.stats.hit_rate == pytest.approx(2 / 3)
    assert pc.insert([0, 1, 2, 3, 9, 9, 9, 9], [10, 20]) == 1 and pc.size == 3
    pc.lookup([0, 1, 2, 3, 9, 9, 9, 9])
    assert pc.insert([7] * 8, [30, 31]) == 2 and pc.size == 3 and pc.stats.evicted_pages >= 2
    assert pc.evict(1) == 1 and pc.size == 2
    pc.clear()
    assert pc.size == 0 and all(v == 0 for v in ref.values())


# ---- pipeline ------------------------------------------------------------------------------------------------------------------------
VOCAB = [b"a", b"b", b"c", b" ", b"STOP", b"!", b"<eos>"]


def _detok(toks):
    return b"".join(VOCAB[t] for t in toks).decode()


def _cycle_logits(tokens):
    x = np.full(len(VOCAB), -9.0)
    x[(tokens[-1] + 1) % 6] = 4.0      # a b c ' ' STOP ! a ...
    return x


def test_pipeline_greedy_stop_sequence_and_eos():
    from oxibonsai_b200.runtime.pipeline import PipelineBuilder, StopReason, greedy_pipeline, chat_pipeline, code_pipeline
    out = greedy_pipeline(5).run([0], _cycle_logits, _detok)
    assert out.tokens == [1, 2, 3, 4, 5] and out.stop_reason == StopReason.MAX_TOKENS and out.prompt_tokens == 1
    out = PipelineBuilder().max_tokens(20).stop_on(["STOP"]).build().run([0], _cycle_logits, _detok)
    assert out.text == "bc " and out.stop_reason == StopReason.STOP_SEQUENCE and out.tokens == [1, 2, 3]
    eos_fn = lambda toks: np.eye(len(VOCAB))[6] * 5 if len(toks) >= 3 else _cycle_logits(toks)
    out = PipelineBuilder().max_tokens(20).eos(6).build().run([0], eos_fn, _detok)
    assert out.stop_reason == StopReason.EOS and out.tokens == [1, 2]
    assert chat_pipeline().stop_sequences() == ["<|im_end|>"] and code_pipeline().max_tokens() == 1024


def test_pipeline_with_constraint_window_beam_and_sampling():
    from oxibonsai_b200.runtime.beam import BeamSearchConfig
    from oxibonsai_b200.runtime.constrained import DfaConstraint, TokenTable
    from oxibonsai_b200.runtime.pipeline import PipelineBuilder, StopReason
    from oxibonsai_b200.runtime.sampling_advanced import SamplerChain
    table = TokenTable(VOCAB)
    c = DfaConstraint.from_regex(table, "(ab)+", eos_token=6)
    flat = lambda toks: np.zeros(len(VOCAB))
    p = PipelineBuilder().max_tokens(6).with_constraint(c).eos(6).with_sampling(SamplerChain(3).add("temperature", 1.0)).build()
    assert p.has_constraint() and not p.has_healing()
    out = p.run([3], flat, _detok, vocab_size=len(VOCAB))
    assert out.text and set(out.text) <= {"a", "b"} and out.text.startswith("ab")
    w = PipelineBuilder().max_tokens(2).context_window(3).build().run([0, 1, 2, 3, 4], _cycle_logits, _detok)
    assert w.truncated_tokens == 2 and w.prompt_tokens == 3 and w.tokens == [5, 0]
    b = PipelineBuilder().max_tokens(4).with_beam_search(BeamSearchConfig(beam_width=3, max_length=10)).build().run([0], _cycle_logits, _detok)
    assert b.tokens == [1, 2, 3, 4] and b.stop_reason == StopReason.MAX_TOKENS
