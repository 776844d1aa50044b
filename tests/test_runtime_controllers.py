"""Host-side runtime controllers (no GPU): KV policy, adaptive lookahead, n-gram drafts, speculative loop."""
import pytest

from oxibonsai_b200.runtime.kv_policy import KvCachePolicy, KvLevel, KvPolicyConfig
from oxibonsai_b200.runtime.speculative import (AdaptiveLookahead, LookaheadConfig, NgramCache, SpeculativeDecoder, greedy_accept,
                                                rejection_accept)


def test_kv_policy_escalates_and_recovers_with_hysteresis():
    p = KvCachePolicy()
    assert p.level == KvLevel.FP16 and p.page_format() == "f16"
    for _ in range(30):
        p.observe(0.85)
    assert p.level == KvLevel.Q8 and p.upgrades == 1 and p.metric_value() == 1
    for _ in range(40):
        p.observe(0.99)
    assert p.level == KvLevel.Q4 and p.page_format() == "q4" and p.metric_value() == 2
    # just below the moderate threshold but inside the hysteresis band: no drop to FP16 yet
    for _ in range(60):
        p.observe(0.78)
    assert p.level == KvLevel.Q8
    for _ in range(60):
        p.observe(0.30)
    assert p.level == KvLevel.FP16 and p.downgrades >= 2
    assert 0.29 < p.smoothed_pressure < 0.31


def test_kv_policy_presets_and_validation():
    p = KvCachePolicy.fp16_only()
    for _ in range(50):
        p.observe(1.0)
    assert p.level == KvLevel.FP16
    a = KvCachePolicy.aggressive()
    for _ in range(50):
        a.observe(0.7)
    assert a.level == KvLevel.Q8
    with pytest.raises(ValueError):
        KvCachePolicy(KvPolicyConfig(alpha=0.0))
    with pytest.raises(ValueError):
        KvCachePolicy(KvPolicyConfig(moderate_threshold=0.9, severe_threshold=0.5))


def test_adaptive_lookahead_tracks_acceptance_within_bounds():
    la = AdaptiveLookahead(LookaheadConfig(min_lookahead=1, max_lookahead=8, initial=5, cooldown_steps=4))
    assert la.current == 5
    for _ in range(40):
        la.record(0)
    assert la.current == 1
    for _ in range(80):
        la.record(8)
    assert la.current == 8 and la.adjustments >= 2
    la2 = AdaptiveLookahead(LookaheadConfig(initial=5, cooldown_steps=4))
    la2.record(0); la2.record(0); la2.record(0)
    assert la2.current == 5          # cooldown: no change before 4 steps
    with pytest.raises(ValueError):
        AdaptiveLookahead(LookaheadConfig(min_lookahead=4, max_lookahead=2))


def test_ngram_cache_and_acceptance_rules():
    c = NgramCache()
    c.observe([1, 2, 3, 1, 2, 3, 1, 2, 4])
    assert c.predict(1, 2) == 3 and c.predict(9, 9) is None
    assert c.draft([7, 1, 2], 3) == [3, 1, 2]
    assert greedy_accept([5, 6, 7], [5, 6, 9, 1]) == (2, 9)
    assert greedy_accept([5], [4, 8]) == (0, 4)
    assert greedy_accept([], [3]) == (0, 3)
    assert rejection_accept([1, 2, 3], [0.5, 0.5, 0.5], [0.5, 0.1, 0.9], [0.9, 0.5, 0.1]) == 1


def test_speculative_loop_reproduces_the_target_stream():
    target = lambda ctx: (ctx[-1] * 7 + len(ctx)) % 50            # deterministic "model"
    def verify(ctx, draft):
        out, c = [], list(ctx)
        for d in list(draft) + [None]:
            out.append(target(c))
            if d is not None:
                c.append(d)
        return out
    def draft(ctx, k):          # right two times out of three
        c, out = list(ctx), []
        for i in range(k):
            t = target(c) if (len(c) % 3) else (target(c) + 1) % 50
            out.append(t); c.append(t)
        return out
    dec = SpeculativeDecoder(draft, verify)
    got = dec.generate([3, 4], 40)
    ref, c = [], [3, 4]
    for _ in range(40):
        t = target(c); ref.append(t); c.append(t)
    assert got == ref
    assert dec.stats.emitted == 40 and dec.stats.target_passes < 40 and 0 < dec.stats.acceptance_rate < 1
    assert dec.stats.tokens_per_target_pass > 1.0 and dec.stats.estimated_speedup(0.1) > 1.0
