"""Speculative decoding with an adaptive draft length.

Reference: ``AdaptiveLookahead`` (crates/oxibonsai-runtime/src/adaptive_lookahead.rs:48-220: EWMA of accepted tokens per
step with alpha 0.2, target = round(ewma + 1) clamped to [min, max], initial 5, cooldown of 4 steps between changes),
``SpeculativeDecoder`` (speculative.rs:43-452: draft k tokens, verify, stats, speed-up estimate) and the trigram
draft cache (ngram_cache.rs).  The reference's verifier uses a mock draft probability and synthetic target logits;
here the target model verifies all drafted tokens in one batched pass through the prefill kernels and accepts the
longest prefix on which its own greedy choice agrees (greedy acceptance), or applies the standard
rejection test min(1, p_target / p_draft) when both distributions are available.
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass, field
from typing import Callable, Sequence


@dataclass
class LookaheadConfig:
    min_lookahead: int = 1
    max_lookahead: int = 8
    initial: int = 5
    alpha: float = 0.2
    cooldown_steps: int = 4


class AdaptiveLookahead:
    """Chooses how many tokens to draft from the recent acceptance history."""

    def __init__(self, config: LookaheadConfig | None = None):
        self.config = config or LookaheadConfig()
        c = self.config
        if not 1 <= c.min_lookahead <= c.max_lookahead:
            raise ValueError("need 1 <= min_lookahead <= max_lookahead")
        self.current = max(c.min_lookahead, min(c.max_lookahead, c.initial))
        self.ewma: float | None = None
        self._since_change = 0
        self.steps = 0
        self.adjustments = 0

    def record(self, accepted: int, drafted: int | None = None) -> int:
        """Records the number of accepted draft tokens of one verify step; returns the next draft length."""
        c = self.config
        a = float(max(0, accepted))
        self.ewma = a if self.ewma is None else c.alpha * a + (1.0 - c.alpha) * self.ewma
        self.steps += 1
        self._since_change += 1
        if self._since_change >= c.cooldown_steps:
            target = int(round(self.ewma + 1.0))
            target = max(c.min_lookahead, min(c.max_lookahead, target))
            if target != self.current:
                self.current = target
                self.adjustments += 1
                self._since_change = 0
        return self.current

    def reset(self) -> None:
        self.__init__(self.config)


class NgramCache:
    """Trigram frequency table: proposes the most frequent continuation of the last two tokens."""

    def __init__(self, max_entries: int = 1 << 16):
        self.table: dict[tuple[int, int], dict[int, int]] = defaultdict(dict)
        self.max_entries = max_entries

    def observe(self, tokens: Sequence[int]) -> None:
        for a, b, c in zip(tokens, tokens[1:], tokens[2:]):
            if len(self.table) >= self.max_entries and (a, b) not in self.table:
                continue
            d = self.table[(a, b)]
            d[c] = d.get(c, 0) + 1

    def predict(self, a: int, b: int) -> int | None:
        d = self.table.get((a, b))
        if not d:
            return None
        best = max(d.values())
        return min(t for t, n in d.items() if n == best)

    def draft(self, context: Sequence[int], k: int) -> list[int]:
        ctx = list(context[-2:])
        out: list[int] = []
        while len(out) < k and len(ctx) >= 2:
            t = self.predict(ctx[-2], ctx[-1])
            if t is None:
                break
            out.append(t)
            ctx.append(t)
        return out


@dataclass
class SpeculativeStats:
    steps: int = 0
    drafted: int = 0
    accepted: int = 0
    emitted: int = 0
    target_passes: int = 0
    prefill_seconds: float = 0.0     # both prompts into the caches (GPU decoder only)
    decode_seconds: float = 0.0      # everything after that
    history: list[int] = field(default_factory=list)

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.drafted if self.drafted else 0.0

    @property
    def tokens_per_target_pass(self) -> float:
        return self.emitted / self.target_passes if self.target_passes else 0.0

    def estimated_speedup(self, draft_cost_ratio: float) -> float:
        """Tokens per unit of target-pass time, counting each drafted token at ``draft_cost_ratio`` target passes."""
        if not self.target_passes:
            return 1.0
        cost = self.target_passes + draft_cost_ratio * self.drafted
        return self.emitted / cost if cost > 0 else 1.0


def greedy_accept(draft: Sequence[int], target_choice: Sequence[int]) -> tuple[int, int]:
    """``target_choice[i]`` is the target's greedy token after the context extended by ``draft[:i]`` (len = len(draft)+1).
    Returns (number of accepted draft tokens, the token the target emits after them)."""
    n = 0
    while n < len(draft) and draft[n] == target_choice[n]:
        n += 1
    return n, target_choice[n]


def rejection_accept(draft: Sequence[int], p_draft: Sequence[float], p_target: Sequence[float], uniforms: Sequence[float]) -> int:
    """Standard speculative-sampling acceptance: token i is kept while u_i <= min(1, p_target_i / p_draft_i)."""
    n = 0
    for pd, pt, u in zip(p_draft, p_target, uniforms):
        ratio = 1.0 if pd <= 0 else min(1.0, pt / pd)
        if u <= ratio:
            n += 1
        else:
            break
    return min(n, len(draft))


class SpeculativeDecoder:
    """Draft-and-verify loop over two step functions.

    ``draft_fn(context, k) -> list[int]`` proposes up to k tokens (a small model's greedy continuation or the n-gram
    cache); ``verify_fn(context, draft) -> list[int]`` returns the target's greedy choice at each of the
    ``len(draft) + 1`` positions, computed in one batched pass.  ``GpuSpeculativeDecoder`` below binds both to engines.
    """

    def __init__(self, draft_fn: Callable[[list[int], int], list[int]], verify_fn: Callable[[list[int], list[int]], list[int]],
                 lookahead: AdaptiveLookahead | None = None, eos_token: int | None = None):
        self.draft_fn, self.verify_fn = draft_fn, verify_fn
        self.lookahead = lookahead or AdaptiveLookahead()
        self.eos = eos_token
        self.stats = SpeculativeStats()

    def generate(self, prompt: Sequence[int], max_tokens: int) -> list[int]:
        ctx = list(prompt)
        out: list[int] = []
        while len(out) < max_tokens:
            k = min(self.lookahead.current, max_tokens - len(out))
            draft = list(self.draft_fn(ctx, k))[:k]
            choice = self.verify_fn(ctx, draft)
            n, nxt = greedy_accept(draft, choice)
            self.stats.steps += 1
            self.stats.target_passes += 1
            self.stats.drafted += len(draft)
            self.stats.accepted += n
            self.stats.history.append(n)
            self.lookahead.record(n, len(draft))
            new = draft[:n] + [nxt]
            for t in new:
                if self.eos is not None and t == self.eos:
                    return out
                out.append(t)
                ctx.append(t)
                self.stats.emitted += 1
                if len(out) >= max_tokens:
                    break
        return out


class GpuSpeculativeDecoder:
    """Speculative decoding with a target engine and a (smaller) draft engine on the same GPU.

    Each round the draft engine proposes ``k`` greedy tokens with its own decode graph, the target verifies
    ``[last, d1..dk]`` in one pass through the prefill kernels, the longest agreeing prefix is kept and the target's
    own token follows it.  Rolling back a rejection costs nothing: the paged caches are indexed by position, so the
    next round simply overwrites the stale entries.  Greedy verification reproduces the target's greedy stream exactly.

    With a ``temperature`` the draft samples its proposals from softmax(logits / T) and the target accepts each with
    probability min(1, p / q), replacing the first rejected one by a draw from max(0, p - q): the rejection test runs on the
    device over the logits of both models (csrc/cuda/spec_verify.cu) and the output is distributed as the target's own
    sampling at that temperature.  Top-k / top-p filters are not applied in this mode (both distributions would need the
    same support).  On tensor-parallel engines every rank draws the same uniforms from ``seed``.
    """

    def __init__(self, target, draft, lookahead: AdaptiveLookahead | None = None, eos_token: int | None = None):
        self.target, self.draft = target, draft
        self.lookahead = lookahead or AdaptiveLookahead(LookaheadConfig(min_lookahead=1, max_lookahead=8, initial=4))
        self.eos = eos_token
        self.stats = SpeculativeStats()

    def generate(self, prompt: Sequence[int], max_tokens: int, temperature: float | None = None, seed: int = 0) -> list[int]:
        from .presets import SamplingParams, SamplingPreset
        import random
        sampled = temperature is not None and temperature > 1e-6
        greedy = SamplingPreset.GREEDY.params()
        t_params = SamplingParams(temperature=float(temperature), top_k=0, top_p=1.0, seed=seed) if sampled else greedy
        d_params = SamplingParams(temperature=float(temperature), top_k=0, top_p=1.0, seed=seed + 1) if sampled else greedy
        rnd = random.Random(seed)
        # every call starts from the same decoder state: the draft length adapts within a generation, and ``stats``
        # describes the last one
        self.lookahead.reset()
        self.stats = SpeculativeStats()
        total = len(prompt) + max_tokens + self.lookahead.config.max_lookahead + 2
        out: list[int] = []
        import time
        import torch
        draft_logits = None
        if sampled:
            kmax = self.lookahead.config.max_lookahead
            draft_logits = torch.empty((kmax, self.draft.config.vocab), dtype=torch.float32, device=self.draft.device)
        t0 = time.perf_counter()
        try:
            last = self.target.open_sequence(prompt, total, 0, t_params)
            self.draft.open_sequence(prompt, total, 0, d_params)
            self.stats.prefill_seconds = time.perf_counter() - t0      # both prompts are in the caches (open_sequence synchronises)
            t0 = time.perf_counter()
            pos = len(prompt)            # position at which `last` will be fed
            draft_pos = pos              # the draft cache holds positions < draft_pos
            while len(out) < max_tokens:
                if self.eos is not None and last == self.eos:
                    break
                out.append(last)
                self.stats.emitted += 1
                if len(out) >= max_tokens:
                    break
                k = max(1, min(self.lookahead.current, max_tokens - len(out)))
                # draft: feed `last`, then its own proposals
                drafts: list[int] = []
                tok = last
                for i in range(k):
                    tok = self.draft.decode_one(tok, pos + i)
                    drafts.append(tok)
                    if sampled:      # the distribution this proposal was drawn from
                        draft_logits[i].copy_(self.draft.runner.logits[0, : draft_logits.shape[1]], non_blocking=True)
                draft_pos = pos + k
                if sampled:
                    n, nxt = self.target.verify_sampled([last] + drafts, pos, draft_logits, float(temperature),
                                                        [rnd.random() for _ in range(2 * (k + 1))])
                else:
                    choice = self.target.verify_greedy([last] + drafts, pos)
                    n, nxt = greedy_accept(drafts, choice)
                self.stats.steps += 1
                self.stats.target_passes += 1
                self.stats.drafted += k
                self.stats.accepted += n
                self.stats.history.append(n)
                self.lookahead.record(n, k)
                for t in drafts[:n]:
                    if self.eos is not None and t == self.eos:
                        return out
                    out.append(t)
                    self.stats.emitted += 1
                    if len(out) >= max_tokens:
                        return out
                if n == k:
                    # the draft model has not consumed its last proposal yet
                    self.draft.decode_one(drafts[-1], pos + k)
                    draft_pos = pos + k + 1
                pos = pos + n + 1
                last = nxt
            return out
        finally:
            self.stats.decode_seconds = time.perf_counter() - t0
            self.target.close_sequence(0)
            self.draft.close_sequence(0)
