"""Beam search and n-best decoding over a ``logits_fn(tokens) -> logits`` callback.

Reference: crates/oxibonsai-runtime/src/beam_search.rs:35-380 (``BeamSearchConfig``, ``Beam`` with a length-penalised
score ``log_prob / len^alpha``, ``BeamSearchEngine::search`` with early stopping, ``apply_no_repeat_ngram``,
``top_k_log_probs``, ``prune_beams``) and nbest.rs:18-280 (``Hypothesis``, bounded ``NBestList`` heap, ``NBestDecoder``).
On a GPU engine ``logits_fn`` is backed by ``InferenceEngine`` slots: the engine exposes one KV slot per live beam.
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass
from typing import Callable, Sequence

import numpy as np

from .sampling_advanced import log_softmax


@dataclass
class BeamSearchConfig:
    beam_width: int = 4
    max_length: int = 64
    length_penalty: float = 1.0
    eos_token: int | None = None
    no_repeat_ngram: int = 0
    early_stopping: bool = True
    top_k_per_beam: int | None = None      # candidates expanded per beam (default: beam_width)


@dataclass
class Beam:
    tokens: list[int]
    log_prob: float = 0.0
    prompt_len: int = 0
    finished: bool = False

    def score(self, length_penalty: float) -> float:
        n = max(1, len(self.tokens) - self.prompt_len)
        return self.log_prob / (n ** length_penalty)

    def extend(self, token: int, log_prob: float, eos: int | None) -> "Beam":
        return Beam(self.tokens + [int(token)], self.log_prob + float(log_prob), self.prompt_len, eos is not None and token == eos)

    def __len__(self) -> int:
        return len(self.tokens)

    @property
    def generated(self) -> list[int]:
        return self.tokens[self.prompt_len:]


@dataclass
class BeamSearchResult:
    beams: list[Beam]
    steps: int
    length_penalty: float = 1.0

    def best(self) -> list[int]:
        return self.beams[0].generated if self.beams else []

    def best_score(self) -> float:
        return self.beams[0].score(self.length_penalty) if self.beams else float("-inf")


def apply_no_repeat_ngram(logits: np.ndarray, tokens: Sequence[int], n: int) -> np.ndarray:
    """Bans every token that would complete an n-gram already present in ``tokens``."""
    out = np.array(logits, dtype=np.float64, copy=True)
    if n <= 0 or len(tokens) < n:
        return out
    prefix = tuple(tokens[len(tokens) - n + 1:]) if n > 1 else ()
    for i in range(len(tokens) - n + 1):
        if tuple(tokens[i:i + n - 1]) == prefix:
            out[tokens[i + n - 1]] = -np.inf
    return out


def top_k_log_probs(logits: np.ndarray, k: int) -> list[tuple[int, float]]:
    lp = log_softmax(logits)
    k = min(k, len(lp))
    idx = np.argpartition(-lp, k - 1)[:k]
    idx = idx[np.argsort(-lp[idx], kind="stable")]
    return [(int(i), float(lp[i])) for i in idx if np.isfinite(lp[i])]


def prune_beams(beams: list[Beam], width: int, length_penalty: float) -> list[Beam]:
    return sorted(beams, key=lambda b: b.score(length_penalty), reverse=True)[:width]


class BeamSearchEngine:
    def __init__(self, config: BeamSearchConfig | None = None):
        self.config = config or BeamSearchConfig()

    def search(self, prompt: Sequence[int], logits_fn: Callable[[list[int]], np.ndarray]) -> BeamSearchResult:
        c = self.config
        live = [Beam(list(prompt), 0.0, len(prompt))]
        done: list[Beam] = []
        steps = 0
        expand = c.top_k_per_beam or c.beam_width
        for steps in range(1, c.max_length + 1):
            cand: list[Beam] = []
            for b in live:
                logits = np.asarray(logits_fn(b.tokens), dtype=np.float64)
                if c.no_repeat_ngram:
                    logits = apply_no_repeat_ngram(logits, b.tokens, c.no_repeat_ngram)
                for tok, lp in top_k_log_probs(logits, expand):
                    cand.append(b.extend(tok, lp, c.eos_token))
            if not cand:
                break
            cand = prune_beams(cand, c.beam_width, c.length_penalty)
            done.extend(b for b in cand if b.finished)
            live = [b for b in cand if not b.finished]
            if not live:
                break
            if c.early_stopping and len(done) >= c.beam_width:
                # no live beam can still beat the worst finished one (log-probs only decrease)
                worst_done = min(b.score(c.length_penalty) for b in prune_beams(done, c.beam_width, c.length_penalty))
                best_live = max(b.log_prob / (max(1, c.max_length) ** c.length_penalty) if c.length_penalty > 0 else b.log_prob for b in live)
                if best_live <= worst_done:
                    break
        final = prune_beams(done + live, c.beam_width, c.length_penalty)
        return BeamSearchResult(final, steps, c.length_penalty)


# ---- n-best --------------------------------------------------------------------------------------------------------
@dataclass(order=False)
class Hypothesis:
    tokens: list[int]
    log_prob: float = 0.0
    complete: bool = False
    length_penalty: float = 0.0

    def score(self) -> float:
        n = max(1, len(self.tokens))
        return self.log_prob / (n ** self.length_penalty) if self.length_penalty else self.log_prob

    def extend(self, token: int, token_log_prob: float) -> "Hypothesis":
        return Hypothesis(self.tokens + [int(token)], self.log_prob + float(token_log_prob), False, self.length_penalty)

    def __len__(self) -> int:
        return len(self.tokens)


class NBestList:
    """Keeps the ``n`` best hypotheses seen (a min-heap on score)."""

    def __init__(self, n: int):
        self.n = max(1, n)
        self._heap: list[tuple[float, int, Hypothesis]] = []
        self._seq = 0

    def push(self, hyp: Hypothesis) -> None:
        item = (hyp.score(), self._seq, hyp)
        self._seq += 1
        if len(self._heap) < self.n:
            heapq.heappush(self._heap, item)
        elif item[0] > self._heap[0][0]:
            heapq.heapreplace(self._heap, item)

    def top(self) -> Hypothesis | None:
        return max(self._heap)[2] if self._heap else None

    def worst_score(self) -> float | None:
        return self._heap[0][0] if self._heap else None

    def is_full(self) -> bool:
        return len(self._heap) >= self.n

    def __len__(self) -> int:
        return len(self._heap)

    def into_sorted(self) -> list[Hypothesis]:
        return [h for _, _, h in sorted(self._heap, key=lambda t: (-t[0], t[1]))]

    def complete_hypotheses(self) -> list[Hypothesis]:
        return [h for h in self.into_sorted() if h.complete]


class NBestDecoder:
    def __init__(self, n: int, eos_id: int, max_len: int, length_penalty: float = 0.0):
        self.n, self.eos, self.max_len, self.alpha = n, eos_id, max_len, length_penalty

    def init(self, prompt: Sequence[int] = ()) -> NBestList:
        l = NBestList(self.n)
        l.push(Hypothesis(list(prompt), 0.0, False, self.alpha))
        return l

    def step(self, current: NBestList, logits_fn: Callable[[list[int]], np.ndarray]) -> NBestList:
        nxt = NBestList(self.n)
        for h in current.into_sorted():
            if h.complete or len(h) >= self.max_len:
                h.complete = True
                nxt.push(h)
                continue
            for tok, lp in top_k_log_probs(np.asarray(logits_fn(h.tokens)), self.n):
                e = h.extend(tok, lp)
                e.complete = tok == self.eos
                nxt.push(e)
        return nxt

    def decode(self, prompt: Sequence[int], logits_fn: Callable[[list[int]], np.ndarray]) -> list[Hypothesis]:
        cur = self.init(prompt)
        for _ in range(self.max_len):
            cur = self.step(cur, logits_fn)
            if all(h.complete for h in cur.into_sorted()):
                break
        return cur.into_sorted()

    @staticmethod
    def partition(hyps: Sequence[Hypothesis]) -> tuple[list[Hypothesis], list[Hypothesis]]:
        return [h for h in hyps if h.complete], [h for h in hyps if not h.complete]
