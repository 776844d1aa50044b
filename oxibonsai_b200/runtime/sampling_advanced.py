"""Host-side advanced samplers over a logits row: Mirostat v1/v2, locally typical, eta, min-p, a composable
``SamplerChain``, repetition penalty, and adaptive strategies that retune the sampling parameters while generating.

Reference: crates/oxibonsai-runtime/src/sampling_advanced.rs:30-778 (``LcgRng``, ``softmax_inplace``, ``log_softmax``,
``entropy``, ``perplexity``, ``apply_repetition_penalty``, ``MirostatV1Sampler``, ``MirostatV2Sampler``, ``TypicalSampler``,
``EtaSampler``, ``MinPSampler``, ``SamplerStep`` / ``SamplerChain`` with greedy / default_chat / creative / precise chains)
and adaptive_sampling.rs:14-306 (``GenerationState``, ``EntropyCooling``, ``RepetitionAdaptation``, ``ScheduledDecay``,
``AdaptiveSamplerChain``).  The GPU sampler (csrc/cuda/sampler.cu) covers temperature / top-k / top-p / masks on the
device; these samplers take the logits row the engine exposes and are used by the pipeline API when a request asks for
them.
"""
from __future__ import annotations

import math
from collections import Counter, deque
from dataclasses import dataclass, field, replace
from typing import Sequence

import numpy as np

from .presets import SamplingParams


class LcgRng:
    """64-bit linear congruential generator (Knuth's MMIX constants); floats use the top 24 bits."""

    MUL, INC, MASK = 6364136223846793005, 1442695040888963407, (1 << 64) - 1

    def __init__(self, seed: int):
        self.state = (int(seed) ^ 0x5DEECE66D) & self.MASK

    def next_u64(self) -> int:
        self.state = (self.state * self.MUL + self.INC) & self.MASK
        return self.state

    def next_f32(self) -> float:
        return (self.next_u64() >> 40) / float(1 << 24)

    def next_below(self, n: int) -> int:
        return self.next_u64() % n if n > 0 else 0


def softmax(logits: np.ndarray) -> np.ndarray:
    x = np.asarray(logits, dtype=np.float64)
    m = np.max(x)
    if not np.isfinite(m):
        out = np.zeros_like(x)
        out[np.argmax(x)] = 1.0
        return out
    e = np.exp(x - m)
    return e / e.sum()


def log_softmax(logits: np.ndarray) -> np.ndarray:
    x = np.asarray(logits, dtype=np.float64)
    m = np.max(x)
    return x - m - math.log(np.exp(x - m).sum())


def entropy(probs: np.ndarray) -> float:
    p = np.asarray(probs, dtype=np.float64)
    p = p[p > 0]
    return float(-(p * np.log(p)).sum())


def perplexity(log_probs: Sequence[float]) -> float:
    lp = np.asarray(log_probs, dtype=np.float64)
    return float(math.exp(-lp.mean())) if lp.size else 1.0


def top_k_indices(logits: np.ndarray, k: int) -> np.ndarray:
    k = min(max(k, 0), len(logits))
    if k == 0:
        return np.empty(0, dtype=np.int64)
    idx = np.argpartition(-np.asarray(logits), k - 1)[:k]
    return idx[np.argsort(-np.asarray(logits)[idx], kind="stable")]


def apply_temperature(logits: np.ndarray, temp: float) -> np.ndarray:
    return np.asarray(logits, dtype=np.float64) / max(temp, 1e-6)


def apply_repetition_penalty(logits: np.ndarray, token_ids: Sequence[int], penalty: float) -> np.ndarray:
    """Divides positive logits of seen tokens by ``penalty`` and multiplies negative ones (the CTRL rule)."""
    out = np.array(logits, dtype=np.float64, copy=True)
    if penalty == 1.0:
        return out
    ids = np.unique(np.asarray([t for t in token_ids if 0 <= t < len(out)], dtype=np.int64))
    sel = out[ids]
    out[ids] = np.where(sel > 0, sel / penalty, sel * penalty)
    return out


def apply_frequency_presence_penalty(logits: np.ndarray, token_ids: Sequence[int], frequency: float = 0.0, presence: float = 0.0) -> np.ndarray:
    out = np.array(logits, dtype=np.float64, copy=True)
    for t, c in Counter(int(t) for t in token_ids if 0 <= t < len(out)).items():
        out[t] -= frequency * c + presence
    return out


def _draw(probs: np.ndarray, rng: LcgRng) -> int:
    u = rng.next_f32() * float(probs.sum())
    c = np.cumsum(probs)
    return int(min(np.searchsorted(c, u, side="right"), len(probs) - 1))


class MirostatV1:
    """Mirostat v1: estimate the Zipf exponent from the top ``m`` tokens, pick k so the expected surprise is ``mu``,
    sample from the top k, then move ``mu`` towards the target surprise ``tau``."""

    def __init__(self, tau: float = 5.0, eta: float = 0.1, m: int = 100):
        self.tau, self.eta, self.m = tau, eta, m
        self.mu = 2.0 * tau

    def sample(self, logits: np.ndarray, rng: LcgRng) -> int:
        p = softmax(logits)
        order = np.argsort(-p, kind="stable")
        ps = p[order]
        m = min(self.m, len(ps) - 1)
        num = den = 0.0
        for i in range(max(m, 1)):
            if ps[i + 1] <= 0 or ps[i] <= 0:
                break
            t = math.log((i + 2) / (i + 1))
            b = math.log(ps[i] / ps[i + 1])
            num += t * b
            den += t * t
        s_hat = num / den if den > 0 else 1.0
        eps = s_hat - 1.0
        n = len(ps)
        if abs(eps) < 1e-6:
            k = n
        else:
            k = ((eps * 2.0 ** self.mu) / (1.0 - n ** (-eps))) ** (1.0 / s_hat)
        k = int(min(max(round(k) if math.isfinite(k) else n, 1), n))
        top = ps[:k] / ps[:k].sum()
        j = _draw(top, rng)
        surprise = -math.log2(max(top[j], 1e-30))
        self.mu -= self.eta * (surprise - self.tau)
        return int(order[j])

    def reset(self) -> None:
        self.mu = 2.0 * self.tau


class MirostatV2:
    """Mirostat v2: drop tokens whose surprise exceeds ``mu``, sample, update ``mu``."""

    def __init__(self, tau: float = 5.0, eta: float = 0.1):
        self.tau, self.eta = tau, eta
        self.mu = 2.0 * tau

    def sample(self, logits: np.ndarray, rng: LcgRng) -> int:
        p = softmax(logits)
        surprise = -np.log2(np.maximum(p, 1e-30))
        keep = surprise <= self.mu
        if not keep.any():
            keep[np.argmax(p)] = True
        q = np.where(keep, p, 0.0)
        q /= q.sum()
        j = _draw(q, rng)
        self.mu -= self.eta * (-math.log2(max(q[j], 1e-30)) - self.tau)
        return j

    def reset(self) -> None:
        self.mu = 2.0 * self.tau


@dataclass
class TypicalSampler:
    """Locally typical sampling: keep the tokens whose surprise is closest to the entropy until mass ``p`` is covered."""
    p: float = 0.9
    min_keep: int = 1

    def filter(self, logits: np.ndarray) -> np.ndarray:
        pr = softmax(logits)
        h = entropy(pr)
        dev = np.abs(-np.log(np.maximum(pr, 1e-30)) - h)
        order = np.argsort(dev, kind="stable")
        c = np.cumsum(pr[order])
        n = max(int(np.searchsorted(c, self.p, side="left")) + 1, self.min_keep)
        keep = np.zeros(len(pr), dtype=bool)
        keep[order[:n]] = True
        return keep

    def sample(self, logits: np.ndarray, rng: LcgRng) -> int:
        keep = self.filter(logits)
        q = np.where(keep, softmax(logits), 0.0)
        return _draw(q / q.sum(), rng)


@dataclass
class EtaSampler:
    """Eta sampling: cutoff = min(epsilon, sqrt(epsilon) * exp(-entropy)); tokens below it are dropped."""
    epsilon: float = 3e-4
    delta: float = 1.0     # multiplies the entropy-dependent term

    def filter(self, logits: np.ndarray) -> np.ndarray:
        pr = softmax(logits)
        cutoff = min(self.epsilon, math.sqrt(self.epsilon) * math.exp(-self.delta * entropy(pr)))
        keep = pr >= cutoff
        if not keep.any():
            keep[np.argmax(pr)] = True
        return keep

    def sample(self, logits: np.ndarray, rng: LcgRng) -> int:
        q = np.where(self.filter(logits), softmax(logits), 0.0)
        return _draw(q / q.sum(), rng)


@dataclass
class MinPSampler:
    """Keep tokens with probability >= ``min_p`` x the top probability."""
    min_p: float = 0.05
    min_keep: int = 1

    def filter(self, logits: np.ndarray) -> np.ndarray:
        pr = softmax(logits)
        keep = pr >= self.min_p * pr.max()
        if keep.sum() < self.min_keep:
            keep[top_k_indices(pr, self.min_keep)] = True
        return keep

    def sample(self, logits: np.ndarray, rng: LcgRng) -> int:
        q = np.where(self.filter(logits), softmax(logits), 0.0)
        return _draw(q / q.sum(), rng)


# ---- sampler chain ------------------------------------------------------------------------------------------------
@dataclass
class SamplerStep:
    kind: str                      # temperature | top_k | top_p | min_p | typical | eta | repetition_penalty | greedy
    value: float = 0.0
    extra: float = 0.0


class SamplerChain:
    """Applies filtering steps in order to the logits, then draws; a ``greedy`` step short-circuits to argmax
    (ties resolve to the highest index, like the engine's greedy path)."""

    def __init__(self, seed: int = 42):
        self.steps: list[SamplerStep] = []
        self.rng = LcgRng(seed)
        self.history: list[int] = []

    def add(self, kind: str, value: float = 0.0, extra: float = 0.0) -> "SamplerChain":
        self.steps.append(SamplerStep(kind, value, extra))
        return self

    def sample(self, logits: np.ndarray) -> int:
        x = np.array(logits, dtype=np.float64, copy=True)
        for st in self.steps:
            if st.kind == "greedy":
                tok = int(len(x) - 1 - np.argmax(x[::-1]))
                self.history.append(tok)
                return tok
            if st.kind == "temperature":
                x = apply_temperature(x, st.value)
            elif st.kind == "repetition_penalty":
                x = apply_repetition_penalty(x, self.history, st.value)
            elif st.kind == "top_k" and 0 < st.value < len(x):
                keep = np.zeros(len(x), dtype=bool)
                keep[top_k_indices(x, int(st.value))] = True
                x = np.where(keep, x, -np.inf)
            elif st.kind == "top_p" and st.value < 1.0:
                p = softmax(x)
                order = np.argsort(-p, kind="stable")
                c = np.cumsum(p[order])
                n = int(np.searchsorted(c, st.value, side="right")) + 1
                keep = np.zeros(len(x), dtype=bool)
                keep[order[:n]] = True
                x = np.where(keep, x, -np.inf)
            elif st.kind == "min_p":
                x = np.where(MinPSampler(st.value, max(1, int(st.extra))).filter(x), x, -np.inf)
            elif st.kind == "typical":
                x = np.where(TypicalSampler(st.value, max(1, int(st.extra))).filter(x), x, -np.inf)
            elif st.kind == "eta":
                x = np.where(EtaSampler(st.value, st.extra or 1.0).filter(x), x, -np.inf)
        tok = _draw(softmax(x), self.rng)
        self.history.append(tok)
        return tok

    @classmethod
    def greedy(cls) -> "SamplerChain":
        return cls(0).add("greedy")

    @classmethod
    def default_chat(cls, seed: int = 42) -> "SamplerChain":
        return cls(seed).add("repetition_penalty", 1.1).add("temperature", 0.7).add("top_k", 40).add("top_p", 0.9)

    @classmethod
    def creative(cls, seed: int = 42) -> "SamplerChain":
        return cls(seed).add("temperature", 1.0).add("top_p", 0.95).add("min_p", 0.02)

    @classmethod
    def precise(cls, seed: int = 42) -> "SamplerChain":
        return cls(seed).add("repetition_penalty", 1.2).add("temperature", 0.1).add("top_k", 10).add("top_p", 0.5)


# ---- adaptive strategies ---------------------------------------------------------------------------------------------
@dataclass
class GenerationState:
    tokens: list[int] = field(default_factory=list)
    entropies: deque = field(default_factory=lambda: deque(maxlen=256))
    step: int = 0

    def update(self, token: int, entropy_value: float) -> None:
        self.tokens.append(int(token))
        self.entropies.append(float(entropy_value))
        self.step += 1

    def recent_repetition_rate(self, window: int = 32) -> float:
        w = self.tokens[-window:]
        return 0.0 if len(w) < 2 else 1.0 - len(set(w)) / len(w)

    def mean_recent_entropy(self, window: int = 16) -> float:
        w = list(self.entropies)[-window:]
        return sum(w) / len(w) if w else 0.0


@dataclass
class EntropyCooling:
    """Lower the temperature when recent entropy runs above the target, raise it when below."""
    target_entropy: float = 2.0
    gain: float = 0.1
    min_temp: float = 0.1
    max_temp: float = 1.5

    def adjust(self, state: GenerationState, p: SamplingParams) -> SamplingParams:
        if not state.entropies:
            return p
        err = state.mean_recent_entropy() - self.target_entropy
        return replace(p, temperature=float(min(self.max_temp, max(self.min_temp, p.temperature - self.gain * err))))


@dataclass
class RepetitionAdaptation:
    """Raise the repetition penalty (and a little temperature) when the recent window repeats itself."""
    threshold: float = 0.3
    max_penalty: float = 1.5
    window: int = 32

    def adjust(self, state: GenerationState, p: SamplingParams) -> SamplingParams:
        r = state.recent_repetition_rate(self.window)
        if r <= self.threshold:
            return p
        over = (r - self.threshold) / max(1e-6, 1.0 - self.threshold)
        return replace(p, repetition_penalty=float(min(self.max_penalty, p.repetition_penalty + over * 0.4)),
                       temperature=float(min(2.0, p.temperature + 0.2 * over)))


@dataclass
class ScheduledDecay:
    """Linear temperature decay from ``initial`` to ``final`` over ``steps`` tokens."""
    initial: float = 1.0
    final: float = 0.3
    steps: int = 256

    def temperature_at_step(self, step: int) -> float:
        if self.steps <= 0 or step >= self.steps:
            return self.final
        return self.initial + (self.final - self.initial) * step / self.steps

    def adjust(self, state: GenerationState, p: SamplingParams) -> SamplingParams:
        return replace(p, temperature=self.temperature_at_step(state.step))


class AdaptiveSamplerChain:
    def __init__(self):
        self.strategies: list = []

    def add(self, strategy) -> "AdaptiveSamplerChain":
        self.strategies.append(strategy)
        return self

    def adjust(self, state: GenerationState, base: SamplingParams) -> SamplingParams:
        p = base
        for s in self.strategies:
            p = s.adjust(state, p)
        return p

    def __len__(self) -> int:
        return len(self.strategies)
