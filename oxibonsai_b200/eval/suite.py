"""Evaluation suite, full form: scored results as objects (BLEU with smoothing and corpus aggregation, ROUGE-N / L / S and
corpus ROUGE, chrF / chrF++, METEOR with alignment, QA scores), calibration tables, bootstrap intervals, online counters,
datasets with sampling and splits, and the benchmark evaluators in both their completion-based and logit-based forms.

Reference: crates/oxibonsai-eval - bleu.rs (Papineni BLEU, Chen & Cherry add-one / exponential-decay smoothing, closest
reference length with shortest-reference tie-break), rouge.rs (``tokenize``: lowercase, punctuation stripped from the
ends of words; ROUGE-N with max-recall multi-reference; ROUGE-L; skip-bigram ROUGE-S; macro-averaged ``CorpusRouge``),
chrf.rs (character n-gram F-beta, word n-grams mixed in for chrF++), meteor.rs (exact-match alignment, fragmentation
penalty), qa.rs, calibration.rs (ECE bins, Brier, NLL from logits), bootstrap.rs, streaming.rs (online perplexity /
accuracy), dataset.rs, accuracy.rs (``McEvaluator`` template ``{question}\\nA) {a}...Answer:``, first-letter answer
extraction), mmlu.rs / arc.rs / hellaswag.rs / winogrande.rs / boolq.rs / truthfulqa.rs (MC1 argmax, MC2 probability mass on
the true answers) / gsm8k.rs, throughput.rs, perplexity.rs (``bits_per_byte``), report.rs.  The compact functional forms
(``bleu``, ``rouge``, ``chrf`` ...) stay in the package's ``__init__``.
"""
from __future__ import annotations

import json
import math
import random
import string
import time
from collections import Counter
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Iterable, Sequence

import numpy as np

from . import AccuracyResult, extract_final_number, normalize_answer

# ---- tokens -------------------------------------------------------------------------------------------------------------------
_PUNCT = string.punctuation


def tokenize(text: str) -> list[str]:
    """Lowercased words; punctuation is stripped from both ends of every word, empty words are dropped."""
    return [w for w in (t.strip(_PUNCT).lower() for t in text.split()) if w]


def ngram_counts(tokens: Sequence[str], n: int) -> Counter:
    return Counter(tuple(tokens[i:i + n]) for i in range(len(tokens) - n + 1)) if n > 0 else Counter()


def _f1(p: float, r: float) -> float:
    return 2 * p * r / (p + r) if p + r > 0 else 0.0


# ---- BLEU ---------------------------------------------------------------------------------------------------------------------
class SmoothingMethod(Enum):
    NONE = "none"
    ADD_ONE = "add_one"          # Chen & Cherry method 2: +1 on numerator and denominator of the orders above 1
    EXP_DECAY = "exp_decay"      # method 3: the k-th zero precision becomes 1 / (2^k * candidate length)


@dataclass
class BleuConfig:
    max_n: int = 4
    smoothing: SmoothingMethod = SmoothingMethod.NONE


@dataclass
class BleuScore:
    bleu: float
    precisions: list[float]
    brevity_penalty: float
    length_ratio: float


def _bleu_stats(cand: Sequence[str], refs: Sequence[Sequence[str]], max_n: int):
    matches, totals = [0] * max_n, [0] * max_n
    for n in range(1, max_n + 1):
        cg = ngram_counts(cand, n)
        best: Counter = Counter()
        for r in refs:
            for g, k in ngram_counts(r, n).items():
                if k > best[g]:
                    best[g] = k
        matches[n - 1] = sum(min(k, best[g]) for g, k in cg.items())
        totals[n - 1] = sum(cg.values())
    closest = min(((abs(len(r) - len(cand)), len(r)) for r in refs), default=(0, 0))[1]      # ties go to the shorter reference
    return matches, totals, len(cand), closest


def _bleu_from(matches, totals, c_len: int, r_len: int, cfg: BleuConfig) -> BleuScore:
    if c_len == 0:
        return BleuScore(0.0, [0.0] * cfg.max_n, 0.0, 0.0)
    precisions, zeros = [], 0
    for n, (m, t) in enumerate(zip(matches, totals), 1):
        if cfg.smoothing is SmoothingMethod.ADD_ONE and n > 1:
            m, t = m + 1, t + 1
        if t == 0:
            p = 0.0
        elif m == 0 and cfg.smoothing is SmoothingMethod.EXP_DECAY:
            zeros += 1
            p = 1.0 / (2 ** zeros * c_len)
        else:
            p = m / t
        precisions.append(p)
    bp = 1.0 if c_len > r_len else math.exp(1.0 - r_len / c_len)
    score = 0.0 if min(precisions) <= 0 else bp * math.exp(sum(math.log(p) for p in precisions) / cfg.max_n)
    return BleuScore(score, precisions, bp, c_len / r_len if r_len else 0.0)


def sentence_bleu_tokens(candidate: Sequence[str], references: Sequence[Sequence[str]], config: BleuConfig | None = None) -> BleuScore:
    cfg = config or BleuConfig()
    return _bleu_from(*_bleu_stats(candidate, references, cfg.max_n), cfg)


def sentence_bleu(candidate: str, references: Sequence[str], config: BleuConfig | None = None) -> BleuScore:
    return sentence_bleu_tokens(tokenize(candidate), [tokenize(r) for r in references], config)


def corpus_bleu_tokens(candidates: Sequence[Sequence[str]], references: Sequence[Sequence[Sequence[str]]], config: BleuConfig | None = None) -> BleuScore:
    """Counts are summed over the corpus before the precisions are formed (not an average of sentence scores)."""
    cfg = config or BleuConfig()
    M, T, C, R = [0] * cfg.max_n, [0] * cfg.max_n, 0, 0
    for cand, refs in zip(candidates, references):
        m, t, c, r = _bleu_stats(cand, refs, cfg.max_n)
        M, T, C, R = [a + b for a, b in zip(M, m)], [a + b for a, b in zip(T, t)], C + c, R + r
    return _bleu_from(M, T, C, R, cfg)


def corpus_bleu(candidates: Sequence[str], references: Sequence[Sequence[str]], config: BleuConfig | None = None) -> BleuScore:
    return corpus_bleu_tokens([tokenize(c) for c in candidates], [[tokenize(r) for r in refs] for refs in references], config)


# ---- ROUGE --------------------------------------------------------------------------------------------------------------------
@dataclass
class RougeNScore:
    n: int
    precision: float
    recall: float
    f1: float

    @classmethod
    def from_tokens(cls, cand: Sequence[str], ref: Sequence[str], n: int) -> "RougeNScore":
        cg, rg = ngram_counts(cand, n), ngram_counts(ref, n)
        if not cg or not rg:
            return cls(n, 0.0, 0.0, 0.0)
        overlap = sum((cg & rg).values())
        p, r = overlap / sum(cg.values()), overlap / sum(rg.values())
        return cls(n, p, r, _f1(p, r))

    @classmethod
    def compute(cls, candidate: str, reference: str, n: int) -> "RougeNScore":
        return cls.from_tokens(tokenize(candidate), tokenize(reference), n)

    @classmethod
    def compute_multi_ref(cls, candidate: str, references: Sequence[str], n: int) -> "RougeNScore":
        """Every reference is scored on its own; the one with the highest recall is reported."""
        best = cls(n, 0.0, 0.0, 0.0)
        for ref in references:
            s = cls.compute(candidate, ref, n)
            if s.recall > best.recall:
                best = s
        return best


def lcs_length(a: Sequence, b: Sequence) -> int:
    from . import _lcs
    return _lcs(a, b)


@dataclass
class RougeLScore:
    precision: float
    recall: float
    f1: float
    lcs_length: int

    @classmethod
    def compute(cls, candidate: str, reference: str) -> "RougeLScore":
        c, r = tokenize(candidate), tokenize(reference)
        if not c or not r:
            return cls(0.0, 0.0, 0.0, 0)
        l = lcs_length(c, r)
        p, rc = l / len(c), l / len(r)
        return cls(p, rc, _f1(p, rc), l)


def skip_bigrams(tokens: Sequence[str]) -> Counter:
    """All ordered pairs of a sentence, n (n - 1) / 2 of them, with multiplicity."""
    return Counter((tokens[i], tokens[j]) for i in range(len(tokens)) for j in range(i + 1, len(tokens)))


@dataclass
class RougeSScore:
    precision: float
    recall: float
    f1: float

    @classmethod
    def compute(cls, candidate: str, reference: str) -> "RougeSScore":
        cg, rg = skip_bigrams(tokenize(candidate)), skip_bigrams(tokenize(reference))
        if not cg or not rg:
            return cls(0.0, 0.0, 0.0)
        overlap = sum((cg & rg).values())
        p, r = overlap / sum(cg.values()), overlap / sum(rg.values())
        return cls(p, r, _f1(p, r))


@dataclass
class CorpusRouge:
    rouge_1: RougeNScore | None
    rouge_2: RougeNScore | None
    rouge_l: RougeLScore | None
    num_samples: int

    @classmethod
    def compute(cls, pairs: Sequence[tuple[str, str]]) -> "CorpusRouge":
        """Macro average of the per-pair scores."""
        if not pairs:
            return cls(None, None, None, 0)
        r1 = [RougeNScore.compute(c, r, 1) for c, r in pairs]
        r2 = [RougeNScore.compute(c, r, 2) for c, r in pairs]
        rl = [RougeLScore.compute(c, r) for c, r in pairs]
        mean = lambda xs, a: sum(getattr(x, a) for x in xs) / len(xs)
        return cls(RougeNScore(1, mean(r1, "precision"), mean(r1, "recall"), mean(r1, "f1")),
                   RougeNScore(2, mean(r2, "precision"), mean(r2, "recall"), mean(r2, "f1")),
                   RougeLScore(mean(rl, "precision"), mean(rl, "recall"), mean(rl, "f1"), round(mean(rl, "lcs_length"))), len(pairs))

    def summary(self) -> str:
        if not self.num_samples:
            return "ROUGE: no samples"
        return f"ROUGE-1 F1 {self.rouge_1.f1:.4f} | ROUGE-2 F1 {self.rouge_2.f1:.4f} | ROUGE-L F1 {self.rouge_l.f1:.4f} ({self.num_samples} samples)"


# ---- chrF ---------------------------------------------------------------------------------------------------------------------
@dataclass
class ChrfScore:
    score: float
    order: int
    beta: float
    word_order: int


def chrf_with(candidate: str, reference: str, order: int = 6, beta: float = 2.0, word_order: int = 0) -> ChrfScore:
    """Mean F-beta over character n-grams up to ``order`` (white space removed) and, for chrF++, word n-grams up to
    ``word_order``.  Orders for which either side has no n-gram are left out of the mean."""
    fs = []

    def add(cg: Counter, rg: Counter) -> None:
        if not cg or not rg:
            return
        m = sum((cg & rg).values())
        p, r = m / sum(cg.values()), m / sum(rg.values())
        fs.append((1 + beta * beta) * p * r / (beta * beta * p + r) if p + r > 0 else 0.0)
    c, r = "".join(candidate.split()), "".join(reference.split())
    for n in range(1, order + 1):
        add(ngram_counts(c, n), ngram_counts(r, n))
    cw, rw = candidate.split(), reference.split()
    for n in range(1, word_order + 1):
        add(ngram_counts(cw, n), ngram_counts(rw, n))
    return ChrfScore(sum(fs) / len(fs) if fs else 0.0, order, beta, word_order)


def chrf_score(candidate: str, reference: str) -> ChrfScore:
    return chrf_with(candidate, reference, 6, 2.0, 0)


def chrf_plus_plus(candidate: str, reference: str) -> ChrfScore:
    return chrf_with(candidate, reference, 6, 2.0, 2)


# ---- METEOR -------------------------------------------------------------------------------------------------------------------
@dataclass
class MeteorConfig:
    alpha: float = 0.9
    beta: float = 3.0
    gamma: float = 0.5


@dataclass
class MeteorScore:
    score: float
    precision: float
    recall: float
    fragmentation: float


def align_tokens(candidate: Sequence[str], reference: Sequence[str]) -> list[tuple[int, int]]:
    """Exact-match alignment: every candidate word takes the first unused equal reference word."""
    used, out = set(), []
    for i, w in enumerate(candidate):
        for j, v in enumerate(reference):
            if j not in used and w == v:
                used.add(j)
                out.append((i, j))
                break
    return out


def meteor_tokens(candidate: Sequence[str], reference: Sequence[str], config: MeteorConfig | None = None) -> MeteorScore:
    cfg = config or MeteorConfig()
    if not candidate or not reference:
        return MeteorScore(0.0, 0.0, 0.0, 0.0)
    al = align_tokens(candidate, reference)
    m = len(al)
    if m == 0:
        return MeteorScore(0.0, 0.0, 0.0, 0.0)
    p, r = m / len(candidate), m / len(reference)
    fmean = p * r / (cfg.alpha * p + (1 - cfg.alpha) * r)
    chunks = 1 + sum(1 for (i0, j0), (i1, j1) in zip(al, al[1:]) if not (i1 == i0 + 1 and j1 == j0 + 1))
    frag = chunks / m
    return MeteorScore(fmean * (1 - cfg.gamma * frag ** cfg.beta), p, r, frag)


def meteor_score(candidate: str, reference: str, config: MeteorConfig | None = None) -> MeteorScore:
    return meteor_tokens(tokenize(candidate), tokenize(reference), config)


def meteor_multi(candidate: str, references: Sequence[str], config: MeteorConfig | None = None) -> MeteorScore:
    """The best score over the references."""
    return max((meteor_score(candidate, r, config) for r in references), key=lambda s: s.score, default=MeteorScore(0.0, 0.0, 0.0, 0.0))


# ---- extractive QA ------------------------------------------------------------------------------------------------------------
@dataclass
class QaScore:
    exact_match: float
    f1: float


def normalize_tokens(text: str) -> list[str]:
    return normalize_answer(text).split()


def f1_score(prediction: str, gold: str) -> float:
    p, g = normalize_tokens(prediction), normalize_tokens(gold)
    if not p or not g:
        return float(p == g)
    common = sum((Counter(p) & Counter(g)).values())
    return _f1(common / len(p), common / len(g)) if common else 0.0


def score_multi(prediction: str, golds: Sequence[str]) -> QaScore:
    """Best exact match and best F1 over the gold answers (SQuAD protocol)."""
    return QaScore(float(any(normalize_answer(prediction) == normalize_answer(g) for g in golds)), max((f1_score(prediction, g) for g in golds), default=0.0))


def corpus_em_f1(predictions: Sequence[str], golds: Sequence[Sequence[str]]) -> QaScore:
    scores = [score_multi(p, g) for p, g in zip(predictions, golds)]
    n = len(scores)
    return QaScore(sum(s.exact_match for s in scores) / n, sum(s.f1 for s in scores) / n) if n else QaScore(0.0, 0.0)


# ---- calibration, bootstrap ---------------------------------------------------------------------------------------------------
@dataclass
class BinStat:
    lo: float
    hi: float
    count: int
    avg_confidence: float
    avg_accuracy: float


@dataclass
class CalibrationResult:
    ece: float
    brier: float
    nll: float
    bin_stats: list[BinStat]


def nll_from_logits(logits: Sequence[Sequence[float]], labels: Sequence[int]) -> float:
    """Mean negative log-likelihood of the labels under softmax(logits)."""
    total, n = 0.0, 0
    for row, y in zip(logits, labels):
        z = np.asarray(row, dtype=np.float64)
        if z.size == 0 or not 0 <= y < z.size:
            continue
        total += float(np.log(np.exp(z - z.max()).sum()) + z.max() - z[y])
        n += 1
    return total / n if n else 0.0


def calibration_all(confidences: Sequence[float], outcomes: Sequence[int], n_bins: int = 10, probs_of_truth: Sequence[float] | None = None) -> CalibrationResult:
    """ECE over equal-width confidence bins with the table of bins, Brier score of the confidences, and the NLL of
    ``probs_of_truth`` (defaults to the confidence where the prediction was right, its complement where it was wrong)."""
    c, o = np.asarray(confidences, dtype=np.float64), np.asarray(outcomes, dtype=np.float64)
    bins, ece = [], 0.0
    idx = np.minimum((c * n_bins).astype(int), n_bins - 1) if c.size else np.zeros(0, dtype=int)
    for b in range(n_bins):
        m = idx == b
        k = int(m.sum())
        conf, acc = (float(c[m].mean()), float(o[m].mean())) if k else (0.0, 0.0)
        bins.append(BinStat(b / n_bins, (b + 1) / n_bins, k, conf, acc))
        if k:
            ece += k / c.size * abs(acc - conf)
    pt = np.asarray(probs_of_truth, dtype=np.float64) if probs_of_truth is not None else np.where(o > 0, c, 1.0 - c)
    nll = float(-np.log(np.clip(pt, 1e-12, 1.0)).mean()) if pt.size else 0.0
    brier = float(((c - o) ** 2).mean()) if c.size else 0.0
    return CalibrationResult(float(ece), brier, nll, bins)


@dataclass
class ConfidenceInterval:
    lo: float
    hi: float
    mean: float
    confidence: float
    n_resamples: int

    def contains(self, x: float) -> bool:
        return self.lo <= x <= self.hi

    @property
    def width(self) -> float:
        return self.hi - self.lo


def bootstrap_interval(values: Sequence[float], n_resamples: int = 1000, confidence: float = 0.95, seed: int = 0) -> ConfidenceInterval:
    """Percentile bootstrap of the mean; deterministic for a seed."""
    v = np.asarray(values, dtype=np.float64)
    if v.size == 0:
        return ConfidenceInterval(0.0, 0.0, 0.0, confidence, n_resamples)
    rng = np.random.default_rng(seed)
    means = v[rng.integers(0, v.size, (n_resamples, v.size))].mean(axis=1)
    lo, hi = np.quantile(means, [(1 - confidence) / 2, 1 - (1 - confidence) / 2])
    return ConfidenceInterval(float(lo), float(hi), float(v.mean()), confidence, n_resamples)


# ---- online counters ----------------------------------------------------------------------------------------------------------
class OnlinePerplexity:
    """Perplexity of a stream of token log-probabilities (natural log) without keeping them."""

    def __init__(self):
        self.reset()

    def reset(self) -> None:
        self._sum, self._n = 0.0, 0

    def push(self, log_prob: float) -> None:
        self._sum += float(log_prob)
        self._n += 1

    def push_chunk(self, log_probs: Iterable[float]) -> None:
        for lp in log_probs:
            self.push(lp)

    def tokens(self) -> int:
        return self._n

    def current(self) -> float:
        return math.exp(-self._sum / self._n) if self._n else float("inf")


class OnlineAccuracy:
    def __init__(self):
        self.reset()

    def reset(self) -> None:
        self._correct = self._total = 0

    def push(self, correct: bool) -> None:
        self._correct += int(bool(correct))
        self._total += 1

    def push_many(self, outcomes: Iterable[bool]) -> None:
        for o in outcomes:
            self.push(o)

    def counts(self) -> tuple[int, int]:
        return self._correct, self._total

    def current(self) -> float:
        return self._correct / self._total if self._total else 0.0
