"""Datasets and benchmark evaluators in their completion-based and logit-based forms, throughput statistics, perplexity
helpers and the report builders.

Reference: crates/oxibonsai-eval - dataset.rs (``EvalDataset``: JSONL round trip, seeded sampling, ordered train / test
split; ``McDataset``: subject filter, sorted subject list), accuracy.rs (``McEvaluator``: template with ``{question}``,
``{a}``..``{d}``, label prefixes such as ``"A: "`` stripped from the choices, the first letter of a completion is the
answer; ``McLogitEvaluator``: argmax over per-choice scores; ``ExactMatchEvaluator``), mmlu.rs (per-subject results), arc.rs
(easy / challenge splits), hellaswag.rs, winogrande.rs (answer 1 / 2), boolq.rs (``Passage: ..\\nQuestion: ..\\nAnswer:``;
a completion answers yes / no by its first characters), truthfulqa.rs (MC1: argmax; MC2: probability mass on the true
answers), gsm8k.rs (the number after the last ``####``), throughput.rs, perplexity.rs, report.rs.
"""
from __future__ import annotations

import json
import math
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable, Sequence

import numpy as np

from . import AccuracyResult


# ---- deterministic sampling ---------------------------------------------------------------------------------------------------
def _lcg_order(n: int, seed: int) -> list[int]:
    """Fisher-Yates shuffle of range(n) driven by a 64-bit linear congruential generator: the same order on every
    platform for a seed."""
    state = (seed ^ 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    order = list(range(n))
    for i in range(n - 1, 0, -1):
        state = (state * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        j = (state >> 33) % (i + 1)
        order[i], order[j] = order[j], order[i]
    return order


# ---- datasets -----------------------------------------------------------------------------------------------------------------
@dataclass
class EvalExample:
    id: str
    input: str
    expected_output: str | None = None
    metadata: dict = field(default_factory=dict)


class EvalDataset:
    def __init__(self, name: str, examples: Iterable[EvalExample] = ()):
        self.name, self.examples = name, list(examples)

    def add(self, example: EvalExample) -> None:
        self.examples.append(example)

    def __len__(self) -> int:
        return len(self.examples)

    def is_empty(self) -> bool:
        return not self.examples

    @classmethod
    def from_jsonl(cls, name: str, text: str) -> "EvalDataset":
        """One JSON object per line (``id``, ``input``, optional ``expected_output`` and ``metadata``); blank lines are
        skipped, a malformed line raises ``ValueError`` with its number."""
        ds = cls(name)
        for n, line in enumerate(text.splitlines(), 1):
            if not line.strip():
                continue
            try:
                row = json.loads(line)
                ds.add(EvalExample(str(row.get("id", n)), row["input"], row.get("expected_output"), dict(row.get("metadata") or {})))
            except (json.JSONDecodeError, KeyError, TypeError) as e:
                raise ValueError(f"{name}: line {n}: {e}") from None
        return ds

    def to_jsonl(self) -> str:
        return "".join(json.dumps({"id": e.id, "input": e.input, "expected_output": e.expected_output, "metadata": e.metadata}, ensure_ascii=False) + "\n"
                       for e in self.examples)

    def sample(self, n: int, seed: int = 0) -> "EvalDataset":
        order = _lcg_order(len(self.examples), seed)
        return EvalDataset(self.name, [self.examples[i] for i in order[:max(0, n)]])

    sample_with_seed = sample

    def split(self, train_ratio: float) -> tuple["EvalDataset", "EvalDataset"]:
        """The first floor(len * ratio) examples train, the rest test; order kept."""
        k = int(math.floor(len(self.examples) * min(max(train_ratio, 0.0), 1.0)))
        return EvalDataset(self.name + "-train", self.examples[:k]), EvalDataset(self.name + "-test", self.examples[k:])


@dataclass
class MultipleChoiceQuestion:
    id: str
    question: str
    choices: list[str]
    correct_answer: int
    subject: str | None = None
    difficulty: str | None = None


class McDataset:
    def __init__(self, name: str, questions: Iterable[MultipleChoiceQuestion] = ()):
        self.name, self.questions = name, list(questions)

    def add(self, q: MultipleChoiceQuestion) -> None:
        self.questions.append(q)

    def __len__(self) -> int:
        return len(self.questions)

    def is_empty(self) -> bool:
        return not self.questions

    @classmethod
    def from_jsonl(cls, name: str, text: str) -> "McDataset":
        ds = cls(name)
        for n, line in enumerate(text.splitlines(), 1):
            if not line.strip():
                continue
            try:
                r = json.loads(line)
                ans = r["correct_answer"] if "correct_answer" in r else r["answer"]
                ans = "ABCDEFGH".index(ans.strip().upper()) if isinstance(ans, str) else int(ans)
                ds.add(MultipleChoiceQuestion(str(r.get("id", n)), r["question"], list(r["choices"]), ans, r.get("subject"), r.get("difficulty")))
            except (json.JSONDecodeError, KeyError, TypeError, ValueError) as e:
                raise ValueError(f"{name}: line {n}: {e}") from None
        return ds

    def filter_by_subject(self, subject: str) -> "McDataset":
        return McDataset(self.name, [q for q in self.questions if q.subject == subject])

    def sample_with_seed(self, n: int, seed: int = 0) -> "McDataset":
        order = _lcg_order(len(self.questions), seed)
        return McDataset(self.name, [self.questions[i] for i in order[:max(0, n)]])

    def subjects(self) -> list[str]:
        return sorted({q.subject for q in self.questions if q.subject})


# ---- multiple choice ----------------------------------------------------------------------------------------------------------
MC_TEMPLATE = "{question}\nA) {a}\nB) {b}\nC) {c}\nD) {d}\nAnswer:"


def _accuracy(pairs: Iterable[tuple[bool, str | None]]) -> AccuracyResult:
    r = AccuracyResult(0, 0)
    for ok, group in pairs:
        r.correct += int(ok)
        r.total += 1
        r.outcomes.append(int(ok))
        if group is not None:
            c, t = r.by_group.get(group, (0, 0))
            r.by_group[group] = (c + int(ok), t + 1)
    return r


def accuracy_pct(r: AccuracyResult) -> float:
    return 100.0 * r.accuracy


class McEvaluator:
    """Completion-based: the prompt is the template filled in, the model's first letter is its answer."""

    def __init__(self, template: str = MC_TEMPLATE):
        self.prompt_template = template

    @classmethod
    def with_template(cls, template: str) -> "McEvaluator":
        return cls(template)

    def format_question(self, q: MultipleChoiceQuestion) -> str:
        def choice(i: int) -> str:
            s = q.choices[i] if i < len(q.choices) else ""
            return s[2:].strip() if len(s) >= 3 and s[1] == ":" else s          # "A: text" -> "text"
        out = self.prompt_template.replace("{question}", q.question)
        for i, key in enumerate("abcd"):
            out = out.replace("{" + key + "}", choice(i))
        return out

    @staticmethod
    def extract_answer(completion: str) -> int | None:
        s = completion.strip()
        return "ABCD".index(s[0].upper()) if s and s[0].upper() in "ABCD" else None

    def score_completion(self, completion: str, correct_answer: int) -> bool:
        return self.extract_answer(completion) == correct_answer

    def evaluate_dataset(self, dataset: McDataset, completions: Sequence[str]) -> AccuracyResult:
        return _accuracy((self.score_completion(c, q.correct_answer), q.subject) for q, c in zip(dataset.questions, completions))


@dataclass
class LogitMcResult:
    predicted: int
    correct: bool
    margin: float            # best score minus the runner-up


class McLogitEvaluator:
    """Logit-based: one score per choice (a log-probability of the choice's text or letter), the largest wins."""

    def __init__(self, template: str = MC_TEMPLATE):
        self.prompt_template = template

    @staticmethod
    def score(choice_scores: Sequence[float], correct_answer: int) -> LogitMcResult:
        s = np.asarray(choice_scores, dtype=np.float64)
        if s.size == 0:
            return LogitMcResult(-1, False, 0.0)
        pred = int(np.argmax(s))
        rest = np.delete(s, pred)
        return LogitMcResult(pred, pred == correct_answer, float(s[pred] - rest.max()) if rest.size else 0.0)

    def evaluate_dataset(self, dataset: McDataset, per_choice_scores: Sequence[Sequence[float]]) -> AccuracyResult:
        return _accuracy((self.score(s, q.correct_answer).correct, q.subject) for q, s in zip(dataset.questions, per_choice_scores))


class ExactMatchEvaluator:
    def __init__(self, case_sensitive: bool = False, strip: bool = True):
        self.case_sensitive, self.strip = case_sensitive, strip

    def _norm(self, s: str) -> str:
        s = s.strip() if self.strip else s
        return s if self.case_sensitive else s.lower()

    def score(self, completion: str, expected: str) -> bool:
        return self._norm(completion) == self._norm(expected)

    def evaluate_dataset(self, dataset: EvalDataset, completions: Sequence[str]) -> AccuracyResult:
        return _accuracy((e.expected_output is not None and self.score(c, e.expected_output), None) for e, c in zip(dataset.examples, completions))


# ---- MMLU, ARC ----------------------------------------------------------------------------------------------------------------
@dataclass
class MmluResult:
    accuracy: float
    accuracy_pct: float
    correct: int
    total: int
    by_subject: dict[str, AccuracyResult]


class MmluEvaluator:
    def __init__(self):
        self.mc, self.logit = McEvaluator(), McLogitEvaluator()

    def evaluate_completions(self, dataset: McDataset, completions: Sequence[str]) -> AccuracyResult:
        return self.mc.evaluate_dataset(dataset, completions)

    def evaluate_logits(self, dataset: McDataset, scores: Sequence[Sequence[float]]) -> AccuracyResult:
        return self.logit.evaluate_dataset(dataset, scores)

    def _by_subject(self, dataset: McDataset, judged: list[bool]) -> MmluResult:
        by: dict[str, AccuracyResult] = {}
        for q, ok in zip(dataset.questions, judged):
            r = by.setdefault(q.subject or "", AccuracyResult(0, 0))
            r.correct += int(ok)
            r.total += 1
        c, t = sum(judged), len(judged)
        return MmluResult(c / t if t else 0.0, 100.0 * c / t if t else 0.0, c, t, by)

    def evaluate_by_subject_completions(self, dataset: McDataset, completions: Sequence[str]) -> MmluResult:
        return self._by_subject(dataset, [self.mc.score_completion(c, q.correct_answer) for q, c in zip(dataset.questions, completions)])

    def evaluate_by_subject_logits(self, dataset: McDataset, scores: Sequence[Sequence[float]]) -> MmluResult:
        return self._by_subject(dataset, [self.logit.score(s, q.correct_answer).correct for q, s in zip(dataset.questions, scores)])


@dataclass
class ArcResult:
    split: str
    accuracy: float
    correct: int
    total: int

    @classmethod
    def from_accuracy_result(cls, split: str, r: AccuracyResult) -> "ArcResult":
        return cls(split, r.accuracy, r.correct, r.total)

    def accuracy_pct(self) -> float:
        return 100.0 * self.accuracy

    def split_name(self) -> str:
        return self.split


class ArcEvaluator:
    def __init__(self, split: str):
        self._split, self.mc, self.logit = split, McEvaluator(), McLogitEvaluator()

    @classmethod
    def easy(cls) -> "ArcEvaluator":
        return cls("ARC-Easy")

    @classmethod
    def challenge(cls) -> "ArcEvaluator":
        return cls("ARC-Challenge")

    def split(self) -> str:
        return self._split

    def evaluate_completions(self, dataset: McDataset, completions: Sequence[str]) -> ArcResult:
        return ArcResult.from_accuracy_result(self._split, self.mc.evaluate_dataset(dataset, completions))

    def evaluate_logits(self, dataset: McDataset, scores: Sequence[Sequence[float]]) -> ArcResult:
        return ArcResult.from_accuracy_result(self._split, self.logit.evaluate_dataset(dataset, scores))


# ---- HellaSwag, WinoGrande, BoolQ, TruthfulQA ---------------------------------------------------------------------------------
@dataclass
class HellaSwagItem:
    id: str
    activity_label: str
    ctx: str
    endings: list[str]
    label: int


class HellaSwagDataset:
    def __init__(self, items: Iterable[HellaSwagItem] = ()):
        self.items = list(items)

    from_items = classmethod(lambda cls, items: cls(items))

    @classmethod
    def from_jsonl(cls, text: str) -> "HellaSwagDataset":
        rows = [json.loads(l) for l in text.splitlines() if l.strip()]
        return cls(HellaSwagItem(str(r.get("ind", r.get("id", i))), r.get("activity_label", ""), r.get("ctx") or (r["ctx_a"] + " " + r.get("ctx_b", "")).strip(),
                                 list(r["endings"]), int(r["label"])) for i, r in enumerate(rows))

    def __len__(self) -> int:
        return len(self.items)

    def is_empty(self) -> bool:
        return not self.items

    def as_mc_dataset(self) -> McDataset:
        return McDataset("hellaswag", [MultipleChoiceQuestion(it.id, it.ctx, list(it.endings), it.label, it.activity_label or None) for it in self.items])


class HellaSwagEvaluator:
    def __init__(self):
        self.mc, self.logit = McEvaluator(), McLogitEvaluator()

    def evaluate_completions(self, dataset: HellaSwagDataset, completions: Sequence[str]) -> AccuracyResult:
        return self.mc.evaluate_dataset(dataset.as_mc_dataset(), completions)

    def evaluate_logits(self, dataset: HellaSwagDataset, scores: Sequence[Sequence[float]], length_normalize: bool = False) -> AccuracyResult:
        """``length_normalize``: divide every ending's log-probability by its length in characters (the acc_norm protocol)."""
        if length_normalize:
            scores = [[s / max(1, len(e)) for s, e in zip(row, it.endings)] for row, it in zip(scores, dataset.items)]
        return self.logit.evaluate_dataset(dataset.as_mc_dataset(), scores)


@dataclass
class WinoGrandeItem:
    sentence: str
    option1: str
    option2: str
    answer: int              # 1 or 2


class WinoGrandeDataset:
    def __init__(self, items: Iterable[WinoGrandeItem] = ()):
        self.items = list(items)

    from_items = classmethod(lambda cls, items: cls(items))

    def __len__(self) -> int:
        return len(self.items)

    def is_empty(self) -> bool:
        return not self.items

    def as_mc_dataset(self) -> McDataset:
        return McDataset("winogrande", [MultipleChoiceQuestion(str(i), it.sentence, [it.option1, it.option2], it.answer - 1) for i, it in enumerate(self.items)])


class WinoGrandeEvaluator:
    def __init__(self):
        self.mc, self.logit = McEvaluator("{question}\nA) {a}\nB) {b}\nAnswer:"), McLogitEvaluator()

    def build_prompt(self, item: WinoGrandeItem) -> str:
        return self.mc.format_question(MultipleChoiceQuestion("", item.sentence, [item.option1, item.option2], 0))

    @staticmethod
    def fill(item: WinoGrandeItem, option: int) -> str:
        """The sentence with its blank replaced by option 1 or 2 (for scoring whole sentences)."""
        return item.sentence.replace("_", item.option1 if option == 1 else item.option2, 1)

    def evaluate_completions(self, dataset: WinoGrandeDataset, completions: Sequence[str]) -> AccuracyResult:
        return self.mc.evaluate_dataset(dataset.as_mc_dataset(), completions)

    def evaluate_logits(self, dataset: WinoGrandeDataset, scores: Sequence[Sequence[float]]) -> AccuracyResult:
        return self.logit.evaluate_dataset(dataset.as_mc_dataset(), scores)


@dataclass
class BoolQItem:
    passage: str
    question: str
    answer: bool


class BoolQDataset:
    def __init__(self, items: Iterable[BoolQItem] = ()):
        self.items = list(items)

    from_items = classmethod(lambda cls, items: cls(items))

    def __len__(self) -> int:
        return len(self.items)

    def is_empty(self) -> bool:
        return not self.items


@dataclass
class BoolQResult:
    accuracy: float
    accuracy_pct: float
    correct: int
    total: int
    yes_predicted: int
    no_predicted: int


class BoolQEvaluator:
    @staticmethod
    def build_prompt(item: BoolQItem) -> str:
        return f"Passage: {item.passage}\nQuestion: {item.question}\nAnswer:"

    @staticmethod
    def extract_answer(completion: str) -> bool | None:
        s = completion.lstrip()[:3].lower()
        if s == "yes":
            return True
        if s.startswith("no"):
            return False
        return None

    def score(self, completion: str, gold: bool) -> bool:
        return self.extract_answer(completion) is gold

    def _result(self, preds: list[bool | None], golds: list[bool]) -> BoolQResult:
        c, t = sum(p is g for p, g in zip(preds, golds)), len(preds)
        return BoolQResult(c / t if t else 0.0, 100.0 * c / t if t else 0.0, c, t, sum(p is True for p in preds), sum(p is False for p in preds))

    def evaluate_completions(self, dataset: BoolQDataset, completions: Sequence[str]) -> BoolQResult:
        n = min(len(dataset), len(completions))
        return self._result([self.extract_answer(c) for c in completions[:n]], [it.answer for it in dataset.items[:n]])

    def evaluate_logits(self, dataset: BoolQDataset, yes_no_scores: Sequence[tuple[float, float]]) -> BoolQResult:
        """``(score of "yes", score of "no")`` per item; the larger one is the prediction (a tie predicts "no")."""
        n = min(len(dataset), len(yes_no_scores))
        return self._result([y > no for y, no in yes_no_scores[:n]], [it.answer for it in dataset.items[:n]])


@dataclass
class TruthfulQaItem:
    question: str
    mc1_correct_idx: int
    mc1_choices: list[str]
    mc2_correct_indices: list[int]
    mc2_choices: list[str]


class TruthfulQaDataset:
    def __init__(self, items: Iterable[TruthfulQaItem] = ()):
        self.items = list(items)

    from_items = classmethod(lambda cls, items: cls(items))

    @classmethod
    def from_jsonl(cls, text: str) -> "TruthfulQaDataset":
        """Rows in the shape of the public release: ``mc1_targets`` / ``mc2_targets`` with ``choices`` and 0/1 ``labels``."""
        items = []
        for line in text.splitlines():
            if not line.strip():
                continue
            r = json.loads(line)
            m1, m2 = r["mc1_targets"], r.get("mc2_targets") or r["mc1_targets"]
            items.append(TruthfulQaItem(r["question"], int(np.argmax(m1["labels"])), list(m1["choices"]),
                                        [i for i, l in enumerate(m2["labels"]) if l], list(m2["choices"])))
        return cls(items)

    def __len__(self) -> int:
        return len(self.items)

    def is_empty(self) -> bool:
        return not self.items


@dataclass
class TruthfulQaResult:
    mode: str
    accuracy: float
    accuracy_pct: float
    correct: int
    total: int


class TruthfulQaEvaluator:
    def __init__(self, mode: str):
        assert mode in ("mc1", "mc2")
        self.mode = mode

    @classmethod
    def mc1(cls) -> "TruthfulQaEvaluator":
        return cls("mc1")

    @classmethod
    def mc2(cls) -> "TruthfulQaEvaluator":
        return cls("mc2")

    def evaluate_logits(self, dataset: TruthfulQaDataset, per_choice_logits: Sequence[Sequence[float]]) -> TruthfulQaResult:
        """MC1: the argmax must be the one true answer.  MC2: an item scores the softmax mass on its true answers, the
        result is the mean of those scores (``correct`` counts items with more than half of the mass on the truth).  Rows
        whose length does not match the item's choices score nothing."""
        total, correct, mass = 0, 0, 0.0
        for it, row in zip(dataset.items, per_choice_logits):
            total += 1
            z = np.asarray(row, dtype=np.float64)
            if self.mode == "mc1":
                if z.size == len(it.mc1_choices) and z.size and int(np.argmax(z)) == it.mc1_correct_idx:
                    correct += 1
                continue
            if z.size != len(it.mc2_choices) or not z.size:
                continue
            p = np.exp(z - z.max())
            p /= p.sum()
            s = float(p[[i for i in it.mc2_correct_indices if 0 <= i < z.size]].sum())
            mass += s
            correct += int(s > 0.5)
        acc = (correct / total if self.mode == "mc1" else mass / total) if total else 0.0
        return TruthfulQaResult(self.mode, acc, 100.0 * acc, correct, total)


# ---- GSM8K --------------------------------------------------------------------------------------------------------------------
@dataclass
class Gsm8kResult:
    correct: int
    total: int
    accuracy: float
    no_answer_extracted: int

    def accuracy_pct(self) -> float:
        return 100.0 * self.accuracy

    def no_answer_rate(self) -> float:
        return self.no_answer_extracted / self.total if self.total else 0.0


def gsm8k_example(question: str, reasoning: str, answer: float | int) -> EvalExample:
    """An example in the corpus' own answer format: free reasoning, then ``#### <number>``."""
    return EvalExample("", question, f"{reasoning}\n#### {answer}")


class Gsm8kAnswerEvaluator:
    """Scores completions by the number after their last ``####`` marker."""

    def __init__(self, tolerance: float = 1e-6):
        self.tolerance = tolerance

    @staticmethod
    def extract_final_answer(text: str) -> float | None:
        pos = text.rfind("####")
        if pos < 0:
            return None
        tail = text[pos + 4:].strip().replace(",", "")
        tail = tail.split()[0] if tail.split() else ""
        try:
            return float(tail)
        except ValueError:
            return None

    def score(self, completion: str, expected: str) -> bool:
        a, b = self.extract_final_answer(completion), self.extract_final_answer(expected)
        return a is not None and b is not None and abs(a - b) <= self.tolerance

    def evaluate_dataset(self, dataset: EvalDataset, completions: Sequence[str]) -> Gsm8kResult:
        correct = total = missing = 0
        for e, c in zip(dataset.examples, completions):
            total += 1
            if self.extract_final_answer(c) is None:
                missing += 1
            elif e.expected_output is not None and self.score(c, e.expected_output):
                correct += 1
        return Gsm8kResult(correct, total, correct / total if total else 0.0, missing)


# ---- throughput ---------------------------------------------------------------------------------------------------------------
def time_fn(f: Callable[[], Any]) -> tuple[Any, float]:
    """(result, seconds)."""
    t = time.perf_counter()
    out = f()
    return out, time.perf_counter() - t


def percentile(values: Sequence[float], p: float) -> float:
    """p in [0, 100], linear interpolation between neighbours, 0.0 for no values."""
    if not values:
        return 0.0
    v = sorted(values)
    idx = min(max(p, 0.0), 100.0) / 100.0 * (len(v) - 1)
    lo = int(math.floor(idx))
    hi = min(lo + 1, len(v) - 1)
    return v[lo] * (1 - (idx - lo)) + v[hi] * (idx - lo)


@dataclass
class ThroughputStats:
    tokens_per_second: float
    prefill_ms: float
    decode_ms_per_token: float
    total_tokens: int
    runs: int
    min_tps: float
    max_tps: float
    p50_tps: float
    p95_tps: float

    def summary(self) -> str:
        return f"Throughput: {self.tokens_per_second:.1f} t/s (p50: {self.p50_tps:.1f}, p95: {self.p95_tps:.1f})"

    def meets_target(self, target_tps: float) -> bool:
        return self.tokens_per_second >= target_tps

    def latency_breakdown(self) -> str:
        return f"Prefill: {self.prefill_ms:.2f} ms | Decode: {self.decode_ms_per_token:.3f} ms/token"


class ThroughputRuns:
    """Aggregates ``(prefill ms, decode ms, tokens generated)`` of measured runs (warm-up runs already left out)."""

    def __init__(self, warmup_runs: int = 1, runs: int = 5):
        self.warmup_runs, self.runs = warmup_runs, runs

    def with_warmup(self, n: int) -> "ThroughputRuns":
        self.warmup_runs = n
        return self

    def with_runs(self, n: int) -> "ThroughputRuns":
        self.runs = n
        return self

    def measure(self, run: Callable[[], tuple[float, float, int]]) -> ThroughputStats:
        for _ in range(self.warmup_runs):
            run()
        return self.from_timings([run() for _ in range(self.runs)])

    @staticmethod
    def from_timings(timings: Sequence[tuple[float, float, int]]) -> ThroughputStats:
        if not timings:
            return ThroughputStats(0.0, 0.0, 0.0, 0, 0, 0.0, 0.0, 0.0, 0.0)
        tps = [n / (d / 1e3) if d > 0 else 0.0 for _, d, n in timings]
        tokens, decode = sum(n for _, _, n in timings), sum(d for _, d, _ in timings)
        return ThroughputStats(tokens / (decode / 1e3) if decode > 0 else 0.0, sum(p for p, _, _ in timings) / len(timings),
                               decode / tokens if tokens else 0.0, tokens, len(timings), min(tps), max(tps), percentile(tps, 50), percentile(tps, 95))


# ---- perplexity helpers -------------------------------------------------------------------------------------------------------
def perplexity_from_log_probs(log_probs: Sequence[float], max_length: int | None = None) -> float:
    lp = list(log_probs)[:max_length] if max_length else list(log_probs)
    return math.exp(-sum(lp) / len(lp)) if lp else float("inf")


def perplexity_from_logits(logits: Sequence[Sequence[float]], targets: Sequence[int]) -> float:
    """``logits[i]`` predicts ``targets[i]``."""
    lps = []
    for row, y in zip(logits, targets):
        z = np.asarray(row, dtype=np.float64)
        lps.append(float(z[y] - z.max() - np.log(np.exp(z - z.max()).sum())))
    return perplexity_from_log_probs(lps)


def perplexity_batch(batch: Sequence[Sequence[float]], max_length: int | None = None) -> float:
    """Token-weighted perplexity over several sequences of log-probabilities."""
    flat = [lp for seq in batch for lp in (list(seq)[:max_length] if max_length else seq)]
    return perplexity_from_log_probs(flat)


def bits_per_byte(log_probs: Sequence[float], n_bytes: int, max_length: int | None = None) -> float:
    lp = list(log_probs)[:max_length] if max_length else list(log_probs)
    return -sum(lp) / math.log(2) / n_bytes if lp and n_bytes > 0 else float("inf")


# ---- report -------------------------------------------------------------------------------------------------------------------
@dataclass
class EvalResultEntry:
    task: str
    metric: str
    value: float
    details: dict = field(default_factory=dict)


class EvalSuiteReport:
    def __init__(self, model: str):
        self.model, self.entries = model, []

    def add(self, task: str, metric: str, value: float, **details) -> "EvalSuiteReport":
        self.entries.append(EvalResultEntry(task, metric, float(value), details))
        return self

    def add_perplexity(self, task: str, perplexity: float, tokens: int = 0) -> "EvalSuiteReport":
        return self.add(task, "perplexity", perplexity, tokens=tokens)

    def add_accuracy(self, task: str, result) -> "EvalSuiteReport":
        return self.add(task, "accuracy", getattr(result, "accuracy", 0.0), correct=getattr(result, "correct", 0), total=getattr(result, "total", 0))

    def add_throughput(self, task: str, stats: ThroughputStats) -> "EvalSuiteReport":
        return self.add(task, "tokens_per_second", stats.tokens_per_second, prefill_ms=stats.prefill_ms, decode_ms_per_token=stats.decode_ms_per_token, runs=stats.runs)

    def to_json(self) -> str:
        return json.dumps({"model": self.model, "results": [{"task": e.task, "metric": e.metric, "value": e.value, **e.details} for e in self.entries]}, indent=2)

    def to_markdown(self) -> str:
        rows = "".join(f"| {e.task} | {e.metric} | {e.value:.4f} | {', '.join(f'{k}={v}' for k, v in e.details.items())} |\n" for e in self.entries)
        return f"# Evaluation report: {self.model}\n\n| Task | Metric | Value | Details |\n|---|---|---|---|\n{rows}"

    def summary(self) -> str:
        return f"{self.model}: " + "; ".join(f"{e.task} {e.metric} {e.value:.4g}" for e in self.entries) if self.entries else f"{self.model}: no results"
