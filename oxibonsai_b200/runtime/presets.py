"""Sampling parameters and presets.

Reference: ``SamplingParams`` (crates/oxibonsai-runtime/src/sampling.rs:19-61), ``SamplingPreset``
(presets.rs:25-86: Balanced 0.7/40/0.9/1.1, Creative 1.0/0/0.95/1.0, Precise 0.1/10/0.5/1.2, Greedy 0/0/1.0/1.0,
Conversational 0.8/50/0.9/1.1) and the README's ``Code`` preset (0.2/10/0.8; README.md:126-131).  All six
names are accepted.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from enum import Enum


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.9
    repetition_penalty: float = 1.1
    max_tokens: int = 512
    seed: int = 42

    def validate(self) -> "SamplingParams":
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0.0 <= self.top_p <= 1.0:
            raise ValueError("top_p must be within [0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if self.repetition_penalty < 1.0:
            raise ValueError("repetition_penalty must be >= 1")
        return self

    @property
    def greedy(self) -> bool:
        return self.temperature < 1e-6


class SamplingPreset(Enum):
    BALANCED = "balanced"
    CREATIVE = "creative"
    PRECISE = "precise"
    GREEDY = "greedy"
    CONVERSATIONAL = "conversational"
    CODE = "code"

    def params(self) -> SamplingParams:
        t, k, p, rp = _TABLE[self]
        return SamplingParams(temperature=t, top_k=k, top_p=p, repetition_penalty=rp)

    @property
    def description(self) -> str:
        return _DESC[self]

    @classmethod
    def parse(cls, name: "str | SamplingPreset") -> "SamplingPreset":
        if isinstance(name, cls):
            return name
        try:
            return cls(str(name).strip().lower())
        except ValueError:
            raise ValueError(f"unknown sampling preset {name!r}; expected one of {[p.value for p in cls]}") from None


_TABLE = {
    SamplingPreset.BALANCED: (0.7, 40, 0.9, 1.1),
    SamplingPreset.CREATIVE: (1.0, 0, 0.95, 1.0),
    SamplingPreset.PRECISE: (0.1, 10, 0.5, 1.2),
    SamplingPreset.GREEDY: (0.0, 0, 1.0, 1.0),
    SamplingPreset.CONVERSATIONAL: (0.8, 50, 0.9, 1.1),
    SamplingPreset.CODE: (0.2, 10, 0.8, 1.1),
}
_DESC = {
    SamplingPreset.BALANCED: "general purpose default",
    SamplingPreset.CREATIVE: "diverse, exploratory text",
    SamplingPreset.PRECISE: "focused, low-variance answers",
    SamplingPreset.GREEDY: "deterministic argmax decoding",
    SamplingPreset.CONVERSATIONAL: "chat-style replies",
    SamplingPreset.CODE: "code generation",
}


def with_overrides(base: SamplingParams, **kw) -> SamplingParams:
    return replace(base, **{k: v for k, v in kw.items() if v is not None}).validate()
