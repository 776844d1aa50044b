"""KV-cache compression policy: FP16 <-> Q8 <-> (FP8) <-> Q4 driven by memory pressure.

Reference: ``KvCachePolicy`` (crates/oxibonsai-runtime/src/kv_cache_policy.rs:50-392): levels Fp16(0) Q8(1) Fp8(2)
Q4(3); an EWMA of the observed pressure (alpha 0.2); the level goes up when the smoothed pressure crosses
0.80 / 0.95 and comes back down only after it has fallen ``hysteresis`` (0.05) below the threshold; clamped to
[min_level, max_level]; upgrade / downgrade counters; presets ``fp16_only`` and ``aggressive``.  In the reference
the policy only reports a level; here :meth:`page_format` maps the level onto the page formats the attention
kernels read (F16 / Q8 / Q4 - the FP8 level is served by the Q8 pages).
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from enum import IntEnum


class KvLevel(IntEnum):
    FP16 = 0
    Q8 = 1
    FP8 = 2
    Q4 = 3

    @property
    def bytes_per_element(self) -> float:
        return {0: 2.0, 1: 1.0, 2: 1.0, 3: 0.5}[int(self)]


@dataclass(frozen=True)
class KvPolicyConfig:
    alpha: float = 0.2
    moderate_threshold: float = 0.80
    severe_threshold: float = 0.95
    hysteresis: float = 0.05
    min_level: KvLevel = KvLevel.FP16
    max_level: KvLevel = KvLevel.Q4
    moderate_level: KvLevel = KvLevel.Q8
    severe_level: KvLevel = KvLevel.Q4

    def validate(self) -> "KvPolicyConfig":
        if not 0.0 < self.alpha <= 1.0:
            raise ValueError("alpha must be in (0, 1]")
        if not 0.0 <= self.moderate_threshold <= self.severe_threshold <= 1.0:
            raise ValueError("thresholds must satisfy 0 <= moderate <= severe <= 1")
        if self.min_level > self.max_level:
            raise ValueError("min_level must not exceed max_level")
        return self


class KvCachePolicy:
    """Thread-safe controller; feed it ``observe(pressure)`` with pressure = used / capacity in [0, 1]."""

    def __init__(self, config: KvPolicyConfig | None = None):
        self.config = (config or KvPolicyConfig()).validate()
        self._lock = threading.Lock()
        self._ewma: float | None = None
        self._level = self.config.min_level
        self.upgrades = 0      # moves toward stronger compression
        self.downgrades = 0    # moves back toward FP16
        self.observations = 0

    @classmethod
    def fp16_only(cls) -> "KvCachePolicy":
        return cls(KvPolicyConfig(max_level=KvLevel.FP16))

    @classmethod
    def aggressive(cls) -> "KvCachePolicy":
        return cls(KvPolicyConfig(moderate_threshold=0.60, severe_threshold=0.80, hysteresis=0.03))

    @property
    def level(self) -> KvLevel:
        return self._level

    @property
    def smoothed_pressure(self) -> float:
        return self._ewma or 0.0

    def _clamp(self, lvl: KvLevel) -> KvLevel:
        return KvLevel(max(int(self.config.min_level), min(int(self.config.max_level), int(lvl))))

    def observe(self, pressure: float) -> KvLevel:
        c = self.config
        p = min(1.0, max(0.0, float(pressure)))
        with self._lock:
            self.observations += 1
            self._ewma = p if self._ewma is None else c.alpha * p + (1.0 - c.alpha) * self._ewma
            e = self._ewma
            cur = self._level
            if e >= c.severe_threshold:
                target = c.severe_level
            elif e >= c.moderate_threshold:
                # stay at the severe level until the pressure is clearly below its threshold
                target = c.severe_level if (cur >= c.severe_level and e >= c.severe_threshold - c.hysteresis) else c.moderate_level
            else:
                if cur >= c.moderate_level and e >= c.moderate_threshold - c.hysteresis:
                    target = min(cur, c.moderate_level) if cur < c.severe_level else c.moderate_level
                else:
                    target = c.min_level
            target = self._clamp(target)
            if target > cur:
                self.upgrades += 1
            elif target < cur:
                self.downgrades += 1
            self._level = target
            return target

    def reset(self) -> None:
        with self._lock:
            self._ewma = None
            self._level = self.config.min_level
            self.upgrades = self.downgrades = self.observations = 0

    def page_format(self) -> str:
        """KV page format for newly allocated sequences at the current level."""
        return {KvLevel.FP16: "f16", KvLevel.Q8: "q8", KvLevel.FP8: "q8", KvLevel.Q4: "q4"}[self._level]

    def metric_value(self) -> int:
        """Value of the ``oxibonsai_kv_cache_compression_level`` gauge (0 FP16, 1 Q8, 2 Q4)."""
        return {KvLevel.FP16: 0, KvLevel.Q8: 1, KvLevel.FP8: 1, KvLevel.Q4: 2}[self._level]
