"""Long-context position encodings: RoPE scaling families (linear, dynamic NTK, Llama-3.1, LongRoPE), YaRN and ALiBi.

Reference: crates/oxibonsai-model/src/layers/rope_scaling.rs:26-383 (``RopeScalingStrategy``, ``compute_rope_frequencies``,
``dynamic_ntk_base``, ``llama31_frequencies``), yarn_rope.rs:12-368 (``YarnConfig`` interpolation ramp, attention scale
``0.1 ln(s) + 1``, ``YarnFreqTable``, ``LongRopeConfig`` position remap) and alibi.rs:37-273 (head slopes ``2^(-8 i / n)``
with the extrapolation rule for head counts that are not powers of two).

Everything here produces frequency / cos / sin / bias tables as torch tensors, so a scaled table can be handed to the
GPU runner in place of the plain one (``Qwen3Runner`` takes its cos/sin tables as device tensors).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


def base_frequencies(head_dim: int, base: float = 1e6) -> torch.Tensor:
    """``1 / base^(2i/d)`` for i in [0, d/2) in float32 (the table the engine uses unscaled)."""
    i = torch.arange(0, head_dim // 2, dtype=torch.float32)
    return 1.0 / (base ** (2.0 * i / head_dim))


def dynamic_ntk_base(base: float, head_dim: int, seq_len: int, original_max: int, factor: float = 1.0) -> float:
    if seq_len <= original_max:
        return base
    s = factor * seq_len / original_max - (factor - 1.0)
    return base * s ** (head_dim / (head_dim - 2))


def llama31_frequencies(freqs: torch.Tensor, factor: float = 8.0, low_freq_factor: float = 1.0, high_freq_factor: float = 4.0,
                        original_max: int = 8192) -> torch.Tensor:
    wavelen = 2 * math.pi / freqs
    low, high = original_max / low_freq_factor, original_max / high_freq_factor
    smooth = ((original_max / wavelen) - low_freq_factor) / (high_freq_factor - low_freq_factor)
    mid = (1 - smooth) * freqs / factor + smooth * freqs
    return torch.where(wavelen < high, freqs, torch.where(wavelen > low, freqs / factor, mid))


@dataclass
class RopeScaling:
    """``strategy``: none | linear | dynamic_ntk | llama31 | yarn | longrope."""
    strategy: str = "none"
    factor: float = 1.0
    original_max: int = 32768
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    short_factors: list[float] | None = None      # LongRoPE per-frequency rescale
    long_factors: list[float] | None = None

    def validate(self) -> "RopeScaling":
        if self.strategy not in ("none", "linear", "dynamic_ntk", "llama31", "yarn", "longrope"):
            raise ValueError(f"unknown RoPE scaling strategy {self.strategy!r}")
        if self.factor < 1.0:
            raise ValueError("scaling factor must be >= 1")
        return self


def compute_rope_frequencies(head_dim: int, base: float, scaling: RopeScaling | None = None, seq_len: int | None = None) -> torch.Tensor:
    sc = (scaling or RopeScaling()).validate()
    f = base_frequencies(head_dim, base)
    if sc.strategy == "none":
        return f
    if sc.strategy == "linear":
        return f / sc.factor
    if sc.strategy == "dynamic_ntk":
        return base_frequencies(head_dim, dynamic_ntk_base(base, head_dim, seq_len or sc.original_max, sc.original_max, sc.factor))
    if sc.strategy == "llama31":
        return llama31_frequencies(f, sc.factor, sc.low_freq_factor, sc.high_freq_factor, sc.original_max)
    if sc.strategy == "yarn":
        return YarnConfig(head_dim, base, sc.factor, sc.original_max, sc.beta_fast, sc.beta_slow).scaled_frequencies()
    factors = sc.long_factors if (seq_len or 0) > sc.original_max else sc.short_factors
    if factors is None:
        return f
    if len(factors) != head_dim // 2:
        raise ValueError("LongRoPE needs one factor per frequency")
    return f / torch.tensor(factors, dtype=torch.float32)


def rope_tables(head_dim: int, max_pos: int, base: float, scaling: RopeScaling | None = None, device=None) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin tables [max_pos, head_dim/2] (float32); YaRN's attention temperature is folded into both."""
    f = compute_rope_frequencies(head_dim, base, scaling, max_pos)
    ang = torch.arange(max_pos, dtype=torch.float32)[:, None] * f[None, :]
    m = 1.0
    if scaling is not None and scaling.strategy == "yarn":
        m = YarnConfig(head_dim, base, scaling.factor, scaling.original_max).attention_scale()
    cos, sin = torch.cos(ang) * m, torch.sin(ang) * m
    return (cos.to(device), sin.to(device)) if device is not None else (cos, sin)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Half-split rotation (the Qwen3 / GPT-NeoX convention) of ``x[..., head_dim]`` at ``positions``."""
    h = x.shape[-1] // 2
    c, s = cos[positions].to(x.dtype), sin[positions].to(x.dtype)
    while c.dim() < x.dim():
        c, s = c.unsqueeze(-2), s.unsqueeze(-2)
    x0, x1 = x[..., :h], x[..., h:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], dim=-1)


@dataclass
class YarnConfig:
    head_dim: int
    base: float = 1e6
    factor: float = 4.0
    original_max: int = 32768
    beta_fast: float = 32.0
    beta_slow: float = 1.0

    def scale(self) -> float:
        return self.factor

    def attention_scale(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0 if self.factor > 1.0 else 1.0

    def _correction_dim(self, rotations: float) -> float:
        return self.head_dim * math.log(self.original_max / (rotations * 2 * math.pi)) / (2 * math.log(self.base))

    def interpolation_factors(self) -> torch.Tensor:
        """Per-frequency blend in [0, 1]: 1 = keep (high frequency, extrapolate), 0 = fully interpolate."""
        lo = max(math.floor(self._correction_dim(self.beta_fast)), 0)
        hi = min(math.ceil(self._correction_dim(self.beta_slow)), self.head_dim // 2 - 1)
        hi = hi if hi > lo else lo + 1e-3
        ramp = ((torch.arange(self.head_dim // 2, dtype=torch.float32) - lo) / (hi - lo)).clamp(0, 1)
        return 1.0 - ramp

    def scaled_frequencies(self) -> torch.Tensor:
        f = base_frequencies(self.head_dim, self.base)
        keep = self.interpolation_factors()
        return f / self.factor * (1 - keep) + f * keep

    def effective_context(self) -> int:
        return int(self.original_max * self.factor)


class YarnFreqTable:
    def __init__(self, config: YarnConfig, max_pos: int):
        self.config = config
        ang = torch.arange(max_pos, dtype=torch.float32)[:, None] * config.scaled_frequencies()[None, :]
        m = config.attention_scale()
        self.cos, self.sin = torch.cos(ang) * m, torch.sin(ang) * m

    def apply(self, x: torch.Tensor, position: int) -> torch.Tensor:
        return apply_rope(x, self.cos, self.sin, torch.tensor(position))

    def apply_batch(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        return apply_rope(x, self.cos, self.sin, positions)

    def num_frequencies(self) -> int:
        return self.cos.shape[1]

    def effective_context(self) -> int:
        return self.config.effective_context()


@dataclass
class LongRopeConfig:
    """Position remap: positions beyond the trained window are compressed by ``factor``."""
    original_max: int
    factor: float

    def remap_position(self, pos: int) -> float:
        return float(pos) if pos < self.original_max else self.original_max + (pos - self.original_max) / self.factor

    def effective_pos(self, pos: int) -> int:
        return int(self.remap_position(pos))


# ---- ALiBi --------------------------------------------------------------------------------------------------------------------
def alibi_slopes(n_heads: int) -> torch.Tensor:
    def pow2(n):
        start = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [start * start ** i for i in range(n)]
    if math.log2(n_heads).is_integer():
        return torch.tensor(pow2(n_heads), dtype=torch.float32)
    closest = 2 ** math.floor(math.log2(n_heads))
    extra = pow2(2 * closest)[0::2][: n_heads - closest]
    return torch.tensor(pow2(closest) + extra, dtype=torch.float32)


class AliBiBias:
    def __init__(self, n_heads: int):
        self.slopes = alibi_slopes(n_heads)

    def bias_for_head(self, head: int, q_pos: int, k_len: int) -> torch.Tensor:
        return -self.slopes[head] * (q_pos - torch.arange(k_len, dtype=torch.float32)).clamp(min=0)

    def biases_for_sequence(self, q_len: int, k_len: int) -> torch.Tensor:
        """[heads, q_len, k_len]; queries are the last ``q_len`` positions of the keys."""
        qp = torch.arange(k_len - q_len, k_len, dtype=torch.float32)[:, None]
        kp = torch.arange(k_len, dtype=torch.float32)[None, :]
        return -self.slopes[:, None, None] * (qp - kp).clamp(min=0)[None]

    def apply(self, scores: torch.Tensor) -> torch.Tensor:
        h, q, k = scores.shape[-3:]
        return scores + self.biases_for_sequence(q, k).to(scores.device, scores.dtype)


def attention_with_alibi(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """q [h, tq, d], k / v [h, tk, d] -> [h, tq, d] with ALiBi biases instead of rotary embeddings."""
    h, tq, d = q.shape
    tk = k.shape[1]
    s = torch.einsum("hqd,hkd->hqk", q.float(), k.float()) / math.sqrt(d)
    s = AliBiBias(h).apply(s)
    if causal:
        qp = torch.arange(tk - tq, tk)[:, None]
        s = s.masked_fill(torch.arange(tk)[None, :] > qp, float("-inf"))
    return torch.einsum("hqk,hkd->hqd", torch.softmax(s, -1), v.float()).to(q.dtype)


@dataclass
class FreqStats:
    min_freq: float
    max_freq: float
    min_wavelength: float
    max_wavelength: float

    @classmethod
    def compute(cls, freqs: torch.Tensor) -> "FreqStats":
        lo, hi = float(freqs.min()), float(freqs.max())
        return cls(lo, hi, 2 * math.pi / hi, 2 * math.pi / lo)

    def summary(self) -> str:
        return f"freq [{self.min_freq:.3e}, {self.max_freq:.3e}] wavelength [{self.min_wavelength:.1f}, {self.max_wavelength:.1f}]"
