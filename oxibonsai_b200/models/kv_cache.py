"""Host-side KV caches: dense FP32 (the oracle's), FP16, INT8 and FP8 row-quantised variants, and activation statistics.

Reference: crates/oxibonsai-model/src/kv_cache.rs:21-240 (``[layer][head][max_seq][head_dim]`` f32 with
``extract_block`` / ``inject_block`` for the prefix cache), kv_cache_fp16.rs:16-222 (f16 store, f32 read),
kv_cache_quant.rs:46-480 (INT8 per (token, head) row: ``scale = absmax / 127`` floored at an epsilon, round, clamp to
+-127) and :502-850 (FP8 rows scaled by ``absmax / 448`` for E4M3 or ``/ 57344`` for E5M2), plus layer_stats.rs
(per-layer activation statistics).  On the GPU the same row formats are the page formats of ``PagedKvCache``
(models/qwen3.py, csrc/cuda/attention_decode.cu); these classes are the CPU counterparts used by the oracle-side tools
and by tests that check the page formats.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ..core.blocks import fp8_decode, fp8_encode

_EPS = 1e-12


class KvCache:
    """Dense f32 cache."""

    def __init__(self, layers: int, kv_heads: int, max_seq: int, head_dim: int):
        self.shape = (layers, kv_heads, max_seq, head_dim)
        self.k = np.zeros(self.shape, dtype=np.float32)
        self.v = np.zeros(self.shape, dtype=np.float32)
        self.len = 0

    def store(self, layer: int, pos: int, k: np.ndarray, v: np.ndarray) -> None:
        """k, v: [kv_heads, head_dim] of one token."""
        if pos >= self.shape[2]:
            raise IndexError(f"position {pos} exceeds the cache length {self.shape[2]}")
        self.k[layer, :, pos], self.v[layer, :, pos] = k, v
        self.len = max(self.len, pos + 1)

    def keys(self, layer: int, head: int, length: int | None = None) -> np.ndarray:
        return self.k[layer, head, : self.len if length is None else length]

    def values(self, layer: int, head: int, length: int | None = None) -> np.ndarray:
        return self.v[layer, head, : self.len if length is None else length]

    def extract_block(self, start: int, n: int) -> tuple[np.ndarray, np.ndarray]:
        return self.k[:, :, start:start + n].copy(), self.v[:, :, start:start + n].copy()

    def inject_block(self, start: int, k: np.ndarray, v: np.ndarray) -> None:
        n = k.shape[2]
        self.k[:, :, start:start + n], self.v[:, :, start:start + n] = k, v
        self.len = max(self.len, start + n)

    def clear(self) -> None:
        self.len = 0

    def is_all_zero(self) -> bool:
        return not self.k[:, :, : self.len].any()

    @property
    def nbytes(self) -> int:
        return self.k.nbytes + self.v.nbytes


class KvCacheFp16(KvCache):
    """Stores f16, reads f32."""

    def __init__(self, layers: int, kv_heads: int, max_seq: int, head_dim: int):
        self.shape = (layers, kv_heads, max_seq, head_dim)
        self.k = np.zeros(self.shape, dtype=np.float16)
        self.v = np.zeros(self.shape, dtype=np.float16)
        self.len = 0

    def keys(self, layer, head, length=None):
        return super().keys(layer, head, length).astype(np.float32)

    def values(self, layer, head, length=None):
        return super().values(layer, head, length).astype(np.float32)


def quantize_row_int8(x: np.ndarray) -> tuple[np.ndarray, float]:
    scale = max(float(np.max(np.abs(x))) / 127.0, _EPS)
    return np.clip(np.rint(x / scale), -127, 127).astype(np.int8), scale


def quantize_row_int4(x: np.ndarray) -> tuple[np.ndarray, float]:
    """The INT4 page format: scale = absmax / 7, codes stored as q + 8, two per byte (low nibble = even element)."""
    scale = max(float(np.max(np.abs(x))) / 7.0, _EPS)
    q = (np.clip(np.rint(x / scale), -7, 7).astype(np.int8) + 8).astype(np.uint8)
    return (q[0::2] | (q[1::2] << 4)).astype(np.uint8), scale


def dequantize_row_int4(packed: np.ndarray, scale: float) -> np.ndarray:
    out = np.empty(packed.size * 2, dtype=np.float32)
    out[0::2] = (packed & 15).astype(np.float32) - 8.0
    out[1::2] = (packed >> 4).astype(np.float32) - 8.0
    return out * scale


class QuantizedKvCache:
    """INT8 rows with one f32 scale per (layer, head, token)."""

    def __init__(self, layers: int, kv_heads: int, max_seq: int, head_dim: int):
        self.shape = (layers, kv_heads, max_seq, head_dim)
        self.k = np.zeros(self.shape, dtype=np.int8)
        self.v = np.zeros(self.shape, dtype=np.int8)
        self.k_scale = np.zeros(self.shape[:3], dtype=np.float32)
        self.v_scale = np.zeros(self.shape[:3], dtype=np.float32)
        self.len = 0

    def store(self, layer: int, pos: int, k: np.ndarray, v: np.ndarray) -> None:
        for h in range(self.shape[1]):
            self.k[layer, h, pos], self.k_scale[layer, h, pos] = quantize_row_int8(k[h])
            self.v[layer, h, pos], self.v_scale[layer, h, pos] = quantize_row_int8(v[h])
        self.len = max(self.len, pos + 1)

    def keys(self, layer: int, head: int, length: int | None = None) -> np.ndarray:
        n = self.len if length is None else length
        return self.k[layer, head, :n].astype(np.float32) * self.k_scale[layer, head, :n, None]

    def values(self, layer: int, head: int, length: int | None = None) -> np.ndarray:
        n = self.len if length is None else length
        return self.v[layer, head, :n].astype(np.float32) * self.v_scale[layer, head, :n, None]

    @property
    def nbytes(self) -> int:
        return self.k.nbytes + self.v.nbytes + self.k_scale.nbytes + self.v_scale.nbytes

    def compression_ratio(self) -> float:
        return (2 * np.prod(self.shape) * 4) / self.nbytes


class Fp8KvCache:
    """FP8 rows (E4M3 or E5M2) with one f32 scale per row chosen so that the row's absmax maps to the format's maximum."""

    def __init__(self, layers: int, kv_heads: int, max_seq: int, head_dim: int, e5m2: bool = False):
        self.shape, self.e5m2 = (layers, kv_heads, max_seq, head_dim), e5m2
        self.max = 57344.0 if e5m2 else 448.0
        self.k = np.zeros(self.shape, dtype=np.uint8)
        self.v = np.zeros(self.shape, dtype=np.uint8)
        self.k_scale = np.zeros(self.shape[:3], dtype=np.float32)
        self.v_scale = np.zeros(self.shape[:3], dtype=np.float32)
        self.len = 0
        self._dec = np.array([fp8_decode(i, e5m2) for i in range(256)], dtype=np.float32)

    def _q(self, x: np.ndarray) -> tuple[np.ndarray, float]:
        scale = max(float(np.max(np.abs(x))) / self.max, _EPS)
        return np.array([fp8_encode(float(t) / scale, self.e5m2) for t in x], dtype=np.uint8), scale

    def store(self, layer: int, pos: int, k: np.ndarray, v: np.ndarray) -> None:
        for h in range(self.shape[1]):
            self.k[layer, h, pos], self.k_scale[layer, h, pos] = self._q(k[h])
            self.v[layer, h, pos], self.v_scale[layer, h, pos] = self._q(v[h])
        self.len = max(self.len, pos + 1)

    def keys(self, layer: int, head: int, length: int | None = None) -> np.ndarray:
        n = self.len if length is None else length
        return self._dec[self.k[layer, head, :n]] * self.k_scale[layer, head, :n, None]

    def values(self, layer: int, head: int, length: int | None = None) -> np.ndarray:
        n = self.len if length is None else length
        return self._dec[self.v[layer, head, :n]] * self.v_scale[layer, head, :n, None]

    @property
    def nbytes(self) -> int:
        return self.k.nbytes + self.v.nbytes + self.k_scale.nbytes + self.v_scale.nbytes


# ---- per-layer activation statistics ---------------------------------------------------------------------------------------------
@dataclass
class LayerStats:
    layer: int
    mean: float
    std: float
    abs_max: float
    l2_norm: float
    zero_fraction: float
    has_nan: bool

    @classmethod
    def compute(cls, layer: int, x: np.ndarray) -> "LayerStats":
        x = np.asarray(x, dtype=np.float64)
        return cls(layer, float(np.nanmean(x)), float(np.nanstd(x)), float(np.nanmax(np.abs(x))), float(np.sqrt(np.nansum(x * x))),
                   float(np.mean(x == 0)), bool(np.isnan(x).any()))

    def summary(self) -> str:
        return f"layer {self.layer:3d}: mean {self.mean:+.4f} std {self.std:.4f} absmax {self.abs_max:.3f} |x| {self.l2_norm:.2f}" + (" NaN!" if self.has_nan else "")


def forward_with_stats(oracle, tokens) -> list[LayerStats]:
    """Runs ``tokens`` through the CPU oracle and returns statistics of the residual stream after every layer at the
    last token."""
    oracle.keep_layer_hidden(True)
    try:
        for pos, t in enumerate(tokens):
            oracle.forward(int(t), pos)
        hidden = oracle.layer_hidden()
    finally:
        oracle.keep_layer_hidden(False)
    return [LayerStats.compute(l, hidden[l]) for l in range(oracle.config.layers)]
