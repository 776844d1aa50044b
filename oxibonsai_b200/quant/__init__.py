"""Post-training quantisation toolbox: Q1 / ternary group quantisers, INT8 (static, per-channel, dynamic), SmoothQuant,
calibration statistics, pruning and a prune -> quantise compression pipeline.

Reference: crates/oxibonsai-model/src/quantize.rs:54-84 (Q1 groups, scale = absmax), quantize_ternary.rs:16-60,
quantize_int8.rs (per-tensor / per-channel INT8 and the W8A8 matvec), dynamic_quant.rs, smoothquant.rs, calibration.rs,
pruning.rs and compression.rs.  Block encodings themselves live in the C++ core (``oxibonsai_b200.core.blocks``);
this module holds the tensor-level policies around them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Iterable, Sequence

import numpy as np

from ..core import gguf as G
from ..core.blocks import dequantize, quantize


# ---- sub-2-bit group quantisers -------------------------------------------------------------------------------
def quantize_q1(values: np.ndarray, scale: str = "mean") -> np.ndarray:
    """Q1_0_g128 blocks; ``scale`` = "mean" (mean |w|, the least-squares optimum for sign codes) or "absmax"
    (what the reference's exporter uses)."""
    return quantize(G.Q1_0_G128, values, q1_absmax=(scale == "absmax"))


def quantize_ternary(values: np.ndarray) -> np.ndarray:
    """TQ2_0_g128 blocks: absmax scale, threshold at half of it, an all-zero group encodes as 0x55 bytes."""
    return quantize(G.TQ2_0_G128, values)


def quantization_error(type_id: int, values: np.ndarray) -> dict:
    """Round-trip error statistics of ``values`` through ``type_id``."""
    v = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    back = dequantize(type_id, quantize(type_id, v))
    err = back - v
    denom = float(np.sqrt(np.mean(v * v))) or 1.0
    _, be, bb = G.type_info(type_id)
    return {"mse": float(np.mean(err * err)), "max_abs": float(np.max(np.abs(err))), "rel_rmse": float(np.sqrt(np.mean(err * err))) / denom,
            "bits_per_weight": 8.0 * bb / be}


# ---- INT8 -----------------------------------------------------------------------------------------------------
@dataclass
class Int8Tensor:
    q: np.ndarray                    # int8, same shape as the source
    scale: np.ndarray                # float32: scalar (per tensor) or [rows] (per output channel)
    zero_point: np.ndarray | None = None

    def dequantize(self) -> np.ndarray:
        s = self.scale if self.scale.ndim == 0 else self.scale.reshape(-1, *([1] * (self.q.ndim - 1)))
        q = self.q.astype(np.float32)
        if self.zero_point is not None:
            z = self.zero_point if self.zero_point.ndim == 0 else self.zero_point.reshape(s.shape)
            q = q - z
        return q * s

    @property
    def nbytes(self) -> int:
        return self.q.nbytes + self.scale.nbytes + (0 if self.zero_point is None else self.zero_point.nbytes)


def quantize_int8(w: np.ndarray, per_channel: bool = False, symmetric: bool = True) -> Int8Tensor:
    w = np.asarray(w, dtype=np.float32)
    axis = tuple(range(1, w.ndim)) if per_channel and w.ndim > 1 else None
    if symmetric:
        amax = np.max(np.abs(w), axis=axis)
        scale = np.maximum(amax, 1e-12) / 127.0
        s = scale if axis is None else scale.reshape(-1, *([1] * (w.ndim - 1)))
        return Int8Tensor(np.clip(np.rint(w / s), -127, 127).astype(np.int8), np.asarray(scale, dtype=np.float32))
    lo, hi = np.min(w, axis=axis), np.max(w, axis=axis)
    scale = np.maximum(hi - lo, 1e-12) / 255.0
    zp = np.rint(-128.0 - lo / scale)
    s = scale if axis is None else scale.reshape(-1, *([1] * (w.ndim - 1)))
    z = zp if axis is None else zp.reshape(s.shape)
    return Int8Tensor(np.clip(np.rint(w / s + z), -128, 127).astype(np.int8), np.asarray(scale, dtype=np.float32), np.asarray(zp, dtype=np.float32))


def int8_matvec(w: Int8Tensor, x: np.ndarray) -> np.ndarray:
    """W8A8 product: the activation is quantised on the fly (dynamic per-vector scale), accumulation is int32."""
    x = np.asarray(x, dtype=np.float32)
    xs = max(float(np.max(np.abs(x))), 1e-12) / 127.0
    xq = np.clip(np.rint(x / xs), -127, 127).astype(np.int32)
    acc = w.q.astype(np.int32) @ xq
    if w.zero_point is not None:
        acc = acc - (w.zero_point.astype(np.int64) * int(xq.sum())).astype(np.int64)
    return acc.astype(np.float32) * w.scale * xs


class DynamicQuantLinear:
    """Weights INT8 per output channel, activations quantised per call."""

    def __init__(self, weight: np.ndarray, bias: np.ndarray | None = None):
        self.w = quantize_int8(weight, per_channel=True)
        self.bias = None if bias is None else np.asarray(bias, dtype=np.float32)

    def __call__(self, x: np.ndarray) -> np.ndarray:
        x = np.asarray(x, dtype=np.float32)
        y = np.stack([int8_matvec(self.w, r) for r in x.reshape(-1, x.shape[-1])]).reshape(*x.shape[:-1], -1)
        return y if self.bias is None else y + self.bias


# ---- calibration + SmoothQuant ----------------------------------------------------------------------------------
@dataclass
class ActivationStats:
    count: int = 0
    absmax: np.ndarray | None = None       # per input channel
    mean: float = 0.0
    m2: float = 0.0
    minimum: float = float("inf")
    maximum: float = float("-inf")

    def update(self, x: np.ndarray) -> None:
        x = np.asarray(x, dtype=np.float32).reshape(-1, np.shape(x)[-1])
        am = np.max(np.abs(x), axis=0)
        self.absmax = am if self.absmax is None else np.maximum(self.absmax, am)
        for v in (x.reshape(-1),):
            n = v.size
            mean_b, m2_b = float(v.mean()), float(((v - v.mean()) ** 2).sum())
            delta = mean_b - self.mean
            tot = self.count + n
            self.mean += delta * n / tot
            self.m2 += m2_b + delta * delta * self.count * n / tot
            self.count = tot
        self.minimum, self.maximum = min(self.minimum, float(x.min())), max(self.maximum, float(x.max()))

    @property
    def std(self) -> float:
        return float(np.sqrt(self.m2 / self.count)) if self.count else 0.0


class CalibrationDb:
    """Per-layer activation statistics gathered from calibration batches."""

    def __init__(self):
        self.layers: dict[str, ActivationStats] = {}

    def observe(self, layer: str, activations: np.ndarray) -> None:
        self.layers.setdefault(layer, ActivationStats()).update(activations)

    def scale_for(self, layer: str, percentile_clip: float = 1.0) -> float:
        st = self.layers[layer]
        return float(np.max(st.absmax)) * percentile_clip / 127.0

    def summary(self) -> dict:
        return {k: {"count": v.count, "mean": v.mean, "std": v.std, "min": v.minimum, "max": v.maximum} for k, v in self.layers.items()}


def smooth_factors(act_absmax: np.ndarray, weight: np.ndarray, alpha: float = 0.5) -> np.ndarray:
    """SmoothQuant per-input-channel factors s_j = max|X_j|^alpha / max|W_j|^(1-alpha)."""
    wmax = np.maximum(np.max(np.abs(weight), axis=0), 1e-8)
    amax = np.maximum(np.asarray(act_absmax, dtype=np.float32), 1e-8)
    return np.maximum(amax ** alpha / wmax ** (1.0 - alpha), 1e-8).astype(np.float32)


def apply_smoothquant(weight: np.ndarray, act_absmax: np.ndarray, alpha: float = 0.5) -> tuple[np.ndarray, np.ndarray]:
    """Returns ``(W * s, s)``; dividing the activations by ``s`` keeps ``W x`` unchanged while flattening activation outliers."""
    s = smooth_factors(act_absmax, weight, alpha)
    return (np.asarray(weight, dtype=np.float32) * s[None, :]), s


# ---- pruning ----------------------------------------------------------------------------------------------------
def magnitude_prune(w: np.ndarray, sparsity: float) -> np.ndarray:
    """Zeroes the ``sparsity`` fraction of smallest-magnitude entries."""
    w = np.array(w, dtype=np.float32, copy=True)
    k = int(round(np.clip(sparsity, 0.0, 1.0) * w.size))
    if k == 0:
        return w
    thr = np.partition(np.abs(w).reshape(-1), k - 1)[k - 1]
    mask = np.abs(w) > thr
    # ties at the threshold: keep just enough of them to hit the requested count
    short = (w.size - k) - int(mask.sum())
    if short > 0:
        ties = np.flatnonzero((np.abs(w) == thr).reshape(-1))[:short]
        mask.reshape(-1)[ties] = True
    return w * mask


def structured_prune_rows(w: np.ndarray, fraction: float) -> tuple[np.ndarray, np.ndarray]:
    """Drops whole output rows with the smallest L2 norm; returns (pruned matrix, kept row indices)."""
    w = np.asarray(w, dtype=np.float32)
    n_drop = int(round(np.clip(fraction, 0.0, 1.0) * w.shape[0]))
    norms = np.linalg.norm(w.reshape(w.shape[0], -1), axis=1)
    keep = np.sort(np.argsort(norms, kind="stable")[n_drop:])
    return w[keep], keep


def n_m_prune(w: np.ndarray, n: int = 2, m: int = 4) -> np.ndarray:
    """N:M sparsity along the input dimension: keeps the ``n`` largest magnitudes of every group of ``m``."""
    w = np.array(w, dtype=np.float32, copy=True)
    if w.shape[-1] % m:
        raise ValueError(f"inner dimension {w.shape[-1]} is not a multiple of {m}")
    g = w.reshape(-1, m)
    drop = np.argsort(np.abs(g), axis=1, kind="stable")[:, : m - n]
    np.put_along_axis(g, drop, 0.0, axis=1)
    return g.reshape(w.shape)


def sparsity(w: np.ndarray) -> float:
    return float(np.mean(np.asarray(w) == 0))


# ---- compression pipeline ---------------------------------------------------------------------------------------
@dataclass
class CompressionReport:
    original_bytes: int = 0
    compressed_bytes: int = 0
    tensors: dict[str, dict] = field(default_factory=dict)

    @property
    def ratio(self) -> float:
        return self.original_bytes / self.compressed_bytes if self.compressed_bytes else 0.0


def compress_tensors(tensors: dict[str, np.ndarray], type_id: int = G.TQ2_0_G128, prune_sparsity: float = 0.0,
                     skip: Callable[[str], bool] = lambda n: n.endswith("norm.weight")) -> tuple[dict[str, tuple[int, np.ndarray]], CompressionReport]:
    """Prune (optional) then quantise every 2-D tensor; 1-D tensors and ``skip`` names stay F32.
    Returns ``{name: (type_id, bytes)}`` and a report."""
    out: dict[str, tuple[int, np.ndarray]] = {}
    rep = CompressionReport()
    _, be, _ = G.type_info(type_id)
    for name, t in tensors.items():
        t = np.asarray(t, dtype=np.float32)
        rep.original_bytes += t.nbytes
        if t.ndim < 2 or skip(name) or t.shape[-1] % be:
            blob, tid = t.view(np.uint8).reshape(-1), G.F32
        else:
            src = magnitude_prune(t, prune_sparsity) if prune_sparsity > 0 else t
            blob, tid = quantize(type_id, src), type_id
            rep.tensors[name] = quantization_error(type_id, src)
        out[name] = (tid, blob)
        rep.compressed_bytes += blob.size
    return out, rep
