"""Quantisation toolbox, full form: calibration statistics with four clipping rules, dynamic INT8 / INT4 quantisation and a
W8A8 product, INT8 modes with error analysis, importance-based pruning with reports, compression pipelines with size
accounting, merge statistics, the SmoothQuant calibrator with FP8 output, and export planning.

Reference: crates/oxibonsai-model/src - calibration.rs (``CalibMethod`` MinMax / Percentile / ACIQ = 2.83 sigma under a
Laplace assumption / MSE by grid search; 256-bin histogram of |x|; INT8 clip 127, INT4 clip 7; ``CalibrationDb``,
``validate_calibration``), dynamic_quant.rs (``DynamicScaleMode``, ``DynQuantFormat``, per-tensor / per-row INT8, INT4 in
[-7, 7], MAE, SmoothQuant factors ``s_j = max|X_j|^alpha / max|W_j|^(1 - alpha)``, ``w8a8_matvec``), quantize_int8.rs
(``Int8Mode``, error analysis, method comparison), pruning.rs (``ImportanceMetric`` L1 / L2 / Taylor proxy / seeded random;
granularity unstructured / row / column; sparsity reports), compression.rs (stages Prune / QuantizeInt8 / Clip; results with
ratios and byte counts), model_merge.rs (``MergeStats``), smoothquant.rs (calibrator, FP8 E4M3 / E5M2 after smoothing),
export.rs (``ExportConfig`` with FP32 exceptions, size estimate, statistics).  The compact functional forms stay in the
package's ``__init__``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from enum import Enum
from typing import Iterable, Mapping, Sequence

import numpy as np

from ..core import gguf as G

Tensors = Mapping[str, np.ndarray]


# ---- calibration --------------------------------------------------------------------------------------------------------------
class CalibMethod(Enum):
    MINMAX = "minmax"
    PERCENTILE = "percentile"
    ACIQ = "aciq"
    MSE = "mse"


class LayerCalibStats:
    """Running statistics of one layer's activations: extremes, mean / variance (Welford) and a 256-bin histogram of |x|
    whose range doubles when a larger value arrives."""

    BINS = 256

    def __init__(self, name: str = ""):
        self.name, self.num_samples = name, 0
        self.running_min, self.running_max = math.inf, -math.inf
        self._mean, self._m2 = 0.0, 0.0
        self.histogram = np.zeros(self.BINS, dtype=np.int64)
        self.histogram_max = 0.0

    def update(self, values) -> None:
        v = np.asarray(values, dtype=np.float64).reshape(-1)
        v = v[np.isfinite(v)]
        if not v.size:
            return
        self.running_min, self.running_max = min(self.running_min, float(v.min())), max(self.running_max, float(v.max()))
        n0, n1 = self.num_samples, v.size
        mean1, m21 = float(v.mean()), float(((v - v.mean()) ** 2).sum())
        delta = mean1 - self._mean
        total = n0 + n1
        self._mean += delta * n1 / total
        self._m2 += m21 + delta * delta * n0 * n1 / total
        self.num_samples = total
        a = np.abs(v)
        top = float(a.max())
        if top > self.histogram_max:
            if self.histogram_max > 0 and self.histogram.any():         # re-bin what was counted into the wider range
                old_edges = (np.arange(self.BINS) + 0.5) / self.BINS * self.histogram_max
                idx = np.minimum((old_edges / top * self.BINS).astype(int), self.BINS - 1)
                rebinned = np.zeros_like(self.histogram)
                np.add.at(rebinned, idx, self.histogram)
                self.histogram = rebinned
            self.histogram_max = top
        if self.histogram_max > 0:
            np.add.at(self.histogram, np.minimum((a / self.histogram_max * self.BINS).astype(int), self.BINS - 1), 1)

    def mean(self) -> float:
        return self._mean

    def std_dev(self) -> float:
        return math.sqrt(self._m2 / self.num_samples) if self.num_samples else 0.0

    def abs_max(self) -> float:
        return max(abs(self.running_min), abs(self.running_max)) if self.num_samples else 0.0

    def percentile_abs(self, p: float) -> float:
        """Upper edge of the histogram bin in which the cumulative count reaches fraction ``p``."""
        total = int(self.histogram.sum())
        if not total:
            return 0.0
        target = p * total
        k = int(np.searchsorted(np.cumsum(self.histogram), target, side="left"))
        return min((min(k, self.BINS - 1) + 1) / self.BINS * self.histogram_max, self.histogram_max)

    def aciq_clip(self) -> float:
        return 2.83 * self.std_dev()

    def mse_optimal_clip(self, clip_val: float) -> float:
        """Grid search over fractions of the absolute maximum: clipping error of what lies beyond the candidate plus the
        rounding noise (step^2 / 12) of what lies inside, both from the histogram."""
        amax = self.abs_max()
        total = int(self.histogram.sum())
        if amax <= 0 or not total:
            return amax
        centres = (np.arange(self.BINS) + 0.5) / self.BINS * self.histogram_max
        best, best_err = amax, math.inf
        for frac in np.linspace(0.3, 1.0, 36):
            c = frac * amax
            step = c / clip_val
            inside = centres <= c
            err = float((self.histogram[~inside] * (centres[~inside] - c) ** 2).sum() + self.histogram[inside].sum() * step * step / 12.0) / total
            if err < best_err:
                best, best_err = c, err
        return best

    def clipping_value(self, method: CalibMethod, percentile: float = 0.9999, clip_val: float = 127.0) -> float:
        amax = self.abs_max()
        if method is CalibMethod.MINMAX:
            return amax
        if method is CalibMethod.PERCENTILE:
            pv = self.percentile_abs(percentile)
            return pv if pv > 0 else amax
        if method is CalibMethod.ACIQ:
            a = self.aciq_clip()
            return min(a, amax) if a > 0 else amax
        return self.mse_optimal_clip(clip_val)

    def compute_scale(self, method: CalibMethod = CalibMethod.MINMAX, percentile: float = 0.9999) -> float:
        """INT8 scale: clipping value / 127 (0.0 before any sample)."""
        return self.clipping_value(method, percentile, 127.0) / 127.0 if self.num_samples else 0.0

    def compute_scale_int4(self, method: CalibMethod = CalibMethod.MINMAX, percentile: float = 0.9999) -> float:
        return self.clipping_value(method, percentile, 7.0) / 7.0 if self.num_samples else 0.0

    def summary(self) -> "CalibSummary":
        return CalibSummary(self.name, self.num_samples, self.running_min if self.num_samples else 0.0, self.running_max if self.num_samples else 0.0,
                            self.mean(), self.std_dev(), self.abs_max())


@dataclass
class CalibSummary:
    layer: str
    num_samples: int
    min: float
    max: float
    mean: float
    std_dev: float
    abs_max: float

    def summary_line(self) -> str:
        return f"{self.layer}: n={self.num_samples} range=[{self.min:.4g}, {self.max:.4g}] mean={self.mean:.4g} std={self.std_dev:.4g} absmax={self.abs_max:.4g}"


@dataclass
class CalibValidation:
    ok: bool
    issues: list[str]


class CalibrationDatabase:
    def __init__(self, method: CalibMethod = CalibMethod.MINMAX, percentile: float = 0.9999):
        self.method, self.percentile = method, percentile
        self.layers: dict[str, LayerCalibStats] = {}

    @classmethod
    def new_minmax(cls) -> "CalibrationDatabase":
        return cls(CalibMethod.MINMAX)

    @classmethod
    def new_percentile(cls, p: float) -> "CalibrationDatabase":
        return cls(CalibMethod.PERCENTILE, p)

    def record(self, layer: str, activations) -> None:
        self.layers.setdefault(layer, LayerCalibStats(layer)).update(activations)

    def get_stats(self, layer: str) -> LayerCalibStats | None:
        return self.layers.get(layer)

    def scale_for_layer(self, layer: str) -> float | None:
        s = self.layers.get(layer)
        return None if s is None else s.compute_scale(self.method, self.percentile)

    def export_scales(self) -> dict[str, float]:
        return {k: v.compute_scale(self.method, self.percentile) for k, v in self.layers.items()}

    def summaries(self) -> list[CalibSummary]:
        return [self.layers[k].summary() for k in sorted(self.layers)]

    def num_layers(self) -> int:
        return len(self.layers)

    def report(self) -> str:
        return "\n".join([f"calibration: {self.num_layers()} layers, method {self.method.value}"] + [s.summary_line() for s in self.summaries()])

    def validate(self, min_samples: int = 1) -> CalibValidation:
        issues = []
        if not self.layers:
            issues.append("no layers recorded")
        for k, s in sorted(self.layers.items()):
            if s.num_samples < min_samples:
                issues.append(f"{k}: only {s.num_samples} samples")
            elif s.abs_max() == 0.0:
                issues.append(f"{k}: all activations are zero")
            elif not math.isfinite(s.compute_scale(self.method, self.percentile)):
                issues.append(f"{k}: non-finite scale")
        return CalibValidation(not issues, issues)


def simulate_calibration(layer_names: Sequence[str], samples: int = 4, width: int = 256, seed: int = 0, method: CalibMethod = CalibMethod.MINMAX) -> CalibrationDatabase:
    """A database filled with seeded Gaussian activations of growing spread per layer (for dry runs of a pipeline)."""
    rng = np.random.default_rng(seed)
    db = CalibrationDatabase(method)
    for i, name in enumerate(layer_names):
        for _ in range(samples):
            db.record(name, rng.normal(scale=1.0 + 0.25 * i, size=width))
    return db


# ---- dynamic quantisation -----------------------------------------------------------------------------------------------------
class DynamicScaleMode(Enum):
    MAX_ABS = "max_abs"
    PERCENTILE = "percentile"


class DynQuantFormat(Enum):
    INT8_PER_TENSOR = "int8_per_tensor"
    INT8_PER_ROW = "int8_per_row"
    INT4_PER_TENSOR = "int4_per_tensor"


class DynQuantError(ValueError):
    pass


def compute_scale(values, clip_val: float, mode: DynamicScaleMode = DynamicScaleMode.MAX_ABS, percentile: float = 0.99) -> float:
    a = np.abs(np.asarray(values, dtype=np.float64).reshape(-1))
    if not a.size:
        raise DynQuantError("empty tensor")
    top = float(a.max()) if mode is DynamicScaleMode.MAX_ABS else float(np.quantile(a, min(max(percentile, 0.0), 1.0)))
    return top / clip_val if top > 0 else 1.0


@dataclass
class DynQuantTensor:
    data: np.ndarray                 # int8 codes (INT4: values in [-7, 7], two per byte when packed for storage)
    scales: np.ndarray               # one scale, or one per row
    shape: tuple[int, ...]
    format: DynQuantFormat

    def dequantize(self) -> np.ndarray:
        s = self.scales.reshape(-1, *([1] * (len(self.shape) - 1))) if self.format is DynQuantFormat.INT8_PER_ROW else self.scales.reshape(())
        return (self.data.astype(np.float32) * s).reshape(self.shape)

    def element_count(self) -> int:
        return int(np.prod(self.shape))

    def memory_bytes(self) -> int:
        payload = (self.element_count() + 1) // 2 if self.format is DynQuantFormat.INT4_PER_TENSOR else self.element_count()
        return payload + 4 * int(self.scales.size)

    def compression_ratio(self) -> float:
        return 4.0 * self.element_count() / self.memory_bytes()


def dynamic_quantize_int8(x, mode: DynamicScaleMode = DynamicScaleMode.MAX_ABS, percentile: float = 0.99) -> DynQuantTensor:
    v = np.asarray(x, dtype=np.float32)
    s = compute_scale(v, 127.0, mode, percentile)
    return DynQuantTensor(np.clip(np.rint(v / s), -127, 127).astype(np.int8), np.asarray([s], dtype=np.float32), v.shape, DynQuantFormat.INT8_PER_TENSOR)


def dynamic_quantize_int8_per_row(x, mode: DynamicScaleMode = DynamicScaleMode.MAX_ABS, percentile: float = 0.99) -> DynQuantTensor:
    v = np.asarray(x, dtype=np.float32)
    if v.ndim != 2:
        raise DynQuantError("per-row quantisation needs a matrix")
    s = np.asarray([compute_scale(r, 127.0, mode, percentile) for r in v], dtype=np.float32)
    return DynQuantTensor(np.clip(np.rint(v / s[:, None]), -127, 127).astype(np.int8), s, v.shape, DynQuantFormat.INT8_PER_ROW)


def dynamic_quantize_int4(x, mode: DynamicScaleMode = DynamicScaleMode.MAX_ABS, percentile: float = 0.99) -> DynQuantTensor:
    v = np.asarray(x, dtype=np.float32)
    s = compute_scale(v, 7.0, mode, percentile)
    return DynQuantTensor(np.clip(np.rint(v / s), -7, 7).astype(np.int8), np.asarray([s], dtype=np.float32), v.shape, DynQuantFormat.INT4_PER_TENSOR)


def quantization_mae(original, q: DynQuantTensor) -> float:
    return float(np.abs(np.asarray(original, dtype=np.float32) - q.dequantize()).mean())


def w8a8_matvec(weight: DynQuantTensor, x) -> np.ndarray:
    """INT8 weights (per row or per tensor) times an activation vector quantised on the fly: integer dot products, one
    float scale per output."""
    if weight.format is DynQuantFormat.INT4_PER_TENSOR or len(weight.shape) != 2:
        raise DynQuantError("w8a8 needs an INT8 matrix")
    xq = dynamic_quantize_int8(np.asarray(x, dtype=np.float32))
    if xq.shape != (weight.shape[1],):
        raise DynQuantError(f"activation of length {xq.shape} against {weight.shape[1]} columns")
    acc = weight.data.astype(np.int32) @ xq.data.astype(np.int32)
    ws = weight.scales if weight.format is DynQuantFormat.INT8_PER_ROW else np.full(weight.shape[0], weight.scales[0], dtype=np.float32)
    return acc.astype(np.float32) * ws * xq.scales[0]


# ---- INT8 modes and error analysis --------------------------------------------------------------------------------------------
class Int8Mode(Enum):
    PER_TENSOR = "per_tensor"
    PER_CHANNEL = "per_channel"


@dataclass
class Int8QuantError:
    mae: float
    mse: float
    max_error: float
    snr_db: float
    relative_error: float


def analyze_int8_error(original, mode: Int8Mode = Int8Mode.PER_TENSOR) -> Int8QuantError:
    v = np.asarray(original, dtype=np.float32)
    q = dynamic_quantize_int8(v) if mode is Int8Mode.PER_TENSOR or v.ndim != 2 else dynamic_quantize_int8_per_row(v)
    err = v - q.dequantize()
    power, noise = float((v.astype(np.float64) ** 2).mean()), float((err.astype(np.float64) ** 2).mean())
    snr = 10.0 * math.log10(power / noise) if noise > 0 and power > 0 else math.inf
    return Int8QuantError(float(np.abs(err).mean()), noise, float(np.abs(err).max()), snr, math.sqrt(noise / power) if power > 0 else 0.0)


@dataclass
class QuantizationComparison:
    per_tensor: Int8QuantError
    per_channel: Int8QuantError
    int4: float                      # mean absolute error of per-tensor INT4
    best: str


def compare_quantization_methods(weight) -> QuantizationComparison:
    w = np.asarray(weight, dtype=np.float32)
    pt, pc = analyze_int8_error(w, Int8Mode.PER_TENSOR), analyze_int8_error(w, Int8Mode.PER_CHANNEL)
    return QuantizationComparison(pt, pc, quantization_mae(w, dynamic_quantize_int4(w)), "per_channel" if pc.mse <= pt.mse else "per_tensor")


# ---- pruning ------------------------------------------------------------------------------------------------------------------
class ImportanceMetric(Enum):
    L1_MAGNITUDE = "l1"
    L2_MAGNITUDE = "l2"
    TAYLOR_PROXY = "taylor"          # |w * gradient| with |w| standing in for the gradient
    RANDOM = "random"


class PruningGranularity(Enum):
    UNSTRUCTURED = "unstructured"
    STRUCTURED_ROW = "row"
    STRUCTURED_COLUMN = "column"


class PruningError(ValueError):
    pass


@dataclass
class PruningConfig:
    sparsity: float
    metric: ImportanceMetric = ImportanceMetric.L1_MAGNITUDE
    granularity: PruningGranularity = PruningGranularity.UNSTRUCTURED
    seed: int = 0
    skip: tuple[str, ...] = ("norm", "embd", "bias")     # tensors whose name contains one of these are left alone

    def __post_init__(self):
        if not 0.0 <= self.sparsity < 1.0:
            raise PruningError(f"sparsity must be in [0, 1), got {self.sparsity}")

    @classmethod
    def unstructured_l1(cls, sparsity: float) -> "PruningConfig":
        return cls(sparsity)

    @classmethod
    def structured_row_l2(cls, sparsity: float) -> "PruningConfig":
        return cls(sparsity, ImportanceMetric.L2_MAGNITUDE, PruningGranularity.STRUCTURED_ROW)


def compute_importance(w, metric: ImportanceMetric, seed: int = 0) -> np.ndarray:
    v = np.asarray(w, dtype=np.float32)
    if metric is ImportanceMetric.L1_MAGNITUDE:
        return np.abs(v)
    if metric in (ImportanceMetric.L2_MAGNITUDE, ImportanceMetric.TAYLOR_PROXY):
        return v * v
    return np.random.default_rng(seed).random(v.shape, dtype=np.float32)


def prune_tensor(w, config: PruningConfig) -> np.ndarray:
    v = np.array(w, dtype=np.float32, copy=True)
    score = compute_importance(v, config.metric, config.seed)
    if config.granularity is PruningGranularity.UNSTRUCTURED:
        k = int(config.sparsity * v.size)
        if k:
            idx = np.argpartition(score.reshape(-1), k - 1)[:k]
            v.reshape(-1)[idx] = 0.0
        return v
    if v.ndim != 2:
        raise PruningError("structured pruning needs a matrix")
    axis = 1 if config.granularity is PruningGranularity.STRUCTURED_ROW else 0
    group = score.sum(axis=axis)
    k = int(config.sparsity * group.size)
    if k:
        idx = np.argpartition(group, k - 1)[:k]
        if axis == 1:
            v[idx, :] = 0.0
        else:
            v[:, idx] = 0.0
    return v


@dataclass
class SparsityReport:
    name: str
    total: int
    zeros: int

    @classmethod
    def compute(cls, name: str, w) -> "SparsityReport":
        v = np.asarray(w)
        return cls(name, int(v.size), int((v == 0).sum()))

    def zero_fraction(self) -> float:
        return self.zeros / self.total if self.total else 0.0

    def density(self) -> float:
        return 1.0 - self.zero_fraction()

    def summary(self) -> str:
        return f"{self.name}: {self.zeros}/{self.total} zero ({100 * self.zero_fraction():.1f} %)"


@dataclass
class ModelSparsitySummary:
    reports: list[SparsityReport]

    @classmethod
    def from_model(cls, tensors: Tensors) -> "ModelSparsitySummary":
        return cls([SparsityReport.compute(k, v) for k, v in tensors.items()])

    def overall(self) -> float:
        t = sum(r.total for r in self.reports)
        return sum(r.zeros for r in self.reports) / t if t else 0.0

    def summary(self) -> str:
        return "\n".join([f"model sparsity {100 * self.overall():.1f} % over {len(self.reports)} tensors"] + [r.summary() for r in self.reports])


def prune_model(tensors: Tensors, config: PruningConfig) -> dict[str, np.ndarray]:
    out = {}
    for k, v in tensors.items():
        a = np.asarray(v)
        skip = a.ndim < 2 or any(s in k for s in config.skip)
        out[k] = np.array(a, dtype=np.float32, copy=True) if skip else prune_tensor(a, config)
    return out


# ---- compression pipeline -----------------------------------------------------------------------------------------------------
@dataclass
class CompressionStage:
    kind: str                        # "prune" | "quantize_int8" | "clip"
    pruning: PruningConfig | None = None
    percentile: float = 0.0

    def name(self) -> str:
        return self.kind

    @classmethod
    def prune(cls, config: PruningConfig) -> "CompressionStage":
        return cls("prune", config)

    @classmethod
    def quantize_int8(cls) -> "CompressionStage":
        return cls("quantize_int8")

    @classmethod
    def clip(cls, percentile: float) -> "CompressionStage":
        if not 0.0 < percentile <= 1.0:
            raise CompressionError("clip percentile must be in (0, 1]")
        return cls("clip", None, percentile)


class CompressionError(ValueError):
    pass


@dataclass
class CompressionConfig:
    stages: list[CompressionStage] = field(default_factory=list)

    def add_stage(self, stage: CompressionStage) -> "CompressionConfig":
        self.stages.append(stage)
        return self

    @classmethod
    def prune_then_quantize(cls, sparsity: float) -> "CompressionConfig":
        return cls([CompressionStage.prune(PruningConfig.unstructured_l1(sparsity)), CompressionStage.quantize_int8()])

    @classmethod
    def quantize_only(cls) -> "CompressionConfig":
        return cls([CompressionStage.quantize_int8()])

    @classmethod
    def prune_only(cls, sparsity: float) -> "CompressionConfig":
        return cls([CompressionStage.prune(PruningConfig.unstructured_l1(sparsity))])


@dataclass
class StageStats:
    stage: str
    params: int
    nonzero: int
    bytes_before: int
    bytes_after: int

    def compression_ratio(self) -> float:
        return self.bytes_before / self.bytes_after if self.bytes_after else math.inf

    def sparsity(self) -> float:
        return 1.0 - self.nonzero / self.params if self.params else 0.0


@dataclass
class CompressionResult:
    tensors: dict[str, np.ndarray]
    stages: list[StageStats]

    def total_params(self) -> int:
        return sum(int(v.size) for v in self.tensors.values())

    def total_nonzero(self) -> int:
        return sum(int(np.count_nonzero(v)) for v in self.tensors.values())

    def overall_sparsity(self) -> float:
        p = self.total_params()
        return 1.0 - self.total_nonzero() / p if p else 0.0

    def memory_before_bytes(self) -> int:
        return self.stages[0].bytes_before if self.stages else 4 * self.total_params()

    def memory_after_bytes(self) -> int:
        return self.stages[-1].bytes_after if self.stages else 4 * self.total_params()

    def total_compression_ratio(self) -> float:
        after = self.memory_after_bytes()
        return self.memory_before_bytes() / after if after else math.inf

    def summary(self) -> str:
        lines = [f"compression: {self.total_params()} parameters, {100 * self.overall_sparsity():.1f} % zero, "
                 f"{self.memory_before_bytes()} -> {self.memory_after_bytes()} bytes ({self.total_compression_ratio():.2f}x)"]
        lines += [f"  {s.stage}: sparsity {100 * s.sparsity():.1f} %, {s.bytes_before} -> {s.bytes_after} bytes" for s in self.stages]
        return "\n".join(lines)


def compress_model(tensors: Tensors, config: CompressionConfig) -> CompressionResult:
    """Runs the stages in order.  Sizes are what the stage's representation would need: 4 bytes per parameter in float
    form, 1 byte per parameter after INT8 (the tensors themselves stay float: INT8 rounding is simulated); pruning and
    clipping change the zero count, not the dense size."""
    if not config.stages:
        raise CompressionError("no stages configured")
    cur = {k: np.array(v, dtype=np.float32, copy=True) for k, v in tensors.items()}
    bytes_per_param, stats = 4, []
    for st in config.stages:
        before = bytes_per_param * sum(int(v.size) for v in cur.values())
        if st.kind == "prune":
            cur = prune_model(cur, st.pruning)
        elif st.kind == "quantize_int8":
            cur = {k: (dynamic_quantize_int8(v).dequantize() if v.ndim >= 2 else v) for k, v in cur.items()}
            bytes_per_param = 1
        elif st.kind == "clip":
            for k, v in cur.items():
                if v.ndim >= 2 and v.size:
                    thr = float(np.quantile(np.abs(v), st.percentile))
                    v[np.abs(v) < thr] = 0.0
        else:
            raise CompressionError(f"unknown stage {st.kind!r}")
        params = sum(int(v.size) for v in cur.values())
        stats.append(StageStats(st.name(), params, sum(int(np.count_nonzero(v)) for v in cur.values()), before, bytes_per_param * params))
    return CompressionResult(cur, stats)


def estimate_compressed_size(total_params: int, config: CompressionConfig) -> int:
    """Dense bytes after the pipeline (pruned weights are still stored)."""
    return total_params * (1 if any(s.kind == "quantize_int8" for s in config.stages) else 4)


# ---- merge statistics ---------------------------------------------------------------------------------------------------------
@dataclass
class MergeStats:
    tensors: int
    parameters: int
    mean_cosine_similarity: float     # between the two inputs, tensor by tensor
    mean_l2_distance: float
    max_abs_change: float             # of the merged model against the first input

    def summary(self) -> str:
        return (f"merged {self.tensors} tensors ({self.parameters} parameters): input cosine {self.mean_cosine_similarity:.4f}, "
                f"input L2 distance {self.mean_l2_distance:.4g}, largest change {self.max_abs_change:.4g}")


def merge_stats(a: Tensors, b: Tensors, merged: Tensors) -> MergeStats:
    cos, dist, change, params = [], [], 0.0, 0
    for k in a:
        x, y = np.asarray(a[k], dtype=np.float64).reshape(-1), np.asarray(b[k], dtype=np.float64).reshape(-1)
        nx, ny = np.linalg.norm(x), np.linalg.norm(y)
        cos.append(float(x @ y / (nx * ny)) if nx > 0 and ny > 0 else 0.0)
        dist.append(float(np.linalg.norm(x - y)))
        change = max(change, float(np.abs(np.asarray(merged[k], dtype=np.float64).reshape(-1) - x).max()) if x.size else 0.0)
        params += x.size
    n = max(1, len(cos))
    return MergeStats(len(cos), params, sum(cos) / n, sum(dist) / n, change)


# ---- SmoothQuant calibrator ---------------------------------------------------------------------------------------------------
class SmoothQuantError(ValueError):
    pass


class SmoothQuantCalibrator:
    """Per-layer running maximum of |activation| per input channel; ``smooth_factors`` balances it against the weights:
    ``s_j = max|X_j|^alpha / max|W_j|^(1 - alpha)``, activations are divided by s and weight columns multiplied by it."""

    def __init__(self, alpha: float = 0.5):
        if not 0.0 <= alpha <= 1.0:
            raise SmoothQuantError("alpha must be in [0, 1]")
        self.alpha = alpha
        self._absmax: dict[str, np.ndarray] = {}

    def record_activation(self, layer: str, activations) -> None:
        a = np.abs(np.asarray(activations, dtype=np.float32))
        a = a.reshape(-1, a.shape[-1]).max(axis=0)
        cur = self._absmax.get(layer)
        if cur is not None and cur.shape != a.shape:
            raise SmoothQuantError(f"{layer}: channel count changed from {cur.shape[0]} to {a.shape[0]}")
        self._absmax[layer] = a if cur is None else np.maximum(cur, a)

    def layer_count(self) -> int:
        return len(self._absmax)

    def has_layer(self, layer: str) -> bool:
        return layer in self._absmax

    def smooth_factors(self, layer: str, weight) -> np.ndarray:
        if layer not in self._absmax:
            raise SmoothQuantError(f"no activations recorded for {layer}")
        w = np.abs(np.asarray(weight, dtype=np.float32))
        if w.ndim != 2 or w.shape[1] != self._absmax[layer].shape[0]:
            raise SmoothQuantError(f"{layer}: weight of shape {w.shape} against {self._absmax[layer].shape[0]} channels")
        act, wmax = np.maximum(self._absmax[layer], 1e-5), np.maximum(w.max(axis=0), 1e-5)
        return (act ** self.alpha / wmax ** (1.0 - self.alpha)).astype(np.float32)

    def quantize_fp8_smooth(self, layer: str, weight, fmt: str = "e4m3") -> tuple[np.ndarray, np.ndarray]:
        """(FP8 block bytes of the smoothed weight, the factors the activations must be divided by)."""
        from ..core.blocks import quantize
        ty = {"e4m3": G.F8_E4M3, "e5m2": G.F8_E5M2}.get(fmt)
        if ty is None:
            raise SmoothQuantError(f"unknown FP8 format {fmt!r}")
        s = self.smooth_factors(layer, weight)
        return quantize(ty, np.asarray(weight, dtype=np.float32) * s[None, :]), s


# ---- export planning ----------------------------------------------------------------------------------------------------------
class ExportFormat(Enum):
    Q1_0_G128 = "q1_0_g128"
    TQ2_0_G128 = "tq2_0_g128"
    Q8_0 = "q8_0"
    F16 = "f16"
    F32 = "f32"

    def type_id(self) -> int:
        return {"q1_0_g128": G.Q1_0_G128, "tq2_0_g128": G.TQ2_0_G128, "q8_0": G.Q8_0, "f16": G.F16, "f32": G.F32}[self.value]


@dataclass
class ExportConfig:
    format: ExportFormat = ExportFormat.TQ2_0_G128
    fp32_layers: tuple[str, ...] = ()
    description: str = ""

    def with_fp32_layers(self, names: Iterable[str]) -> "ExportConfig":
        self.fp32_layers = tuple(names)
        return self

    def with_description(self, text: str) -> "ExportConfig":
        self.description = text
        return self

    @staticmethod
    def default_fp32_exceptions() -> tuple[str, ...]:
        """Name fragments of tensors that are never quantised: normalisation weights and biases."""
        return ("norm", "bias")

    def type_for(self, name: str, shape: Sequence[int]) -> int:
        if len(shape) < 2 or any(f in name for f in self.default_fp32_exceptions()) or name in self.fp32_layers:
            return G.F32
        _, block, _ = G.type_info(self.format.type_id())
        return self.format.type_id() if shape[-1] % block == 0 else G.F16       # rows that do not fill blocks stay in F16


@dataclass
class ExportStats:
    tensors: int
    quantized: int
    kept_float: int
    bytes_f32: int
    bytes_out: int

    def compression_ratio(self) -> float:
        return self.bytes_f32 / self.bytes_out if self.bytes_out else math.inf


def export_stats(shapes: Mapping[str, Sequence[int]], config: ExportConfig) -> ExportStats:
    q = kept = b32 = bout = 0
    for name, shape in shapes.items():
        n = int(np.prod(shape)) if len(shape) else 1
        ty = config.type_for(name, shape)
        b32 += 4 * n
        bout += G.data_size(ty, n)
        if ty in (G.F32, G.F16):
            kept += 1
        else:
            q += 1
    return ExportStats(len(shapes), q, kept, b32, bout)


def estimate_export_size(shapes: Mapping[str, Sequence[int]], config: ExportConfig) -> int:
    return export_stats(shapes, config).bytes_out


def export_to_gguf(tensors: Tensors, path: str, config: ExportConfig, metadata: Mapping[str, object] | None = None) -> ExportStats:
    """Writes ``tensors`` (row-major float arrays) as a GGUF file in the configured format."""
    from ..core.blocks import quantize
    w = G.GgufWriter()
    for k, v in (metadata or {}).items():
        w.add(k, v)
    if config.description:
        w.add("general.description", config.description)
    for name, arr in tensors.items():
        a = np.asarray(arr, dtype=np.float32)
        ty = config.type_for(name, a.shape)
        if ty == G.F32:
            blob = np.ascontiguousarray(a).view(np.uint8).reshape(-1)
        elif ty == G.F16:
            blob = a.astype(np.float16).view(np.uint8).reshape(-1)
        else:
            blob = quantize(ty, a)
        w.add_tensor(name, tuple(reversed(a.shape)), ty, blob)
    w.write(path)
    return export_stats({k: np.asarray(v).shape for k, v in tensors.items()}, config)
