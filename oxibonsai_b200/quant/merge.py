"""Model merging on named float tensors: linear, SLERP, task vectors, TIES and DARE.

Reference: crates/oxibonsai-model/src/model_merge.rs (linear / SLERP / TIES / DARE / task-vector merges over tensor maps).
"""
from __future__ import annotations

from typing import Mapping, Sequence

import numpy as np

Tensors = Mapping[str, np.ndarray]


def _check(models: Sequence[Tensors]) -> list[str]:
    keys = list(models[0].keys())
    for m in models[1:]:
        if set(m.keys()) != set(keys):
            raise ValueError("models have different tensor names")
        for k in keys:
            if m[k].shape != models[0][k].shape:
                raise ValueError(f"shape mismatch for {k}: {m[k].shape} vs {models[0][k].shape}")
    return keys


def linear_merge(models: Sequence[Tensors], weights: Sequence[float] | None = None, normalize: bool = True) -> dict[str, np.ndarray]:
    w = np.ones(len(models)) if weights is None else np.asarray(weights, dtype=np.float64)
    if len(w) != len(models):
        raise ValueError("one weight per model")
    if normalize:
        w = w / w.sum()
    return {k: sum(wi * m[k].astype(np.float32) for wi, m in zip(w, models)).astype(np.float32) for k in _check(models)}


def slerp(a: np.ndarray, b: np.ndarray, t: float, eps: float = 1e-8) -> np.ndarray:
    """Spherical interpolation of two tensors seen as flat vectors; falls back to lerp when nearly colinear."""
    a32, b32 = a.astype(np.float32).reshape(-1), b.astype(np.float32).reshape(-1)
    na, nb = np.linalg.norm(a32), np.linalg.norm(b32)
    if na < eps or nb < eps:
        return ((1 - t) * a32 + t * b32).reshape(a.shape)
    cos = float(np.clip(np.dot(a32 / na, b32 / nb), -1.0, 1.0))
    omega = np.arccos(cos)
    if abs(np.sin(omega)) < 1e-6:
        return ((1 - t) * a32 + t * b32).reshape(a.shape)
    out = (np.sin((1 - t) * omega) * a32 + np.sin(t * omega) * b32) / np.sin(omega)
    return out.astype(np.float32).reshape(a.shape)


def slerp_merge(a: Tensors, b: Tensors, t: float) -> dict[str, np.ndarray]:
    return {k: slerp(a[k], b[k], t) for k in _check([a, b])}


def task_vector(finetuned: Tensors, base: Tensors) -> dict[str, np.ndarray]:
    return {k: finetuned[k].astype(np.float32) - base[k].astype(np.float32) for k in _check([finetuned, base])}


def apply_task_vectors(base: Tensors, vectors: Sequence[Tensors], scale: float = 1.0) -> dict[str, np.ndarray]:
    return {k: (base[k].astype(np.float32) + scale * sum(v[k] for v in vectors)).astype(np.float32) for k in base}


def ties_merge(base: Tensors, finetuned: Sequence[Tensors], density: float = 0.2, scale: float = 1.0) -> dict[str, np.ndarray]:
    """TIES: trim each task vector to its top-``density`` magnitudes, elect a sign per entry by total mass, average the
    entries that agree with the elected sign."""
    out = {}
    for k in _check([base, *finetuned]):
        tv = np.stack([f[k].astype(np.float32) - base[k].astype(np.float32) for f in finetuned]).reshape(len(finetuned), -1)
        keep = max(1, int(round(density * tv.shape[1])))
        if keep < tv.shape[1]:
            thr = np.partition(np.abs(tv), tv.shape[1] - keep, axis=1)[:, tv.shape[1] - keep][:, None]
            tv = np.where(np.abs(tv) >= thr, tv, 0.0)
        sign = np.sign(tv.sum(axis=0))
        agree = (np.sign(tv) == sign[None, :]) & (tv != 0)
        cnt = np.maximum(agree.sum(axis=0), 1)
        merged = (tv * agree).sum(axis=0) / cnt
        out[k] = (base[k].astype(np.float32) + scale * merged.reshape(base[k].shape)).astype(np.float32)
    return out


def dare_merge(base: Tensors, finetuned: Sequence[Tensors], drop_rate: float = 0.9, seed: int = 0, weights: Sequence[float] | None = None) -> dict[str, np.ndarray]:
    """DARE: randomly drop a fraction of every task vector and rescale the survivors by 1/(1-p), then add them up."""
    if not 0.0 <= drop_rate < 1.0:
        raise ValueError("drop_rate must be in [0, 1)")
    rng = np.random.default_rng(seed)
    w = np.ones(len(finetuned)) if weights is None else np.asarray(weights, dtype=np.float64)
    out = {}
    for k in _check([base, *finetuned]):
        acc = np.zeros(base[k].shape, dtype=np.float32)
        for wi, f in zip(w, finetuned):
            tv = f[k].astype(np.float32) - base[k].astype(np.float32)
            mask = rng.random(tv.shape) >= drop_rate
            acc += wi * tv * mask / (1.0 - drop_rate)
        out[k] = base[k].astype(np.float32) + acc
    return out
