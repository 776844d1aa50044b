"""CPU kernel tiers and the kernel dispatcher.

Reference: crates/oxibonsai-kernels/src/dispatch.rs:26-201 (``KernelTier`` Reference / Avx2 / Avx512 / Neon / Gpu,
``KernelDispatcher::auto_detect``, GPU first for matrices of at least ``GPU_MIN_ROWS`` rows, GPU errors fall back to the
CPU), traits.rs (``OneBitKernel`` / ``TernaryKernel``: dequant, gemv, gemm, cached device weights), error.rs
(``KernelError``: NotBlockAligned, DimensionMismatch, BufferTooSmall, GpuError, UnsupportedOperation), weight_cache.rs
(``GpuWeightHandle``), aligned.rs and tuning.rs.  This project has exactly two backends: the sm_100a kernels and the C++
CPU tiers (csrc/cpu/kernels.cpp); there is no multi-vendor dispatch.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from enum import IntEnum

import numpy as np

from .. import _native
from ..core import gguf as G

GPU_MIN_ROWS = 1024


class KernelError(RuntimeError):
    pass


class NotBlockAligned(KernelError):
    pass


class DimensionMismatch(KernelError):
    pass


class BufferTooSmall(KernelError):
    pass


class GpuError(KernelError):
    pass


class UnsupportedOperation(KernelError):
    pass


class KernelTier(IntEnum):
    REFERENCE = 0
    AVX2 = 1
    AVX512 = 2
    GPU = 10

    @property
    def is_accelerated(self) -> bool:
        return self != KernelTier.REFERENCE


def _lib():
    lib = _native.host()
    if "bcpu_gemv_tiered" not in lib._declared:
        vp, i, u32, u64, f = C.c_void_p, C.c_int, C.c_uint32, C.c_uint64, C.c_float
        _native.declare(lib, {
            "bcpu_detect_tier": (i, []), "bcpu_active_tier": (i, []), "bcpu_set_tier": (i, [i]), "bcpu_tier_name": (C.c_char_p, [i]),
            "bcpu_gemv_tiered": (i, [u32, vp, u64, u64, vp, vp, i, i]), "bcpu_gemm_tiered": (i, [u32, vp, u64, u64, vp, u64, vp, i]),
            "bcpu_rmsnorm_tiered": (None, [vp, vp, vp, u64, f, i]), "bcpu_silu": (None, [vp, vp, u64]), "bcpu_swiglu_tiered": (None, [vp, vp, vp, u64]),
            "bcpu_softmax": (None, [vp, vp, u64]), "bcpu_rope_apply": (None, [vp, u64, u64, vp, vp]),
            "bcpu_silu_t": (None, [vp, vp, u64, i]), "bcpu_swiglu_t": (None, [vp, vp, vp, u64, i]), "bcpu_softmax_t": (None, [vp, vp, u64, i]),
            "bcpu_rope_apply_t": (None, [vp, u64, u64, vp, vp, i]),
            "bcpu_aligned_alloc": (vp, [u64]), "bcpu_aligned_free": (None, [vp]),
            "bcpu_working_set_bytes": (u64, [u32, u64, u64]), "bcpu_optimal_tile_rows": (u64, [u32, u64, u64]),
            "bcpu_select_strategy": (i, [u64, u64, u64]), "bcpu_prefetch_range": (None, [vp, u64, i, i]),
            "bcpu_pack_rows_tiled": (i, [vp, u64, u64, u64, u64, vp, i]),
            "bcpu_gemv_tiled": (i, [u32, vp, u64, u64, vp, vp, u64, i]), "bcpu_gemm_tiled": (i, [u32, vp, u64, u64, vp, u64, vp, u64, u64, i]),
            "bcpu_gemv_adaptive": (i, [u32, vp, u64, u64, vp, vp]), "bcpu_gemm_adaptive": (i, [u32, vp, u64, u64, vp, u64, vp])})
        lib._declared.add("bcpu_gemv_tiered")
    return lib


def detect_tier() -> KernelTier:
    return KernelTier(_lib().bcpu_detect_tier())


def set_tier(tier: KernelTier | int | None) -> KernelTier:
    return KernelTier(_lib().bcpu_set_tier(-1 if tier is None else int(tier)))


def tier_name(tier: int) -> str:
    return "gpu" if tier == KernelTier.GPU else _lib().bcpu_tier_name(int(tier)).decode()


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# (elements, bytes) of one block of the row formats the CPU tiers read
_ROW_FORMATS = {G.Q1_0_G128: (128, 18), G.TQ2_0_G128: (128, 34), G.F8_E4M3: (32, 34), G.F8_E5M2: (32, 34)}


def _check_matrix(type_id: int, data: np.ndarray, rows: int, cols: int) -> np.ndarray:
    if type_id not in _ROW_FORMATS:
        raise UnsupportedOperation(f"tiered CPU kernels cover Q1_0_g128, TQ2_0_g128 and the FP8 blocks, not type {type_id}")
    elems, nbytes = _ROW_FORMATS[type_id]
    if cols % elems:
        raise NotBlockAligned(f"row length {cols} is not a multiple of {elems}")
    raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    need = rows * (cols // elems) * nbytes
    if raw.size < need:
        raise BufferTooSmall(f"matrix needs {need} bytes, got {raw.size}")
    return raw


def gemv(type_id: int, data, rows: int, cols: int, x, tier: KernelTier | int | None = None, threads: int = 0) -> np.ndarray:
    raw, xv = _check_matrix(type_id, data, rows, cols), _f32(x)
    if xv.size != cols:
        raise DimensionMismatch(f"x has {xv.size} elements, expected {cols}")
    out = np.empty(rows, dtype=np.float32)
    rc = _lib().bcpu_gemv_tiered(type_id, raw.ctypes.data, rows, cols, xv.ctypes.data, out.ctypes.data, -1 if tier is None else int(tier), threads)
    if rc != 0:
        raise KernelError(f"cpu gemv failed with code {rc}")
    return out


def gemm(type_id: int, data, rows: int, cols: int, x, threads: int = 0) -> np.ndarray:
    """``x`` [batch, cols] -> [batch, rows]."""
    raw, xv = _check_matrix(type_id, data, rows, cols), _f32(x)
    if xv.ndim != 2 or xv.shape[1] != cols:
        raise DimensionMismatch(f"x has shape {xv.shape}, expected [batch, {cols}]")
    out = np.empty((xv.shape[0], rows), dtype=np.float32)
    rc = _lib().bcpu_gemm_tiered(type_id, raw.ctypes.data, rows, cols, xv.ctypes.data, xv.shape[0], out.ctypes.data, threads)
    if rc != 0:
        raise KernelError(f"cpu gemm failed with code {rc}")
    return out


class Strategy(IntEnum):
    """How the adaptive entry points run a product (reference: ``AdaptiveStrategy``, parallel_tiled.rs:259-281)."""
    DIRECT = 0
    PARALLEL_ROWS = 1
    PARALLEL_TILED = 2


def select_strategy(rows: int, cols: int, batch: int = 1) -> Strategy:
    return Strategy(_lib().bcpu_select_strategy(rows, cols, batch))


def working_set_bytes(type_id: int, rows: int, cols: int) -> int:
    """Packed weights + input + output of a GEMV (0 for an unknown format or a ragged row)."""
    return int(_lib().bcpu_working_set_bytes(type_id, rows, cols))


def fits_in_cache(type_id: int, rows: int, cols: int, cache_bytes: int = 32 * 1024) -> bool:
    ws = working_set_bytes(type_id, rows, cols)
    return 0 < ws <= cache_bytes


def optimal_tile_rows(type_id: int, cols: int, cache_bytes: int = 0) -> int:
    """Rows per tile whose weights stay in ``cache_bytes`` beside the input vector (default: a 32 KB L1), within [4, 256]."""
    return int(_lib().bcpu_optimal_tile_rows(type_id, cols, cache_bytes))


def prefetch_range(array: np.ndarray, locality: int = 3, write: bool = False) -> None:
    """Prefetch hints for every cache line of ``array`` (locality 0 = streamed once .. 3 = keep in all cache levels)."""
    a = np.ascontiguousarray(array)
    _lib().bcpu_prefetch_range(a.ctypes.data, a.nbytes, int(locality), int(write))


def pack_rows_tiled(type_id: int, data, rows: int, cols: int, tile: int = 32, unpack: bool = False) -> np.ndarray:
    """Block order for a GEMV that walks ``tile`` rows block column by block column: inside every tile, block 0 of every row,
    then block 1 of every row, ...  ``unpack=True`` inverts it (reference: ``pack_blocks_for_gemv`` / ``unpack_blocks_from_gemv``,
    packing.rs:122-215)."""
    raw = _check_matrix(type_id, data, rows, cols)
    elems, nbytes = _ROW_FORMATS[type_id]
    n = rows * (cols // elems) * nbytes
    out = np.empty(n, dtype=np.uint8)
    rc = _lib().bcpu_pack_rows_tiled(raw.ctypes.data, rows, cols // elems, nbytes, tile, out.ctypes.data, int(unpack))
    if rc != 0:
        raise KernelError(f"pack_rows_tiled failed with code {rc}")
    return out


def gemv_tiled(type_id: int, data, rows: int, cols: int, x, tile_rows: int = 0, threads: int = 0) -> np.ndarray:
    """GEMV over row tiles sized for the cache (``tile_rows`` 0 = :func:`optimal_tile_rows`), tiles handed to threads from a
    shared counter with the next tile prefetched (reference: ``gemv_tiled_par``, ``gemv_parallel_tiled``)."""
    raw, xv = _check_matrix(type_id, data, rows, cols), _f32(x)
    if xv.size != cols:
        raise DimensionMismatch(f"x has {xv.size} elements, expected {cols}")
    out = np.empty(rows, dtype=np.float32)
    rc = _lib().bcpu_gemv_tiled(type_id, raw.ctypes.data, rows, cols, xv.ctypes.data, out.ctypes.data, tile_rows, threads)
    if rc != 0:
        raise KernelError(f"cpu tiled gemv failed with code {rc}")
    return out


def gemm_tiled(type_id: int, data, rows: int, cols: int, x, tile_rows: int = 0, tile_batch: int = 0, threads: int = 0) -> np.ndarray:
    """Batch GEMM tiled over weight rows (decoded once per tile) and over the batch (reference: ``gemm_tiled_par``)."""
    raw, xv = _check_matrix(type_id, data, rows, cols), _f32(x)
    if xv.ndim != 2 or xv.shape[1] != cols:
        raise DimensionMismatch(f"x has shape {xv.shape}, expected [batch, {cols}]")
    out = np.empty((xv.shape[0], rows), dtype=np.float32)
    rc = _lib().bcpu_gemm_tiled(type_id, raw.ctypes.data, rows, cols, xv.ctypes.data, xv.shape[0], out.ctypes.data, tile_rows, tile_batch, threads)
    if rc != 0:
        raise KernelError(f"cpu tiled gemm failed with code {rc}")
    return out


def gemv_adaptive(type_id: int, data, rows: int, cols: int, x) -> tuple[np.ndarray, Strategy]:
    """GEMV by the strategy :func:`select_strategy` picks for the shape; returns the result and the strategy used."""
    raw, xv = _check_matrix(type_id, data, rows, cols), _f32(x)
    if xv.size != cols:
        raise DimensionMismatch(f"x has {xv.size} elements, expected {cols}")
    out = np.empty(rows, dtype=np.float32)
    rc = _lib().bcpu_gemv_adaptive(type_id, raw.ctypes.data, rows, cols, xv.ctypes.data, out.ctypes.data)
    if rc < 0:
        raise KernelError(f"cpu adaptive gemv failed with code {rc}")
    return out, Strategy(rc)


def gemm_adaptive(type_id: int, data, rows: int, cols: int, x) -> tuple[np.ndarray, Strategy]:
    raw, xv = _check_matrix(type_id, data, rows, cols), _f32(x)
    if xv.ndim != 2 or xv.shape[1] != cols:
        raise DimensionMismatch(f"x has shape {xv.shape}, expected [batch, {cols}]")
    out = np.empty((xv.shape[0], rows), dtype=np.float32)
    rc = _lib().bcpu_gemm_adaptive(type_id, raw.ctypes.data, rows, cols, xv.ctypes.data, xv.shape[0], out.ctypes.data)
    if rc < 0:
        raise KernelError(f"cpu adaptive gemm failed with code {rc}")
    return out, Strategy(rc)


def rms_norm(x, w, eps: float = 1e-6, tier: int = 1) -> np.ndarray:
    xv, wv = _f32(x), _f32(w)
    if xv.size != wv.size:
        raise DimensionMismatch("x and weight differ in length")
    out = np.empty_like(xv)
    _lib().bcpu_rmsnorm_tiered(xv.ctypes.data, wv.ctypes.data, out.ctypes.data, xv.size, eps, tier)
    return out


def silu(x, tier: int = 0) -> np.ndarray:
    """``tier`` 0: scalar body (the oracle's arithmetic); >= 1: AVX2 + FMA with a polynomial exp (agrees to rounding)."""
    xv = _f32(x)
    out = np.empty_like(xv)
    _lib().bcpu_silu_t(xv.ctypes.data, out.ctypes.data, xv.size, int(tier))
    return out


def swiglu(gate, up, tier: int = 0) -> np.ndarray:
    g, u = _f32(gate), _f32(up)
    if g.size != u.size:
        raise DimensionMismatch("gate and up differ in length")
    out = np.empty_like(g)
    _lib().bcpu_swiglu_t(g.ctypes.data, u.ctypes.data, out.ctypes.data, g.size, int(tier))
    return out


def softmax(x, tier: int = 0) -> np.ndarray:
    xv = _f32(x)
    out = np.empty_like(xv)
    _lib().bcpu_softmax_t(xv.ctypes.data, out.ctypes.data, xv.size, int(tier))
    return out


def rope_apply(x, cos, sin, tier: int = 0) -> np.ndarray:
    """x [heads, head_dim] rotated in the half-split convention by cos / sin [head_dim / 2].  The vectorised tier uses
    separate multiplies and adds, so its result equals the scalar one bit for bit."""
    xv = np.array(x, dtype=np.float32, copy=True, order="C")
    c, s = _f32(cos), _f32(sin)
    if xv.ndim != 2 or c.size != xv.shape[1] // 2 or s.size != c.size:
        raise DimensionMismatch("need x [heads, head_dim] and cos / sin [head_dim / 2]")
    _lib().bcpu_rope_apply_t(xv.ctypes.data, xv.shape[0], xv.shape[1], c.ctypes.data, s.ctypes.data, int(tier))
    return xv


class AlignedBuffer:
    """64-byte aligned host memory exposed as a numpy array."""

    def __init__(self, n: int, dtype=np.float32):
        self._lib = _lib()
        nbytes = int(n) * np.dtype(dtype).itemsize
        self._p = self._lib.bcpu_aligned_alloc(max(nbytes, 1))
        if not self._p:
            raise MemoryError(f"cannot allocate {nbytes} aligned bytes")
        self.array = np.frombuffer((C.c_uint8 * nbytes).from_address(self._p), dtype=dtype)

    @property
    def address(self) -> int:
        return self._p

    def __del__(self):
        if getattr(self, "_p", None):
            self._lib.bcpu_aligned_free(self._p)
            self._p = None


@dataclass(frozen=True)
class GpuWeightHandle:
    """Opaque id of a matrix cached on the device."""
    id: int


@dataclass
class TuningThresholds:
    gpu_min_rows: int = GPU_MIN_ROWS
    parallel_min_rows: int = 64
    threads: int = 0

    @classmethod
    def for_this_machine(cls) -> "TuningThresholds":
        return cls(threads=os.cpu_count() or 1)


class KernelDispatcher:
    """Chooses between the GPU kernels and the CPU tiers per call, falling back to the CPU when a GPU call fails."""

    def __init__(self, tier: KernelTier | None = None, thresholds: TuningThresholds | None = None):
        self.thresholds = thresholds or TuningThresholds.for_this_machine()
        self.tier = tier if tier is not None else self.auto_detect_tier()
        self.gpu_fallbacks = 0
        self._weights: dict[int, object] = {}
        self._next = 1

    @staticmethod
    def auto_detect_tier() -> KernelTier:
        try:
            import torch
            if torch.cuda.is_available():
                return KernelTier.GPU
        except Exception:
            pass
        return detect_tier()

    @classmethod
    def auto_detect(cls) -> "KernelDispatcher":
        return cls()

    def cpu_tier(self) -> KernelTier:
        return detect_tier() if self.tier == KernelTier.GPU else self.tier

    def upload_weights(self, type_id: int, data, rows: int, cols: int) -> GpuWeightHandle:
        """Repacks a matrix into the device layout once; later ``gemv_cached`` calls reuse it."""
        import torch
        from . import cuda_ops as K
        raw = torch.from_numpy(np.ascontiguousarray(data).view(np.uint8).reshape(-1).copy()).cuda()
        pw = K.PlanarWeight(rows, cols, raw.device).fill_from_gguf(raw, type_id, cols, 0, rows)
        h = GpuWeightHandle(self._next)
        self._next += 1
        self._weights[h.id] = pw
        return h

    def gemv_cached(self, handle: GpuWeightHandle, x) -> np.ndarray:
        import torch
        from . import cuda_ops as K
        pw = self._weights[handle.id]
        return K.bitgemv(pw, torch.as_tensor(np.asarray(x, dtype=np.float32)).cuda()).cpu().numpy()

    def gemv(self, type_id: int, data, rows: int, cols: int, x) -> np.ndarray:
        if self.tier == KernelTier.GPU and rows >= self.thresholds.gpu_min_rows:
            try:
                h = self.upload_weights(type_id, data, rows, cols)
                try:
                    return self.gemv_cached(h, x)
                finally:
                    self._weights.pop(h.id, None)
            except Exception:
                self.gpu_fallbacks += 1
        return gemv(type_id, data, rows, cols, x, self.cpu_tier(), self.thresholds.threads if rows >= self.thresholds.parallel_min_rows else 1)

    def gemm(self, type_id: int, data, rows: int, cols: int, x) -> np.ndarray:
        return gemm(type_id, data, rows, cols, x, self.thresholds.threads)

    def describe(self) -> str:
        return f"tier={tier_name(self.tier)} cpu={tier_name(self.cpu_tier())} gpu_min_rows={self.thresholds.gpu_min_rows} threads={self.thresholds.threads}"
