"""Block codecs: quantise / dequantise GGUF weight blocks with the C++ implementations.

Reference surface: ``BlockQ1_0G128`` (crates/oxibonsai-core/src/tensor.rs:25), ``BlockTQ2_0_g128``
(quant_ternary.rs:64), ``BlockTQ2_0``, ``BlockQ4_0`` / ``BlockQ8_0`` (quant_std.rs), FP8 blocks
(quant_fp8.rs).
"""
from __future__ import annotations

import numpy as np

from .. import _native
from .gguf import type_info


def dequantize(type_id: int, data: bytes | np.ndarray) -> np.ndarray:
    """Decodes whole blocks of ``type_id`` into float32."""
    lib = _native.host()
    src = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1))
    _, be, bb = type_info(type_id)
    if src.size % bb:
        raise ValueError(f"{src.size} bytes is not a whole number of {bb}-byte blocks")
    nblk = src.size // bb
    out = np.empty(nblk * be, dtype=np.float32)
    _native.check(lib.bonsai_dequant(type_id, src.ctypes.data, nblk, out.ctypes.data))
    return out


def quantize(type_id: int, values: np.ndarray, q1_absmax: bool = False) -> np.ndarray:
    """Encodes float32 values (a whole number of blocks) into ``type_id`` bytes."""
    lib = _native.host()
    src = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    _, be, bb = type_info(type_id)
    if src.size % be:
        raise ValueError(f"{src.size} values is not a multiple of the block size {be}")
    nblk = src.size // be
    out = np.empty(nblk * bb, dtype=np.uint8)
    _native.check(lib.bonsai_quant(type_id, src.ctypes.data, nblk, out.ctypes.data, 1 if q1_absmax else 0))
    return out


def fp8_encode(v: float, e5m2: bool = False) -> int:
    return _native.host().bonsai_fp8_encode(float(v), int(e5m2))


def fp8_decode(q: int, e5m2: bool = False) -> float:
    return _native.host().bonsai_fp8_decode(int(q), int(e5m2))
