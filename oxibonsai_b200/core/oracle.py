"""CPU oracle and CPU reference ops (C++), plus the synthetic checkpoint generator.

The oracle restates the reference's scalar forward (crates/oxibonsai-model/src/model/types/mod.rs:633-934)
and is the ground truth for the greedy token-stream gate.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .. import _native
from .._native import check
from .gguf import GgufFile, Qwen3Config, TQ2_0_G128

EOS_TOKEN = 151645


class Oracle:
    def __init__(self, gguf: GgufFile, max_seq: int = 4096):
        self._lib = _native.host()
        self._gguf = gguf
        self._h = self._lib.boracle_new(gguf.handle, max_seq)
        if not self._h:
            raise _native.last_error()
        self.config = gguf.config()

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.boracle_free(self._h)
            self._h = None

    def forward(self, token: int, pos: int) -> np.ndarray:
        logits = np.empty(self.config.vocab, dtype=np.float32)
        check(self._lib.boracle_forward(self._h, token, pos, logits.ctypes.data))
        return logits

    def last_hidden(self) -> np.ndarray:
        out = np.empty(self.config.hidden, dtype=np.float32)
        check(self._lib.boracle_last_hidden(self._h, out.ctypes.data, out.size))
        return out

    def keep_layer_hidden(self, on: bool = True) -> None:
        """Keeps the residual stream after every layer of each forward (read it with :meth:`layer_hidden`)."""
        self._lib.boracle_keep_layer_hidden.argtypes = [C.c_void_p, C.c_int]
        self._lib.boracle_keep_layer_hidden(self._h, int(on))

    def layer_hidden(self) -> np.ndarray:
        out = np.empty((self.config.layers, self.config.hidden), dtype=np.float32)
        self._lib.boracle_layer_hidden.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        self._lib.boracle_layer_hidden.restype = C.c_int
        if self._lib.boracle_layer_hidden(self._h, out.ctypes.data, out.size) != 0:
            raise RuntimeError("layer hidden states are not being kept; call keep_layer_hidden() before forward()")
        return out

    def generate_greedy(self, prompt, max_new: int, stop_at_eos: bool = True):
        """Returns (token ids, per-step top-1 minus top-2 logit gaps)."""
        p = np.ascontiguousarray(prompt, dtype=np.uint32)
        out = np.zeros(max_new, dtype=np.uint32)
        gaps = np.zeros(max_new, dtype=np.float32)
        n = check(self._lib.boracle_generate(self._h, p.ctypes.data, p.size, max_new, out.ctypes.data, gaps.ctypes.data, int(stop_at_eos)))
        return out[:n].tolist(), gaps[: min(max_new, n + 1)].tolist()


def cpu_gemv(type_id: int, data: np.ndarray, rows: int, cols: int, x: np.ndarray) -> np.ndarray:
    lib = _native.host()
    d = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    xv = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(rows, dtype=np.float32)
    check(lib.bcpu_gemv(type_id, d.ctypes.data, rows, cols, xv.ctypes.data, out.ctypes.data))
    return out


def cpu_rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    xv, wv = np.ascontiguousarray(x, dtype=np.float32), np.ascontiguousarray(w, dtype=np.float32)
    out = np.empty_like(xv)
    _native.host().bcpu_rmsnorm(xv.ctypes.data, wv.ctypes.data, out.ctypes.data, xv.size, eps)
    return out


def cpu_rope(x: np.ndarray, pos: int, base: float) -> np.ndarray:
    out = np.array(x, dtype=np.float32, copy=True)
    _native.host().bcpu_rope(out.ctypes.data, out.size, pos, base)
    return out


def cpu_argmax_last(x: np.ndarray) -> int:
    xv = np.ascontiguousarray(x, dtype=np.float32)
    return _native.host().bcpu_argmax_last(xv.ctypes.data, xv.size)


def write_synthetic_gguf(path: str, cfg: Qwen3Config, weight_type: int = TQ2_0_G128, tied: bool = True,
                         seed: int = 42, llm_keys: bool = False) -> str:
    """Writes a seeded random-init checkpoint of shape ``cfg`` (see csrc/cpu/oracle.hpp)."""
    check(_native.host().bonsai_write_synthetic(str(path).encode(), cfg.packed_u32(), cfg.packed_f32(), cfg.name.encode(),
                                                weight_type, int(tied), seed, int(llm_keys)))
    return str(path)


def rope_table(head_dim: int, max_pos: int, base: float) -> tuple[np.ndarray, np.ndarray]:
    """cos / sin tables [max_pos, head_dim // 2] in f32, bit-identical to the oracle's per-token values."""
    cos = np.empty((max_pos, head_dim // 2), dtype=np.float32)
    sin = np.empty_like(cos)
    _native.host().bcpu_rope_table(head_dim, max_pos, base, cos.ctypes.data, sin.ctypes.data)
    return cos, sin
