"""GGUF container access (thin wrappers over the C++ reader / writer / streaming parser).

Reference surface: ``GgufFile::parse``, ``tensor_data``, ``mmap_gguf_file``, ``GgufWriter``,
``GgufStreamParser`` (crates/oxibonsai-core/src/gguf/reader.rs:32-99, writer.rs:175-330,
streaming.rs:110-219).
"""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import dataclass
from typing import Any, Iterable

import numpy as np

from .. import _native
from .._native import check

# on-disk tensor type ids
F32, F16, Q4_0, Q8_0, BF16 = 0, 1, 2, 8, 30
Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, Q8_K = 10, 11, 12, 13, 14, 15
TQ2_0, Q1_0_G128, TQ2_0_G128, F8_E4M3, F8_E5M2 = 35, 41, 42, 43, 44

# metadata value type ids
META_U8, META_I8, META_U16, META_I16, META_U32, META_I32, META_F32, META_BOOL, META_STRING, META_ARRAY, META_U64, META_I64, META_F64 = range(13)


def type_info(type_id: int) -> tuple[str, int, int]:
    """Returns (name, elements per block, bytes per block) of a tensor type id."""
    lib = _native.host()
    be, bb = C.c_uint32(), C.c_uint32()
    name = C.create_string_buffer(32)
    if lib.bonsai_type_info(type_id, C.byref(be), C.byref(bb), name, 32) < 0:
        raise _native.NativeError(7, "unsupported_quant_type", f"unsupported tensor type id {type_id}", False)
    return name.value.decode(), be.value, bb.value


def data_size(type_id: int, n_elements: int) -> int:
    _, be, bb = type_info(type_id)
    return (n_elements + be - 1) // be * bb


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dims: tuple[int, ...]  # innermost first: (in_features, out_features)
    type: int
    offset: int
    nbytes: int

    @property
    def type_name(self) -> str:
        return type_info(self.type)[0]

    @property
    def n_elements(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n


@dataclass(frozen=True)
class Qwen3Config:
    hidden: int = 4096
    inter: int = 14336
    layers: int = 36
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    vocab: int = 151936
    context: int = 65536
    eps: float = 1e-6
    rope_base: float = 1e6
    arch: str = "qwen3"
    name: str = "Bonsai-8B"

    @property
    def q_dim(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    def packed_u32(self):
        return (C.c_uint32 * 8)(self.hidden, self.inter, self.layers, self.heads, self.kv_heads, self.head_dim,
                                self.vocab, self.context)

    def packed_f32(self):
        return (C.c_float * 2)(self.eps, self.rope_base)


class GgufFile:
    """Parsed GGUF file.  ``open`` maps the file; ``parse`` works over a bytes-like object."""

    def __init__(self, handle: int, keepalive: Any = None, borrowed: bool = False):
        self._h = handle
        self._keep = keepalive
        self._borrowed = borrowed
        self._lib = _native.host()
        self._meta: dict | None = None
        self._tensors: list[TensorInfo] | None = None

    @classmethod
    def open(cls, path: str) -> "GgufFile":
        lib = _native.host()
        h = lib.bgguf_open(str(path).encode())
        if not h:
            raise _native.last_error()
        return cls(h)

    @classmethod
    def parse(cls, data: bytes | bytearray | memoryview | np.ndarray) -> "GgufFile":
        lib = _native.host()
        arr = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data
        h = lib.bgguf_parse(arr.ctypes.data, arr.size)
        if not h:
            raise _native.last_error()
        return cls(h, keepalive=(data, arr))

    def close(self) -> None:
        if self._h and not self._borrowed:
            self._lib.bgguf_close(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def handle(self) -> int:
        return self._h

    @property
    def version(self) -> int:
        return self._lib.bgguf_version(self._h)

    @property
    def alignment(self) -> int:
        return self._lib.bgguf_alignment(self._h)

    @property
    def data_offset(self) -> int:
        return self._lib.bgguf_data_offset(self._h)

    @property
    def metadata(self) -> dict:
        if self._meta is None:
            p = self._lib.bgguf_metadata_json(self._h, 0)
            if not p:
                raise _native.last_error()
            try:
                self._meta = json.loads(C.string_at(p).decode("utf-8", errors="replace"))
            finally:
                self._lib.bonsai_free(p)
        return self._meta

    @property
    def tensors(self) -> list[TensorInfo]:
        if self._tensors is None:
            out = []
            name = C.create_string_buffer(512)
            dims = (C.c_uint64 * 8)()
            nd, ty, off, nb = C.c_uint32(), C.c_uint32(), C.c_uint64(), C.c_uint64()
            for i in range(self._lib.bgguf_n_tensors(self._h)):
                check(self._lib.bgguf_tensor_info(self._h, i, name, 512, dims, C.byref(nd), C.byref(ty), C.byref(off), C.byref(nb)))
                out.append(TensorInfo(name.value.decode("utf-8", errors="replace"), tuple(dims[d] for d in range(nd.value)), ty.value, off.value, nb.value))
            self._tensors = out
        return self._tensors

    def tensor_index(self, name: str) -> int:
        return self._lib.bgguf_find_tensor(self._h, name.encode())

    def has_tensor(self, name: str) -> bool:
        return self.tensor_index(name) >= 0

    def tensor_info(self, name: str) -> TensorInfo:
        i = self.tensor_index(name)
        if i < 0:
            raise KeyError(name)
        return self.tensors[i]

    def tensor_bytes(self, name_or_index: str | int) -> np.ndarray:
        """Zero-copy uint8 view of a tensor's bytes (valid while this object is alive)."""
        i = name_or_index if isinstance(name_or_index, int) else self.tensor_index(name_or_index)
        if i < 0:
            raise KeyError(name_or_index)
        nb = C.c_uint64()
        p = self._lib.bgguf_tensor_data(self._h, i, C.byref(nb))
        if not p:
            raise _native.last_error()
        buf = (C.c_uint8 * nb.value).from_address(p)
        arr = np.frombuffer(buf, dtype=np.uint8)
        arr.flags.writeable = False
        return arr

    def config(self) -> Qwen3Config:
        u = (C.c_uint32 * 8)()
        f = (C.c_float * 2)()
        arch, name = C.create_string_buffer(64), C.create_string_buffer(256)
        check(self._lib.bgguf_config(self._h, u, f, arch, 64, name, 256))
        return Qwen3Config(u[0], u[1], u[2], u[3], u[4], u[5], u[6], u[7], float(f[0]), float(f[1]), arch.value.decode(), name.value.decode())


class GgufWriter:
    """GGUF v3 writer.  Tensor offsets are a running sum; padding only before the data section."""

    def __init__(self, version: int = 3, alignment: int = 32):
        self._lib = _native.host()
        self._h = self._lib.bggufw_new(version, alignment)
        self._keep: list[Any] = []

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.bggufw_free(self._h)
            self._h = None

    def add(self, key: str, value: Any, type_id: int | None = None) -> "GgufWriter":
        k = key.encode()
        lib, h = self._lib, self._h
        if isinstance(value, (list, tuple)):
            n = len(value)
            if n and all(isinstance(v, str) for v in value) or type_id == META_STRING:
                enc = [v.encode() for v in value]
                arr = (C.c_char_p * n)(*enc)
                lens = (C.c_uint64 * n)(*[len(e) for e in enc])
                lib.bggufw_add_str_array(h, k, arr, lens, n)
            elif all(isinstance(v, (int, np.integer)) for v in value) and type_id not in (META_F32, META_F64):
                iv = (C.c_int64 * n)(*[int(v) for v in value])
                lib.bggufw_add_num_array(h, k, META_I32 if type_id is None else type_id, iv, None, n)
            else:
                fv = (C.c_double * n)(*[float(v) for v in value])
                lib.bggufw_add_num_array(h, k, META_F32 if type_id is None else type_id, None, fv, n)
        elif type_id is not None and type_id != META_STRING:
            lib.bggufw_add_scalar(h, k, type_id, int(value) if type_id not in (META_F32, META_F64) else 0, float(value))
        elif isinstance(value, bool):
            lib.bggufw_add_bool(h, k, int(value))
        elif isinstance(value, str):
            lib.bggufw_add_str(h, k, value.encode())
        elif isinstance(value, (int, np.integer)):
            if value < 0:
                lib.bggufw_add_i32(h, k, int(value))
            elif value < 2**32:
                lib.bggufw_add_u32(h, k, int(value))
            else:
                lib.bggufw_add_u64(h, k, int(value))
        elif isinstance(value, (float, np.floating)):
            lib.bggufw_add_f32(h, k, float(value))
        else:
            raise TypeError(f"unsupported metadata value for {key!r}: {type(value)}")
        return self

    def add_tensor(self, name: str, dims: Iterable[int], type_id: int, data: bytes | np.ndarray) -> "GgufWriter":
        arr = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1))
        d = list(dims)
        da = (C.c_uint64 * len(d))(*d)
        check(self._lib.bggufw_add_tensor(self._h, name.encode(), da, len(d), type_id, arr.ctypes.data, arr.size, 1))
        return self

    def write(self, path: str) -> None:
        check(self._lib.bggufw_write(self._h, str(path).encode()))

    def to_bytes(self) -> bytes:
        n = C.c_uint64()
        p = self._lib.bggufw_to_bytes(self._h, C.byref(n))
        if not p:
            raise _native.last_error()
        try:
            return C.string_at(p, n.value)
        finally:
            self._lib.bonsai_free(p)


class GgufStreamParser:
    """Incremental header parser for checkpoints arriving in chunks (e.g. over a socket)."""

    NEED_MORE, HEADER_COMPLETE, FAILED = 0, 1, 2

    def __init__(self):
        self._lib = _native.host()
        self._h = self._lib.bggufs_new()

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.bggufs_free(self._h)
            self._h = None

    def feed(self, chunk: bytes) -> int:
        buf = np.frombuffer(chunk, dtype=np.uint8)
        return self._lib.bggufs_feed(self._h, buf.ctypes.data if buf.size else None, buf.size)

    @property
    def file(self) -> GgufFile | None:
        h = self._lib.bggufs_file(self._h)
        return GgufFile(h, keepalive=self, borrowed=True) if h else None

    @property
    def error(self) -> str:
        return self._lib.bggufs_error(self._h).decode()

    @property
    def bytes_consumed(self) -> int:
        return self._lib.bggufs_bytes_consumed(self._h)

    @property
    def data_bytes_seen(self) -> int:
        return self._lib.bggufs_data_seen(self._h)

    @property
    def data_bytes_expected(self) -> int:
        return self._lib.bggufs_data_expected(self._h)
