"""Checkpoint containers: ``OXCK`` (named f32 tensors + string metadata), ``OXCA`` (cache of already-quantised tensors),
the repacked-weight cache of the B200 engine, and weight tying helpers.

Reference file formats (crates/oxibonsai-model/src/checkpoint.rs:1-40, disk_cache.rs:7-19), both little endian:

``OXCK`` v1: ``"OXCK" | u32 version=1 | u64 flags=0 | u64 num_tensors | u32 metadata_len | metadata JSON`` then per tensor
``u32 name_len | name | u32 ndim | u64 shape[ndim] | u64 n_elements | f32 data``.

``OXCA`` v1: ``"OXCA" | u32 version=1 | u64 num_entries | u32 metadata_len | metadata JSON`` then per entry
``u32 name_len | name | u32 quant_type_len | quant_type | u64 data_len | data``; a cache is fresh when it is newer than
its source file (disk_cache.rs:277).

Files written here load in the reference and vice versa.  Weight tying mirrors weight_tying.rs: a tied model shares the
embedding matrix with the LM head; GGUF files for the reference's loader carry a duplicate ``output.weight``.
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
from dataclasses import dataclass, field
from typing import BinaryIO

import numpy as np

OXCK_MAGIC, OXCA_MAGIC = b"OXCK", b"OXCA"


class CheckpointError(ValueError):
    pass


def _read(f: BinaryIO, n: int) -> bytes:
    b = f.read(n)
    if len(b) != n:
        raise CheckpointError("unexpected end of file")
    return b


def _flat_json(meta: dict[str, str]) -> bytes:
    for k, v in meta.items():
        if any(c in str(k) + str(v) for c in '"\\'):
            raise CheckpointError("metadata keys and values must not contain quotes or backslashes")
    return json.dumps({str(k): str(v) for k, v in meta.items()}, separators=(",", ":")).encode("utf-8")


@dataclass
class Checkpoint:
    metadata: dict[str, str] = field(default_factory=dict)
    tensors: dict[str, np.ndarray] = field(default_factory=dict)
    version: int = 1

    def add(self, name: str, array: np.ndarray) -> "Checkpoint":
        if name in self.tensors:
            raise CheckpointError(f"duplicate tensor {name!r}")
        self.tensors[name] = np.ascontiguousarray(array, dtype="<f4")
        return self

    def save(self, path: str) -> None:
        meta = _flat_json(self.metadata)
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(OXCK_MAGIC + struct.pack("<IQQI", 1, 0, len(self.tensors), len(meta)) + meta)
            for name, a in self.tensors.items():
                nb = name.encode("utf-8")
                f.write(struct.pack("<I", len(nb)) + nb + struct.pack("<I", a.ndim) + struct.pack(f"<{a.ndim}Q", *a.shape))
                f.write(struct.pack("<Q", a.size))
                f.write(np.ascontiguousarray(a, dtype="<f4").tobytes())
        os.replace(tmp, path)

    @classmethod
    def load(cls, path: str) -> "Checkpoint":
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            if _read(f, 4) != OXCK_MAGIC:
                raise CheckpointError("not an OXCK checkpoint")
            version, _flags, n, mlen = struct.unpack("<IQQI", _read(f, 24))
            if version != 1:
                raise CheckpointError(f"unsupported checkpoint version {version}")
            if mlen > size:
                raise CheckpointError("metadata length exceeds the file size")
            meta = json.loads(_read(f, mlen).decode("utf-8")) if mlen else {}
            ck = cls({str(k): str(v) for k, v in meta.items()}, {}, version)
            for _ in range(n):
                (nl,) = struct.unpack("<I", _read(f, 4))
                if nl > 1 << 16:
                    raise CheckpointError("tensor name too long")
                name = _read(f, nl).decode("utf-8")
                (nd,) = struct.unpack("<I", _read(f, 4))
                if nd > 8:
                    raise CheckpointError("too many dimensions")
                shape = struct.unpack(f"<{nd}Q", _read(f, 8 * nd))
                (cnt,) = struct.unpack("<Q", _read(f, 8))
                if cnt != int(np.prod(shape, dtype=np.uint64)) if nd else cnt != 1 and cnt != 0:
                    raise CheckpointError(f"tensor {name!r}: {cnt} elements do not match shape {shape}")
                if cnt * 4 > size:
                    raise CheckpointError("tensor data exceeds the file size")
                ck.tensors[name] = np.frombuffer(_read(f, 4 * cnt), dtype="<f4").reshape(shape).copy()
            return ck


@dataclass
class DiskCacheEntry:
    quant_type: str
    data: bytes


class DiskCache:
    """``.oxcache`` container of quantised tensors."""

    def __init__(self, metadata: dict[str, str] | None = None):
        self.metadata: dict[str, str] = dict(metadata or {})
        self.entries: dict[str, DiskCacheEntry] = {}

    def put(self, name: str, quant_type: str, data: bytes | np.ndarray) -> None:
        self.entries[name] = DiskCacheEntry(quant_type, bytes(data) if not isinstance(data, np.ndarray) else data.tobytes())

    def get(self, name: str) -> DiskCacheEntry | None:
        return self.entries.get(name)

    def save(self, path: str) -> None:
        meta = _flat_json(self.metadata)
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(OXCA_MAGIC + struct.pack("<IQI", 1, len(self.entries), len(meta)) + meta)
            for name, e in self.entries.items():
                nb, qb = name.encode(), e.quant_type.encode()
                f.write(struct.pack("<I", len(nb)) + nb + struct.pack("<I", len(qb)) + qb + struct.pack("<Q", len(e.data)))
                f.write(e.data)
        os.replace(tmp, path)

    @classmethod
    def load(cls, path: str) -> "DiskCache":
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            if _read(f, 4) != OXCA_MAGIC:
                raise CheckpointError("invalid cache magic")
            version, n, mlen = struct.unpack("<IQI", _read(f, 16))
            if version != 1:
                raise CheckpointError(f"unsupported cache version: {version}")
            c = cls(json.loads(_read(f, mlen).decode()) if mlen else {})
            for _ in range(n):
                (nl,) = struct.unpack("<I", _read(f, 4))
                name = _read(f, nl).decode()
                (ql,) = struct.unpack("<I", _read(f, 4))
                qt = _read(f, ql).decode()
                (dl,) = struct.unpack("<Q", _read(f, 8))
                if dl > size:
                    raise CheckpointError("entry exceeds the file size")
                c.entries[name] = DiskCacheEntry(qt, _read(f, dl))
            return c

    @staticmethod
    def is_valid(path: str) -> bool:
        try:
            with open(path, "rb") as f:
                return f.read(4) == OXCA_MAGIC and struct.unpack("<I", f.read(4))[0] == 1
        except (OSError, struct.error):
            return False

    @staticmethod
    def is_fresh(cache_path: str, source_path: str) -> bool:
        """True when the cache exists, is valid and is not older than its source."""
        try:
            return DiskCache.is_valid(cache_path) and os.path.getmtime(cache_path) >= os.path.getmtime(source_path)
        except OSError:
            return False


def repack_cache_key(model_path: str, tp_rank: int, tp_size: int, layout: str = "planar-sm") -> str:
    """Key of the device-layout weight cache: file identity (size, mtime, first MiB hash) + layout + TP coordinates."""
    st = os.stat(model_path)
    h = hashlib.blake2b(digest_size=16)
    with open(model_path, "rb") as f:
        h.update(f.read(1 << 20))
    h.update(f"{st.st_size}:{int(st.st_mtime_ns)}:{layout}:{tp_rank}/{tp_size}".encode())
    return h.hexdigest()


REPACK_MAGIC = b"OXRP"
_REPACK_ALIGN = 4096


def save_repacked(path: str, tensors: dict, meta: dict | None = None) -> None:
    """Writes named tensors (torch, any device) as one file: ``"OXRP" | u32 version=1 | u64 header_len | header JSON`` and
    the raw bytes of every tensor at a 4096-byte aligned offset.  The header lists name, dtype, shape, offset and byte
    count, plus ``meta``.  The file is written under a temporary name and renamed, so a reader never sees a partial one."""
    import torch
    entries, off = [], 0
    flat = {}
    for name, t in tensors.items():
        c = t.detach().contiguous().cpu()
        flat[name] = c
        nbytes = c.numel() * c.element_size()
        entries.append({"name": name, "dtype": str(c.dtype).replace("torch.", ""), "shape": list(c.shape), "offset": off, "nbytes": nbytes})
        off += -(-nbytes // _REPACK_ALIGN) * _REPACK_ALIGN
    header = json.dumps({"meta": meta or {}, "tensors": entries}).encode("utf-8")
    base = -(-(16 + len(header)) // _REPACK_ALIGN) * _REPACK_ALIGN
    tmp = f"{path}.{os.getpid()}.tmp"
    with open(tmp, "wb") as f:
        f.write(REPACK_MAGIC + struct.pack("<IQ", 1, len(header)) + header)
        for e in entries:
            f.seek(base + e["offset"])
            if e["nbytes"]:
                f.write(flat[e["name"]].reshape(-1).view(torch.uint8).numpy().tobytes())
        f.truncate(base + off)
    os.replace(tmp, path)


def load_repacked(path: str, device="cpu") -> tuple[dict, dict]:
    """Reads a file written by :func:`save_repacked`; returns ``(tensors, meta)`` with the tensors on ``device`` (uploaded
    from the page cache through pinned staging copies when it is a CUDA device)."""
    import torch
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        if _read(f, 4) != REPACK_MAGIC:
            raise CheckpointError("not a repacked-weight cache")
        version, hlen = struct.unpack("<IQ", _read(f, 12))
        if version != 1 or hlen > size:
            raise CheckpointError("unsupported or damaged repacked-weight cache")
        header = json.loads(_read(f, hlen).decode("utf-8"))
    base = -(-(16 + hlen) // _REPACK_ALIGN) * _REPACK_ALIGN
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    dev = torch.device(device)
    out = {}
    for e in header["tensors"]:
        lo = base + e["offset"]
        if lo + e["nbytes"] > size:
            raise CheckpointError(f"tensor {e['name']!r} exceeds the file size")
        if e["nbytes"] == 0:
            out[e["name"]] = torch.empty(e["shape"], dtype=getattr(torch, e["dtype"]), device=dev)
            continue
        raw = torch.from_numpy(np.array(mm[lo: lo + e["nbytes"]], copy=True))
        if dev.type == "cuda":
            raw = raw.pin_memory().to(dev, non_blocking=True)
        out[e["name"]] = raw.view(getattr(torch, e["dtype"])).reshape(e["shape"])
    return out, header.get("meta", {})


def tie_weights(tensors: dict[str, np.ndarray], embed: str = "token_embd.weight", head: str = "output.weight") -> dict[str, np.ndarray]:
    """Makes the LM head an alias of the embedding table (shared storage)."""
    if embed not in tensors:
        raise KeyError(embed)
    out = dict(tensors)
    out[head] = out[embed]
    return out


def is_tied(tensors: dict[str, np.ndarray], embed: str = "token_embd.weight", head: str = "output.weight") -> bool:
    if head not in tensors:
        return True
    a, b = tensors[embed], tensors[head]
    return a is b or (a.shape == b.shape and np.shares_memory(a, b)) or (a.shape == b.shape and bool(np.array_equal(a, b)))


def untie_weights(tensors: dict[str, np.ndarray], embed: str = "token_embd.weight", head: str = "output.weight") -> dict[str, np.ndarray]:
    out = dict(tensors)
    out[head] = np.array(out.get(head, out[embed]), copy=True)
    return out
