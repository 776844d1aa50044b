"""ONNX (``MatMulNBits``, 2-bit) -> GGUF conversion with a self-contained protobuf reader.

Reference: crates/oxibonsai-model/src/convert/onnx/* (graph walk over ``MatMulNBits`` nodes with ``bits = 2``, role map
from node / initializer names to GGUF tensor names, 2-bit dequantisation ``(q - zero_point) * scale`` per block along K,
requantisation into the target block format) and the ``onnx_inspect`` / ``onnx_convert`` examples.  No ONNX package is
needed: the handful of message types involved (ModelProto, GraphProto, NodeProto, AttributeProto, TensorProto) are read
straight from the protobuf wire format.
"""
from __future__ import annotations

import re
import struct
from dataclasses import dataclass, field
from typing import Iterator

import numpy as np

from ..core import gguf as G
from ..core.blocks import quantize
from . import QUANT_TYPES, ConvertStats


# ---- protobuf wire format ----------------------------------------------------------------------------------------------------
def _varint(buf: memoryview, i: int) -> tuple[int, int]:
    v = shift = 0
    while True:
        b = buf[i]
        i += 1
        v |= (b & 0x7F) << shift
        if b < 0x80:
            return v, i
        shift += 7
        if shift > 70:
            raise ValueError("malformed varint")


def _fields(buf: memoryview) -> Iterator[tuple[int, int, object]]:
    """Yields ``(field_number, wire_type, value)``; length-delimited values are memoryviews."""
    i, n = 0, len(buf)
    while i < n:
        key, i = _varint(buf, i)
        fn, wt = key >> 3, key & 7
        if wt == 0:
            v, i = _varint(buf, i)
        elif wt == 1:
            v, i = bytes(buf[i:i + 8]), i + 8
        elif wt == 2:
            ln, i = _varint(buf, i)
            if i + ln > n:
                raise ValueError("length-delimited field runs past the end of its message")
            v, i = buf[i:i + ln], i + ln
        elif wt == 5:
            v, i = bytes(buf[i:i + 4]), i + 4
        else:
            raise ValueError(f"unsupported protobuf wire type {wt}")
        yield fn, wt, v


_DTYPES = {1: np.float32, 2: np.uint8, 3: np.int8, 6: np.int32, 7: np.int64, 10: np.float16, 11: np.float64}


@dataclass
class OnnxTensor:
    name: str = ""
    dims: list[int] = field(default_factory=list)
    data_type: int = 0
    raw: bytes = b""
    floats: list[float] = field(default_factory=list)
    ints: list[int] = field(default_factory=list)

    def numpy(self) -> np.ndarray:
        if self.data_type == 16:   # bfloat16
            a = (np.frombuffer(self.raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif self.raw:
            a = np.frombuffer(self.raw, dtype=np.dtype(_DTYPES[self.data_type]).newbyteorder("<"))
        elif self.floats:
            a = np.asarray(self.floats, dtype=np.float32)
        else:
            a = np.asarray(self.ints, dtype=_DTYPES.get(self.data_type, np.int64))
        return a.reshape(self.dims) if self.dims else a


def _tensor(buf: memoryview) -> OnnxTensor:
    t = OnnxTensor()
    for fn, wt, v in _fields(buf):
        if fn == 1:
            if wt == 0:
                t.dims.append(v)
            else:
                j = 0
                while j < len(v):
                    d, j = _varint(v, j)
                    t.dims.append(d)
        elif fn == 2:
            t.data_type = v
        elif fn == 4:
            t.floats.extend(struct.unpack(f"<{len(v) // 4}f", bytes(v)) if wt == 2 else struct.unpack("<f", v))
        elif fn in (5, 7):
            if wt == 0:
                t.ints.append(v)
            else:
                j = 0
                while j < len(v):
                    d, j = _varint(v, j)
                    t.ints.append(d)
        elif fn == 8:
            t.name = bytes(v).decode("utf-8")
        elif fn == 9:
            t.raw = bytes(v)
        elif fn == 13:
            raise ValueError(f"tensor {t.name!r} uses external data, which is not supported")
    return t


@dataclass
class OnnxNode:
    name: str = ""
    op_type: str = ""
    domain: str = ""
    inputs: list[str] = field(default_factory=list)
    outputs: list[str] = field(default_factory=list)
    attrs: dict = field(default_factory=dict)


def _node(buf: memoryview) -> OnnxNode:
    n = OnnxNode()
    for fn, wt, v in _fields(buf):
        if fn == 1:
            n.inputs.append(bytes(v).decode())
        elif fn == 2:
            n.outputs.append(bytes(v).decode())
        elif fn == 3:
            n.name = bytes(v).decode()
        elif fn == 4:
            n.op_type = bytes(v).decode()
        elif fn == 7:
            n.domain = bytes(v).decode()
        elif fn == 5:
            name, val = "", None
            for afn, awt, av in _fields(v):
                if afn == 1:
                    name = bytes(av).decode()
                elif afn == 2:
                    val = struct.unpack("<f", av)[0]
                elif afn == 3:
                    val = av if av < (1 << 63) else av - (1 << 64)
                elif afn == 4:
                    val = bytes(av).decode("utf-8", errors="replace")
            n.attrs[name] = val
    return n


@dataclass
class OnnxGraph:
    name: str = ""
    nodes: list[OnnxNode] = field(default_factory=list)
    initializers: dict[str, OnnxTensor] = field(default_factory=dict)


def read_onnx(path: str) -> OnnxGraph:
    data = memoryview(np.memmap(path, dtype=np.uint8, mode="r"))
    g = OnnxGraph()
    for fn, wt, v in _fields(data):
        if fn == 7 and wt == 2:           # ModelProto.graph
            for gfn, gwt, gv in _fields(v):
                if gfn == 1:
                    g.nodes.append(_node(gv))
                elif gfn == 2:
                    g.name = bytes(gv).decode()
                elif gfn == 5:
                    t = _tensor(gv)
                    g.initializers[t.name] = t
    return g


def inspect_onnx(path: str) -> dict:
    g = read_onnx(path)
    ops: dict[str, int] = {}
    for n in g.nodes:
        ops[n.op_type] = ops.get(n.op_type, 0) + 1
    nbits = [n for n in g.nodes if n.op_type == "MatMulNBits"]
    return {"graph": g.name, "nodes": len(g.nodes), "initializers": len(g.initializers), "ops": ops,
            "matmul_nbits": [{"name": n.name, "K": n.attrs.get("K"), "N": n.attrs.get("N"), "bits": n.attrs.get("bits"), "block_size": n.attrs.get("block_size")}
                             for n in nbits]}


# ---- MatMulNBits ------------------------------------------------------------------------------------------------------------------
def dequant_matmul_nbits(b: np.ndarray, scales: np.ndarray, zero_points: np.ndarray | None, K: int, N: int, bits: int, block_size: int) -> np.ndarray:
    """Packed ``B`` [N][blocks][block_size*bits/8] -> f32 [N][K]:  w = (q - zero_point) * scale per (row, block)."""
    if bits not in (2, 4, 8):
        raise ValueError(f"unsupported bits {bits}")
    nblk = (K + block_size - 1) // block_size
    per = 8 // bits
    raw = np.ascontiguousarray(b, dtype=np.uint8).reshape(N, nblk, block_size // per)
    q = np.empty((N, nblk, block_size), dtype=np.float32)
    mask = (1 << bits) - 1
    for j in range(per):
        q[:, :, j::per] = (raw >> (bits * j)) & mask
    sc = np.asarray(scales, dtype=np.float32).reshape(N, nblk, 1)
    if zero_points is None:
        zp = np.float32(1 << (bits - 1))
    else:
        z = np.ascontiguousarray(zero_points, dtype=np.uint8).reshape(N, -1)
        zq = np.empty((N, z.shape[1] * per), dtype=np.float32)
        for j in range(per):
            zq[:, j::per] = (z >> (bits * j)) & mask
        zp = zq[:, :nblk].reshape(N, nblk, 1)
    return ((q - zp) * sc).reshape(N, nblk * block_size)[:, :K]


_ROLES = [("q_proj", "attn_q"), ("k_proj", "attn_k"), ("v_proj", "attn_v"), ("o_proj", "attn_output"), ("gate_proj", "ffn_gate"),
          ("up_proj", "ffn_up"), ("down_proj", "ffn_down")]
_NORMS = [("input_layernorm", "attn_norm"), ("post_attention_layernorm", "ffn_norm"), ("q_norm", "attn_q_norm"), ("k_norm", "attn_k_norm")]
_LAYER = re.compile(r"layers?[._/](\d+)[._/]")


def role_for(name: str) -> str | None:
    """GGUF tensor name for an ONNX node / initializer name, or None."""
    low = name.replace("/", ".")
    m = _LAYER.search(low)
    if m:
        for key, role in _ROLES + _NORMS:
            if key in low:
                return f"blk.{int(m.group(1))}.{role}.weight"
        return None
    if "lm_head" in low:
        return "output.weight"
    if "embed_tokens" in low:
        return "token_embd.weight"
    if re.search(r"(^|\.)(model\.)?(final_)?norm(\.|$)", low) and "layernorm" not in low:
        return "output_norm.weight"
    return None


def convert_onnx_to_gguf(src: str, dst: str, quant: str = "tq2_0_g128", name: str | None = None) -> ConvertStats:
    if quant not in QUANT_TYPES:
        raise ValueError(f"unknown quantisation {quant!r}")
    qtype = QUANT_TYPES[quant]
    _, qblock, _ = G.type_info(qtype)
    g = read_onnx(src)
    w = G.GgufWriter()
    st = ConvertStats()
    seen: dict[str, tuple[int, ...]] = {}

    def emit(gname: str, arr: np.ndarray, as_norm: bool) -> None:
        if gname in seen:
            return
        arr = np.asarray(arr, dtype=np.float32)
        if as_norm or arr.ndim < 2 or arr.shape[-1] % qblock:
            tid, blob = (G.F32, arr.reshape(-1).view(np.uint8)) if (as_norm or arr.ndim < 2) else (G.F16, arr.astype(np.float16).reshape(-1).view(np.uint8))
        else:
            tid, blob = qtype, quantize(qtype, arr)
        w.add_tensor(gname, tuple(reversed(arr.shape)), tid, blob)
        seen[gname] = tuple(reversed(arr.shape))
        st.tensors += 1
        st.bytes_out += blob.size

    for n in g.nodes:
        if n.op_type != "MatMulNBits":
            continue
        gname = role_for(n.name) or role_for(n.inputs[1] if len(n.inputs) > 1 else "")
        if gname is None:
            st.skipped += 1
            continue
        K, N, bits, bs = int(n.attrs["K"]), int(n.attrs["N"]), int(n.attrs.get("bits", 4)), int(n.attrs.get("block_size", 32))
        b = g.initializers[n.inputs[1]]
        sc = g.initializers[n.inputs[2]]
        zp = g.initializers.get(n.inputs[3]) if len(n.inputs) > 3 and n.inputs[3] else None
        st.bytes_in += len(b.raw) + len(sc.raw)
        emit(gname, dequant_matmul_nbits(b.numpy(), sc.numpy(), None if zp is None else zp.numpy(), K, N, bits, bs), False)
    for iname, t in g.initializers.items():
        gname = role_for(iname)
        if gname is None or gname in seen or t.data_type not in (1, 10, 16):
            continue
        arr = t.numpy().astype(np.float32)
        if gname.endswith("norm.weight") or arr.ndim >= 2:
            st.bytes_in += arr.nbytes
            emit(gname, arr, gname.endswith("norm.weight"))
    if "output.weight" not in seen and "token_embd.weight" in seen:
        t = next(t for n_, t in g.initializers.items() if role_for(n_) == "token_embd.weight")
        seen.pop("output.weight", None)
        emit("output.weight", t.numpy().astype(np.float32), False)
        st.tied = True
    layers = 1 + max((int(k.split(".")[1]) for k in seen if k.startswith("blk.")), default=-1)
    hidden = seen.get("blk.0.attn_q.weight", (0, 0))[0] or seen.get("token_embd.weight", (0, 0))[0]
    hd = seen.get("blk.0.attn_q_norm.weight", (128,))[0]
    w.add("general.architecture", "qwen3")
    w.add("general.name", name or g.name or "onnx-import")
    w.add("qwen3.block_count", layers)
    w.add("qwen3.embedding_length", int(hidden))
    w.add("qwen3.feed_forward_length", int(seen.get("blk.0.ffn_gate.weight", (0, 0))[1]))
    w.add("qwen3.attention.head_count", int(seen.get("blk.0.attn_q.weight", (0, hd))[1] // hd))
    w.add("qwen3.attention.head_count_kv", int(seen.get("blk.0.attn_k.weight", (0, hd))[1] // hd))
    w.add("qwen3.attention.key_length", int(hd))
    w.add("qwen3.attention.layer_norm_rms_epsilon", 1e-6)
    w.add("qwen3.rope.freq_base", 1e6)
    w.add("qwen3.context_length", 32768)
    w.write(dst)
    return st
