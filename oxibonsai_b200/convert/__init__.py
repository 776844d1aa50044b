"""Checkpoint conversion: Hugging Face safetensors -> GGUF with sub-2-bit weights.

Reference: ``convert_safetensors_to_gguf`` (crates/oxibonsai-model/src/convert/mod.rs:54-240) maps the Hugging Face
Qwen3 tensor names to GGUF names (convert/name_map.rs:15-75), stores norm vectors as F32 and every other tensor in the
requested block format, reverses the shape (GGUF lists the contiguous dimension first), duplicates tied embeddings as
``output.weight`` and writes the model metadata under ``llm.*`` keys (convert/common.rs:43-150).

The safetensors container (8-byte little-endian header length, JSON header, raw little-endian tensor data) is read here
directly through a memory map, shard by shard, so a conversion never holds more than one tensor in float32.
"""
from __future__ import annotations

import glob
import json
import os
import re
import struct
from dataclasses import dataclass
from typing import Iterator

import numpy as np

from ..core import gguf as G
from ..core.blocks import quantize

_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "F64": np.float64, "I64": np.int64, "I32": np.int32, "I16": np.int16, "I8": np.int8,
              "U8": np.uint8, "BOOL": np.bool_}

_LAYER_SUFFIX = {
    "input_layernorm.weight": ("attn_norm.weight", True), "post_attention_layernorm.weight": ("ffn_norm.weight", True),
    "self_attn.q_proj.weight": ("attn_q.weight", False), "self_attn.k_proj.weight": ("attn_k.weight", False),
    "self_attn.v_proj.weight": ("attn_v.weight", False), "self_attn.o_proj.weight": ("attn_output.weight", False),
    "mlp.gate_proj.weight": ("ffn_gate.weight", False), "mlp.up_proj.weight": ("ffn_up.weight", False),
    "mlp.down_proj.weight": ("ffn_down.weight", False), "self_attn.q_norm.weight": ("attn_q_norm.weight", True),
    "self_attn.k_norm.weight": ("attn_k_norm.weight", True),
}
_TOP = {"model.embed_tokens.weight": ("token_embd.weight", False), "model.norm.weight": ("output_norm.weight", True),
        "lm_head.weight": ("output.weight", False)}
_LAYER_RE = re.compile(r"^model\.layers\.(\d+)\.(.+)$")

QUANT_TYPES = {"tq2_0_g128": G.TQ2_0_G128, "q1_0_g128": G.Q1_0_G128, "tq2_0": G.TQ2_0, "q4_0": G.Q4_0, "q8_0": G.Q8_0,
               "f8_e4m3": G.F8_E4M3, "f8_e5m2": G.F8_E5M2, "f16": G.F16, "f32": G.F32}


def hf_to_gguf_name(name: str) -> tuple[str, bool] | None:
    """``(gguf_name, is_norm)`` for a Hugging Face Qwen3 tensor name; None for tensors that are not exported."""
    if name in _TOP:
        return _TOP[name]
    m = _LAYER_RE.match(name)
    if m and m.group(2) in _LAYER_SUFFIX:
        suffix, is_norm = _LAYER_SUFFIX[m.group(2)]
        return f"blk.{int(m.group(1))}.{suffix}", is_norm
    return None


@dataclass
class SafeTensor:
    name: str
    dtype: str
    shape: tuple[int, ...]
    data: np.ndarray          # raw bytes (a view into the memory map)

    def to_f32(self) -> np.ndarray:
        if self.dtype == "BF16":
            u = np.frombuffer(self.data, dtype="<u2").astype(np.uint32) << 16
            return u.view(np.float32).reshape(self.shape)
        if self.dtype not in _ST_DTYPES:
            raise ValueError(f"unsupported safetensors dtype {self.dtype} for {self.name}")
        return np.frombuffer(self.data, dtype=np.dtype(_ST_DTYPES[self.dtype]).newbyteorder("<")).astype(np.float32).reshape(self.shape)


def read_safetensors(path: str) -> Iterator[SafeTensor]:
    """Yields the tensors of one ``.safetensors`` file in file order (views into a read-only memory map)."""
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    if mm.size < 8:
        raise ValueError(f"{path}: too short for a safetensors header")
    (hlen,) = struct.unpack("<Q", bytes(mm[:8]))
    if hlen > mm.size - 8 or hlen > 100 << 20:
        raise ValueError(f"{path}: implausible header length {hlen}")
    header = json.loads(bytes(mm[8:8 + hlen]).decode("utf-8"))
    base = 8 + hlen
    entries = [(k, v) for k, v in header.items() if k != "__metadata__"]
    entries.sort(key=lambda kv: kv[1]["data_offsets"][0])
    for name, e in entries:
        lo, hi = e["data_offsets"]
        if not 0 <= lo <= hi <= mm.size - base:
            raise ValueError(f"{path}: tensor {name} lies outside the file")
        yield SafeTensor(name, e["dtype"], tuple(int(d) for d in e["shape"]), mm[base + lo: base + hi])


def write_safetensors(path: str, tensors: dict[str, np.ndarray]) -> None:
    """Writes float32 / float16 arrays as a safetensors file (used by tests and by the export tools)."""
    names = {np.dtype(np.float32): "F32", np.dtype(np.float16): "F16", np.dtype(np.int64): "I64", np.dtype(np.int32): "I32"}
    header, blobs, off = {}, [], 0
    for k, a in tensors.items():
        a = np.ascontiguousarray(a)
        b = a.tobytes()
        header[k] = {"dtype": names[a.dtype], "shape": list(a.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


@dataclass
class ConvertStats:
    tensors: int = 0
    skipped: int = 0
    bytes_in: int = 0
    bytes_out: int = 0
    tied: bool = False
    tokenizer_tokens: int = 0          # size of the vocabulary copied into the file's metadata (0: none found)


def _shards(src: str) -> list[str]:
    if os.path.isdir(src):
        files = sorted(glob.glob(os.path.join(src, "*.safetensors")))
        if not files:
            raise FileNotFoundError(f"no .safetensors files in {src}")
        return files
    return [src]


def _hf_config(src: str) -> dict:
    d = src if os.path.isdir(src) else os.path.dirname(os.path.abspath(src))
    p = os.path.join(d, "config.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f)
    return {}


def convert_safetensors_to_gguf(src: str, dst: str, quant: str = "tq2_0_g128", quantize_embeddings: bool = True,
                                key_prefix: str = "llm", name: str | None = None, embed_tokenizer: bool = True) -> ConvertStats:
    """Converts a Hugging Face Qwen3 checkpoint (a directory of shards or a single file) to GGUF.

    ``quantize_embeddings=True`` reproduces the reference (embedding table and LM head in the block format too);
    False keeps them in F16, which is what the B200 engine serves from anyway.
    """
    if quant not in QUANT_TYPES:
        raise ValueError(f"unknown quantisation {quant!r}; choose from {sorted(QUANT_TYPES)}")
    qtype = QUANT_TYPES[quant]
    _, qblock, _ = G.type_info(qtype)
    cfg = _hf_config(src)
    w = G.GgufWriter()
    stats = ConvertStats()
    seen: dict[str, tuple[int, ...]] = {}
    embd: tuple[tuple[int, ...], int, np.ndarray] | None = None
    for shard in _shards(src):
        for t in read_safetensors(shard):
            m = hf_to_gguf_name(t.name)
            if m is None:
                stats.skipped += 1
                continue
            gname, is_norm = m
            v = t.to_f32()
            stats.bytes_in += t.data.size
            if is_norm or v.ndim < 2:
                ttype, blob = G.F32, np.ascontiguousarray(v, dtype=np.float32).view(np.uint8).reshape(-1)
            else:
                ttype = qtype
                if gname in ("token_embd.weight", "output.weight") and not quantize_embeddings:
                    ttype = G.F16
                if ttype == G.F16:
                    blob = v.astype(np.float16).view(np.uint8).reshape(-1)
                elif ttype == G.F32:
                    blob = np.ascontiguousarray(v).view(np.uint8).reshape(-1)
                else:
                    if v.shape[-1] % qblock:
                        raise ValueError(f"{t.name}: inner dimension {v.shape[-1]} is not a multiple of the {quant} block size {qblock}")
                    blob = quantize(ttype, v)
            dims = tuple(reversed(v.shape))
            w.add_tensor(gname, dims, ttype, blob)
            seen[gname] = dims
            stats.tensors += 1
            stats.bytes_out += blob.size
            if gname == "token_embd.weight":
                embd = (dims, ttype, blob)
    if "output.weight" not in seen and embd is not None:
        # tied embeddings: loaders of this format expect an explicit output.weight
        w.add_tensor("output.weight", embd[0], embd[1], embd[2])
        stats.tensors += 1
        stats.bytes_out += embd[2].size
        stats.tied = True
    layers = 1 + max((int(k.split(".")[1]) for k in seen if k.startswith("blk.")), default=-1)
    hidden = seen.get("token_embd.weight", (cfg.get("hidden_size", 0),))[0]
    heads = int(cfg.get("num_attention_heads", 0)) or max(1, seen.get("blk.0.attn_q.weight", (0, hidden))[1] // 128)
    kv_heads = int(cfg.get("num_key_value_heads", 0)) or max(1, seen.get("blk.0.attn_k.weight", (0, hidden))[1] // 128)
    head_dim = int(cfg.get("head_dim", 0)) or (seen.get("blk.0.attn_q.weight", (0, hidden))[1] // heads)
    p = key_prefix
    w.add("general.architecture", "qwen3" if p != "llm" else "llm")
    w.add("general.name", name or cfg.get("_name_or_path") or os.path.basename(os.path.normpath(src)))
    w.add("general.quantization_version", 2)
    w.add(f"{p}.block_count", layers)
    w.add(f"{p}.embedding_length", int(hidden))
    w.add(f"{p}.feed_forward_length", int(cfg.get("intermediate_size", seen.get("blk.0.ffn_gate.weight", (0, 0))[1])))
    w.add(f"{p}.attention.head_count", heads)
    w.add(f"{p}.attention.head_count_kv", kv_heads)
    w.add(f"{p}.attention.key_length", head_dim)
    w.add(f"{p}.attention.layer_norm_rms_epsilon", float(cfg.get("rms_norm_eps", 1e-6)))
    w.add(f"{p}.rope.freq_base", float(cfg.get("rope_theta", 1e6)))
    w.add(f"{p}.context_length", int(cfg.get("max_position_embeddings", 32768)))
    w.add(f"{p}.vocab_size", int(cfg.get("vocab_size", seen.get("token_embd.weight", (0, 0))[1])))
    if embed_tokenizer:
        stats.tokenizer_tokens = embed_tokenizer_metadata(w, src)
    w.write(dst)
    return stats


def embed_tokenizer_metadata(w: "G.GgufWriter", src: str) -> int:
    """Copies a byte-level BPE ``tokenizer.json`` found beside the checkpoint into the GGUF metadata (``tokenizer.ggml.model``
    "gpt2", ``tokens``, ``token_type`` with 3 for added / special tokens, ``merges``, ``pre``, ``eos`` / ``bos_token_id``), so
    that the converted file needs no side file.  Returns the number of tokens written (0: no usable tokenizer found)."""
    folder = src if os.path.isdir(src) else os.path.dirname(os.path.abspath(src))
    path = os.path.join(folder, "tokenizer.json")
    if not os.path.exists(path):
        return 0
    try:
        with open(path, encoding="utf-8") as f:
            j = json.load(f)
        model = j["model"]
        if model.get("type", "BPE") != "BPE":
            return 0
        vocab: dict[str, int] = dict(model["vocab"])
        added = {t["content"]: int(t["id"]) for t in j.get("added_tokens", [])}
        size = 1 + max(list(vocab.values()) + list(added.values()))
        tokens, types = [f"[PAD{i}]" for i in range(size)], [5] * size          # 5 = unused id
        for t, i in vocab.items():
            tokens[i], types[i] = t, 1
        for t, i in added.items():
            tokens[i], types[i] = t, 3
        merges = [m if isinstance(m, str) else " ".join(m) for m in model.get("merges", [])]
    except (KeyError, ValueError, TypeError, OSError):
        return 0
    w.add("tokenizer.ggml.model", "gpt2")
    w.add("tokenizer.ggml.pre", "qwen2" if "Split" in json.dumps(j.get("pre_tokenizer")) else "default")
    w.add("tokenizer.ggml.tokens", tokens)
    w.add("tokenizer.ggml.token_type", types)
    w.add("tokenizer.ggml.merges", merges)
    for key, names in (("eos", ("<|im_end|>", "<|endoftext|>", "</s>")), ("bos", ("<|begin_of_text|>", "<s>"))):
        tid = next((added[n] for n in names if n in added), None)
        if tid is not None:
            w.add(f"tokenizer.ggml.{key}_token_id", tid)
    return size

