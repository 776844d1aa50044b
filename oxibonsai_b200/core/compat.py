"""GGUF compatibility report and model card.

Reference: crates/oxibonsai-core/src/gguf/compat.rs:27-455 (``GgufVersion`` capabilities, ``ExtendedQuantType`` ids with
bits per weight, ``GgufCompatReport`` with warnings and unknown quantisation ids, ``check_gguf_header``,
``build_compat_report``) and model_card.rs:70-454 (``ModelCard`` extracted from ``general.*`` and architecture metadata,
rendered as Markdown with a parameter table, plus a one-line summary and an estimated parameter count).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

from . import gguf as G
from .gguf import GgufFile

GGUF_MAGIC = 0x46554747


class GgufVersion:
    SUPPORTED = (2, 3)

    def __init__(self, v: int):
        self.v = v

    @classmethod
    def from_u32(cls, v: int) -> "GgufVersion | None":
        return cls(v) if v in (1, 2, 3) else None

    def to_u32(self) -> int:
        return self.v

    def is_supported(self) -> bool:
        return self.v in self.SUPPORTED

    def supports_f16_kv(self) -> bool:
        return self.v >= 2

    def supports_aligned_tensors(self) -> bool:
        return self.v >= 2

    def supports_64bit_counts(self) -> bool:
        return self.v >= 2


KNOWN_QUANT_IDS = (0, 1, 2, 8, 10, 11, 12, 13, 14, 15, 30, 35, 41, 42, 43, 44)


def quant_name(type_id: int) -> str:
    try:
        return G.type_info(type_id)[0]
    except Exception:
        return f"unknown({type_id})"


def quant_is_known(type_id: int) -> bool:
    return type_id in KNOWN_QUANT_IDS


def quant_bits_per_weight(type_id: int) -> float | None:
    if not quant_is_known(type_id):
        return None
    _, be, bb = G.type_info(type_id)
    return 8.0 * bb / be


class CompatError(ValueError):
    pass


def check_gguf_header(data: bytes) -> tuple[int, int, int]:
    """``(version, tensor_count, metadata_count)`` of a GGUF header, or CompatError."""
    if len(data) < 24:
        raise CompatError("file is shorter than a GGUF header")
    magic, version = struct.unpack_from("<II", data, 0)
    if magic != GGUF_MAGIC:
        raise CompatError(f"bad magic 0x{magic:08x}")
    v = GgufVersion.from_u32(version)
    if v is None or not v.is_supported():
        raise CompatError(f"unsupported GGUF version {version}")
    nt, nkv = struct.unpack_from("<QQ", data, 8)
    return version, nt, nkv


@dataclass
class GgufCompatReport:
    version: int
    tensor_count: int = 0
    metadata_count: int = 0
    warnings: list[str] = field(default_factory=list)
    unknown_quants: dict[int, int] = field(default_factory=dict)     # type id -> tensor count
    quant_histogram: dict[str, int] = field(default_factory=dict)
    compatible: bool = True
    servable_on_gpu: bool = True

    def add_warning(self, w: str) -> None:
        self.warnings.append(w)

    def add_unknown_quant(self, type_id: int) -> None:
        self.unknown_quants[type_id] = self.unknown_quants.get(type_id, 0) + 1

    def finalize(self) -> "GgufCompatReport":
        self.compatible = not self.unknown_quants and GgufVersion(self.version).is_supported()
        return self

    def summary(self) -> str:
        q = ", ".join(f"{k} x{v}" for k, v in sorted(self.quant_histogram.items()))
        s = f"GGUF v{self.version}: {self.tensor_count} tensors ({q}), {self.metadata_count} metadata entries; "
        s += "compatible" if self.compatible else f"NOT compatible (unknown quant ids {sorted(self.unknown_quants)})"
        if self.warnings:
            s += f"; {len(self.warnings)} warning(s): " + "; ".join(self.warnings)
        return s


def build_compat_report(f: GgufFile) -> GgufCompatReport:
    r = GgufCompatReport(f.version, len(f.tensors), len(f.metadata))
    for t in f.tensors:
        if not quant_is_known(t.type):
            r.add_unknown_quant(t.type)
        else:
            n = quant_name(t.type)
            r.quant_histogram[n] = r.quant_histogram.get(n, 0) + 1
    md = f.metadata
    if "general.architecture" not in md:
        r.add_warning("general.architecture is missing")
    if f.alignment not in (32, 64, 128, 256):
        r.add_warning(f"unusual alignment {f.alignment}")
    if not any(t.name == "output.weight" for t in f.tensors):
        r.add_warning("no output.weight tensor (tied embeddings)")
    # the B200 decode kernels take the 128-group sub-2-bit formats natively; other formats are dequantised on load
    native = {G.Q1_0_G128, G.TQ2_0_G128}
    lin = [t for t in f.tensors if t.name.startswith("blk.") and len(t.dims) == 2]
    if lin and any(t.type not in native for t in lin):
        r.servable_on_gpu = all(quant_is_known(t.type) for t in lin)
        r.add_warning("some linear layers are not Q1_0_g128 / TQ2_0_g128 and are requantised to ternary groups for the GPU path")
    return r.finalize()


# ---- model card ------------------------------------------------------------------------------------------------------------------
class render:
    @staticmethod
    def heading(level: int, text: str) -> str:
        return f"{'#' * level} {text}\n\n"

    @staticmethod
    def field(name: str, value: str) -> str:
        return f"- **{name}**: {value}\n"

    @staticmethod
    def table_row(cells: list[str]) -> str:
        return "| " + " | ".join(cells) + " |\n"

    @staticmethod
    def code(text: str) -> str:
        return f"`{text}`"

    @staticmethod
    def bold(text: str) -> str:
        return f"**{text}**"


@dataclass
class ModelCard:
    name: str | None = None
    architecture: str | None = None
    author: str | None = None
    license: str | None = None
    description: str | None = None
    quantization: str | None = None
    file_size_bytes: int | None = None
    context_length: int | None = None
    embedding_length: int | None = None
    block_count: int | None = None
    head_count: int | None = None
    head_count_kv: int | None = None
    feed_forward_length: int | None = None
    vocab_size: int | None = None
    rope_freq_base: float | None = None
    bits_per_weight: float | None = None

    def populated_count(self) -> int:
        return sum(v is not None for v in self.__dict__.values())

    def is_empty(self) -> bool:
        return self.populated_count() == 0

    def estimated_param_count(self) -> int | None:
        if None in (self.embedding_length, self.block_count, self.feed_forward_length, self.vocab_size):
            return None
        h, L, f, v = self.embedding_length, self.block_count, self.feed_forward_length, self.vocab_size
        heads, kv = self.head_count or 1, self.head_count_kv or self.head_count or 1
        hd = h // heads
        attn = h * (heads * hd + 2 * kv * hd) + heads * hd * h
        return L * (attn + 3 * h * f + 2 * h) + 2 * v * h + h

    def to_markdown(self) -> str:
        out = render.heading(1, self.name or "Unnamed model") + render.heading(2, "Model Information")
        for label, v in (("Architecture", self.architecture), ("Author", self.author), ("License", self.license), ("Description", self.description)):
            if v:
                out += render.field(label, str(v))
        if self.quantization:
            out += render.field("Quantization", render.code(self.quantization) + (f" ({self.bits_per_weight:.3f} bits per weight)" if self.bits_per_weight else ""))
        if self.file_size_bytes:
            out += render.field("File Size", f"{self.file_size_bytes} bytes ({self.file_size_bytes / 1e9:.2f} GB)")
        out += "\n" + render.heading(2, "Architecture Details") + render.table_row(["Parameter", "Value"]) + render.table_row(["---", "---"])
        pc = self.estimated_param_count()
        if pc:
            out += render.table_row(["Parameter Count", f"{pc / 1e9:.2f}B"])
        for label, v in (("Context Length", self.context_length), ("Embedding Length", self.embedding_length), ("Layers", self.block_count),
                         ("Attention Heads", self.head_count), ("KV Heads", self.head_count_kv), ("Feed-Forward Length", self.feed_forward_length),
                         ("Vocabulary Size", self.vocab_size), ("RoPE Base", self.rope_freq_base)):
            if v is not None:
                out += render.table_row([label, str(v)])
        return out

    def to_summary(self) -> str:
        pc = self.estimated_param_count()
        parts = [self.name or "model", self.architecture or "?", f"{pc / 1e9:.2f}B params" if pc else None, self.quantization,
                 f"ctx {self.context_length}" if self.context_length else None]
        return " | ".join(p for p in parts if p)


def extract_model_card(f: GgufFile, file_size_bytes: int | None = None) -> ModelCard:
    md = f.metadata
    arch = md.get("general.architecture")
    pre = [arch, "llm"] if arch else ["llm"]

    def get(key):
        for p in pre:
            if f"{p}.{key}" in md:
                return md[f"{p}.{key}"]
        return None
    from ..models.registry import dominant_weight_type
    dom = dominant_weight_type(f)
    vocab = get("vocab_size")
    if vocab is None and any(t.name == "token_embd.weight" for t in f.tensors):
        vocab = f.tensor_info("token_embd.weight").dims[1]
    return ModelCard(name=md.get("general.name"), architecture=arch, author=md.get("general.author"), license=md.get("general.license"),
                     description=md.get("general.description"), quantization=quant_name(dom) if dom is not None else None,
                     file_size_bytes=file_size_bytes, context_length=get("context_length"), embedding_length=get("embedding_length"),
                     block_count=get("block_count"), head_count=get("attention.head_count"), head_count_kv=get("attention.head_count_kv"),
                     feed_forward_length=get("feed_forward_length"), vocab_size=vocab, rope_freq_base=get("rope.freq_base"),
                     bits_per_weight=quant_bits_per_weight(dom) if dom is not None else None)
