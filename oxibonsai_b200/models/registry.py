"""Model registry: variant detection, specs, capability profiles, fluent config builder and GGUF loading utilities.

Reference: crates/oxibonsai-model/src/model_registry.rs:39-80 (variant from ``(layers, hidden)``: (36, 4096) -> 8B,
(24, 2560) -> 4B, (16, 1536) -> 1.7B, else Custom; ternary / FP8 variants from a sample tensor type), model_variants.rs:39-437
(``ModelSpec``, ``CapabilityProfile``), model_config_builder.rs:71- (``ModelConfigBuilder``) and gguf_loader.rs:19-509
(validation, memory budget, chunked tensor iteration).  The shapes the B200 benchmarks use (36 x 4096, 36 x 2560,
28 x 2048 - the published Qwen3 8B / 4B / 1.7B shapes) are recognised too.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from enum import Enum
from typing import Iterator

from ..core import gguf as G
from ..core.gguf import GgufFile, Qwen3Config


class ModelVariant(Enum):
    BONSAI_8B = "Bonsai-8B"
    BONSAI_4B = "Bonsai-4B"
    BONSAI_1_7B = "Bonsai-1.7B"
    TERNARY_8B = "Ternary-Bonsai-8B"
    TERNARY_4B = "Ternary-Bonsai-4B"
    TERNARY_1_7B = "Ternary-Bonsai-1.7B"
    FP8_8B = "FP8-Bonsai-8B"
    FP8_4B = "FP8-Bonsai-4B"
    FP8_1_7B = "FP8-Bonsai-1.7B"
    CUSTOM = "Custom"


_SIZE_BY_SHAPE = {(36, 4096): "8B", (24, 2560): "4B", (36, 2560): "4B", (16, 1536): "1_7B", (28, 2048): "1_7B"}
_TERNARY_TYPES = (G.TQ2_0_G128, G.TQ2_0)
_FP8_TYPES = (G.F8_E4M3, G.F8_E5M2)


def variant_from_config(cfg: Qwen3Config, sample_tensor_type: int | None = None) -> ModelVariant:
    size = _SIZE_BY_SHAPE.get((cfg.layers, cfg.hidden))
    if size is None:
        return ModelVariant.CUSTOM
    family = "TERNARY" if sample_tensor_type in _TERNARY_TYPES else ("FP8" if sample_tensor_type in _FP8_TYPES else "BONSAI")
    return ModelVariant[f"{family}_{size}"]


def default_config(variant: ModelVariant) -> Qwen3Config:
    size = variant.name.rsplit("_", 2)[-1] if variant != ModelVariant.CUSTOM else "8B"
    if variant.name.endswith("1_7B"):
        size = "1_7B"
    shapes = {"8B": dict(hidden=4096, inter=12288, layers=36, heads=32, kv_heads=8), "4B": dict(hidden=2560, inter=9728, layers=36, heads=32, kv_heads=8),
              "1_7B": dict(hidden=2048, inter=6144, layers=28, heads=16, kv_heads=8)}
    return Qwen3Config(head_dim=128, vocab=151936, context=65536, name=variant.value, **shapes[size])


def param_count(cfg: Qwen3Config, tied: bool = False) -> int:
    q, kv = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
    per_layer = cfg.hidden * (q + 2 * kv) + q * cfg.hidden + 3 * cfg.hidden * cfg.inter + 2 * cfg.hidden + 2 * cfg.head_dim
    return cfg.layers * per_layer + cfg.vocab * cfg.hidden * (1 if tied else 2) + cfg.hidden


def bits_per_weight(type_id: int) -> float:
    _, be, bb = G.type_info(type_id)
    return 8.0 * bb / be


def expected_model_size_bytes(cfg: Qwen3Config, weight_type: int = G.TQ2_0_G128, embedding_type: int = G.F16, tied: bool = False) -> int:
    q, kv = cfg.heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
    lin = cfg.layers * (cfg.hidden * (q + 2 * kv) + q * cfg.hidden + 3 * cfg.hidden * cfg.inter)
    emb = cfg.vocab * cfg.hidden * (1 if tied else 2)
    norms = (cfg.layers * (2 * cfg.hidden + 2 * cfg.head_dim) + cfg.hidden) * 4
    return int(lin * bits_per_weight(weight_type) / 8 + emb * bits_per_weight(embedding_type) / 8 + norms)


@dataclass
class ModelSpec:
    name: str
    variant: ModelVariant
    config: Qwen3Config
    param_count: int
    weights_size_bytes: int
    kv_cache_4k_bytes: int
    min_memory_bytes: int
    description: str = ""


def spec_for_variant(variant: ModelVariant) -> ModelSpec:
    cfg = default_config(variant)
    wt = G.TQ2_0_G128 if variant.name.startswith("TERNARY") else (G.F8_E4M3 if variant.name.startswith("FP8") else G.Q1_0_G128)
    w = expected_model_size_bytes(cfg, wt)
    kv4k = 4096 * cfg.layers * 2 * cfg.kv_heads * cfg.head_dim * 2
    kind = {"TERNARY": "ternary (1.58-bit) weights in 128-wide groups", "FP8": "FP8 E4M3 block weights", "BONSAI": "1-bit sign weights in 128-wide groups"}
    fam = variant.name.split("_")[0]
    return ModelSpec(variant.value, variant, cfg, param_count(cfg), w, kv4k, int((w + kv4k) * 1.15),
                     f"Qwen3-shaped decoder with {kind.get(fam, 'custom weights')}")


def all_specs() -> list[ModelSpec]:
    return [spec_for_variant(v) for v in ModelVariant if v != ModelVariant.CUSTOM]


def known_variants() -> list[ModelVariant]:
    return [v for v in ModelVariant if v != ModelVariant.CUSTOM]


@dataclass
class CapabilityProfile:
    max_context_len: int
    supports_system_prompt: bool = True
    supports_streaming: bool = True
    supports_tensor_parallel: bool = True
    recommended_temperature: float = 0.7
    recommended_top_p: float = 0.9
    languages: tuple[str, ...] = ("en", "zh", "ja", "ko", "fr", "de", "es")
    use_cases: tuple[str, ...] = ("chat", "code", "summarisation")


def capability_profile(variant: ModelVariant) -> CapabilityProfile:
    p = CapabilityProfile(max_context_len=65536)
    if variant.name.endswith("1_7B"):
        return replace(p, use_cases=("chat", "draft model for speculative decoding", "edge"), recommended_temperature=0.6)
    if variant.name.endswith("8B"):
        return replace(p, use_cases=("chat", "code", "reasoning", "tool use"))
    return p


class ConfigError(ValueError):
    pass


class ModelConfigBuilder:
    def __init__(self):
        self._v = dict(hidden=4096, inter=12288, layers=36, heads=32, kv_heads=8, head_dim=None, vocab=151936, context=32768, rope_base=1e6,
                       eps=1e-6, arch="qwen3", name="custom")

    def _set(self, k, v):
        self._v[k] = v
        return self

    def layers(self, n): return self._set("layers", n)
    def hidden_size(self, n): return self._set("hidden", n)
    def num_attention_heads(self, n): return self._set("heads", n)
    def num_kv_heads(self, n): return self._set("kv_heads", n)
    def head_dim(self, n): return self._set("head_dim", n)
    def intermediate_size(self, n): return self._set("inter", n)
    def vocab_size(self, n): return self._set("vocab", n)
    def max_position_embeddings(self, n): return self._set("context", n)
    def rope_freq_base(self, x): return self._set("rope_base", float(x))
    def rms_norm_eps(self, x): return self._set("eps", float(x))
    def architecture(self, s): return self._set("arch", s)
    def model_name(self, s): return self._set("name", s)

    def build(self) -> Qwen3Config:
        v = dict(self._v)
        if v["head_dim"] is None:
            if v["hidden"] % v["heads"]:
                raise ConfigError("hidden_size must be divisible by num_attention_heads when head_dim is not given")
            v["head_dim"] = v["hidden"] // v["heads"]
        for k in ("layers", "hidden", "heads", "kv_heads", "inter", "vocab", "context", "head_dim"):
            if v[k] <= 0:
                raise ConfigError(f"{k} must be positive")
        if v["heads"] % v["kv_heads"]:
            raise ConfigError("num_attention_heads must be a multiple of num_kv_heads")
        if v["hidden"] % 128 or v["inter"] % 128:
            raise ConfigError("hidden_size and intermediate_size must be multiples of the 128-weight group")
        if v["head_dim"] % 2:
            raise ConfigError("head_dim must be even for rotary embeddings")
        return Qwen3Config(**v)

    def build_tiny(self) -> Qwen3Config:
        return self.layers(2).hidden_size(256).intermediate_size(512).num_attention_heads(4).num_kv_heads(2).head_dim(64).vocab_size(1000) \
            .max_position_embeddings(512).model_name("tiny").build()


# ---- GGUF loading utilities ----------------------------------------------------------------------------------------------------
@dataclass
class GgufValidation:
    ok: bool
    errors: list[str] = field(default_factory=list)
    warnings: list[str] = field(default_factory=list)
    dominant_type: int | None = None
    variant: ModelVariant = ModelVariant.CUSTOM


def dominant_weight_type(f: GgufFile) -> int | None:
    sizes: dict[int, int] = {}
    for t in f.tensors:
        if t.name.startswith("blk.") and len(t.dims) == 2:
            sizes[t.type] = sizes.get(t.type, 0) + t.n_elements
    return max(sizes, key=sizes.get) if sizes else None


def validate_gguf(f: GgufFile) -> GgufValidation:
    """Checks that every tensor a Qwen3 decoder needs is present with consistent shapes."""
    v = GgufValidation(True)
    try:
        cfg = f.config()
    except Exception as e:
        return GgufValidation(False, [f"cannot read the model configuration: {e}"])
    need = ["token_embd.weight", "output_norm.weight"]
    for l in range(cfg.layers):
        need += [f"blk.{l}.{s}.weight" for s in ("attn_norm", "attn_q", "attn_k", "attn_v", "attn_output", "ffn_norm", "ffn_gate", "ffn_up", "ffn_down")]
    for n in need:
        if not f.has_tensor(n):
            v.errors.append(f"missing tensor {n}")
    if not f.has_tensor("output.weight"):
        v.warnings.append("no output.weight: the embedding table is used as the LM head")
    if f.has_tensor("blk.0.attn_q.weight"):
        k, n = f.tensor_info("blk.0.attn_q.weight").dims
        if k != cfg.hidden or n != cfg.heads * cfg.head_dim:
            v.errors.append(f"blk.0.attn_q.weight is {n}x{k}, expected {cfg.heads * cfg.head_dim}x{cfg.hidden}")
    if not f.has_tensor("blk.0.attn_q_norm.weight"):
        v.warnings.append("no QK-norm tensors")
    v.dominant_type = dominant_weight_type(f)
    v.variant = variant_from_config(cfg, v.dominant_type)
    v.ok = not v.errors
    return v


def iter_tensor_chunks(f: GgufFile, name: str, chunk_bytes: int = 64 << 20) -> Iterator[memoryview]:
    """Streams one tensor's bytes in bounded chunks (for uploads that must not stage the whole tensor)."""
    raw = f.tensor_bytes(name)
    for off in range(0, len(raw), chunk_bytes):
        yield raw[off:off + chunk_bytes]


def memory_budget_check(f: GgufFile, available_bytes: int, context: int = 4096, batch: int = 1, kv_bytes_per_elem: float = 2.0) -> dict:
    cfg = f.config()
    weights = sum(G.data_size(t.type, t.n_elements) for t in f.tensors)
    kv = int(context * batch * cfg.layers * 2 * cfg.kv_heads * cfg.head_dim * kv_bytes_per_elem)
    return {"weights": weights, "kv_cache": kv, "total": weights + kv, "available": available_bytes, "fits": weights + kv <= available_bytes}
