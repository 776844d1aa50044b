"""Fluent builders: ``EngineBuilder``, ``SamplerBuilder``, ``ConfigBuilder``.

Reference: crates/oxibonsai-runtime/src/builders.rs:34-300 (validation rules T >= 0, 0 <= top_p <= 1,
repetition_penalty >= 1) and the README surface ``EngineBuilder::new().model_path(..).preset(..).max_seq_len(..).build()``
(README.md:112-131).
"""
from __future__ import annotations

from dataclasses import replace

from .presets import SamplingParams, SamplingPreset


class SamplerBuilder:
    def __init__(self, base: SamplingParams | None = None):
        self._p = base or SamplingParams()

    def temperature(self, v: float) -> "SamplerBuilder":
        self._p = replace(self._p, temperature=float(v)); return self

    def top_k(self, v: int) -> "SamplerBuilder":
        self._p = replace(self._p, top_k=int(v)); return self

    def top_p(self, v: float) -> "SamplerBuilder":
        self._p = replace(self._p, top_p=float(v)); return self

    def repetition_penalty(self, v: float) -> "SamplerBuilder":
        self._p = replace(self._p, repetition_penalty=float(v)); return self

    def max_tokens(self, v: int) -> "SamplerBuilder":
        self._p = replace(self._p, max_tokens=int(v)); return self

    def seed(self, v: int) -> "SamplerBuilder":
        self._p = replace(self._p, seed=int(v)); return self

    def preset(self, name) -> "SamplerBuilder":
        base = SamplingPreset.parse(name).params()
        self._p = replace(base, max_tokens=self._p.max_tokens, seed=self._p.seed); return self

    def build(self) -> SamplingParams:
        return self._p.validate()


class EngineBuilder:
    """Collects engine options; ``build()`` loads the checkpoint and returns an ``InferenceEngine`` (Q1_0_g128 / TQ2_0_g128
    weights) or a ``GenericFormatEngine`` (any other block format)."""

    def __init__(self):
        self._model_path: str | None = None
        self._sampler = SamplerBuilder()
        self._max_seq_len = 4096
        self._max_batch = 1
        self._kv_dtype = "f16"
        self._device = "cuda:0"
        self._tp_size = 1
        self._tp_rank = 0
        self._page_size = 64
        self._kv_pages: int | None = None
        self._warmup = True
        self._exact: bool | None = None
        self._repack_cache: str | None = None
        self._prefill_chunk: int | None = None

    def model_path(self, path: str) -> "EngineBuilder":
        self._model_path = str(path); return self

    def preset(self, name) -> "EngineBuilder":
        self._sampler.preset(name); return self

    def sampler(self, params: SamplingParams) -> "EngineBuilder":
        self._sampler = SamplerBuilder(params); return self

    def max_seq_len(self, n: int) -> "EngineBuilder":
        if n <= 0:
            raise ValueError("max_seq_len must be positive")
        self._max_seq_len = int(n); return self

    def max_batch(self, n: int) -> "EngineBuilder":
        self._max_batch = int(n); return self

    def kv_cache(self, dtype: str, page_size: int | None = None, pages: int | None = None) -> "EngineBuilder":
        self._kv_dtype = dtype
        if page_size:
            self._page_size = page_size
        self._kv_pages = pages
        return self

    def device(self, dev: str) -> "EngineBuilder":
        self._device = dev; return self

    def tensor_parallel(self, rank: int, size: int) -> "EngineBuilder":
        self._tp_rank, self._tp_size = int(rank), int(size); return self

    def seed(self, seed: int) -> "EngineBuilder":
        self._sampler.seed(seed); return self

    def warmup(self, on: bool) -> "EngineBuilder":
        self._warmup = bool(on); return self

    def exact(self, on: bool | None) -> "EngineBuilder":
        """``True``: f32 activations end to end (the mode held to the CPU scalar path token for token); ``False``: f16
        activations on the tensor-core kernels; ``None`` (default): exact only with an f32 KV cache."""
        self._exact = on; return self

    def repack_cache(self, directory: str | None) -> "EngineBuilder":
        """Directory in which the device layouts of the weights are kept between starts (None = no cache)."""
        self._repack_cache = directory; return self

    def prefill_chunk(self, tokens: int | None) -> "EngineBuilder":
        """Tokens per prompt chunk of the batched prefill path (a multiple of 64; default 4096)."""
        self._prefill_chunk = None if tokens is None else int(tokens); return self

    def options(self) -> dict:
        return dict(model_path=self._model_path, max_seq_len=self._max_seq_len, max_batch=self._max_batch, kv_dtype=self._kv_dtype,
                    device=self._device, sampling=self._sampler.build(), page_size=self._page_size, kv_pages=self._kv_pages,
                    tp_rank=self._tp_rank, tp_size=self._tp_size, warmup=self._warmup, exact=self._exact,
                    repack_cache=self._repack_cache, prefill_chunk=self._prefill_chunk)

    def build(self):
        if not self._model_path:
            raise ValueError("EngineBuilder: model_path is required")
        from .engine import load_engine
        return load_engine(**self.options())     # the sub-2-bit runner, or the generic-format engine for other weight types
