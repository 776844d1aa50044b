"""oxibonsai_b200: a Blackwell-native sub-2-bit LLM inference engine.

PyTorch is the tensor/stream/allocator layer; every hot op is a hand-written sm_100a CUDA kernel
in ``csrc/cuda`` and ``csrc/comm``; the host runtime is C++ in ``csrc/core``, ``csrc/cpu`` and
``csrc/runtime``.

The package root is the facade (reference: the ``oxibonsai`` crate re-exporting core, kernels, model, runtime, tokenizer,
rag and eval, crates/oxibonsai/src/lib.rs): the names below resolve on first use, so ``import oxibonsai_b200`` stays light
(no torch, no native build) until something is asked for.

    from oxibonsai_b200 import EngineBuilder, SamplingParams
    engine = EngineBuilder().model_path("model.gguf").preset("balanced").build()
"""
__version__ = "0.1.0"

_EXPORTS = {
    # core
    "GgufFile": "core", "GgufWriter": "core", "GgufStreamParser": "core", "Qwen3Config": "core", "Oracle": "core", "write_synthetic_gguf": "core",
    "quantize": "core.blocks", "dequantize": "core.blocks",
    # runtime
    "EngineBuilder": "runtime", "SamplingParams": "runtime.presets", "SamplingPreset": "runtime.presets", "BatchScheduler": "runtime.scheduler",
    "GpuSpeculativeDecoder": "runtime.speculative", "KvCachePolicy": "runtime.kv_policy", "InferenceMetrics": "runtime.metrics",
    "TokenTable": "runtime.constrained", "GrammarConstraint": "runtime.constrained", "DfaConstraint": "runtime.constrained",
    "json_constraint": "runtime.constrained", "json_schema_constraint": "runtime.constrained", "build_tool_constraint": "runtime.tools",
    "ContinuousBatchScheduler": "runtime.batching", "AsyncSchedulerFront": "runtime.batching", "batch_generate": "runtime.batching",
    "ElasticGroup": "runtime.elastic",
    # tokenizer, retrieval, evaluation
    "BpeTokenizer": "tokenizer", "ByteTokenizer": "tokenizer", "load_tokenizer": "tokenizer", "chat_prompt": "tokenizer", "ChatTemplateKind": "tokenizer.toolkit",
    "RagPipeline": "rag", "VectorStore": "rag", "TfIdfEmbedder": "rag",
    "PerplexityEvaluator": "eval", "MultipleChoiceEvaluator": "eval", "EvalReport": "eval",
    # conversion, server
    "convert_safetensors_to_gguf": "convert", "convert_onnx_to_gguf": "convert.onnx",
    "create_app": "server.app", "serve": "server.app", "ServerConfig": "server.config",
}
__all__ = sorted(_EXPORTS) + ["__version__"]


def __getattr__(name: str):
    mod = _EXPORTS.get(name)
    if mod is None:
        raise AttributeError(f"module 'oxibonsai_b200' has no attribute {name!r}")
    import importlib
    value = getattr(importlib.import_module(f"{__name__}.{mod}"), name)
    globals()[name] = value
    return value


def __dir__():
    return __all__
