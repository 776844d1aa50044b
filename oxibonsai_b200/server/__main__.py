"""``python -m oxibonsai_b200.server``: the standalone OpenAI-compatible server.

Reference: the ``oxibonsai-serve`` binary (crates/oxibonsai-serve/src/main.rs:37-197): layered configuration
(defaults < TOML < OXIBONSAI_* environment < command line), validation, tokenizer auto-discovery beside the model,
a banner with the effective settings, then the HTTP server with graceful shutdown.
"""
from __future__ import annotations

import sys


def banner(cfg, info: dict) -> str:
    lines = ["oxibonsai_b200 server",
             f"  model        {cfg.model_path}",
             f"  shape        {info.get('layers')} layers x {info.get('hidden')} hidden, vocab {info.get('vocab')}",
             f"  weights      {info.get('weight_bytes', 0) / 1e9:.2f} GB on device, KV cache {cfg.kv_cache} ({info.get('kv_bytes', 0) / 1e9:.2f} GB)",
             f"  batching     up to {cfg.max_concurrent} concurrent sequences, max_seq_len {cfg.max_seq_len}",
             f"  listening    http://{cfg.host}:{cfg.port}  (metrics {cfg.metrics_path if cfg.metrics_enabled else 'off'}, auth {'on' if cfg.bearer_token else 'off'})"]
    return "\n".join(lines)


def main(argv: list[str] | None = None) -> int:
    from ..cli import no_tokenizer_warning, resolve_tokenizer
    from ..runtime import EngineBuilder
    from ..runtime.observability import init_tracing
    from ..runtime.presets import SamplingParams
    from ..runtime.scheduler import BatchScheduler
    from ..tokenizer import load_tokenizer
    from .app import SchedulerBackend, SerialBackend, create_app
    from .config import load_config
    cfg = load_config(sys.argv[1:] if argv is None else argv)
    if cfg.model_path is None:
        print("error: --model-path (or OXIBONSAI_MODEL_PATH, or [model] model_path in the TOML file) is required", file=sys.stderr)
        return 2
    init_tracing(cfg.log_level, cfg.json_logs)
    tok_path, searched = resolve_tokenizer(cfg.model_path, cfg.tokenizer_path)
    if tok_path is None:
        print(no_tokenizer_warning(searched), file=sys.stderr)
    tokenizer = load_tokenizer(tok_path, cfg.tokenizer_kind)
    sp = SamplingParams(temperature=cfg.temperature, top_k=cfg.top_k, top_p=cfg.top_p, repetition_penalty=cfg.repetition_penalty,
                        max_tokens=cfg.max_tokens, seed=cfg.seed)
    engine = (EngineBuilder().model_path(cfg.model_path).sampler(sp).max_seq_len(cfg.max_seq_len).max_batch(cfg.max_concurrent)
              .kv_cache(cfg.kv_cache).build())
    sched = None
    if hasattr(engine, "open_sequence"):          # the sub-2-bit runner: continuous batching over its sequence slots
        if not engine.exact:
            engine.enable_prefix_cache()
        sched = BatchScheduler(engine, queue_capacity=cfg.queue_capacity).start()
        backend = SchedulerBackend(sched, engine.config.name)
    else:                                         # generic block formats: one request at a time
        backend = SerialBackend(engine, engine.config.name)
    app = create_app(backend, tokenizer, cfg)
    print(banner(cfg, engine.model_info()), file=sys.stderr)
    import uvicorn
    try:
        uvicorn.run(app, host=cfg.host, port=cfg.port, log_level=cfg.log_level if cfg.log_level in ("debug", "info", "warning", "error") else "info")
    finally:
        if sched is not None:
            sched.stop()
    return 0


if __name__ == "__main__":
    sys.exit(main())
