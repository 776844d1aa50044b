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
             f"  batching     up to {cfg.max_concurrent} concurrent sequences per engine, max_seq_len {cfg.max_seq_len}",
             f"  GPUs         " + (f"tensor parallel over {cfg.tensor_parallel}" if cfg.tensor_parallel > 1 else f"{cfg.replicas} replica(s)"),
             f"  listening    http://{cfg.host}:{cfg.port}  (metrics {cfg.metrics_path if cfg.metrics_enabled else 'off'}, auth {'on' if cfg.bearer_token else 'off'})"]
    return "\n".join(lines)


def main(argv: list[str] | None = None) -> int:
    from ..cli import no_tokenizer_warning, resolve_tokenizer
    from ..runtime import EngineBuilder
    from ..runtime.observability import init_tracing
    from ..runtime.presets import SamplingParams
    from ..runtime.scheduler import BatchScheduler
    from ..tokenizer import load_tokenizer
    from .app import ReplicaBackend, SchedulerBackend, SerialBackend, create_app
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
    import os
    tp = cfg.tensor_parallel
    rank, leader = 0, None
    builder = lambda dev: (EngineBuilder().model_path(cfg.model_path).sampler(sp).max_seq_len(cfg.max_seq_len).max_batch(cfg.max_concurrent)
                           .kv_cache(cfg.kv_cache).device(dev))
    if tp > 1:
        # one process per GPU (torchrun): NCCL carries the bootstrap of the symmetric buffers, a gloo group the commands
        import torch
        import torch.distributed as dist
        from ..runtime.tp_serving import CommandChannel, LeaderEngine, follower_loop
        rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
        if world != tp:
            print(f"error: --tensor-parallel {tp} needs {tp} processes (torchrun --nproc-per-node {tp}), found WORLD_SIZE={world}", file=sys.stderr)
            return 2
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        channel = CommandChannel(dist.new_group(backend="gloo"))
        engine = builder(f"cuda:{local}").tensor_parallel(rank, world).build()
        if rank != 0:
            n = follower_loop(engine, channel, on_error=lambda op, e: print(f"[rank {rank}] {op}: {e}", file=sys.stderr))
            print(f"[rank {rank}] leader shut down after {n} commands", file=sys.stderr)
            dist.destroy_process_group()
            return 0
        leader = engine = LeaderEngine(engine, channel)
    engines = [engine] if tp > 1 else [builder(f"cuda:{i}").build() for i in range(cfg.replicas)]
    engine = engines[0]
    scheds = []
    policy = None
    if cfg.kv_policy != "off" and hasattr(engine, "enable_kv_formats"):
        from ..runtime.kv_policy import KvCachePolicy
        policy = KvCachePolicy.aggressive() if cfg.kv_policy == "aggressive" else KvCachePolicy()
    if hasattr(engine, "step_batch"):             # continuous batching over the engine's sequence slots
        for e in engines:
            if not e.exact and hasattr(e, "enable_prefix_cache"):
                e.enable_prefix_cache()
                if policy is not None:
                    e.enable_kv_formats(("f16", "q8", "q4"))      # the levels of the policy that the engine does not have yet
            scheds.append(BatchScheduler(e, queue_capacity=cfg.queue_capacity, prefill_chunk_tokens=cfg.prefill_chunk_tokens, prefill_chunk_boost=cfg.prefill_chunk_boost,
                                         kv_policy=policy).start())
        backend = SchedulerBackend(scheds[0], engine.config.name) if len(scheds) == 1 else ReplicaBackend(scheds, engine.config.name)
    else:                                         # an engine without sequence slots: one request at a time
        backend = SerialBackend(engine, engine.config.name)
    app = create_app(backend, tokenizer, cfg, kv_policy=policy)
    print(banner(cfg, engine.model_info()), file=sys.stderr)
    import uvicorn
    try:
        uvicorn.run(app, host=cfg.host, port=cfg.port, log_level=cfg.log_level if cfg.log_level in ("debug", "info", "warning", "error") else "info")
    finally:
        for sc in scheds:
            sc.stop()
        if leader is not None:
            leader.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
