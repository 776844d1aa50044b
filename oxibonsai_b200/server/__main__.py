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
             f"  listening    http://{cfg.host}:{cfg.port}  (metrics {cfg.metrics_path if cfg.metrics_enabled else 'off'}, auth {'on' if cfg.bearer_token else 'off'}, front {'native' if cfg.native_front else 'uvicorn'})"]
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
    tokenizer = load_tokenizer(tok_path, cfg.tokenizer_kind, model_path=cfg.model_path)
    if tok_path is None:
        if type(tokenizer).__name__ == "BpeTokenizer":
            print(f"no tokenizer.json found; using the vocabulary embedded in {cfg.model_path} ({tokenizer.vocab_size} tokens)", file=sys.stderr)
        else:
            print(no_tokenizer_warning(searched), file=sys.stderr)
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
        if cfg.tp_elastic:
            return _serve_elastic(cfg, tokenizer, builder, rank, world, local)
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
            scheds.append(BatchScheduler(e, eos_token=getattr(tokenizer, "eos_token_id", None), queue_capacity=cfg.queue_capacity, prefill_chunk_tokens=cfg.prefill_chunk_tokens, prefill_chunk_boost=cfg.prefill_chunk_boost,
                                         kv_policy=policy, idle_hook=getattr(leader, "keepalive", None), overlap=cfg.overlap_steps,
                                         admit_tokens_per_step=cfg.admit_tokens_per_step).start())
        backend = SchedulerBackend(scheds[0], engine.config.name) if len(scheds) == 1 else ReplicaBackend(scheds, engine.config.name)
    else:                                         # an engine without sequence slots: one request at a time
        backend = SerialBackend(engine, engine.config.name)
    app = create_app(backend, tokenizer, cfg, kv_policy=policy)
    print(banner(cfg, engine.model_info()), file=sys.stderr)
    from .app import serve
    try:
        serve(app, cfg.host, cfg.port, cfg.log_level, tokenizer=tokenizer, native=cfg.native_front, vocab_size=engine.config.vocab)
    finally:
        for sc in scheds:
            sc.stop()
        if leader is not None:
            leader.shutdown()
    return 0


def _serve_elastic(cfg, tokenizer, builder, uid: int, world: int, local: int) -> int:
    """Tensor-parallel serving that survives the loss of a follower rank: heartbeats through the job's TCP store, a check
    before every launch, and on a loss a new generation at the largest degree the survivors fill (8 -> 4 -> 2 -> 1), the
    engine rebuilt from the checkpoint for that degree.  Rank 0 keeps the HTTP front up throughout; requests that arrive
    while the group re-forms get 503."""
    import os
    import threading

    import torch
    import torch.distributed as dist

    from ..runtime.elastic import ElasticGroup, RankLost
    from ..runtime.scheduler import BatchScheduler
    from ..runtime.tp_serving import CommandChannel, ElasticBackend, lead_with_scheduler, run_elastic_rank
    from .app import create_app
    port = int(os.environ.get("MASTER_PORT", "29500")) + 1          # next to torchrun's own rendezvous store
    store = dist.TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"), port, is_master=(uid == 0), wait_for_workers=False)
    device = torch.device("cuda", local)

    def init_group(prefix_store, rank, size):
        from datetime import timedelta
        dist.init_process_group("nccl", store=prefix_store, rank=rank, world_size=size, device_id=device, timeout=timedelta(seconds=60))

    group = ElasticGroup(store, uid, world, backend="nccl", interval=min(0.5, cfg.tp_heartbeat_timeout / 5), timeout=cfg.tp_heartbeat_timeout,
                         init_group=init_group)

    def build_engine(rank: int, size: int):
        b = builder(f"cuda:{local}")
        return (b.tensor_parallel(rank, size) if size > 1 else b).build()

    stop = threading.Event()
    backend = ElasticBackend(os.path.basename(cfg.model_path), cfg.max_seq_len)

    def fatal(e: Exception) -> bool:
        # a lost rank shows up as the watchdog's exception, or first as a kernel whose bounded wait ran out
        return isinstance(e, RankLost) or (type(e).__name__ == "CudaKernelError" and group.confirm_loss())

    def make_scheduler(le, g):
        if hasattr(le, "enable_prefix_cache") and not le.exact:
            le.enable_prefix_cache()
        return BatchScheduler(le, eos_token=getattr(tokenizer, "eos_token_id", None), queue_capacity=cfg.queue_capacity,
                              prefill_chunk_tokens=cfg.prefill_chunk_tokens, prefill_chunk_boost=cfg.prefill_chunk_boost, before_launch=g.check,
                              on_fatal=lambda e: fatal(e), idle_hook=le.keepalive, admit_tokens_per_step=cfg.admit_tokens_per_step)

    def lead(le, g):
        inner = lead_with_scheduler(make_scheduler, backend, stop)
        try:
            inner(le, g)
        except Exception as e:  # noqa: BLE001 - a kernel time-out that the watchdog attributes to a lost rank re-forms the group
            if isinstance(e, RankLost) or g.confirm_loss(0.0):
                raise RankLost(g.lost(), g.generation) from e
            raise

    make_channel = lambda: CommandChannel(dist.new_group(backend="gloo"))
    on_error = lambda op, e: print(f"[uid {uid}] {op}: {e}", file=sys.stderr)
    if uid != 0:
        history = run_elastic_rank(group, build_engine, make_channel, lead, on_error)
        print(f"[uid {uid}] done after {len(history)} re-formation(s)", file=sys.stderr)
        return 0
    worker = threading.Thread(target=lambda: run_elastic_rank(group, build_engine, make_channel, lead, on_error), name="bonsai-elastic-leader", daemon=True)
    worker.start()
    app = create_app(backend, tokenizer, cfg)
    from .app import serve
    try:
        serve(app, cfg.host, cfg.port, cfg.log_level, tokenizer=tokenizer, native=cfg.native_front)
    finally:
        stop.set()
        worker.join(timeout=30)
    return 0


if __name__ == "__main__":
    sys.exit(main())
