"""Serving-side services on CPU: caches, registries, vector index, profiler, request ids, stream metrics, quality
metrics, auto tuner, hash ring / registry / replica pool, asyncio front."""
import asyncio
import io
import json
import time

import numpy as np
import pytest

from oxibonsai_b200.core import Qwen3Config
from oxibonsai_b200.runtime import caches as CA
from oxibonsai_b200.runtime import distributed as D
from oxibonsai_b200.runtime import observability as OB

CFG_8B = Qwen3Config(hidden=4096, inter=12288, layers=36, heads=32, kv_heads=8, head_dim=128, vocab=151936, context=65536, name="8b")


def test_hot_reload_and_model_registry_router():
    h = CA.HotReloadCoordinator().with_max_history(2)
    assert h.current_generation() == 0 and h.current_version() is None
    assert h.reload("a.gguf", lambda p: p.upper()) == "A.GGUF" and h.current_generation() == 1
    with pytest.raises(OSError):
        h.reload("b.gguf", lambda p: (_ for _ in ()).throw(OSError("gone")))
    h.record_reload("c.gguf")
    h.record_reload("d.gguf")
    assert h.reload_count() == 3 and [v.path for v in h.version_history()] == ["c.gguf", "d.gguf"]
    assert h.log.total_events() == 4 and not h.log.recent_events(4)[1].success and "reloads" in h.log.summary()
    reg = CA.ModelRegistry()
    reg.register(CA.ModelEndpoint(CA.ModelId("bonsai-8b"), "/m/8b.gguf", context_length=32768, is_default=True))
    reg.register(CA.ModelEndpoint(CA.ModelId("bonsai-8b:sql"), "/m/8b.gguf", adapter="sql", context_length=8192))
    reg.add_alias("default-chat", "bonsai-8b")
    r = CA.ModelRouter(reg)
    assert r.route(None).model_id == "bonsai-8b" and r.route("default-chat").path == "/m/8b.gguf"
    assert r.route("bonsai-8b:sql").adapter == "sql" and CA.ModelId("bonsai-8b:sql").adapter_name() == "sql" and CA.ModelId("x").is_base()
    assert r.route_for_context(4000).model_id == "bonsai-8b:sql" and r.route_for_context(20000).model_id == "bonsai-8b"
    reg.set_status("bonsai-8b", "draining")
    with pytest.raises(CA.RoutingError):
        r.route("bonsai-8b")
    with pytest.raises(CA.RoutingError):
        r.route("nope")
    assert len(r.models_list()) == 2 and reg.unregister("bonsai-8b") and len(reg) == 1
    st = CA.AdapterStack().add("a", 1.0).add("b", 3.0)
    st.normalize_weights()
    assert [a.weight for a in st.adapters] == [0.25, 0.75]


def test_model_cache_and_warmup():
    c = CA.ModelCache(CA.ModelCacheConfig(max_models=2, max_idle_seconds=0.0))
    loads = []
    load = lambda k: (lambda: (loads.append(k) or f"model-{k}", 10))
    assert c.get_or_insert("a", load("a")) == "model-a" and c.get_or_insert("a", load("a")) == "model-a" and loads == ["a"]
    c.get_or_insert("b", load("b"))
    c.get_or_insert("c", load("c"))
    assert len(c) == 2 and not c.contains("a") and c.hit_rate() == pytest.approx(0.25) and c.total_memory_bytes() == 20
    time.sleep(0.01)
    assert c.evict_stale() == 2 and c.stats()["evictions"] == 3
    w = CA.ModelWarmup().with_tokens(2).with_prompt([1, 2, 3])
    seen = []
    assert w.needs_warmup() and w.run(lambda p, n: seen.append((p, n))) >= 0 and not w.needs_warmup() and seen == [([1, 2, 3], 2)]


def test_dedup_and_semantic_cache_and_nsw_index():
    k1 = CA.request_key("hello", temperature=0, max_tokens=5)
    assert k1 == CA.request_key("hello", max_tokens=5, temperature=0) != CA.request_key("hello", temperature=1, max_tokens=5)
    assert CA.request_key([{"role": "user", "content": "a"}]) != CA.request_key([{"role": "system", "content": "a"}])
    d = CA.DedupCache(capacity=2, default_ttl=None)
    assert d.get(k1) is None
    d.insert(k1, "world")
    assert d.get(k1) == "world" and d.hit_rate() == 0.5
    d.insert("t", "x", ttl=0.0)
    time.sleep(0.005)
    assert d.get("t") is None and d.evict_expired() == 0
    d.insert("a", "1"), d.insert("b", "2")
    assert len(d) == 2 and d.get(k1) is None
    rng = np.random.default_rng(0)
    pts = rng.normal(size=(300, 16)).astype(np.float32)
    idx = CA.NswIndex(16)
    for p in pts:
        idx.insert(p)
    hits = 0
    for q in range(0, 300, 10):
        exact = int(np.argmax((pts / np.linalg.norm(pts, axis=1, keepdims=True)) @ (pts[q] / np.linalg.norm(pts[q]))))
        hits += idx.search(pts[q] + 0.01 * rng.normal(size=16), 1)[0].index == exact
    assert hits >= 27 and len(idx) == 300
    with pytest.raises(ValueError):
        idx.insert([1.0, 2.0])
    vocab = {}
    def embed(text):
        v = np.zeros(32)
        for w in text.lower().split():
            v[vocab.setdefault(w, len(vocab)) % 32] += 1
        return v
    sc = CA.SemanticCache(embed, 32, CA.SemanticCacheConfig(similarity_threshold=0.8))
    calls = []
    run = lambda p: calls.append(p) or f"answer to {p}"
    assert sc.run_or_cache("what is the capital of france", run) == ("answer to what is the capital of france", False)
    assert sc.run_or_cache("what is the capital of france please", run)[1] is True and len(calls) == 1
    assert sc.run_or_cache("how do i sort a list in python", run)[1] is False and sc.stats()["hits"] == 1


def test_profiler_memory_logging_request_ids():
    p = OB.Profiler()
    p.begin_trace("step")
    with p.scoped("layer0.qkv", flops=OB.flop_counter.linear(1, 4096, 6144)):
        time.sleep(0.002)
    p.profile("layer0.attn", lambda: time.sleep(0.001))
    t = p.end_trace()
    assert [e.name for e in t.events] == ["layer0.qkv", "layer0.attn"] and t.duration_for_prefix("layer0") >= 3.0
    assert t.events[0].gflops_per_second() > 0 and t.layer_breakdown()["layer0"] >= 3.0 and "trace step" in t.summary()
    assert p.aggregate_stats()["layer0.qkv"]["count"] == 1 and p.last_trace() is t
    off = OB.Profiler(enabled=False)
    with off.scoped("x") as ev:
        assert ev is None
    assert OB.flop_counter.matmul(2, 3, 4) == 48 and OB.flop_counter.decoder_step(CFG_8B, 4096) > 1.4e10
    m = OB.MemoryProfiler()
    blob = bytearray(32 << 20)
    assert m.sample() > 0 and m.peak_rss_bytes() >= m.start_rss_bytes() and m.take_snapshot("x").label == "x" and m.sample_count() == 2
    del blob
    buf = io.StringIO()
    log = OB.init_tracing("debug", json_logs=True, stream=buf)
    log.info("served", extra={"request_id": "abc", "tokens": 5})
    rec = json.loads(buf.getvalue())
    assert rec["message"] == "served" and rec["request_id"] == "abc" and rec["level"] == "info"
    a, b = OB.RequestId.new(), OB.RequestId.new()
    assert a != b and len(a.as_hex()) == 32 and a.as_uuid()[14] == "4" and a.as_uuid()[19] in "89ab"
    assert OB.RequestId.from_hex(a.as_hex()) == a == OB.RequestId.from_uuid(a.as_uuid()) == OB.RequestId.from_bytes(a.as_bytes())
    with pytest.raises(ValueError):
        OB.RequestId.from_hex("xyz")


def test_stream_metrics_quality_autotuner_formatting():
    m = OB.RequestStreamMetrics(prompt_tokens=10)
    t0 = m.t0
    for i in range(5):
        m.record_token(t0 + 0.1 + 0.02 * i)
    m.finish(t0 + 0.2)
    assert m.ttft() == pytest.approx(0.1) and m.median_tbt() == pytest.approx(0.02) and m.tokens_per_second() == pytest.approx(25.0)
    agg = OB.StreamingMetricsAggregator()
    agg.record(m)
    assert agg.report()["requests"] == 1 and agg.avg_ttft_ms() == pytest.approx(100.0) and agg.total_completion_tokens() == 5
    loop = [1, 2, 3] * 10
    rm = OB.RepetitionMetrics.compute(loop)
    assert rm.is_degenerate() and rm.trigram_repetition > 0.8
    good = list(range(30))
    assert not OB.RepetitionMetrics.compute(good).is_degenerate() and OB.DiversityMetrics.compute(good).distinct_1 == 1.0
    assert OB.bleu([1, 2, 3, 4, 5], [[1, 2, 3, 4, 5]]) == pytest.approx(1.0) and OB.bleu([9, 9], [[1, 2, 3]]) == 0.0
    assert OB.perplexity_from_logprobs([np.log(0.5)] * 3) == pytest.approx(2.0)
    ba = OB.BatchQualityAnalyzer()
    ba.add_generation(loop), ba.add_generation(good)
    assert ba.degenerate_fraction() == 0.5 and 0 < ba.mean_quality_score() < 1 and ba.report()["n"] == 2
    b = OB.MemoryBudget.estimate(CFG_8B, "f16")
    assert 2.5e9 < b.weight_bytes < 5e9 and b.kv_bytes_per_token == 36 * 2 * 8 * 128 * 2 and b.max_context_length() > 1_000_000
    rec = OB.AutoTuner(148, 180 * 10 ** 9, 8).recommend(CFG_8B, 4096, 64)
    assert rec.kv_cache == "f16" and rec.tensor_parallel == 1 and rec.attention_splits == 37
    tight = OB.AutoTuner(148, 16 << 30, 8).recommend(CFG_8B, 32768, 8)
    assert tight.kv_cache in ("q8", "q4") or tight.tensor_parallel > 1
    assert OB.format_bytes(1536) == "1.5 KiB" and OB.format_token_count(1500) == "1.5K" and OB.format_duration(0.0025) == "2.5 ms"
    assert OB.format_duration(125) == "2m05s" and OB.format_tokens_per_second(1234.56) == "1,234.6 tok/s"
    assert OB.estimate_memory_requirements(CFG_8B, 4096, 64)["kv_cache"] == 64 * 4096 * 147456


def test_validate_model_file(tmp_path, tiny_gguf):
    assert OB.validate_model_file(tiny_gguf)["valid"] and OB.validate_model_file(tiny_gguf)["version"] == 3
    bad = tmp_path / "x.gguf"
    bad.write_bytes(b"nope" * 10)
    assert not OB.validate_model_file(str(bad))["valid"] and not OB.validate_model_file(str(tmp_path / "missing"))["exists"]


def test_hash_ring_registry_coordinator_and_replica_pool():
    assert D.fnv1a_hash("") == 0xCBF29CE484222325 and D.fnv1a_hash("a") == 0xAF63DC4C8601EC8C
    ring = D.ConsistentHashRing(64)
    for n in ("n0", "n1", "n2", "n3"):
        ring.add_node(n)
    keys = [f"session-{i}" for i in range(2000)]
    before = {k: ring.get_node(k) for k in keys}
    counts = {n: sum(v == n for v in before.values()) for n in ("n0", "n1", "n2", "n3")}
    assert min(counts.values()) > 250 and ring.vnode_count() == 256
    ring.remove_node("n2")
    moved = sum(before[k] != ring.get_node(k) for k in keys)
    assert moved == counts["n2"] and ring.node_count() == 3                 # only the removed node's keys move
    assert len(ring.get_nodes("k", 2)) == 2 and len(set(ring.get_nodes("k", 5))) == 3
    co = D.DistributedCoordinator()
    co.register_self()
    co.add_peer("gpu1", "127.0.0.1:8081")
    owner = co.route("user-42").node_id
    co.set_peer_health(owner, False)
    assert co.route("user-42").node_id != owner and co.healthy_count() == 1 and "down" in co.topology_summary()
    co.set_peer_health(owner, True)
    co.update_peer_load(owner, 0.99)
    assert co.route("user-42").node_id != owner and co.cluster_size() == 2

    class B:
        def __init__(self, fail=False):
            self.n, self.fail = 0, fail

        def submit(self, x):
            if self.fail:
                raise RuntimeError("device lost")
            self.n += 1
            return x * 2
    pool = D.ReplicaPool({"gpu0": B(), "gpu1": B()}, capacity=4)
    nid, out = pool.submit("conv-1", 21)
    assert out == 42 and pool.pick("conv-1") == nid       # a session sticks to its replica
    pool.finished(nid)
    bad = D.ReplicaPool({"gpu0": B(fail=True), "gpu1": B()}, capacity=4)
    key = next(k for k in (f"s{i}" for i in range(100)) if bad.pick(k) == "gpu0")
    with pytest.raises(RuntimeError):
        bad.submit(key, 1)
    assert bad.pick(key) == "gpu1"                         # the failed replica is taken out of rotation


def test_sse_formatter_token_stream_and_middleware_pieces():
    from oxibonsai_b200.runtime import streaming as ST
    f = ST.SseFormatter("rid", "m", created=1, include_usage=True)
    first = f.first_chunk()
    assert first.startswith("data: ") and first.endswith("\n\n") and json.loads(first[6:])["choices"][0]["delta"] == {"role": "assistant"}
    tok = json.loads(f.token_chunk("héllo\nwörld")[6:])
    assert tok["choices"][0]["delta"]["content"] == "héllo\nwörld" and tok["object"] == "chat.completion.chunk"
    fin = json.loads(f.final_chunk("length", {"total_tokens": 3})[6:])
    assert fin["choices"][0]["finish_reason"] == "length" and fin["usage"] == {"total_tokens": 3}
    assert ST.SseFormatter.done_sentinel() == "data: [DONE]\n\n" and f.error_event("boom").startswith("event: error\ndata: ")
    assert ST.SseFormatter.format_event("a\nb") == "data: a\ndata: b\n\n"
    ts = ST.TokenStream()
    assert ts.is_empty() and ts.push_token_bytes(b"\xc3") == "" and ts.push_token_bytes(b"\xa9x") == "éx" and ts.flush() == "" and ts.emitted == "éx"
    st = ST.StreamStats(prompt_tokens=4)
    st.on_token(), st.on_token(), st.finish()
    assert st.to_usage_chunk() == {"prompt_tokens": 4, "completion_tokens": 2, "total_tokens": 6} and st.ttft() >= 0 and st.throughput() > 0
    ctx = ST.RequestContext("r1", "POST", "/v1/completions")
    assert ST.RequestLogger.format_request_line(ctx) == "--> POST /v1/completions [r1]" and "<-- 200 POST" in ST.RequestLogger.format_response_line(ctx, 200)
    g = ST.RequestIdGen("t")
    assert [g.next(), g.next()] == ["t-00000001", "t-00000002"]
    c = ST.CorsConfig(allowed_origins=("https://a.example",))
    assert c.is_origin_allowed("https://a.example") and not c.access_control_headers("https://evil.example")
    assert ST.CorsConfig().access_control_headers("x")["access-control-allow-origin"] == "*"


def test_async_engine_bounds_concurrency_and_streams():
    running, peak = [0], [0]

    def gen(prompt, n):
        running[0] += 1
        peak[0] = max(peak[0], running[0])
        time.sleep(0.02)
        running[0] -= 1
        return [prompt] * n

    def stream(prompt, n):
        for i in range(n):
            yield prompt + i
    eng = D.AsyncInferenceEngine(gen, stream, max_concurrent=2)

    async def main():
        outs = await asyncio.gather(*[eng.generate(i, 2) for i in range(6)])
        toks = [t async for t in eng.generate_streaming(10, 3)]
        return outs, toks
    outs, toks = asyncio.run(main())
    assert outs == [[i, i] for i in range(6)] and toks == [10, 11, 12] and peak[0] <= 2 and eng.active_requests() == 0 and eng.has_capacity()
