"""Model-side library on CPU: RoPE scaling / YaRN / ALiBi, attention variants, MoE, registry, mesh / collectives / sharded
linears / pipeline schedules, quantisation toolbox, model merging, checkpoint containers, converters."""
import json
import math
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

from oxibonsai_b200.core import Qwen3Config


# ---- position encodings -------------------------------------------------------------------------------------------------------
def test_rope_scaling_families():
    from oxibonsai_b200.core.oracle import rope_table
    from oxibonsai_b200.models import rope_scaling as RS
    f = RS.base_frequencies(128, 1e6)
    assert f.shape == (64,) and f[0] == 1.0 and f[-1] == pytest.approx(1e6 ** (-126 / 128), rel=1e-5)
    cos, sin = RS.rope_tables(128, 16, 1e6)
    c0, s0 = rope_table(128, 16, 1e6)
    assert np.allclose(cos.numpy(), c0, atol=1e-6) and np.allclose(sin.numpy(), s0, atol=1e-6)       # unscaled table = the engine's
    assert torch.allclose(RS.compute_rope_frequencies(128, 1e6, RS.RopeScaling("linear", 4.0)), f / 4)
    assert RS.dynamic_ntk_base(1e4, 128, 4096, 4096) == 1e4 and RS.dynamic_ntk_base(1e4, 128, 16384, 4096) > 3e4
    l31 = RS.llama31_frequencies(RS.base_frequencies(128, 5e5), 8.0, 1.0, 4.0, 8192)
    b = RS.base_frequencies(128, 5e5)
    assert torch.equal(l31[:8], b[:8]) and torch.allclose(l31[-1], b[-1] / 8) and (l31 <= b).all()
    y = RS.YarnConfig(128, 1e6, 4.0, 32768)
    keep = y.interpolation_factors()
    assert keep[0] == 1.0 and keep[-1] == 0.0 and (keep[:-1] >= keep[1:]).all()
    sf = y.scaled_frequencies()
    assert sf[0] == f[0] and sf[-1] == pytest.approx(float(f[-1]) / 4) and y.attention_scale() == pytest.approx(0.1 * math.log(4) + 1)
    t = RS.YarnFreqTable(y, 64)
    x = torch.randn(2, 128)
    assert t.apply(x, 0).norm() == pytest.approx(float(x.norm()) * y.attention_scale(), rel=1e-5) and t.effective_context() == 131072
    assert t.apply_batch(torch.randn(3, 4, 128), torch.tensor([1, 2, 3])).shape == (3, 4, 128)
    lr = RS.LongRopeConfig(100, 4.0)
    assert lr.remap_position(50) == 50 and lr.remap_position(140) == 110 and lr.effective_pos(141) == 110
    with pytest.raises(ValueError):
        RS.RopeScaling("bogus").validate()
    assert "wavelength" in RS.FreqStats.compute(f).summary()
    # rotation preserves norms and relative angles
    q = torch.randn(5, 128)
    r = RS.apply_rope(q, cos, sin, torch.arange(5))
    assert torch.allclose(r.norm(dim=-1), q.norm(dim=-1), rtol=1e-5)


def test_alibi():
    from oxibonsai_b200.models import rope_scaling as RS
    s8 = RS.alibi_slopes(8)
    assert torch.allclose(s8, torch.tensor([2.0 ** -(i + 1) for i in range(8)]))
    s12 = RS.alibi_slopes(12)
    assert s12.shape == (12,) and torch.equal(s12[:8], s8) and (s12 > 0).all()
    b = RS.AliBiBias(4).biases_for_sequence(2, 5)
    assert b.shape == (4, 2, 5) and b[0, 1, 4] == 0 and b[0, 1, 0] == -RS.alibi_slopes(4)[0] * 4
    out = RS.attention_with_alibi(torch.randn(4, 3, 16), torch.randn(4, 6, 16), torch.randn(4, 6, 16))
    assert out.shape == (4, 3, 16) and torch.isfinite(out).all()


# ---- attention variants ---------------------------------------------------------------------------------------------------------
def test_attention_variants_agree_with_dense():
    from oxibonsai_b200.models import attention_variants as AV
    g = torch.Generator().manual_seed(0)
    h, t, d = 4, 50, 32
    q1, k, v = torch.randn(h, d, generator=g), torch.randn(h, t, d, generator=g), torch.randn(h, t, d, generator=g)
    dense = AV.masked_attention(q1[:, None], k, v)[:, 0]
    assert torch.allclose(AV.online_softmax_attention(q1, k, v, block=7), dense, atol=1e-5)
    assert torch.allclose(AV.flash_decode(q1, k, v, n_splits=4), dense, atol=1e-5)
    q = torch.randn(8, 10, d, generator=g)
    ref = AV.masked_attention(q, k.repeat_interleave(2, 0), v.repeat_interleave(2, 0), AV.causal_mask(10, t))
    assert torch.allclose(AV.gqa_attention(q, k, v), ref, atol=1e-6)
    cfg = AV.SlidingWindowConfig(8, sinks=2)
    m = AV.sliding_window_mask(t, t, cfg)
    assert m[20].nonzero().flatten().tolist() == [0, 1] + list(range(13, 21)) and AV.attention_range(20, cfg) == (13, 21)
    assert AV.is_in_window(20, 1, cfg) and not AV.is_in_window(20, 5, cfg) and not AV.is_in_window(20, 21, cfg)
    assert AV.evict_outside_window(list(range(30)), 29, cfg) == [0, 1] + list(range(22, 30)) and AV.SlidingWindowConfig().is_disabled()
    full = AV.sliding_window_mask(5, 5, AV.SlidingWindowConfig())
    assert torch.equal(full, AV.causal_mask(5, 5))


def test_sink_cache_sparse_masks_cross_attention_mod():
    from oxibonsai_b200.models import attention_variants as AV
    c = AV.AttentionSinkCache(2, 4, n_heads=1, head_dim=1)
    for i in range(10):
        c.push_step(torch.tensor([[float(i)]]), torch.tensor([[float(i)]]))
    assert c.get_keys().flatten().tolist() == [0, 1, 6, 7, 8, 9] and c.is_streaming() and c.total_evicted() == 4
    assert c.get_remapped_positions().tolist() == list(range(6)) and c.cache_len() == 6 and c.memory_bytes() == 2 * 6 * 4
    loc = AV.SparseAttentionMask.build(AV.SparsePattern.LOCAL, 32, window=4)
    assert loc.keys_for_query(10) == [7, 8, 9, 10] and not loc.can_attend(10, 11) and 0 < loc.density() < 0.3
    st = AV.SparseAttentionMask.build(AV.SparsePattern.STRIDED, 32, window=2, stride=8)
    assert st.keys_for_query(17) == [1, 9, 16, 17]
    bb = AV.SparseAttentionMask.build(AV.SparsePattern.BIGBIRD, 32, window=2, n_global=2, n_random=1)
    assert bb.can_attend(20, 0) and bb.can_attend(20, 1) and bb.nnz() <= 32 * 33 // 2 and AV.memory_reduction(bb) > 0.5
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(2, 32, 8, generator=g) for _ in range(3))
    wide = AV.SparseAttentionMask.build(AV.SparsePattern.LOCAL, 32, window=32)
    assert AV.sparse_vs_dense_error(q, k, v, wide) < 1e-6 and AV.sparse_vs_dense_error(q, k, v, loc) > 1e-3
    ca = AV.CrossAttention(16, 4, memory_dim=8)
    y = ca(torch.randn(3, 16), torch.randn(5, 8), torch.tensor([True, True, True, False, False]))
    assert y.shape == (3, 16)
    mod = AV.MixtureOfDepthsRouter(16, 0.5)
    x = torch.randn(8, 16)
    out = mod(x, lambda z: z * 2)
    idx, _ = mod.route(x)
    untouched = [i for i in range(8) if i not in idx.tolist()]
    assert len(idx) == 4 and torch.equal(out[untouched], x[untouched]) and not torch.equal(out[idx], x[idx])
    ac = AV.AttentionConfig.alternating(4, window=8)
    assert [l.kind for l in ac.layers] == ["sliding_window", "full", "sliding_window", "full"]
    assert ac.kv_tokens_needed(0, 100) == 8 and ac.kv_tokens_needed(1, 100) == 100 and ac.mask_for_layer(0, 4, 20).shape == (4, 20)


def test_moe_routing_and_layer():
    from oxibonsai_b200.models import moe as M
    torch.manual_seed(0)
    cfg = M.moe_tiny_config()
    layer = M.MoeFfnLayer(cfg)
    x = torch.randn(64, cfg.hidden)
    y = layer(x)
    d = layer.last_decision
    assert y.shape == x.shape and d.num_tokens() == 64 and torch.allclose(d.weights.sum(-1), torch.ones(64), atol=1e-6)
    # dense reference of the same computation for the tokens that were not dropped
    ref = torch.zeros_like(x)
    for t in range(64):
        for s in range(cfg.top_k):
            if not d.dropped[t, s]:
                ref[t] += d.weights[t, s] * layer.experts[int(d.expert_ids[t, s])](x[t])
    assert torch.allclose(y, ref, atol=1e-5)
    assert d.max_expert_load(4) <= layer.router.capacity(64) and 0 <= d.overflow_rate() < 0.5 and 0 < d.load_balance_score(4) <= 1
    assert layer.router.aux_loss(d) > 0 and layer.router.z_loss(d) > 0
    assert layer.active_param_count() < layer.total_param_count() and 0 < layer.sparsity() < 1
    buf = M.ExpertBuffer(2, 2)
    assert [buf.try_assign(0, t) for t in range(3)] == [True, True, False] and buf.overflow_count() == 1 and buf.expert_utilization() == [1.0, 0.0]
    out = M.combine_expert_outputs(torch.ones(3, 2, 4), torch.tensor([[0.25, 0.75]] * 3))
    assert torch.allclose(out, torch.ones(3, 4)) and M.moe_8x7b_config().n_experts == 8


# ---- registry ---------------------------------------------------------------------------------------------------------------------
def test_registry_variants_specs_and_builder(tiny_gguf):
    from oxibonsai_b200.core import GgufFile, gguf as G
    from oxibonsai_b200.models import registry as R
    c8 = Qwen3Config(hidden=4096, inter=12288, layers=36, heads=32, kv_heads=8, head_dim=128)
    assert R.variant_from_config(c8) == R.ModelVariant.BONSAI_8B and R.variant_from_config(c8, G.TQ2_0_G128) == R.ModelVariant.TERNARY_8B
    assert R.variant_from_config(c8, G.F8_E4M3) == R.ModelVariant.FP8_8B
    assert R.variant_from_config(Qwen3Config(hidden=1536, layers=16)) == R.ModelVariant.BONSAI_1_7B
    assert R.variant_from_config(Qwen3Config(hidden=512, layers=3)) == R.ModelVariant.CUSTOM
    spec = R.spec_for_variant(R.ModelVariant.TERNARY_8B)
    assert 8.0e9 < spec.param_count < 8.4e9 and 4.2e9 < spec.weights_size_bytes < 4.5e9 and spec.kv_cache_4k_bytes == 4096 * 147456
    assert len(R.all_specs()) == 9 and R.ModelVariant.CUSTOM not in R.known_variants()
    assert R.bits_per_weight(G.TQ2_0_G128) == 2.125 and R.bits_per_weight(G.Q1_0_G128) == 1.125
    assert "draft" in " ".join(R.capability_profile(R.ModelVariant.TERNARY_1_7B).use_cases)
    cfg = R.ModelConfigBuilder().layers(4).hidden_size(512).num_attention_heads(8).num_kv_heads(2).intermediate_size(1024).build()
    assert cfg.head_dim == 64 and cfg.layers == 4
    with pytest.raises(R.ConfigError):
        R.ModelConfigBuilder().num_attention_heads(6).num_kv_heads(4).build()
    with pytest.raises(R.ConfigError):
        R.ModelConfigBuilder().hidden_size(1000).build()
    assert R.ModelConfigBuilder().build_tiny().hidden == 256
    f = GgufFile.open(tiny_gguf)
    v = R.validate_gguf(f)
    assert v.ok and v.dominant_type == G.TQ2_0_G128 and v.variant == R.ModelVariant.CUSTOM
    assert sum(len(c) for c in R.iter_tensor_chunks(f, "token_embd.weight", 1000)) == len(f.tensor_bytes("token_embd.weight"))
    assert R.memory_budget_check(f, 1 << 30)["fits"] and not R.memory_budget_check(f, 1000)["fits"]


# ---- mesh / collectives / pipeline ---------------------------------------------------------------------------------------------------
def test_mesh_simulated_collectives_sharded_linear_and_pipeline_schedule():
    from oxibonsai_b200.parallel import collectives as PC
    mesh = PC.DeviceMesh(4, 2)
    assert mesh.size() == 8 and mesh.tp_group(1) == [4, 5, 6, 7] and mesh.pp_group(2) == [2, 6] and mesh.get(3, 1).rank == 7
    co = PC.Collectives()
    xs = [torch.full((4,), float(r)) for r in range(4)]
    assert all(torch.equal(t, torch.full((4,), 6.0)) for t in co.all_reduce_sum(xs))
    assert torch.equal(co.all_reduce_max(xs)[2], torch.full((4,), 3.0))
    assert co.all_gather(xs)[0].shape == (16,) and torch.equal(co.reduce_scatter(xs)[1], torch.tensor([6.0]))
    assert torch.equal(co.broadcast(xs, src=3)[0], xs[3]) and co.bytes_moved > 0
    g = torch.Generator().manual_seed(0)
    w, b, x = torch.randn(12, 8, generator=g), torch.randn(12, generator=g), torch.randn(3, 8, generator=g)
    ref = x @ w.T + b
    for kind in ("column", "row"):
        shards = PC.ShardedLinear.shard(w, b, kind, 4)
        assert torch.allclose(PC.tensor_parallel_forward(shards, x), ref, atol=1e-5), kind
    assert torch.equal(PC.merge_column_shards(PC.partition_weights_column(w, 3)), w)
    assert torch.equal(PC.merge_row_shards(PC.partition_weights_row(w, 2)), w)
    with pytest.raises(ValueError):
        PC.partition_weights_column(w, 5)
    plan = PC.ShardingPlan.standard_transformer_plan()
    assert plan.kind_for("blk.3.attn_q.weight") == "column" and plan.kind_for("blk.3.ffn_down.weight") == "row"
    assert plan.kind_for("blk.0.attn_norm.weight") == "replicated" and plan.collectives_per_layer() == {"all_reduce": 2}
    stages = PC.partition_layers(36, 8)
    assert [s.layer_count() for s in stages] == [5, 5, 5, 5, 4, 4, 4, 4] and stages[1].contains_layer(7) and list(stages[0].layer_range()) == [0, 1, 2, 3, 4]
    sch = PC.PipelineSchedule.gpipe_schedule(4, 8)
    assert sch.total_steps() == 11 and sch.bubble_fraction() == pytest.approx(3 / 11) and sch.steps[0] == [(0, 0)] and (3, 7) in sch.steps[-1]
    mem = PC.pipeline_memory_per_stage(stages, 100, 1000, 10, 8)
    assert mem[0] == 5 * 100 + 80 + 1000 and mem[-1] == 4 * 100 + 10 + 1000
    assert PC.MicroBatch(0, 128).is_first_stage()


def test_collectives_over_gloo_process_group(tmp_path):
    script = tmp_path / "w.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys, json, torch, torch.distributed as dist
        sys.path.insert(0, {os.path.dirname(os.path.dirname(os.path.abspath(__file__)))!r})
        from oxibonsai_b200.parallel.collectives import Collectives
        dist.init_process_group("gloo")
        r, w = dist.get_rank(), dist.get_world_size()
        co = Collectives(dist.group.WORLD)
        a = co.all_reduce_sum(torch.full((4,), float(r + 1)))
        g = co.all_gather(torch.tensor([float(r)]))
        rs = co.reduce_scatter(torch.arange(4.0) + r)
        b = co.broadcast(torch.tensor([float(r)]), src=1)
        json.dump(dict(a=a.tolist(), g=g.tolist(), rs=rs.tolist(), b=b.tolist()), open(os.path.join({str(tmp_path)!r}, f"r{{r}}.json"), "w"))
        dist.destroy_process_group()
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29611", str(script)], capture_output=True, text=True, timeout=300, env=env)
    assert p.returncode == 0, p.stderr[-2000:]
    r0, r1 = (json.load(open(tmp_path / f"r{i}.json")) for i in range(2))
    assert r0["a"] == r1["a"] == [3.0] * 4 and r0["g"] == [0.0, 1.0] and r0["b"] == r1["b"] == [1.0]
    assert r0["rs"] == [1.0, 3.0] and r1["rs"] == [5.0, 7.0]


# ---- quantisation toolbox, merging, checkpoints, conversion -------------------------------------------------------------------------------
def test_quant_toolbox():
    from oxibonsai_b200 import quant as Q
    from oxibonsai_b200.core import gguf as G
    rng = np.random.default_rng(0)
    w = rng.normal(size=(64, 256)).astype(np.float32) * 0.05
    e_t, e_q = Q.quantization_error(G.TQ2_0_G128, w), Q.quantization_error(G.Q1_0_G128, w)
    assert e_t["bits_per_weight"] == 2.125 and 0 < e_t["rel_rmse"] < 1.0 and e_q["bits_per_weight"] == 1.125
    assert Q.quantize_q1(w).size == w.size // 128 * 18 and Q.quantize_ternary(w).size == w.size // 128 * 34
    t = Q.quantize_int8(w)
    pc = Q.quantize_int8(w, per_channel=True)
    asym = Q.quantize_int8(w + 0.1, symmetric=False)
    assert np.abs(t.dequantize() - w).max() <= float(t.scale) and pc.scale.shape == (64,) and np.abs(asym.dequantize() - (w + 0.1)).max() < 2e-3
    assert np.abs(pc.dequantize() - w).mean() <= np.abs(t.dequantize() - w).mean() + 1e-9
    x = rng.normal(size=256).astype(np.float32)
    assert np.allclose(Q.int8_matvec(pc, x), w @ x, atol=0.05)
    lin = Q.DynamicQuantLinear(w, bias=np.ones(64, dtype=np.float32))
    assert np.allclose(lin(np.stack([x, 2 * x])), np.stack([w @ x, 2 * (w @ x)]) + 1, atol=0.1)
    db = Q.CalibrationDb()
    acts = rng.normal(size=(100, 256)).astype(np.float32)
    acts[:, 3] *= 50
    db.observe("l0", acts[:50]), db.observe("l0", acts[50:])
    st = db.layers["l0"]
    assert st.count == acts.size and st.std == pytest.approx(float(acts.std()), rel=1e-3) and int(np.argmax(st.absmax)) == 3
    ws, s = Q.apply_smoothquant(w, st.absmax, 0.5)
    assert np.allclose((acts / s) @ ws.T, acts @ w.T, rtol=1e-3, atol=1e-3) and (acts / s)[:, 3].std() < acts[:, 3].std()
    assert db.scale_for("l0") > 0 and "l0" in db.summary()
    p = Q.magnitude_prune(w, 0.75)
    assert Q.sparsity(p) == pytest.approx(0.75, abs=1e-3) and np.abs(p[p != 0]).min() >= np.abs(w[p == 0]).max()
    kept, rows = Q.structured_prune_rows(w, 0.25)
    assert kept.shape == (48, 256) and len(rows) == 48
    nm = Q.n_m_prune(w, 2, 4)
    assert ((nm.reshape(-1, 4) != 0).sum(1) == 2).all()
    out, rep = Q.compress_tensors({"blk.0.attn_q.weight": w, "blk.0.attn_norm.weight": np.ones(256, dtype=np.float32)}, prune_sparsity=0.5)
    assert out["blk.0.attn_q.weight"][0] == G.TQ2_0_G128 and out["blk.0.attn_norm.weight"][0] == G.F32 and rep.ratio > 8


def test_model_merging():
    from oxibonsai_b200.quant import merge as MG
    rng = np.random.default_rng(1)
    base = {"w": rng.normal(size=(4, 8)).astype(np.float32)}
    a = {"w": base["w"] + 1.0}
    b = {"w": base["w"] - 1.0}
    assert np.allclose(MG.linear_merge([a, b])["w"], base["w"]) and np.allclose(MG.linear_merge([a, b], [3, 1])["w"], base["w"] + 0.5)
    u, v = np.array([1.0, 0.0]), np.array([0.0, 1.0])
    assert np.allclose(MG.slerp(u, v, 0.5), [math.sqrt(0.5)] * 2) and np.allclose(MG.slerp(u, u, 0.3), u)
    tv = MG.task_vector(a, base)
    assert np.allclose(tv["w"], 1.0) and np.allclose(MG.apply_task_vectors(base, [tv, tv], 0.5)["w"], a["w"])
    t = MG.ties_merge(base, [a, a, b], density=1.0)
    assert np.allclose(t["w"], base["w"] + 1.0)                      # the majority sign wins, dissenters are dropped
    d = MG.dare_merge(base, [a], drop_rate=0.5, seed=0)["w"] - base["w"]
    assert set(np.unique(d.round(6))) <= {0.0, 2.0} and 0.2 < (d != 0).mean() < 0.8
    with pytest.raises(ValueError):
        MG.linear_merge([a, {"x": a["w"]}])


def test_checkpoint_containers_and_weight_tying(tmp_path):
    from oxibonsai_b200.models import checkpoint as CK
    ck = CK.Checkpoint({"step": "12", "loss": "0.5"})
    ck.add("layer.0.weight", np.arange(6, dtype=np.float32).reshape(2, 3)).add("bias", np.zeros(3))
    p = str(tmp_path / "m.oxck")
    ck.save(p)
    raw = open(p, "rb").read()
    assert raw[:4] == b"OXCK" and raw[4:8] == (1).to_bytes(4, "little")
    back = CK.Checkpoint.load(p)
    assert back.metadata == ck.metadata and np.array_equal(back.tensors["layer.0.weight"], ck.tensors["layer.0.weight"]) and list(back.tensors) == ["layer.0.weight", "bias"]
    with pytest.raises(CK.CheckpointError):
        ck.add("bias", np.zeros(1))
    open(p, "wb").write(raw[:40])
    with pytest.raises(CK.CheckpointError):
        CK.Checkpoint.load(p)
    dc = CK.DiskCache({"source": "model.gguf"})
    dc.put("blk.0.attn_q.weight", "TQ2_0_g128", b"\x55" * 34)
    cp, src = str(tmp_path / "m.oxcache"), str(tmp_path / "src")
    open(src, "w").write("x")
    dc.save(cp)
    got = CK.DiskCache.load(cp)
    assert got.get("blk.0.attn_q.weight").quant_type == "TQ2_0_g128" and got.metadata["source"] == "model.gguf"
    assert CK.DiskCache.is_valid(cp) and CK.DiskCache.is_fresh(cp, src) and not CK.DiskCache.is_valid(src)
    os.utime(src, (os.path.getmtime(cp) + 10,) * 2)
    assert not CK.DiskCache.is_fresh(cp, src)
    k1 = CK.repack_cache_key(src, 0, 2)
    assert k1 != CK.repack_cache_key(src, 1, 2) and len(k1) == 32
    t = CK.tie_weights({"token_embd.weight": np.ones((4, 2))})
    assert CK.is_tied(t) and not CK.is_tied({**CK.untie_weights(t), "output.weight": np.zeros((4, 2))})


def test_safetensors_to_gguf_conversion_roundtrip(tmp_path):
    from oxibonsai_b200 import convert as CV
    from oxibonsai_b200.core import GgufFile, dequantize, gguf as G
    rng = np.random.default_rng(0)
    h, inter, v, hd = 256, 512, 300, 64
    t = {"model.embed_tokens.weight": rng.normal(size=(v, h)).astype(np.float32) * 0.02, "model.norm.weight": np.ones(h, dtype=np.float32)}
    for l in range(2):
        p = f"model.layers.{l}."
        t.update({p + "input_layernorm.weight": np.ones(h, np.float32), p + "post_attention_layernorm.weight": np.ones(h, np.float32),
                  p + "self_attn.q_proj.weight": rng.normal(size=(4 * hd, h)).astype(np.float16), p + "self_attn.k_proj.weight": rng.normal(size=(2 * hd, h)).astype(np.float32),
                  p + "self_attn.v_proj.weight": rng.normal(size=(2 * hd, h)).astype(np.float32), p + "self_attn.o_proj.weight": rng.normal(size=(h, 4 * hd)).astype(np.float32),
                  p + "self_attn.q_norm.weight": np.ones(hd, np.float32), p + "self_attn.k_norm.weight": np.ones(hd, np.float32),
                  p + "mlp.gate_proj.weight": rng.normal(size=(inter, h)).astype(np.float32), p + "mlp.up_proj.weight": rng.normal(size=(inter, h)).astype(np.float32),
                  p + "mlp.down_proj.weight": rng.normal(size=(h, inter)).astype(np.float32), p + "self_attn.rotary_emb.inv_freq": np.ones(4, np.float32)})
    d = tmp_path / "hf"
    d.mkdir()
    CV.write_safetensors(str(d / "model.safetensors"), t)
    (d / "config.json").write_text(json.dumps({"hidden_size": h, "intermediate_size": inter, "num_attention_heads": 4, "num_key_value_heads": 2,
                                               "head_dim": hd, "vocab_size": v, "rms_norm_eps": 1e-6, "rope_theta": 1e6}))
    names = [s.name for s in CV.read_safetensors(str(d / "model.safetensors"))]
    assert names[0] == "model.embed_tokens.weight" and CV.hf_to_gguf_name("model.layers.7.mlp.up_proj.weight") == ("blk.7.ffn_up.weight", False)
    assert CV.hf_to_gguf_name("model.layers.0.self_attn.rotary_emb.inv_freq") is None
    out = str(tmp_path / "m.gguf")
    st = CV.convert_safetensors_to_gguf(str(d), out, quantize_embeddings=False, key_prefix="qwen3")
    assert st.tied and st.skipped == 2 and st.tensors == 2 + 2 * 11 + 1
    f = GgufFile.open(out)
    cfg = f.config()
    assert (cfg.hidden, cfg.inter, cfg.layers, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.vocab) == (h, inter, 2, 4, 2, hd, v)
    q = f.tensor_info("blk.1.attn_q.weight")
    assert q.type == G.TQ2_0_G128 and tuple(q.dims) == (h, 4 * hd) and f.tensor_info("token_embd.weight").type == G.F16
    w = t["model.layers.1.self_attn.k_proj.weight"]
    deq = dequantize(G.TQ2_0_G128, f.tensor_bytes("blk.1.attn_k.weight")).reshape(w.shape)
    assert np.corrcoef(deq.reshape(-1), w.reshape(-1))[0, 1] > 0.7   # absmax-scaled ternary codes of Gaussian weights
    st2 = CV.convert_safetensors_to_gguf(str(d), str(tmp_path / "ref.gguf"))       # reference behaviour: llm.* keys, quantised embeddings
    g = GgufFile.open(str(tmp_path / "ref.gguf"))
    assert g.metadata["llm.block_count"] == 2 and g.tensor_info("output.weight").type == G.TQ2_0_G128 and g.config().hidden == h
    with pytest.raises(ValueError):
        CV.convert_safetensors_to_gguf(str(d), out, quant="q9")
    # a tokenizer.json beside the checkpoint travels into the GGUF metadata: the converted file is self-contained
    assert st.tokenizer_tokens == 0 and "tokenizer.ggml.tokens" not in f.metadata
    from oxibonsai_b200 import tokenizer as T
    from oxibonsai_b200.tokenizer.extras import save_bpe_text                                   # noqa: F401 - (the text format is not the HF one)
    tok = T.train_bpe(["the quick brown fox " * 10, "héllo wörld " * 10], 290, special_tokens=["<|endoftext|>", "<|im_end|>"])
    hf = {"model": {"type": "BPE", "vocab": tok.vocab, "merges": [f"{tok.id_to_token[a]} {tok.id_to_token[b]}" for a, b, _ in tok.merges]},
          "added_tokens": [{"id": i, "content": c, "special": True} for c, i in tok.special.items()],
          "pre_tokenizer": {"type": "ByteLevel"}, "decoder": {"type": "ByteLevel"}}
    (d / "tokenizer.json").write_text(json.dumps(hf))
    st3 = CV.convert_safetensors_to_gguf(str(d), str(tmp_path / "with_tok.gguf"), key_prefix="qwen3")
    assert st3.tokenizer_tokens == tok.vocab_size
    emb = T.BpeTokenizer.from_gguf(str(tmp_path / "with_tok.gguf"))
    text = "the quick héllo<|im_end|>"
    assert emb.encode(text) == tok.encode(text) and emb.decode(emb.encode(text)) == text and emb.eos_token_id == tok.special["<|im_end|>"]
    assert CV.convert_safetensors_to_gguf(str(d), str(tmp_path / "no_tok.gguf"), embed_tokenizer=False).tokenizer_tokens == 0


def test_host_kv_caches_and_layer_stats(tiny_gguf):
    from oxibonsai_b200.core import GgufFile, Oracle
    from oxibonsai_b200.models import kv_cache as KV
    rng = np.random.default_rng(0)
    L, H, T, D = 2, 2, 8, 16
    k, v = rng.normal(size=(H, D)).astype(np.float32), rng.normal(size=(H, D)).astype(np.float32)
    for cls, tol in ((KV.KvCache, 0.0), (KV.KvCacheFp16, 2e-3), (KV.QuantizedKvCache, 0.02), (lambda *a: KV.Fp8KvCache(*a), 0.08),
                     (lambda *a: KV.Fp8KvCache(*a, e5m2=True), 0.15)):
        c = cls(L, H, T, D)
        c.store(1, 3, k, v)
        assert c.len == 4 and np.abs(c.keys(1, 0)[3] - k[0]).max() <= tol * np.abs(k[0]).max() + 1e-7
        assert np.abs(c.values(1, 1, 4)[3] - v[1]).max() <= tol * np.abs(v[1]).max() + 1e-7 and c.nbytes > 0
    d = KV.KvCache(L, H, T, D)
    assert d.is_all_zero()
    d.store(0, 0, k, v), d.store(0, 1, v, k)
    kb, vb = d.extract_block(0, 2)
    e = KV.KvCache(L, H, T, D)
    e.inject_block(4, kb, vb)
    assert e.len == 6 and np.array_equal(e.keys(0, 1)[5], v[1]) and not e.is_all_zero()
    with pytest.raises(IndexError):
        d.store(0, T, k, v)
    q, s = KV.quantize_row_int8(k[0])
    assert s == pytest.approx(np.abs(k[0]).max() / 127) and q.dtype == np.int8 and np.abs(q).max() == 127
    p4, s4 = KV.quantize_row_int4(k[0])
    assert p4.size == D // 2 and np.abs(KV.dequantize_row_int4(p4, s4) - k[0]).max() <= s4 / 2 + 1e-6
    assert KV.QuantizedKvCache(L, H, T, D).compression_ratio() > 3
    stats = KV.forward_with_stats(Oracle(GgufFile.open(tiny_gguf), 16), [1, 2, 3])
    assert len(stats) == 2 and all(s.std > 0 and not s.has_nan for s in stats) and "layer   1" in stats[1].summary()


def test_repacked_weight_cache_file_roundtrip(tmp_path):
    import torch
    from oxibonsai_b200.models import checkpoint as CK
    t = {"a.codes": torch.arange(24, dtype=torch.int32).reshape(2, 12), "a.scales": torch.linspace(0, 1, 6).to(torch.float16).reshape(2, 3),
         "bytes": torch.arange(5000, dtype=torch.int64).to(torch.uint8), "empty": torch.zeros((0, 4), dtype=torch.float32),
         "norm": torch.randn(7)}
    path = str(tmp_path / "w.oxrp")
    CK.save_repacked(path, t, {"layers": 3})
    got, meta = CK.load_repacked(path)
    assert meta == {"layers": 3} and set(got) == set(t)
    for k in t:
        assert got[k].dtype == t[k].dtype and got[k].shape == t[k].shape and torch.equal(got[k], t[k])
    # damaged files are refused, not half-read
    with open(path, "r+b") as f:
        f.write(b"XXXX")
    with pytest.raises(CK.CheckpointError):
        CK.load_repacked(path)


def test_nvtx_ranges_are_off_by_default_and_nest():
    from oxibonsai_b200.ops import nvtx
    assert not nvtx.enabled() and nvtx.push("x") is False
    nvtx.pop(False)
    with nvtx.range("nothing happens on CPU when off"):
        pass


def test_package_facade_resolves_lazily():
    """``import oxibonsai_b200`` imports nothing heavy; every advertised name resolves to the object of its home module."""
    import subprocess
    import sys
    code = ("import sys, oxibonsai_b200 as ob\n"
            "assert 'torch' not in sys.modules and 'numpy' not in sys.modules\n"
            "missing = [n for n in ob.__all__ if not hasattr(ob, n)]\n"
            "assert not missing, missing\n"
            "from oxibonsai_b200.runtime.presets import SamplingParams\n"
            "assert ob.SamplingParams is SamplingParams and 'EngineBuilder' in dir(ob)\n"
            "try:\n    ob.nothing_here\nexcept AttributeError as e:\n    assert 'nothing_here' in str(e)\nelse:\n    raise SystemExit(1)\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0, r.stderr[-2000:]
