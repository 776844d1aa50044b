"""Quantisation toolbox: calibration rules, dynamic quantisation, INT8 error analysis, pruning, compression pipelines, merge
statistics, SmoothQuant, export planning."""
import math

import numpy as np
import pytest

from oxibonsai_b200.core import GgufFile, dequantize, gguf as G
from oxibonsai_b200.quant import toolbox as Q


def test_calibration_rules_and_database():
    rng = np.random.default_rng(0)
    s = Q.LayerCalibStats("l0")
    assert s.compute_scale() == 0.0 and s.percentile_abs(0.5) == 0.0
    data = rng.laplace(scale=1.0, size=20000).astype(np.float32)
    for part in np.array_split(data, 7):                 # streamed in pieces: same statistics as in one go
        s.update(part)
    assert s.num_samples == 20000 and s.mean() == pytest.approx(float(data.mean()), abs=1e-4) and s.std_dev() == pytest.approx(float(data.std()), rel=1e-4)
    amax = float(np.abs(data).max())
    assert s.abs_max() == pytest.approx(amax) and s.compute_scale(Q.CalibMethod.MINMAX) == pytest.approx(amax / 127)
    p99 = s.percentile_abs(0.99)
    assert abs(p99 - float(np.quantile(np.abs(data), 0.99))) < 2 * amax / 256            # histogram resolution
    assert s.compute_scale(Q.CalibMethod.PERCENTILE, 0.99) == pytest.approx(p99 / 127)
    assert s.aciq_clip() == pytest.approx(2.83 * s.std_dev()) and s.compute_scale(Q.CalibMethod.ACIQ) == pytest.approx(min(s.aciq_clip(), amax) / 127)
    mse = s.clipping_value(Q.CalibMethod.MSE)
    assert 0.3 * amax <= mse <= amax and s.compute_scale_int4(Q.CalibMethod.MSE) < s.compute_scale_int4(Q.CalibMethod.MINMAX)   # INT4 wants a tighter clip than the tail
    # clipping at the MSE choice beats clipping at the maximum for a heavy-tailed tensor at 4 bits
    def err(clip, levels):
        q = np.clip(np.rint(data / (clip / levels)), -levels, levels) * (clip / levels)
        return float(((data - q) ** 2).mean())
    assert err(s.clipping_value(Q.CalibMethod.MSE, clip_val=7.0), 7) < err(amax, 7)
    assert "l0: n=20000" in s.summary().summary_line()
    db = Q.CalibrationDatabase.new_percentile(0.999)
    db.record("a", data[:100])
    db.record("a", data[100:5000])
    db.record("z", np.zeros(10))
    assert db.num_layers() == 2 and db.get_stats("a").num_samples == 5000 and db.scale_for_layer("missing") is None
    assert set(db.export_scales()) == {"a", "z"} and db.export_scales()["z"] == 0.0 and "method percentile" in db.report()
    v = db.validate(min_samples=50)
    assert not v.ok and any("z" in i for i in v.issues) and len(v.issues) == 1
    sim = Q.simulate_calibration(["x", "y", "w"], seed=1)
    assert sim.validate().ok and sim.scale_for_layer("w") > sim.scale_for_layer("x") and Q.CalibrationDatabase.new_minmax().validate().issues == ["no layers recorded"]


def test_dynamic_quantisation_and_w8a8():
    rng = np.random.default_rng(1)
    w = rng.normal(size=(64, 96)).astype(np.float32)
    w[3] *= 20                                            # one loud row: per-row scales pay off
    pt, pr, i4 = Q.dynamic_quantize_int8(w), Q.dynamic_quantize_int8_per_row(w), Q.dynamic_quantize_int4(w)
    assert pt.format is Q.DynQuantFormat.INT8_PER_TENSOR and pr.scales.shape == (64,) and np.abs(i4.data).max() <= 7
    assert Q.quantization_mae(w, pr) < Q.quantization_mae(w, pt) < Q.quantization_mae(w, i4)
    assert pt.element_count() == 64 * 96 and pt.memory_bytes() == 64 * 96 + 4 and pr.memory_bytes() == 64 * 96 + 4 * 64 and i4.memory_bytes() == 64 * 96 // 2 + 4
    assert pt.compression_ratio() == pytest.approx(4 * 6144 / 6148) and i4.compression_ratio() > 7.9
    assert np.abs(pt.dequantize() - w).max() <= pt.scales[0] / 2 + 1e-6
    robust = Q.dynamic_quantize_int8(w, Q.DynamicScaleMode.PERCENTILE, 0.99)
    assert robust.scales[0] < pt.scales[0]
    x = rng.normal(size=96).astype(np.float32)
    y = Q.w8a8_matvec(pr, x)
    assert np.abs(y - w @ x).max() < 0.02 * np.abs(w @ x).max() + 0.05
    with pytest.raises(Q.DynQuantError):
        Q.w8a8_matvec(i4, x)
    with pytest.raises(Q.DynQuantError):
        Q.w8a8_matvec(pr, x[:10])
    with pytest.raises(Q.DynQuantError):
        Q.dynamic_quantize_int8_per_row(x)
    with pytest.raises(Q.DynQuantError):
        Q.compute_scale([], 127)
    assert Q.compute_scale(np.zeros(4), 127) == 1.0
    e_pt, e_pc = Q.analyze_int8_error(w, Q.Int8Mode.PER_TENSOR), Q.analyze_int8_error(w, Q.Int8Mode.PER_CHANNEL)
    assert e_pc.mse < e_pt.mse and e_pc.snr_db > e_pt.snr_db > 20 and e_pt.max_error <= pt.scales[0] / 2 + 1e-6 and 0 < e_pc.relative_error < 0.05
    cmp = Q.compare_quantization_methods(w)
    assert cmp.best == "per_channel" and cmp.int4 > cmp.per_tensor.mae


def test_pruning_metrics_granularity_and_reports():
    w = np.array([[0.1, -2.0, 0.3, 4.0], [0.05, 0.06, -0.07, 0.08], [1.0, 1.0, -1.0, 1.0]], dtype=np.float32)
    p = Q.prune_tensor(w, Q.PruningConfig.unstructured_l1(0.5))
    assert (p == 0).sum() == 6 and p[0, 3] == 4.0 and np.all(p[1] == 0) and w[1, 0] == np.float32(0.05)      # a copy: the input is untouched
    rows = Q.prune_tensor(w, Q.PruningConfig.structured_row_l2(0.34))
    assert np.all(rows[1] == 0) and np.all(rows[0] == w[0]) and np.all(rows[2] == w[2])
    cols = Q.prune_tensor(w, Q.PruningConfig(0.5, Q.ImportanceMetric.L1_MAGNITUDE, Q.PruningGranularity.STRUCTURED_COLUMN))
    assert np.all(cols[:, 0] == 0) and np.all(cols[:, 2] == 0) and np.all(cols[:, 3] == w[:, 3])
    r1 = Q.prune_tensor(w, Q.PruningConfig(0.5, Q.ImportanceMetric.RANDOM, seed=3))
    assert np.array_equal(r1, Q.prune_tensor(w, Q.PruningConfig(0.5, Q.ImportanceMetric.RANDOM, seed=3))) and (r1 == 0).sum() == 6
    assert np.array_equal(Q.compute_importance(w, Q.ImportanceMetric.TAYLOR_PROXY), w * w)
    with pytest.raises(Q.PruningError):
        Q.PruningConfig(1.0)
    with pytest.raises(Q.PruningError):
        Q.prune_tensor(np.ones(4), Q.PruningConfig.structured_row_l2(0.5))
    rep = Q.SparsityReport.compute("w", p)
    assert rep.zero_fraction() == 0.5 and rep.density() == 0.5 and "6/12 zero (50.0 %)" in rep.summary()
    model = {"blk.0.ffn_up.weight": np.random.default_rng(0).normal(size=(8, 16)).astype(np.float32), "blk.0.attn_norm.weight": np.ones(16, np.float32),
             "token_embd.weight": np.ones((4, 16), np.float32)}
    pruned = Q.prune_model(model, Q.PruningConfig.unstructured_l1(0.75))
    summ = Q.ModelSparsitySummary.from_model(pruned)
    assert (pruned["blk.0.ffn_up.weight"] == 0).sum() == 96 and np.all(pruned["token_embd.weight"] == 1) and np.all(pruned["blk.0.attn_norm.weight"] == 1)
    assert summ.overall() == pytest.approx(96 / (128 + 16 + 64)) and "model sparsity" in summ.summary()


def test_compression_pipeline_and_merge_stats():
    rng = np.random.default_rng(2)
    model = {"a.weight": rng.normal(size=(32, 64)).astype(np.float32), "b.weight": rng.normal(size=(16, 64)).astype(np.float32), "a.norm": np.ones(64, np.float32)}
    res = Q.compress_model(model, Q.CompressionConfig.prune_then_quantize(0.5))
    assert [s.stage for s in res.stages] == ["prune", "quantize_int8"] and res.total_params() == 32 * 64 + 16 * 64 + 64
    assert res.stages[0].sparsity() == pytest.approx(1536 / 3136) and res.stages[0].compression_ratio() == 1.0 and res.stages[1].compression_ratio() == 4.0
    assert res.memory_before_bytes() == 4 * 3136 and res.memory_after_bytes() == 3136 and res.total_compression_ratio() == 4.0
    assert res.overall_sparsity() >= 0.48 and "4.00x" in res.summary()
    # INT8 rounding was simulated: values sit on the grid of the tensor's scale
    q = res.tensors["a.weight"]
    nz = q[q != 0]
    step = np.abs(nz).min()
    assert np.abs(model["a.weight"] - q)[q != 0].max() < 0.02 and step > 0
    clip = Q.compress_model(model, Q.CompressionConfig().add_stage(Q.CompressionStage.clip(0.25)))
    assert clip.overall_sparsity() == pytest.approx(0.25 * 3072 / 3136, abs=0.01) and clip.memory_after_bytes() == 4 * 3136
    assert Q.estimate_compressed_size(1000, Q.CompressionConfig.quantize_only()) == 1000 and Q.estimate_compressed_size(1000, Q.CompressionConfig.prune_only(0.9)) == 4000
    with pytest.raises(Q.CompressionError):
        Q.compress_model(model, Q.CompressionConfig())
    with pytest.raises(Q.CompressionError):
        Q.CompressionStage.clip(0.0)
    from oxibonsai_b200.quant.merge import linear_merge
    other = {k: v + 0.1 for k, v in model.items()}
    merged = linear_merge([model, other], [0.5, 0.5])
    st = Q.merge_stats(model, other, merged)
    assert st.tensors == 3 and st.parameters == 3136 and st.max_abs_change == pytest.approx(0.05, abs=1e-6) and 0.9 < st.mean_cosine_similarity <= 1.0
    assert "merged 3 tensors" in st.summary()


def test_smoothquant_calibrator_and_export(tmp_path):
    rng = np.random.default_rng(4)
    x = rng.normal(size=(50, 128)).astype(np.float32)
    x[:, 7] *= 40                                         # an outlier channel, the case SmoothQuant is for
    w = rng.normal(size=(64, 128)).astype(np.float32) * 0.05
    cal = Q.SmoothQuantCalibrator(0.5)
    cal.record_activation("ffn", x[:25])
    cal.record_activation("ffn", x[25:].reshape(5, 5, 128))
    assert cal.layer_count() == 1 and cal.has_layer("ffn") and not cal.has_layer("attn")
    s = cal.smooth_factors("ffn", w)
    assert s.shape == (128,) and s[7] > 4 * np.median(s)
    y = x @ w.T
    assert np.allclose((x / s) @ (w * s[None, :]).T, y, rtol=1e-3, atol=1e-3)                   # the product is unchanged
    assert np.abs(x / s).max() < np.abs(x).max() / 4                                            # and the activations are tamer
    blob, s2 = cal.quantize_fp8_smooth("ffn", w, "e4m3")
    back = dequantize(G.F8_E4M3, blob).reshape(w.shape) / s2[None, :]
    assert np.abs(back - w).max() < 0.1 * np.abs(w).max()
    for bad in (lambda: cal.smooth_factors("attn", w), lambda: cal.smooth_factors("ffn", w[:, :64]), lambda: cal.record_activation("ffn", x[:, :64]),
                lambda: Q.SmoothQuantCalibrator(1.5), lambda: cal.quantize_fp8_smooth("ffn", w, "e3m4")):
        with pytest.raises(Q.SmoothQuantError):
            bad()
    tensors = {"blk.0.ffn_up.weight": rng.normal(size=(256, 128)).astype(np.float32), "blk.0.attn_norm.weight": np.ones(128, np.float32),
               "odd.weight": rng.normal(size=(8, 100)).astype(np.float32), "keep.weight": rng.normal(size=(4, 128)).astype(np.float32)}
    cfg = Q.ExportConfig(Q.ExportFormat.TQ2_0_G128).with_fp32_layers(["keep.weight"]).with_description("toolbox test")
    shapes = {k: v.shape for k, v in tensors.items()}
    st = Q.export_stats(shapes, cfg)
    assert (st.tensors, st.quantized, st.kept_float) == (4, 1, 3) and st.bytes_f32 == 4 * sum(v.size for v in tensors.values())
    assert cfg.type_for("odd.weight", (8, 100)) == G.F16 and cfg.type_for("blk.0.attn_norm.weight", (128,)) == G.F32 and Q.ExportConfig.default_fp32_exceptions() == ("norm", "bias")
    path = str(tmp_path / "export.gguf")
    written = Q.export_to_gguf(tensors, path, cfg, {"general.architecture": "qwen3"})
    f = GgufFile.open(path)
    assert written.bytes_out == Q.estimate_export_size(shapes, cfg) == sum(t.nbytes for t in f.tensors) and written.compression_ratio() > 2
    assert f.tensor_info("blk.0.ffn_up.weight").type == G.TQ2_0_G128 and f.tensor_info("keep.weight").type == G.F32 and f.tensor_info("odd.weight").type == G.F16
    assert f.metadata["general.description"] == "toolbox test" and tuple(f.tensor_info("blk.0.ffn_up.weight").dims) == (128, 256)
    assert Q.ExportFormat.Q8_0.type_id() == G.Q8_0
