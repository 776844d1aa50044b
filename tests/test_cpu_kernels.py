"""CPU kernel tiers: reference tier bit-identical to the oracle, AVX2 tier close, float ops, dispatcher (CPU)."""
import numpy as np
import pytest

from oxibonsai_b200.core import gguf as G
from oxibonsai_b200.core.blocks import dequantize, quantize
from oxibonsai_b200.core.oracle import cpu_gemv
from oxibonsai_b200.ops import cpu_ops as CK


@pytest.mark.parametrize("ty", [G.TQ2_0_G128, G.Q1_0_G128])
def test_tiers_against_oracle(ty):
    rng = np.random.default_rng(0)
    rows, cols = 300, 512
    w = rng.normal(size=(rows, cols)).astype(np.float32) * 0.05
    q = quantize(ty, w)
    x = rng.normal(size=cols).astype(np.float32)
    oracle = cpu_gemv(ty, q, rows, cols, x)
    ref = CK.gemv(ty, q, rows, cols, x, CK.KernelTier.REFERENCE, threads=3)
    assert np.array_equal(ref, oracle)                                     # same summation order, any thread count
    best = CK.detect_tier()
    for tier in (CK.KernelTier.AVX2, CK.KernelTier.AVX512):                # each vector tier the host has runs its own body
        if tier <= best:
            assert np.allclose(CK.gemv(ty, q, rows, cols, x, tier), oracle, rtol=1e-4, atol=1e-5)
    xb = rng.normal(size=(5, cols)).astype(np.float32)
    want = xb.astype(np.float64) @ dequantize(ty, q).reshape(rows, cols).astype(np.float64).T
    assert np.allclose(CK.gemm(ty, q, rows, cols, xb), want, rtol=1e-4, atol=1e-4)


def test_tier_control_and_errors():
    best = CK.detect_tier()
    assert CK.set_tier(CK.KernelTier.REFERENCE) == CK.KernelTier.REFERENCE and CK.set_tier(None) == best and CK.set_tier(99) == best
    assert CK.tier_name(0) == "reference" and CK.tier_name(CK.KernelTier.GPU) == "gpu" and CK.KernelTier.AVX2.is_accelerated
    q = quantize(G.TQ2_0_G128, np.zeros((2, 128), np.float32))
    with pytest.raises(CK.UnsupportedOperation):
        CK.gemv(G.Q4_0, q, 2, 128, np.zeros(128))
    with pytest.raises(CK.NotBlockAligned):
        CK.gemv(G.TQ2_0_G128, q, 2, 100, np.zeros(100))
    with pytest.raises(CK.BufferTooSmall):
        CK.gemv(G.TQ2_0_G128, q, 3, 128, np.zeros(128))
    with pytest.raises(CK.DimensionMismatch):
        CK.gemv(G.TQ2_0_G128, q, 2, 128, np.zeros(64))
    assert issubclass(CK.GpuError, CK.KernelError)


def test_float_ops():
    rng = np.random.default_rng(1)
    x, w = rng.normal(size=300).astype(np.float32), rng.uniform(0.5, 1.5, 300).astype(np.float32)
    want = w * x / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-6)
    assert np.allclose(CK.rms_norm(x, w, 1e-6, tier=0), want, rtol=1e-5) and np.allclose(CK.rms_norm(x, w, 1e-6, tier=1), want, rtol=1e-5)
    assert np.allclose(CK.rms_norm(x, w, 1e-6, tier=2), want, rtol=1e-5)
    assert np.allclose(CK.silu(x), x / (1 + np.exp(-x)), rtol=1e-5) and np.allclose(CK.swiglu(x, w), x / (1 + np.exp(-x)) * w, rtol=1e-5)
    s = CK.softmax(x)
    assert abs(s.sum() - 1) < 1e-5 and int(np.argmax(s)) == int(np.argmax(x))
    from oxibonsai_b200.core.oracle import rope_table
    cos, sin = rope_table(64, 8, 1e6)
    v = rng.normal(size=(3, 64)).astype(np.float32)
    r = CK.rope_apply(v, cos[5], sin[5])
    assert np.allclose(np.linalg.norm(r, axis=1), np.linalg.norm(v, axis=1), rtol=1e-5)
    assert np.allclose(r[:, :32], v[:, :32] * cos[5] - v[:, 32:] * sin[5], rtol=1e-5, atol=1e-6) and np.allclose(CK.rope_apply(v, cos[0], sin[0]), v)
    b = CK.AlignedBuffer(100)
    assert b.address % 64 == 0 and b.array.shape == (100,)
    b.array[:] = 3.0
    assert float(b.array.sum()) == 300.0


def test_dispatcher_on_cpu():
    d = CK.KernelDispatcher(tier=CK.detect_tier())
    rng = np.random.default_rng(2)
    w = rng.normal(size=(64, 256)).astype(np.float32)
    q = quantize(G.Q1_0_G128, w)
    x = rng.normal(size=256).astype(np.float32)
    assert np.allclose(d.gemv(G.Q1_0_G128, q, 64, 256, x), cpu_gemv(G.Q1_0_G128, q, 64, 256, x), rtol=1e-4, atol=1e-5)
    assert d.gemm(G.Q1_0_G128, q, 64, 256, x[None]).shape == (1, 64) and "threads=" in d.describe() and d.gpu_fallbacks == 0
    assert CK.KernelDispatcher.auto_detect().tier in tuple(CK.KernelTier) and CK.GpuWeightHandle(3).id == 3


def test_vector_tiers_agree_with_the_reference_tier_on_random_shapes():
    """Property test: every vector tier against tier 0 over random shapes, scales and sparsity (edge rows, all-zero blocks)."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=25, deadline=None)
    @given(ty=st.sampled_from([G.TQ2_0_G128, G.Q1_0_G128]), rows=st.integers(1, 70), blocks=st.integers(1, 8),
           scale=st.floats(1e-3, 10.0), zero_frac=st.floats(0.0, 1.0), seed=st.integers(0, 2**31 - 1))
    def check(ty, rows, blocks, scale, zero_frac, seed):
        rng = np.random.default_rng(seed)
        cols = 128 * blocks
        w = (rng.normal(size=(rows, cols)) * scale).astype(np.float32)
        w[rng.random(size=w.shape) < zero_frac] = 0.0
        q = quantize(ty, w)
        x = rng.normal(size=cols).astype(np.float32)
        ref = CK.gemv(ty, q, rows, cols, x, CK.KernelTier.REFERENCE, threads=1)
        tol = 1e-4 * max(1.0, float(np.abs(ref).max()))
        for tier in (CK.KernelTier.AVX2, CK.KernelTier.AVX512):
            if tier <= CK.detect_tier():
                assert np.abs(CK.gemv(ty, q, rows, cols, x, tier, threads=2) - ref).max() <= tol
        xb = rng.normal(size=(3, cols)).astype(np.float32)
        got = CK.gemm(ty, q, rows, cols, xb)
        want = np.stack([CK.gemv(ty, q, rows, cols, xb[i], CK.KernelTier.REFERENCE, threads=1) for i in range(3)])
        assert np.abs(got - want).max() <= 1e-4 * max(1.0, float(np.abs(want).max()))

    check()


@pytest.mark.parametrize("ty", [G.F8_E4M3, G.F8_E5M2])
def test_fp8_rows_on_every_tier(ty):
    """FP8 blocks (32 codes + f16 scale): the scalar body and the table-gather vector bodies agree with the decoded matrix."""
    rng = np.random.default_rng(2)
    rows, cols = 130, 224                                   # 7 blocks per row: not a multiple of 128
    q = quantize(ty, rng.normal(size=(rows, cols)).astype(np.float32) * 0.05)
    wd = dequantize(ty, q).reshape(rows, cols).astype(np.float64)
    x = rng.normal(size=cols).astype(np.float32)
    want = wd @ x.astype(np.float64)
    best = CK.detect_tier()
    for tier in (CK.KernelTier.REFERENCE, CK.KernelTier.AVX2, CK.KernelTier.AVX512):
        if tier <= best:
            assert np.allclose(CK.gemv(ty, q, rows, cols, x, tier, threads=2), want, rtol=1e-4, atol=1e-5), tier
    xb = rng.normal(size=(3, cols)).astype(np.float32)
    assert np.allclose(CK.gemm(ty, q, rows, cols, xb), xb.astype(np.float64) @ wd.T, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("ty", [G.TQ2_0_G128, G.Q1_0_G128, G.F8_E4M3])
def test_tiled_and_adaptive_products_match_the_plain_ones(ty):
    rng = np.random.default_rng(6)
    rows, cols = 523, 384
    q = quantize(ty, rng.normal(size=(rows, cols)).astype(np.float32) * 0.05)
    x = rng.normal(size=cols).astype(np.float32)
    plain = CK.gemv(ty, q, rows, cols, x, threads=1)
    for tile, threads in ((0, 0), (7, 3), (600, 2), (1, 1)):
        assert np.array_equal(CK.gemv_tiled(ty, q, rows, cols, x, tile_rows=tile, threads=threads), plain), (tile, threads)
    xb = rng.normal(size=(11, cols)).astype(np.float32)
    plain_mm = CK.gemm(ty, q, rows, cols, xb, threads=1)
    for tr, tb, threads in ((0, 0, 0), (5, 3, 2), (64, 16, 4)):
        assert np.array_equal(CK.gemm_tiled(ty, q, rows, cols, xb, tile_rows=tr, tile_batch=tb, threads=threads), plain_mm), (tr, tb)
    y, st = CK.gemv_adaptive(ty, q, rows, cols, x)
    assert st == CK.Strategy.PARALLEL_TILED and np.array_equal(y, plain)
    y, st = CK.gemv_adaptive(ty, q[: 20 * (cols // (128 if ty != G.F8_E4M3 else 32)) * (34 if ty != G.Q1_0_G128 else 18)], 20, cols, x)
    assert st == CK.Strategy.DIRECT and np.array_equal(y, plain[:20])
    ym, st = CK.gemm_adaptive(ty, q, rows, cols, xb)
    assert st == CK.Strategy.PARALLEL_TILED and np.array_equal(ym, plain_mm)


def test_strategy_tiles_packing_and_prefetch_helpers():
    assert CK.select_strategy(16, 4096) == CK.Strategy.DIRECT
    assert CK.select_strategy(200, 4096) == CK.Strategy.PARALLEL_ROWS
    assert CK.select_strategy(200, 4096, batch=8) == CK.Strategy.PARALLEL_TILED
    assert CK.select_strategy(4096, 4096) == CK.Strategy.PARALLEL_TILED
    # working set: packed rows + f32 input + f32 output
    assert CK.working_set_bytes(G.TQ2_0_G128, 10, 256) == 10 * 2 * 34 + 256 * 4 + 10 * 4
    assert CK.working_set_bytes(G.Q4_0, 10, 256) == 0 and CK.working_set_bytes(G.TQ2_0_G128, 10, 100) == 0
    assert CK.fits_in_cache(G.Q1_0_G128, 64, 1024) and not CK.fits_in_cache(G.Q1_0_G128, 4096, 4096)
    t = CK.optimal_tile_rows(G.Q1_0_G128, 4096)                   # (32 KB - 16 KB input) / 576 bytes per row
    assert t == (32 * 1024 - 4096 * 4) // (32 * 18)
    assert CK.optimal_tile_rows(G.TQ2_0_G128, 16384) == 4 and CK.optimal_tile_rows(G.Q1_0_G128, 128, 1 << 20) == 256
    # tile packing: a permutation of the blocks with an exact inverse; a ragged last tile is handled
    rng = np.random.default_rng(1)
    rows, cols = 70, 512
    q = quantize(G.TQ2_0_G128, rng.normal(size=(rows, cols)).astype(np.float32))
    packed = CK.pack_rows_tiled(G.TQ2_0_G128, q, rows, cols, tile=32)
    assert packed.shape == q.reshape(-1).shape and not np.array_equal(packed, q.reshape(-1))
    blocks, pblocks = q.reshape(rows, 4, 34), packed.reshape(-1, 34)
    assert np.array_equal(pblocks[0], blocks[0, 0]) and np.array_equal(pblocks[1], blocks[1, 0]) and np.array_equal(pblocks[32], blocks[0, 1])
    assert np.array_equal(pblocks[2 * 32 * 4 + 6], blocks[64, 1])            # last tile has 6 rows: block 1 starts after 6 entries
    assert np.array_equal(CK.pack_rows_tiled(G.TQ2_0_G128, packed, rows, cols, tile=32, unpack=True), q.reshape(-1))
    CK.prefetch_range(q, locality=1)
    CK.prefetch_range(np.zeros(1000, np.float32), locality=3, write=True)     # hints only: nothing observable, must not fault


def test_vectorised_float_ops_agree_with_the_scalar_bodies():
    """SiLU / SwiGLU / softmax with the polynomial exp agree with the scalar bodies to rounding (relative 1e-6); the rotation
    uses the same multiplies and adds and is equal bit for bit.  Lengths that are not multiples of the vector width and
    extreme arguments are included."""
    rng = np.random.default_rng(3)
    for n in (1, 7, 8, 9, 64, 1000, 4099):
        x = (rng.normal(size=n) * 4).astype(np.float32)
        up = rng.normal(size=n).astype(np.float32)
        np.testing.assert_allclose(CK.silu(x, tier=1), CK.silu(x, tier=0), rtol=2e-6, atol=1e-7)
        np.testing.assert_allclose(CK.swiglu(x, up, tier=1), CK.swiglu(x, up, tier=0), rtol=2e-6, atol=1e-7)
        a, b = CK.softmax(x, tier=1), CK.softmax(x, tier=0)
        np.testing.assert_allclose(a, b, rtol=3e-6, atol=1e-9)
        assert abs(float(a.sum()) - 1.0) < 1e-5
    extreme = np.array([-200.0, -88.0, -30.0, 0.0, 30.0, 88.0, 200.0, -0.0, 1e-8], dtype=np.float32)
    s1, s0 = CK.silu(extreme, tier=1), CK.silu(extreme, tier=0)
    assert np.all(np.isfinite(s1)) and np.allclose(s1, s0, rtol=1e-5, atol=1e-30)
    sm = CK.softmax(np.array([1000.0, 999.0, -1000.0] * 5, dtype=np.float32), tier=1)
    assert np.all(np.isfinite(sm)) and abs(sm.sum() - 1.0) < 1e-5 and sm[2] < 1e-30      # (the vector body clamps exp at e^-87)
    # against float64 references
    x = (rng.normal(size=513) * 3).astype(np.float32)
    ref = x.astype(np.float64) / (1.0 + np.exp(-x.astype(np.float64)))
    assert np.abs(CK.silu(x, tier=1) - ref).max() < 2e-6
    for heads, hd in ((1, 64), (4, 128), (3, 20), (2, 6)):
        v = rng.normal(size=(heads, hd)).astype(np.float32)
        ang = rng.uniform(0, 6.28, size=hd // 2)
        c, s = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
        assert np.array_equal(CK.rope_apply(v, c, s, tier=1), CK.rope_apply(v, c, s, tier=0))
