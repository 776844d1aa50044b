"""Block codecs against closed-form expectations (hand-built blocks, as the reference's unit tests do)."""
import numpy as np
import pytest

from oxibonsai_b200.core import dequantize, quantize, Q1_0_G128, TQ2_0_G128
from oxibonsai_b200.core import gguf as G
from oxibonsai_b200.core.blocks import fp8_decode, fp8_encode
from oxibonsai_b200.core.oracle import cpu_argmax_last, cpu_gemv, cpu_rmsnorm, cpu_rope, rope_table


def f16(v):
    return np.array([v], dtype=np.float16).view(np.uint8).tobytes()


def test_q1_layout_scale_first_bit_set_is_positive():
    qs = bytes([0b00000101] + [0] * 15)
    w = dequantize(Q1_0_G128, f16(0.5) + qs)
    assert w.shape == (128,)
    assert w[0] == 0.5 and w[1] == -0.5 and w[2] == 0.5 and (w[3:] == -0.5).all()


def test_tq2_layout_codes_first_scale_last_and_code_map():
    # codes 0,1,2,3 in the first byte -> -1, 0, +1, 0
    qs = bytes([0b11100100] + [0x55] * 31)
    w = dequantize(TQ2_0_G128, qs + f16(2.0))
    assert w[:4].tolist() == [-2.0, 0.0, 2.0, 0.0] and (w[4:] == 0).all()


def test_tq2_quantiser_threshold_and_zero_block():
    x = np.zeros(128, dtype=np.float32)
    q = quantize(TQ2_0_G128, x)
    assert bytes(q[:32]) == b"\x55" * 32 and bytes(q[32:]) == b"\0\0"
    x[0], x[1], x[2], x[3] = 1.0, -1.0, 0.49, 0.5
    w = dequantize(TQ2_0_G128, quantize(TQ2_0_G128, x))
    assert w[:4].tolist() == [1.0, -1.0, 0.0, 1.0]
    w256 = dequantize(G.TQ2_0, quantize(G.TQ2_0, np.tile(x, 2)))
    assert w256[:4].tolist() == [1.0, -1.0, 0.0, 1.0] and w256[128:132].tolist() == [1.0, -1.0, 0.0, 1.0]


def test_q1_quantiser_uses_loader_polarity():
    rng = np.random.default_rng(0)
    x = rng.standard_normal(256).astype(np.float32)
    w = dequantize(Q1_0_G128, quantize(Q1_0_G128, x))
    assert (np.sign(w) == np.where(x >= 0, 1, -1)).all()
    assert np.allclose(np.abs(w[:128]), np.abs(x[:128]).mean(), rtol=1e-3)
    wmax = dequantize(Q1_0_G128, quantize(Q1_0_G128, x, q1_absmax=True))
    assert np.allclose(np.abs(wmax[:128]), np.abs(x[:128]).max(), rtol=1e-3)


@pytest.mark.parametrize("ty,tol", [(G.Q4_0, 0.08), (G.Q8_0, 0.005), (G.F8_E4M3, 0.07), (G.F8_E5M2, 0.13)])
def test_standard_formats_round_trip(ty, tol):
    rng = np.random.default_rng(1)
    x = rng.standard_normal(32 * 16).astype(np.float32)
    y = dequantize(ty, quantize(ty, x))
    assert np.abs(x - y).max() <= tol * np.abs(x).max() + 1e-6


def test_q4_0_nibble_order_and_centre():
    blk = f16(1.0) + bytes([0x80 | 0x09] + [0x88] * 15)  # elem0 = 9-8 = 1, elem1 = 8-8 = 0
    w = dequantize(G.Q4_0, blk)
    assert w[0] == 1.0 and w[1] == 0.0 and (w[2:] == 0).all()


def test_fp8_codes_are_bit_exact():
    assert fp8_decode(0x7E) == 448.0 and fp8_decode(0x38) == 1.0 and fp8_decode(0x01) == 2.0 ** -9
    assert fp8_encode(448.0) == 0x7E and fp8_encode(1e9) == 0x7E and fp8_encode(-1.0) == 0xB8
    assert fp8_decode(0x7B, e5m2=True) == 57344.0 and fp8_encode(57344.0, e5m2=True) == 0x7B
    # every finite code survives decode -> encode
    for e5 in (False, True):
        for q in range(256):
            v = fp8_decode(q, e5)
            if np.isfinite(v):
                assert fp8_encode(v, e5) == q or v == 0.0
    # round to nearest even between 1.0 (0x38) and 1.125 (0x39)
    assert fp8_encode(1.0625) == 0x38 and fp8_encode(1.0626) == 0x39


def test_cpu_gemv_matches_dequantised_matmul():
    rng = np.random.default_rng(2)
    for ty in (TQ2_0_G128, Q1_0_G128, G.Q8_0, G.F16):
        rows, cols = 24, 256
        w = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32)
        raw = w.astype(np.float16).view(np.uint8).reshape(-1) if ty == G.F16 else quantize(ty, w)
        wd = w.astype(np.float16).astype(np.float32) if ty == G.F16 else dequantize(ty, raw).reshape(rows, cols)
        x = rng.standard_normal(cols).astype(np.float32)
        y = cpu_gemv(ty, raw, rows, cols, x)
        assert np.allclose(y, wd @ x, rtol=1e-4, atol=1e-4)


def test_float_ops_and_argmax_tie_rule():
    x = np.array([3.0, 4.0], dtype=np.float32)
    y = cpu_rmsnorm(x, np.array([1.0, 2.0], dtype=np.float32), 0.0)
    assert np.allclose(y, [3 / np.sqrt(12.5), 8 / np.sqrt(12.5)], rtol=1e-6)
    assert cpu_argmax_last(np.array([1, 5, 2, 5, 0], dtype=np.float32)) == 3
    v = np.arange(8, dtype=np.float32)
    assert np.allclose(cpu_rope(v, 0, 1e6), v)
    r = cpu_rope(v, 3, 1e4)
    cos, sin = rope_table(8, 4, 1e4)
    assert np.allclose(r[:4], v[:4] * cos[3] - v[4:] * sin[3]) and np.allclose(r[4:], v[:4] * sin[3] + v[4:] * cos[3])
    assert np.allclose(np.linalg.norm(r.reshape(2, 4), axis=0), np.linalg.norm(v.reshape(2, 4), axis=0), rtol=1e-5)
