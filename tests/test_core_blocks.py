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


# ---- K-quant super-blocks: the C++ decoders against an independent decode of the documented layouts -------------------------
def _f16(b, off):
    return float(np.frombuffer(bytes(b[off:off + 2]), dtype="<f2")[0])


def _k6(s):
    sc = [0] * 8
    mn = [0] * 8
    for i in range(4):
        sc[2 * i], sc[2 * i + 1] = s[i] & 15, s[i] >> 4
        mn[2 * i], mn[2 * i + 1] = s[4 + i] & 15, s[4 + i] >> 4
    for i in range(4):
        sc[i] |= ((s[8] >> (2 * i)) & 3) << 4
        sc[4 + i] |= ((s[9] >> (2 * i)) & 3) << 4
        mn[i] |= ((s[10] >> (2 * i)) & 3) << 4
        mn[4 + i] |= ((s[11] >> (2 * i)) & 3) << 4
    return sc, mn


def _py_decode(name, b):
    out = np.zeros(256, dtype=np.float64)
    b = [int(v) for v in b]
    bits = lambda arr, i, n: (arr[(i * n) // 8] >> ((i * n) % 8)) & ((1 << n) - 1)
    if name == "Q2_K":
        d, dm = _f16(b, 80), _f16(b, 82)
        for i in range(256):
            out[i] = d * (b[i // 16] & 15) * bits(b[16:80], i, 2) - dm * (b[i // 16] >> 4)
    elif name == "Q3_K":
        d = _f16(b, 108)
        for i in range(256):
            q = bits(b[32:96], i, 2) | (bits(b[0:32], i, 1) << 2)
            out[i] = d * (bits(b[96:108], i // 16, 4) - 8) * (q - 4)
    elif name in ("Q4_K", "Q5_K"):
        d, dm = _f16(b, 0), _f16(b, 2)
        sc, mn = _k6(b[4:16])
        for i in range(256):
            q = bits(b[16:144], i, 4) if name == "Q4_K" else (bits(b[48:176], i, 4) | (bits(b[16:48], i, 1) << 4))
            out[i] = d * sc[i // 32] * q - dm * mn[i // 32]
    elif name == "Q6_K":
        d = _f16(b, 208)
        sc = np.frombuffer(bytes(b[192:208]), dtype=np.int8)
        for i in range(256):
            out[i] = d * int(sc[i // 16]) * ((bits(b[0:128], i, 4) | (bits(b[128:192], i, 2) << 4)) - 32)
    else:
        d = float(np.frombuffer(bytes(b[0:4]), dtype="<f4")[0])
        out[:] = d * np.frombuffer(bytes(b[4:260]), dtype=np.int8)
    return out


@pytest.mark.parametrize("name,bytes_per_block,max_rel", [("Q2_K", 84, 0.45), ("Q3_K", 110, 0.25), ("Q4_K", 144, 0.1), ("Q5_K", 176, 0.05),
                                                          ("Q6_K", 210, 0.03), ("Q8_K", 292, 0.01)])
def test_kquant_layouts_and_roundtrip(name, bytes_per_block, max_rel):
    from oxibonsai_b200.core import gguf as G
    from oxibonsai_b200.core.blocks import dequantize, quantize
    from oxibonsai_b200.core.oracle import cpu_gemv
    tid = getattr(G, name)
    assert G.type_info(tid) == (name, 256, bytes_per_block)
    rng = np.random.default_rng(5)
    raw = rng.integers(0, 256, size=3 * bytes_per_block, dtype=np.uint8)
    for blk in range(3):          # finite scales in the f16 / f32 header fields
        b = raw[blk * bytes_per_block:(blk + 1) * bytes_per_block]
        for off in {"Q2_K": (80, 82), "Q3_K": (108,), "Q4_K": (0, 2), "Q5_K": (0, 2), "Q6_K": (208,)}.get(name, ()):
            b[off:off + 2] = np.frombuffer(np.float16(rng.uniform(0.01, 0.1)).tobytes(), dtype=np.uint8)
        if name == "Q8_K":
            b[0:4] = np.frombuffer(np.float32(0.02).tobytes(), dtype=np.uint8)
    got = dequantize(tid, raw).reshape(3, 256)
    for blk in range(3):
        want = _py_decode(name, raw[blk * bytes_per_block:(blk + 1) * bytes_per_block])
        assert np.allclose(got[blk], want, rtol=1e-6, atol=1e-7), (name, blk)
    x = rng.normal(size=(6, 512)).astype(np.float32)
    q = quantize(tid, x)
    back = dequantize(tid, q).reshape(x.shape)
    assert q.size == x.size // 256 * bytes_per_block and np.sqrt(((back - x) ** 2).mean()) / x.std() < max_rel
    v = rng.normal(size=512).astype(np.float32)
    assert np.allclose(cpu_gemv(tid, q, 6, 512, v), back.astype(np.float64) @ v, rtol=1e-4, atol=1e-4)
    if name == "Q8_K":
        b0 = q[:292]
        sums = np.frombuffer(bytes(b0[260:292]), dtype="<i2")
        assert np.array_equal(sums, np.frombuffer(bytes(b0[4:260]), dtype=np.int8).reshape(16, 16).sum(1))
    zeros = dequantize(tid, quantize(tid, np.zeros(256, dtype=np.float32)))
    assert np.all(zeros == 0)


def test_compat_report_and_model_card(tiny_gguf):
    from oxibonsai_b200.core import GgufFile, compat as CP, gguf as G
    f = GgufFile.open(tiny_gguf)
    head = open(tiny_gguf, "rb").read(24)
    assert CP.check_gguf_header(head)[0] == 3
    with pytest.raises(CP.CompatError):
        CP.check_gguf_header(b"XXXX" + head[4:])
    with pytest.raises(CP.CompatError):
        CP.check_gguf_header(head[:4] + (9).to_bytes(4, "little") + head[8:])
    assert CP.GgufVersion.from_u32(7) is None and CP.GgufVersion(3).supports_aligned_tensors() and not CP.GgufVersion(1).supports_f16_kv()
    assert CP.quant_bits_per_weight(G.TQ2_0_G128) == 2.125 and CP.quant_bits_per_weight(99) is None and CP.quant_name(99) == "unknown(99)"
    r = CP.build_compat_report(f)
    assert r.compatible and r.servable_on_gpu and r.quant_histogram["TQ2_0_g128"] == 14 and "compatible" in r.summary()
    r.add_unknown_quant(99)
    assert not r.finalize().compatible and "NOT compatible" in r.summary()
    card = CP.extract_model_card(f, file_size_bytes=12345)
    md = card.to_markdown()
    assert card.architecture and card.block_count == 2 and card.quantization == "TQ2_0_g128" and not card.is_empty()
    assert "## Architecture Details" in md and "| Layers | 2 |" in md and "`TQ2_0_g128`" in md and "12345 bytes" in md
    assert card.estimated_param_count() > 1e5 and "params" in card.to_summary() and CP.ModelCard().is_empty()
