"""Host statement of the streamed decode layout: packing, the one-instruction decode and the integer arithmetic."""
import numpy as np

from oxibonsai_b200.ops import s16_layout as L


def _random(n, k, seed):
    rng = np.random.default_rng(seed)
    w = rng.integers(-1, 2, size=(n, k)).astype(np.int8)
    s = np.abs(rng.normal(0.02, 0.002, size=(n, k // 128))).astype(np.float16)
    return w, s, rng


def test_pack_round_trip_with_ragged_tile():
    w, s, _ = _random(40, 384, 0)
    b = L.pack(w, s)
    assert b.size == 3 * 3 * L.BLOCK_BYTES
    w2, s2 = L.unpack(b, 40, 384)
    assert (w2 == w).all() and (s2 == s).all()


def test_every_input_is_covered_once_per_row():
    seen = []
    for step in range(4):
        for t in range(4):
            for word in (0, 2):          # words 1 and 3 hold the same inputs for rows g + 8
                for byte in range(4):
                    seen.append(L.input_of(0, step, t, word, byte))
    assert sorted(seen) == list(range(128))


def test_step_operand_is_the_scaled_code_and_ignores_other_fields():
    for step in range(4):
        for codes in ((0, 1, 2, 1), (2, 2, 0, 0)):
            word = 0xFFFFFFFF
            for b, c in enumerate(codes):
                word &= ~(3 << (8 * b + 2 * step))
                word |= c << (8 * b + 2 * step)
            got = L.step_operand(np.array([word], dtype=np.uint32), step)[0]
            assert got.tolist() == [c << (2 * step) for c in codes] and max(got) <= 128


def test_two_term_quantisation_is_sixteen_bits_of_the_group_maximum():
    rng = np.random.default_rng(5)
    x = (rng.normal(size=512) * np.repeat([0.01, 1.0, 30.0, 1e-4], 128)).astype(np.float32)
    q1, q2, s = L.quantize_activations(x)
    assert np.abs(q1).max() <= 127 and np.abs(q2).max() <= 127
    back = np.repeat(s, 128) * (q1 + q2 / L.TERM2)
    amax = np.repeat(np.abs(x.reshape(-1, 128)).max(axis=1), 128)
    assert (np.abs(back - x) <= amax / (127 * 2 * L.TERM2) * 1.01 + 1e-12).all()
    assert (L.quantize_activations(np.zeros(128, np.float32))[0] == 0).all()


def test_emulated_kernel_arithmetic_matches_a_plain_product():
    w, s, rng = _random(50, 512, 3)
    x = rng.normal(size=512).astype(np.float32) * 3.0
    x[::37] *= 8.0
    b = L.pack(w, s)
    y = L.emulate_gemv(b, 50, 512, x)
    ref = (w.astype(np.float64) * np.repeat(s.astype(np.float64), 128, axis=1)) @ x.astype(np.float64)
    assert np.abs(y - ref).max() <= 2e-4 * np.abs(ref).mean() * 2.0
