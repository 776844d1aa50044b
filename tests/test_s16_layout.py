"""Host statement of the streamed decode layout: packing, the one-instruction decode and the offset arithmetic."""
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
    seen = set()
    for step in range(8):
        for t in range(4):
            for word in (0, 2):          # words 1 and 3 hold the same inputs for rows g + 8
                for half in range(2):
                    seen.add(L.input_of(0, step, t, word, half))
    assert seen == set(range(128))


def test_decode_is_offset_plus_code_for_every_slot():
    for step in range(8):
        for c_lo in range(3):
            for c_hi in range(3):
                word = np.array([(c_lo << (2 * step)) | (c_hi << (2 * step + 16)) | 0xFFFFFFFF & ~((3 << (2 * step)) | (3 << (2 * step + 16)))], dtype=np.uint32)
                # every other slot is filled with ones: the mask must remove them
                dec = L.decode_word(word, step)[0]
                off = L.SLOTS[step][3]
                assert dec[0] == off + c_lo and dec[1] == off + c_hi


def test_emulated_kernel_arithmetic_matches_a_plain_product():
    w, s, rng = _random(50, 512, 3)
    x = rng.normal(size=512).astype(np.float32) * 3.0
    b = L.pack(w, s)
    y = L.emulate_gemv(b, 50, 512, x)
    ref = (w.astype(np.float64) * np.repeat(s.astype(np.float64), 128, axis=1)) @ x.astype(np.float16).astype(np.float64)
    assert np.abs(y - ref).max() <= 1e-5 * np.abs(ref).max() + 1e-6
