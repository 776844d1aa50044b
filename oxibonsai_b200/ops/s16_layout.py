"""Host-side statement of the S16 packed-weight layout consumed by the streamed decode GEMV.

``csrc/cuda/bitgemv_stream.cu`` reads a ternary / sign matrix as tiles of 16 output rows.  One 544-byte block covers a
(tile, 128-input group) pair: 32 lanes x 16 bytes of 2-bit codes followed by 16 f16 group scales.  This module packs a
dense matrix into that form, decodes it back and restates the kernel's arithmetic (offset decode, per-group offset sum,
f32 accumulation) with numpy, so the layout and the bit tricks can be checked without a GPU and the device repack can be
compared byte for byte.  Reference counterpart: the reference's array-of-blocks -> structure-of-arrays re-layout
(crates/oxibonsai-kernels/src/gpu_backend/cuda_graph/cudagraph_reformat_tq2_blocks_to_soa_group.rs:16-74).
"""
from __future__ import annotations

import numpy as np

BLOCK_BYTES = 544
#: (shift applied to the word, mask, exponent pattern, offset) of code slot / MMA step 0..7
SLOTS = [(+6, 0x00C000C0, 0x4C004C00, 16.0), (+6, 0x03000300, 0x44004400, 4.0),
         (0, 0x00300030, 0x54005400, 64.0), (0, 0x00C000C0, 0x4C004C00, 16.0), (0, 0x03000300, 0x44004400, 4.0),
         (-6, 0x00300030, 0x54005400, 64.0), (-6, 0x00C000C0, 0x4C004C00, 16.0), (-6, 0x03000300, 0x44004400, 4.0)]


def input_of(group: int, step: int, t: int, word: int, half: int) -> int:
    """Input index covered by MMA step ``step`` of lane-quad position ``t``, code word ``word`` (0..3), 16-bit half ``half``."""
    return group * 128 + 32 * (step >> 1) + 8 * t + 4 * (step & 1) + (2 if word & 2 else 0) + half


def pack(weights: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """``weights`` int8 [N, K] in {-1, 0, 1}, ``scales`` f16 [N, K/128] -> uint8 array of S16 blocks [tile][group]."""
    n, k = weights.shape
    assert k % 128 == 0 and scales.shape == (n, k // 128)
    ntiles, ng = (n + 15) // 16, k // 128
    wp = np.zeros((ntiles * 16, k), dtype=np.int8)
    wp[:n] = weights
    sp = np.zeros((ntiles * 16, ng), dtype=np.float16)
    sp[:n] = scales
    codes = (wp.astype(np.int32) + 1).astype(np.uint32)          # c = w + 1
    out = np.zeros((ntiles, ng, BLOCK_BYTES // 4), dtype=np.uint32)
    tiles = np.arange(ntiles)[:, None]
    for grp in range(ng):
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            for word in range(4):
                rows = tiles[:, 0] * 16 + g + (8 if word & 1 else 0)
                acc = np.zeros(ntiles, dtype=np.uint32)
                for step in range(8):
                    for half in range(2):
                        kk = input_of(grp, step, t, word, half)
                        acc |= codes[rows, kk] << np.uint32(2 * step + 16 * half)
                out[:, grp, lane * 4 + word] = acc
        for g in range(8):
            lo = sp[tiles[:, 0] * 16 + g, grp].view(np.uint16).astype(np.uint32)
            hi = sp[tiles[:, 0] * 16 + g + 8, grp].view(np.uint16).astype(np.uint32)
            out[:, grp, 128 + g] = lo | (hi << np.uint32(16))
    return out.reshape(-1).view(np.uint8)


def unpack(blocks: np.ndarray, n: int, k: int) -> tuple[np.ndarray, np.ndarray]:
    """Inverse of :func:`pack`: returns (weights int8 [N, K], scales f16 [N, K/128])."""
    ntiles, ng = (n + 15) // 16, k // 128
    w32 = np.ascontiguousarray(blocks).view(np.uint32).reshape(ntiles, ng, BLOCK_BYTES // 4)
    weights = np.zeros((ntiles * 16, k), dtype=np.int8)
    scales = np.zeros((ntiles * 16, ng), dtype=np.float16)
    tiles = np.arange(ntiles)
    for grp in range(ng):
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            for word in range(4):
                rows = tiles * 16 + g + (8 if word & 1 else 0)
                v = w32[:, grp, lane * 4 + word]
                for step in range(8):
                    for half in range(2):
                        c = (v >> np.uint32(2 * step + 16 * half)) & np.uint32(3)
                        weights[rows, input_of(grp, step, t, word, half)] = c.astype(np.int8) - 1
        for g in range(8):
            v = w32[:, grp, 128 + g]
            scales[tiles * 16 + g, grp] = (v & np.uint32(0xFFFF)).astype(np.uint16).view(np.float16)
            scales[tiles * 16 + g + 8, grp] = (v >> np.uint32(16)).astype(np.uint16).view(np.float16)
    return weights[:n], scales[:n]


def decode_word(word: np.ndarray, step: int) -> np.ndarray:
    """The kernel's one-instruction decode of code slot ``step``: returns the two f16 numbers (offset + code) held by the
    halves of ``(shifted word & mask) | exponent`` as float32 [..., 2]."""
    shift, mask, expo, _ = SLOTS[step]
    w = word.astype(np.uint32)
    v = (w << np.uint32(shift)) if shift > 0 else (w >> np.uint32(-shift)) if shift < 0 else w
    v = (v & np.uint32(mask)) | np.uint32(expo)
    halves = np.stack([(v & np.uint32(0xFFFF)).astype(np.uint16), (v >> np.uint32(16)).astype(np.uint16)], axis=-1)
    return halves.view(np.float16).astype(np.float32)


def emulate_gemv(blocks: np.ndarray, n: int, k: int, x: np.ndarray) -> np.ndarray:
    """W x as the kernel computes it: f16 activations, offset-coded weights, the per-group offset sum removed, group
    scales applied in f32.  Returns float32 [N]."""
    ntiles, ng = (n + 15) // 16, k // 128
    w32 = np.ascontiguousarray(blocks).view(np.uint32).reshape(ntiles, ng, BLOCK_BYTES // 4)
    xh = x.astype(np.float16).astype(np.float32)
    out = np.zeros(ntiles * 16, dtype=np.float32)
    tiles = np.arange(ntiles)
    for grp in range(ng):
        og = np.float32(0.0)
        acc = np.zeros(ntiles * 16, dtype=np.float32)
        for step in range(8):
            off1 = np.float32(SLOTS[step][3] + 1.0)
            for t in range(4):
                for word in range(4):
                    ks = [input_of(grp, step, t, word, h) for h in range(2)]
                    for g in range(8):
                        rows = tiles * 16 + g + (8 if word & 1 else 0)
                        dec = decode_word(w32[:, grp, (g * 4 + t) * 4 + word], step)       # [ntiles, 2] = offset + code
                        acc[rows] += dec[:, 0] * xh[ks[0]] + dec[:, 1] * xh[ks[1]]
                for word in (0, 2):                                                          # each input once for the offset sum
                    for h in range(2):
                        og += off1 * xh[input_of(grp, step, t, word, h)]
        sc = np.zeros(ntiles * 16, dtype=np.float32)
        for g in range(8):
            v = w32[:, grp, 128 + g]
            sc[tiles * 16 + g] = (v & np.uint32(0xFFFF)).astype(np.uint16).view(np.float16).astype(np.float32)
            sc[tiles * 16 + g + 8] = (v >> np.uint32(16)).astype(np.uint16).view(np.float16).astype(np.float32)
        out += sc * (acc - og)
    return out[:n]
