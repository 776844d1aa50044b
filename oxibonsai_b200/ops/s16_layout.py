"""Host-side statement of the S16 packed-weight layout consumed by the streamed decode GEMV.

``csrc/cuda/bitgemv_stream.cu`` reads a ternary / sign matrix as tiles of 16 output rows.  One 544-byte block covers a
(tile, 128-input group) pair: 32 lanes x 16 bytes of 2-bit codes followed by 16 f16 group scales.  This module packs a
dense matrix into that form, decodes it back and restates the kernel's arithmetic (two-term int8 activations, 4^j-scaled
u8 weights per MMA step, integer sums, f32 scales) with numpy, so the layout and the bit tricks can be checked without a GPU
and the device repack can be compared byte for byte.  Reference counterpart: the reference's array-of-blocks ->
structure-of-arrays re-layout (crates/oxibonsai-kernels/src/gpu_backend/cuda_graph/cudagraph_reformat_tq2_blocks_to_soa_group.rs:16-74).
"""
from __future__ import annotations

import numpy as np

BLOCK_BYTES = 544
TERM2 = 254.0      # activations: x = s * (q1 + q2 / 254), |q| <= 127


def input_of(group: int, step: int, t: int, word: int, byte: int) -> int:
    """Input index held by 2-bit field ``step`` of byte ``byte`` of code word ``word`` (0..3) of lane-quad position ``t``."""
    return group * 128 + 32 * step + 8 * t + (4 if word & 2 else 0) + byte


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
    tiles = np.arange(ntiles)
    for grp in range(ng):
        for lane in range(32):
            g, t = lane >> 2, lane & 3
            for word in range(4):
                rows = tiles * 16 + g + (8 if word & 1 else 0)
                acc = np.zeros(ntiles, dtype=np.uint32)
                for byte in range(4):
                    for step in range(4):
                        acc |= codes[rows, input_of(grp, step, t, word, byte)] << np.uint32(8 * byte + 2 * step)
                out[:, grp, lane * 4 + word] = acc
        for g in range(8):
            lo = sp[tiles * 16 + g, grp].view(np.uint16).astype(np.uint32)
            hi = sp[tiles * 16 + g + 8, grp].view(np.uint16).astype(np.uint32)
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
                for byte in range(4):
                    for step in range(4):
                        c = (v >> np.uint32(8 * byte + 2 * step)) & np.uint32(3)
                        weights[rows, input_of(grp, step, t, word, byte)] = c.astype(np.int8) - 1
        for g in range(8):
            v = w32[:, grp, 128 + g]
            scales[tiles * 16 + g, grp] = (v & np.uint32(0xFFFF)).astype(np.uint16).view(np.float16)
            scales[tiles * 16 + g + 8, grp] = (v >> np.uint32(16)).astype(np.uint16).view(np.float16)
    return weights[:n], scales[:n]


def quantize_activations(x: np.ndarray) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Two int8 terms per 128-input group, as the kernel's prologue computes them: returns (q1, q2 int32 [K], s f32 [K/128])
    with x ~ s[group] * (q1 + q2 / 254)."""
    xg = x.astype(np.float32).reshape(-1, 128)
    amax = np.abs(xg).max(axis=1)
    s = np.where(amax > 0, amax * np.float32(1.0 / 127.0), np.float32(1.0)).astype(np.float32)
    f = xg * (np.float32(1.0) / s)[:, None]
    q1 = np.clip(np.rint(f), -127, 127).astype(np.int32)
    q2 = np.clip(np.rint((f - q1.astype(np.float32)) * np.float32(TERM2)), -127, 127).astype(np.int32)
    return q1.reshape(-1), q2.reshape(-1), s


def step_operand(word: np.ndarray, step: int) -> np.ndarray:
    """The kernel's one-instruction decode of MMA step ``step``: ``word & (0x03030303 << 2 * step)`` as four u8 values
    (4^step * code) [..., 4]."""
    v = word.astype(np.uint32) & np.uint32(0x03030303 << (2 * step))
    return np.stack([(v >> np.uint32(8 * b)) & np.uint32(0xFF) for b in range(4)], axis=-1).astype(np.int64)


def emulate_gemv(blocks: np.ndarray, n: int, k: int, x: np.ndarray) -> np.ndarray:
    """W x as the kernel computes it: integer dot products of the 4^j-scaled codes with the two activation terms per MMA
    step, minus the part the +1 of the codes adds, combined and scaled in f32.  Returns float32 [N]."""
    ntiles, ng = (n + 15) // 16, k // 128
    w32 = np.ascontiguousarray(blocks).view(np.uint32).reshape(ntiles, ng, BLOCK_BYTES // 4)
    q1, q2, sx = quantize_activations(x)
    out = np.zeros(ntiles * 16, dtype=np.float32)
    tiles = np.arange(ntiles)
    for grp in range(ng):
        sc = np.zeros(ntiles * 16, dtype=np.float32)
        for g in range(8):
            v = w32[:, grp, 128 + g]
            sc[tiles * 16 + g] = (v & np.uint32(0xFFFF)).astype(np.uint16).view(np.float16).astype(np.float32)
            sc[tiles * 16 + g + 8] = (v >> np.uint32(16)).astype(np.uint16).view(np.float16).astype(np.float32)
        for step in range(4):
            acc1 = np.zeros(ntiles * 16, dtype=np.int64)
            acc2 = np.zeros(ntiles * 16, dtype=np.int64)
            lo = grp * 128 + 32 * step
            og1, og2 = int(q1[lo:lo + 32].sum()) << (2 * step), int(q2[lo:lo + 32].sum()) << (2 * step)
            for lane in range(32):
                g, t = lane >> 2, lane & 3
                for word in range(4):
                    rows = tiles * 16 + g + (8 if word & 1 else 0)
                    a = step_operand(w32[:, grp, lane * 4 + word], step)            # [ntiles, 4] = 4^step * code
                    ks = [input_of(grp, step, t, word, b) for b in range(4)]
                    acc1[rows] += a @ q1[ks].astype(np.int64)
                    acc2[rows] += a @ q2[ks].astype(np.int64)
            v = (acc1 - og1).astype(np.float32) + (acc2 - og2).astype(np.float32) * np.float32(1.0 / TERM2)
            out += sc * (sx[grp] * np.float32(1.0 / (1 << (2 * step)))) * v
    return out[:n]
