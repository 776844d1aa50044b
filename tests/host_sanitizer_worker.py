"""Worker of tests/test_host_sanitizers.py: drives the native host library (loaded from OXIBONSAI_HOST_LIB, an ASan + UBSan
build) through its codecs, GGUF reader / writer, CPU kernels, tokenizer merges and vocabulary masks."""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np

from oxibonsai_b200.core import GgufFile, Oracle, Qwen3Config, write_synthetic_gguf
from oxibonsai_b200.core import gguf as G
from oxibonsai_b200.core.blocks import dequantize, quantize
from oxibonsai_b200.ops import cpu_ops as CK


def main() -> None:
    rng = np.random.default_rng(0)
    # every block codec, both directions, including a ragged tail of the float side
    for ty in (G.Q1_0_G128, G.TQ2_0_G128, G.TQ2_0, G.Q4_0, G.Q8_0, G.F8_E4M3, G.F8_E5M2, G.Q2_K, G.Q3_K, G.Q4_K, G.Q5_K, G.Q6_K, G.Q8_K):
        w = rng.normal(size=(3, 512)).astype(np.float32)
        q = quantize(ty, w)
        assert dequantize(ty, q).size == w.size
    # GGUF writer -> reader -> oracle forward on a tiny model
    cfg = Qwen3Config(hidden=256, inter=512, layers=1, heads=2, kv_heads=1, head_dim=128, vocab=300, context=64, name="san")
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        write_synthetic_gguf(path, cfg, tied=False, seed=3)
        f = GgufFile.open(path)
        toks, _ = Oracle(f, 32).generate_greedy([1, 2, 3], 4)
        assert len(toks) == 4
        blob = open(path, "rb").read()
        GgufFile.parse(blob)
        for cut in (10, 100, len(blob) // 2):       # truncated files must be refused, not read past their end
            try:
                GgufFile.parse(blob[:cut])
            except Exception:
                pass
    # CPU tiers, tiled and adaptive products, packing
    for ty in (G.TQ2_0_G128, G.Q1_0_G128, G.F8_E4M3):
        rows, cols = 77, 384
        q = quantize(ty, rng.normal(size=(rows, cols)).astype(np.float32) * 0.05)
        x = rng.normal(size=cols).astype(np.float32)
        for tier in (0, 1, 2):
            CK.gemv(ty, q, rows, cols, x, tier, threads=2)
        CK.gemv_tiled(ty, q, rows, cols, x, tile_rows=5, threads=3)
        CK.gemm_tiled(ty, q, rows, cols, rng.normal(size=(4, cols)).astype(np.float32), tile_rows=9, tile_batch=3, threads=2)
        CK.pack_rows_tiled(ty, q, rows, cols, tile=32)
    CK.rms_norm(rng.normal(size=300).astype(np.float32), np.ones(300, np.float32))
    # tokenizer merges and vocabulary masks
    from oxibonsai_b200.tokenizer import train_bpe
    tok = train_bpe(["the quick brown fox jumps over the lazy dog " * 4, "pack my box with five dozen liquor jugs"], 300)
    ids = tok.encode("the quick dog jumps")
    assert tok.decode(ids) == "the quick dog jumps"
    from oxibonsai_b200.runtime.constrained import DfaConstraint, TokenTable
    table = TokenTable([bytes([b]) for b in range(256)] + [b"true", b"false"])
    c = DfaConstraint.from_regex(table, r"(true|false)+", eos_token=None)
    assert c.allowed_mask().any() and c.advance(256) and c.is_complete()
    print("sanitizer worker ok")


if __name__ == "__main__":
    main()
