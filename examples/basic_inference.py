"""Load a GGUF checkpoint and generate (reference example: examples/basic_inference.rs).

    python examples/basic_inference.py model.gguf "Hello" [--tokenizer tokenizer.json]
Without a model path a tiny random-init checkpoint is written to a temporary file and used instead.
"""
import argparse
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.core import Qwen3Config, write_synthetic_gguf
from oxibonsai_b200.runtime import EngineBuilder
from oxibonsai_b200.tokenizer import load_tokenizer

ap = argparse.ArgumentParser()
ap.add_argument("model", nargs="?")
ap.add_argument("prompt", nargs="?", default="Hello")
ap.add_argument("--tokenizer")
ap.add_argument("--max-tokens", type=int, default=32)
a = ap.parse_args()
path = a.model
if path is None:
    path = os.path.join(tempfile.mkdtemp(), "tiny.gguf")
    write_synthetic_gguf(path, Qwen3Config(hidden=256, inter=512, layers=2, heads=4, kv_heads=2, head_dim=64, vocab=1000, context=512, name="tiny"))
tok = load_tokenizer(a.tokenizer)
engine = EngineBuilder().model_path(path).preset("greedy").max_seq_len(512).build()
ids = [t % engine.config.vocab for t in tok.encode(a.prompt)]
out = engine.generate(ids, a.max_tokens, stop_at_eos=False)
print("prompt ids:", ids)
print("generated :", out)
print(f"{engine.last_stats.decode_tokens_per_second:.1f} tok/s decode, prefill {engine.last_stats.prefill_seconds * 1e3:.1f} ms")
