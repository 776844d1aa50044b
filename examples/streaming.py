"""Token streaming with UTF-8-safe incremental decoding (reference example: examples/streaming.rs)."""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.core import Qwen3Config, write_synthetic_gguf
from oxibonsai_b200.runtime import EngineBuilder
from oxibonsai_b200.tokenizer import ByteTokenizer, StreamingDecoder

path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(tempfile.mkdtemp(), "tiny.gguf")
if not os.path.exists(path):
    write_synthetic_gguf(path, Qwen3Config(hidden=256, inter=512, layers=2, heads=4, kv_heads=2, head_dim=64, vocab=256, context=512, name="tiny"))
tok, dec = ByteTokenizer(), StreamingDecoder()
engine = EngineBuilder().model_path(path).preset("creative").seed(7).max_seq_len(512).build()
for t in engine.generate_stream(tok.encode("stream: "), 48, stop_at_eos=False):
    sys.stdout.write(dec.push(tok.token_bytes(t)))
    sys.stdout.flush()
print(dec.flush())
