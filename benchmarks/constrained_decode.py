"""Decode throughput with and without a grammar constraint on one GPU.

    python benchmarks/constrained_decode.py [--model 4b] [--tokens 256]

A synthetic checkpoint of the chosen shape (vocabulary 151 936) decodes one stream three ways: free, under a JSON-schema
constraint (an array of at least 24 {name, score} objects: a long output whatever the random weights prefer) and under the free-form
JSON constraint.  The vocabulary is 256 byte tokens plus random 2-8 character tokens, as in ``benchmarks/grammar_mask.py``.
Before every step the constraint's allowed-token mask (19 KB) is computed on the host and uploaded; the sampler kernel
applies it.  The second constrained run of each kind starts with the masks of the first in the grammar's cache, which is
the steady state of a server that sees the same schema again.  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SHAPES = {
    "1.7b": dict(hidden=2048, inter=6144, layers=28, heads=16, kv_heads=8, head_dim=128, vocab=151936, name="Ternary-Bonsai-1.7B-shaped"),
    "4b": dict(hidden=2560, inter=9728, layers=36, heads=32, kv_heads=8, head_dim=128, vocab=151936, name="Ternary-Bonsai-4B-shaped"),
    "8b": dict(hidden=4096, inter=12288, layers=36, heads=32, kv_heads=8, head_dim=128, vocab=151936, name="Ternary-Bonsai-8B-shaped"),
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="4b", choices=list(SHAPES))
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--model-dir", default=os.environ.get("BONSAI_BENCH_DIR", "/tmp/oxibonsai_b200_bench"))
    a = ap.parse_args()
    import torch
    from oxibonsai_b200.core import Qwen3Config, write_synthetic_gguf
    from oxibonsai_b200.runtime import EngineBuilder
    from oxibonsai_b200.runtime.constrained import TokenTable, json_constraint, json_schema_constraint
    from oxibonsai_b200.runtime.presets import SamplingParams
    os.makedirs(a.model_dir, exist_ok=True)
    path = os.path.join(a.model_dir, f"{a.model}_tq2_seed42.gguf")
    if not os.path.exists(path):
        write_synthetic_gguf(path + ".tmp", Qwen3Config(context=65536, **SHAPES[a.model]), tied=a.model != "8b", seed=42)
        os.replace(path + ".tmp", path)
    rng = random.Random(0)
    alphabet = 'abcdefghijklmnopqrstuvwxyz ABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789{}[]":,.-_\n'
    vocab = SHAPES[a.model]["vocab"]
    table = TokenTable([bytes([b]) for b in range(256)] + ["".join(rng.choice(alphabet) for _ in range(rng.randint(2, 8))).encode() for _ in range(vocab - 256)])
    sp = SamplingParams(temperature=0.7, top_k=40, top_p=0.9, seed=7)
    eng = EngineBuilder().model_path(path).sampler(sp).max_seq_len(1024).build()
    prompt = list(range(300, 332))
    schema = {"type": "array", "items": {"type": "object", "required": ["name", "score"], "properties": {"name": {"type": "string"}, "score": {"type": "integer"}}},
              "minItems": 24}

    def run(constraint) -> dict:
        torch.cuda.synchronize()
        t = time.perf_counter()
        toks = eng.generate(prompt, a.tokens, sp, stop_at_eos=False, constraint=constraint)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t
        st = eng.last_stats
        out = {"tokens": len(toks), "decode_tok_s": round(st.generated_tokens / st.decode_seconds, 1) if st.decode_seconds else None, "wall_s": round(dt, 3)}
        if constraint is not None:
            text = b"".join(table.tokens[t] for t in toks)
            out["mask_cache_hits"] = int(constraint.cache_hits)
            out["output_is_a_prefix_of_the_language"] = bool(constraint.rec.__class__(constraint.rec.compiled).feed_bytes(text))
        return out

    run(None)                                                     # warm-up: graph capture
    res = {"model": SHAPES[a.model]["name"], "vocab": vocab, "max_tokens": a.tokens, "sampling": "T 0.7, top-k 40, top-p 0.9",
           "free": run(None),
           "json_schema_first": run(json_schema_constraint(table, schema)), "json_schema_again": run(json_schema_constraint(table, schema)),
           "json_object_first": run(json_constraint(table)), "json_object_again": run(json_constraint(table))}
    print(json.dumps(res))
    return 0


if __name__ == "__main__":
    sys.exit(main())
