"""Speculative decoding with a draft checkpoint, greedy and sampled (needs a GPU).

    python examples/speculative.py target.gguf draft.gguf
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.runtime import EngineBuilder
from oxibonsai_b200.runtime.speculative import GpuSpeculativeDecoder

target = EngineBuilder().model_path(sys.argv[1]).preset("greedy").max_seq_len(1024).build()
draft = EngineBuilder().model_path(sys.argv[2]).preset("greedy").max_seq_len(1024).build()
decoder = GpuSpeculativeDecoder(target, draft)
prompt = list(range(10, 40))
greedy = decoder.generate(prompt, 64)
print("greedy:", greedy[:16], "...", f"acceptance {decoder.stats.acceptance_rate:.2f}, {decoder.stats.tokens_per_target_pass:.2f} tokens per verify pass")
sampled = decoder.generate(prompt, 64, temperature=0.8, seed=1)
print("sampled:", sampled[:16], "...", f"acceptance {decoder.stats.acceptance_rate:.2f}")
