"""Sampler presets, a custom sampler chain, and a grammar-constrained generation (reference: examples/custom_sampling.rs)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np

from oxibonsai_b200.runtime.constrained import DfaConstraint, TokenTable
from oxibonsai_b200.runtime.pipeline import PipelineBuilder
from oxibonsai_b200.runtime.presets import SamplingPreset
from oxibonsai_b200.runtime.sampling_advanced import MirostatV2, LcgRng, SamplerChain

for p in SamplingPreset:
    print(f"{p.name:<15} {p.params()}")
rng = np.random.default_rng(0)
logits_fn = lambda toks: rng.normal(size=256) * 2            # a stand-in model over a byte vocabulary
chain = SamplerChain(seed=1).add("repetition_penalty", 1.2).add("temperature", 0.8).add("min_p", 0.05).add("typical", 0.9)
print("chain   :", [chain.sample(logits_fn([])) for _ in range(8)])
m = MirostatV2(tau=3.0)
print("mirostat:", [m.sample(logits_fn([]), LcgRng(2)) for _ in range(8)], "mu", round(m.mu, 2))
table = TokenTable([bytes([b]) for b in range(256)])
pipe = PipelineBuilder().max_tokens(12).with_sampling(SamplerChain(3).add("temperature", 1.0)).with_constraint(
    DfaConstraint.from_regex(table, r"[A-Z][a-z]+ [0-9]{2,4}", eos_token=0)).eos(0).build()
out = pipe.run([65], logits_fn, lambda t: bytes(t).decode("latin1"), vocab_size=256)
print("regex-constrained text:", repr(out.text), out.stop_reason.value)
