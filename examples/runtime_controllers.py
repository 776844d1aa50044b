"""The adaptive controllers in isolation: speculative lookahead and KV cache policy (reference: examples/runtime_controllers.rs)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.runtime.kv_policy import KvCachePolicy
from oxibonsai_b200.runtime.speculative import AdaptiveLookahead

la = AdaptiveLookahead()
for accepted in [5, 5, 4, 1, 0, 0, 1, 3, 6, 6, 6]:
    print(f"accepted {accepted} -> next lookahead {la.record(accepted)}")
pol = KvCachePolicy()
for pressure in [0.2, 0.9, 0.99, 0.5, 0.2]:
    for _ in range(12):                      # the policy smooths pressure (EWMA) and applies hysteresis
        level = pol.observe(pressure)
    print(f"kv pressure held at {pressure:.2f} -> level {level.name}")
