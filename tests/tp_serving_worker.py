"""Worker of tests/test_tp_serving_cpu.py: two gloo ranks, rank 0 schedules requests on a fake engine through LeaderEngine,
rank 1 follows.  Each rank writes the calls its engine received to <out_dir>/rank<r>.json."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch.distributed as dist

from oxibonsai_b200.runtime.presets import SamplingParams
from oxibonsai_b200.runtime.scheduler import BatchScheduler
from oxibonsai_b200.runtime.tp_serving import CommandChannel, LeaderEngine, follower_loop
from test_scheduler_cpu import FakeEngine


def main(out_dir: str) -> None:
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    eng = FakeEngine()
    eng.enable_prefix_cache = lambda: eng.log.append(("prefix_cache",))
    ch = CommandChannel(dist.new_group(backend="gloo"))
    result = {}
    if rank == 0:
        lead = LeaderEngine(eng, ch)
        lead.enable_prefix_cache()
        sched = BatchScheduler(lead, eos_token=-1, prefill_chunk_tokens=32).start()
        reqs = [sched.submit([i + 1] * n, SamplingParams(), m) for i, (n, m) in enumerate([(20, 12), (100, 5), (40, 30), (17, 3)])]
        result["tokens"] = [r.wait(30) for r in reqs]
        sched.stop()
        lead.shutdown()
    else:
        result["commands"] = follower_loop(eng, ch)
    result["log"] = [list(e) for e in eng.log]
    result["slots_left"] = len(eng.slots)
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(result, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
