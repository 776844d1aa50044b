"""One process of the elastic tensor-parallel test (CPU, gloo).  Usage: elastic_worker.py <uid> <world> <port> <out dir>.

The fake engine's decode step is an all-reduce over the generation's process group: it only completes while every member
of the generation is there, like the tensor-parallel kernels.  uid 3 leaves between steps in generation 0, uid 1 in
generation 1 (both with ``os._exit``: no farewell, as a crashed process)."""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.runtime.elastic import ElasticGroup  # noqa: E402
from oxibonsai_b200.runtime.tp_serving import CommandChannel, run_elastic_rank  # noqa: E402

uid, world, port, out = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
LEAVE = {3: (0, 4), 1: (1, 3)}            # uid -> (generation, after this many steps of that generation)
TOTAL_STEPS = 16
log: list = []
done_steps = 0


class FakeEngine:
    def __init__(self, group, rank, size):
        self.group, self.rank, self.size, self.steps = group, rank, size, 0
        log.append(["build", group.generation, rank, size])

    def bind_thread(self):
        pass

    def step_batch(self, positions):
        t = torch.tensor([float(self.group.uid + 1)])
        dist.all_reduce(t)
        self.steps += 1
        log.append(["step", self.group.generation, self.size, list(positions), t.item()])
        leave = LEAVE.get(self.group.uid)
        if leave == (self.group.generation, self.steps):
            json.dump({"log": log, "left": True}, open(os.path.join(out, f"uid{uid}.json"), "w"))
            os._exit(0)
        return [0] * len(positions)

    def close(self):
        log.append(["close", self.group.generation])


def lead(le, group):
    global done_steps
    while done_steps < TOTAL_STEPS:
        le.step_batch([done_steps, done_steps + 1])
        done_steps += 1
        time.sleep(0.05)


store = dist.TCPStore("127.0.0.1", port, is_master=(uid == 0), wait_for_workers=False)
group = ElasticGroup(store, uid, world, backend="gloo", interval=0.05, timeout=0.6, pg_timeout=5.0)
history = run_elastic_rank(group, lambda r, n: FakeEngine(group, r, n), lambda: CommandChannel(dist.new_group(backend="gloo")), lead)
json.dump({"log": log, "history": history, "left": False, "members": group.members, "spares": group.spares},
          open(os.path.join(out, f"uid{uid}.json"), "w"))
