"""One process of the elastic serving test (CPU, gloo): the leader runs the real scheduler over a leader engine and an
``ElasticBackend``; uid 2 exits in the middle of the first batch of requests.  Usage: <uid> <world> <port> <out dir>."""
import json
import os
import sys
import threading
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.runtime.elastic import ElasticGroup, RankLost  # noqa: E402
from oxibonsai_b200.runtime.presets import SamplingParams  # noqa: E402
from oxibonsai_b200.runtime.scheduler import BatchScheduler  # noqa: E402
from oxibonsai_b200.runtime.tp_serving import CommandChannel, ElasticBackend, Unavailable, lead_with_scheduler, run_elastic_rank  # noqa: E402

uid, world, port, out = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
builds: list = []


class Engine:
    """The scheduler's engine interface; a decode step is an all-reduce over the generation's ranks."""
    max_batch, max_seq_len, prefill_min_tokens, exact = 4, 4096, 16, True

    def __init__(self, group, rank, size):
        self.group, self.rank, self.size, self.steps = group, rank, size, 0
        builds.append([group.generation, rank, size])

    def bind_thread(self):
        pass

    def begin_sequence(self, prompt, max_total, slot, params=None):
        return 0

    def prefill(self, part, slot, pos0):
        pass

    def finish_sequence(self, prompt, slot):
        return 1

    def step_batch(self, positions):
        t = torch.ones(1)
        dist.all_reduce(t)
        self.steps += 1
        if self.group.uid == 2 and self.group.generation == 0 and self.steps == 6:
            json.dump({"left": True, "builds": builds}, open(os.path.join(out, f"uid{uid}.json"), "w"))
            os._exit(0)
        time.sleep(0.01)
        return [int(t.item())] * len(positions)          # the token is the number of ranks that took part in the step

    def move_slot(self, src, dst):
        pass

    def close_sequence(self, slot=0):
        pass

    def kv_utilization(self):
        return 0.0


store = dist.TCPStore("127.0.0.1", port, is_master=(uid == 0), wait_for_workers=False)
group = ElasticGroup(store, uid, world, backend="gloo", interval=0.05, timeout=0.6, pg_timeout=5.0)
backend = ElasticBackend("fake", 4096)
stop = threading.Event()
record: dict = {"first": [], "retry": [], "unavailable": 0}


def fatal(e: Exception) -> bool:
    return isinstance(e, RankLost) or group.confirm_loss()


def make_scheduler(le, g):
    return BatchScheduler(le, eos_token=-1, before_launch=g.check, on_fatal=fatal, idle_hook=le.keepalive, idle_hook_seconds=0.2)


def client():
    """What the HTTP front does: submit, wait; a request that fails or is refused while the group re-forms is retried."""
    while backend.s is None:
        time.sleep(0.01)
    reqs = [backend.submit([1, 2, 3], SamplingParams(), 12, None, f"r{i}") for i in range(3)]
    for r in reqs:
        r.done.wait(30)
        record["first"].append({"tokens": list(r.tokens), "error": None if r.error is None else type(r.error).__name__})
    deadline = time.monotonic() + 30
    while time.monotonic() < deadline:
        try:
            r = backend.submit([4, 5], SamplingParams(), 8, None, "retry")
        except Unavailable:
            record["unavailable"] += 1
            time.sleep(0.05)
            continue
        r.done.wait(30)
        if r.error is None:
            record["retry"] = list(r.tokens)
            break
        time.sleep(0.05)
    time.sleep(0.5)                                    # an idle stretch: the keep-alive must hold the followers' receive open
    stop.set()


def lead(le, g):
    inner = lead_with_scheduler(make_scheduler, backend, stop)
    try:
        inner(le, g)
    except Exception as e:  # noqa: BLE001
        if isinstance(e, RankLost) or g.confirm_loss(0.0):
            raise RankLost(g.lost(), g.generation) from e
        raise


if uid == 0:
    threading.Thread(target=client, daemon=True).start()
history = run_elastic_rank(group, lambda r, n: Engine(group, r, n), lambda: CommandChannel(dist.new_group(backend="gloo")), lead)
json.dump({"left": False, "builds": builds, "history": history, "record": record, "generations": backend.generations},
          open(os.path.join(out, f"uid{uid}.json"), "w"))
