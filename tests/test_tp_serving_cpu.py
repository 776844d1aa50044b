"""Tensor-parallel serving protocol on CPU: the leader's scheduler drives a fake engine, a follower rank (gloo) must see
exactly the same engine calls in the same order."""
import json
import os
import socket
import subprocess
import sys


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_follower_executes_the_leaders_engine_calls_in_order(tmp_path):
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_serving_worker.py")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), worker, str(tmp_path)]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    r0 = json.load(open(tmp_path / "rank0.json"))
    r1 = json.load(open(tmp_path / "rank1.json"))
    assert r0["log"] == r1["log"] and len(r0["log"]) > 20
    assert r1["commands"] == len(r1["log"]) + 4          # the four close_sequence calls are not logged by the fake engine
    assert r0["slots_left"] == 0 and r1["slots_left"] == 0
    assert [len(t) for t in r0["tokens"]] == [12, 5, 30, 3]
    ops = {e[0] for e in r1["log"]}
    assert {"prefix_cache", "begin", "prefill", "finish", "step"} <= ops
