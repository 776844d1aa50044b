"""Watchdog and re-formation of a tensor-parallel group: failures are host events (a rank that stops beating or exits
between steps), the ranks are threads over an in-memory store or gloo processes on CPU."""
import json
import os
import socket
import subprocess
import sys
import threading
import time

import pytest

from oxibonsai_b200.runtime.elastic import ElasticGroup, RankLost, shrink_world


def test_shrink_world():
    assert [shrink_world(n) for n in (8, 7, 5, 4, 3, 2, 1)] == [8, 4, 4, 4, 2, 2, 1]
    assert shrink_world(6, supported=(6, 3, 1)) == 6
    with pytest.raises(ValueError):
        shrink_world(0)


def _thread_groups(n, **kw):
    import torch.distributed as dist
    store = dist.HashStore()
    events = []
    groups = [ElasticGroup(store, u, n, interval=0.02, timeout=0.25, settle=1.0, monitor_store=store,
                           init_group=lambda s, r, w, u=u: events.append(("init", u, r, w)), destroy_group=lambda u=u: events.append(("destroy", u)), **kw)
              for u in range(n)]
    for g in groups:
        g.start()
    return groups, events


def test_watchdog_flags_a_silent_rank_and_the_survivors_reform():
    groups, events = _thread_groups(4)
    time.sleep(0.15)
    for g in groups:
        g.check()                                         # everyone beats: nothing to report
    groups[2].close()                                     # uid 2 stops beating (no farewell)
    deadline = time.monotonic() + 5
    while time.monotonic() < deadline:
        try:
            groups[0].check()
            time.sleep(0.02)
        except RankLost as e:
            assert e.lost == [2] or e.lost == []          # seen directly, or through a peer's announcement
            break
    else:
        pytest.fail("the lost rank was never reported")
    results = {}
    ts = [threading.Thread(target=lambda u=u: results.__setitem__(u, groups[u].rebuild())) for u in (0, 1, 3)]
    [t.start() for t in ts]
    [t.join(20) for t in ts]
    assert results == {0: (0, 2), 1: (1, 2), 3: (None, 2)}     # 3 survivors fill degree 2; the third is a spare
    assert groups[0].members == [0, 1] and groups[0].spares == [3] and groups[3].rank is None
    assert groups[0].history[0]["lost"] == [2] and groups[0].generation == 1
    assert ("init", 0, 0, 2) in events and ("init", 1, 1, 2) in events and ("destroy", 0) in events
    assert not any(e[:2] == ("init", 3) and e[3] == 2 for e in events)
    time.sleep(0.1)
    for u in (0, 1, 3):
        groups[u].check()
    # second loss: an active rank goes, the spare is promoted and takes its place
    groups[1].close()
    assert groups[0].confirm_loss(5.0) and groups[3].confirm_loss(5.0)
    ts = [threading.Thread(target=lambda u=u: results.__setitem__(u, groups[u].rebuild())) for u in (0, 3)]
    [t.start() for t in ts]
    [t.join(20) for t in ts]
    assert results[0] == (0, 2) and results[3] == (1, 2) and groups[0].members == [0, 3] and groups[0].spares == []
    for u in (0, 3):
        groups[u].close(shutdown=True)


def test_a_follower_that_leaves_the_generation_makes_the_others_leave_too():
    groups, _ = _thread_groups(2)
    time.sleep(0.1)
    # uid 1 suspects something (say, a failed collective) and announces itself for generation 1; the leader must follow
    t = threading.Thread(target=groups[1].rebuild)
    t.start()
    assert groups[0].confirm_loss(5.0)
    with pytest.raises(RankLost):
        groups[0].check()
    assert groups[0].rebuild() == (0, 2)                      # nobody was lost: the same two ranks form generation 1
    t.join(10)
    assert groups[1].rank == 1 and groups[1].generation == 1 and groups[0].history[0]["lost"] == []
    for g in groups:
        g.close(shutdown=True)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_gloo_ranks_lose_two_members_and_keep_serving(tmp_path):
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "elastic_worker.py")
    port = _free_port()
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    procs = [subprocess.Popen([sys.executable, worker, str(u), "4", str(port), str(tmp_path)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for u in range(4)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=180)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0])
    assert all(p.returncode == 0 for p in procs), "\n----\n".join(o[-1500:] for o in outs)
    r = {u: json.load(open(tmp_path / f"uid{u}.json")) for u in range(4)}
    assert r[3]["left"] and r[1]["left"] and not r[0]["left"] and not r[2]["left"]
    steps0 = [e for e in r[0]["log"] if e[0] == "step"]
    assert len(steps0) == 16 + 0 and [e[3] for e in steps0] == [[i, i + 1] for i in range(16)]     # no step lost, none repeated by the leader
    by_gen = {}
    for e in steps0:
        by_gen.setdefault(e[1], set()).add((e[2], e[4]))
    # generation 0: four ranks (1+2+3+4); generation 1: uids 0, 1 (1+2), uid 2 spare; generation 2: uids 0, 2 (1+3)
    assert by_gen == {0: {(4, 10.0)}, 1: {(2, 3.0)}, 2: {(2, 4.0)}}
    assert [h["lost"] for h in r[0]["history"]] == [[3], [1]] and r[0]["members"] == [0, 2] and r[0]["spares"] == []
    builds2 = [e for e in r[2]["log"] if e[0] == "build"]
    assert builds2 == [["build", 0, 2, 4], ["build", 2, 1, 2]]                                   # parked as a spare during generation 1
    assert all(h["seconds"] < 30 for h in r[0]["history"])


def test_scheduler_behind_an_elastic_backend_survives_a_lost_follower(tmp_path):
    """The serving path: real scheduler + leader engine + ``ElasticBackend`` on the leader, followers mirroring its commands.
    A follower exits in the middle of the first requests: those fail (the client sees an error, not a hang), the group
    re-forms at degree 2, the retried request is served by two ranks."""
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "elastic_sched_worker.py")
    port = _free_port()
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    procs = [subprocess.Popen([sys.executable, worker, str(u), "3", str(port), str(tmp_path)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for u in range(3)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=180)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0])
    assert all(p.returncode == 0 for p in procs), "\n----\n".join(o[-1500:] for o in outs)
    r = {u: json.load(open(tmp_path / f"uid{u}.json")) for u in range(3)}
    assert r[2]["left"] and not r[0]["left"] and not r[1]["left"]
    rec = r[0]["record"]
    assert len(rec["first"]) == 3 and all(f["error"] == "RankLost" for f in rec["first"])            # in flight when the rank went: failed, not hung
    assert all(set(f["tokens"]) <= {1, 3} for f in rec["first"])                                     # what they got before came from three ranks
    assert rec["retry"] and set(rec["retry"][1:]) == {2} and len(rec["retry"]) == 8                  # served by the two survivors
    assert r[0]["generations"] == 2 and [h["lost"] for h in r[0]["history"]] == [[2]]
    assert r[0]["builds"] == [[0, 0, 3], [1, 0, 2]] and r[1]["builds"] == [[0, 1, 3], [1, 1, 2]]
