"""Watchdog and re-formation of a tensor-parallel group after a rank is lost.

The reference has no multi-process group to lose; its failure handling is the circuit breaker and the retry / time-out
helpers of one process (crates/oxibonsai-runtime/src/circuit_breaker.rs:109-246, recovery.rs:12-199, health.rs:10-245), and
its tensor-parallel plan is a pure description of shards (crates/oxibonsai-model/src/tensor_parallel.rs:405-468).  With one
process per GPU a rank can go away, and the kernels of the others would then wait for a peer that never writes (their waits
are bounded and report through a status word, but the step is lost).  This module keeps that from happening silently and
brings the service back at a smaller tensor-parallel degree:

* every process beats a counter into the job's key-value store (``torch.distributed`` ``TCPStore``, held by rank 0); a
  monitor thread watches the peers' counters against its own monotonic clock and the store's ``generation`` key;
* ``ElasticGroup.check()`` is what an engine owner calls before every launch: it raises :class:`RankLost` as soon as a
  peer has been silent for ``timeout`` seconds or the leader has opened a new generation, so no kernel that would wait
  for the lost peer is launched;
* ``ElasticGroup.rebuild()`` tears the process group down, lets the survivors announce themselves, has the leader (the
  process that holds the store) fix the member list - the largest supported tensor-parallel degree that the survivors can
  fill, the rest become spares that later generations can promote - and initialises a fresh process group under a
  store prefix of its own.  The caller then rebuilds its engine for ``(group.rank, group.world)``: the weight shards
  come from the memory-mapped GGUF (or the re-layout cache of that degree) again, nothing of the old group's device
  state is reused.

The store lives in the first process; losing that one ends the job (it is also the one that fronts HTTP).  Failures are
host events here - a process that exits or stops beating between steps - never a faulting kernel.
"""
from __future__ import annotations

import json
import threading
import time
from datetime import timedelta
from typing import Callable, Sequence

SUPPORTED_DEGREES = (8, 4, 2, 1)


class RankLost(RuntimeError):
    """A member of the current generation is gone (or the leader has already opened the next generation)."""

    def __init__(self, lost: Sequence[int], generation: int):
        super().__init__(f"rank(s) {sorted(lost)} lost in generation {generation}" if lost else f"generation {generation} was closed by the leader")
        self.lost, self.generation = sorted(lost), generation


class Evicted(RuntimeError):
    """This process announced itself too late for the new generation (the leader had already fixed the member list)."""


def _second_client(store):
    try:
        from torch.distributed import TCPStore
        if isinstance(store, TCPStore):
            return TCPStore(store.host, store.port, is_master=False, wait_for_workers=False, timeout=timedelta(seconds=30))
    except Exception:  # noqa: BLE001 - fall back to sharing the handle
        pass
    return store


def shrink_world(alive: int, supported: Sequence[int] = SUPPORTED_DEGREES) -> int:
    """Largest supported tensor-parallel degree that ``alive`` processes can fill."""
    fits = [d for d in supported if d <= alive]
    if not fits:
        raise ValueError(f"no supported degree fits {alive} processes")
    return max(fits)


class ElasticGroup:
    """Membership of one process in a group that can lose ranks and re-form.

    ``uid`` is the process's rank at start-up and never changes; ``rank`` / ``world`` are its position in the current
    generation (``rank`` is None for a spare).  ``init_group(store, rank, world)`` / ``destroy_group()`` create and drop the
    communication group of a generation; the defaults use ``torch.distributed`` with ``backend``."""

    def __init__(self, store, uid: int, world: int, *, backend: str = "gloo", supported: Sequence[int] = SUPPORTED_DEGREES,
                 interval: float = 0.1, timeout: float = 1.0, settle: float | None = None, pg_timeout: float = 30.0,
                 init_group: Callable | None = None, destroy_group: Callable | None = None, clock: Callable[[], float] = time.monotonic,
                 monitor_store=None):
        """``monitor_store``: the store handle of the monitor thread.  By default a second client connection is opened when
        ``store`` is a ``TCPStore``: a client serialises its operations, and the rendezvous of a new process group blocks
        inside the store for as long as the slowest peer needs - the heartbeat must not wait behind that."""
        self.store, self.uid, self.backend = store, int(uid), backend
        self._mstore = monitor_store if monitor_store is not None else _second_client(store)
        self.supported = tuple(sorted(supported, reverse=True))
        self.interval, self.timeout = float(interval), float(timeout)
        self.settle = 3.0 * self.timeout if settle is None else float(settle)
        self.pg_timeout = float(pg_timeout)
        self._init_group, self._destroy_group = init_group or self._default_init, destroy_group or self._default_destroy
        self._clock = clock
        self.generation = 0
        self.members: list[int] = list(range(world))        # uids of the active ranks, index = rank in the group
        self.spares: list[int] = []
        self.history: list[dict] = []                       # one record per re-formation
        self._lock = threading.Lock()
        self._lost: set[int] = set()
        self._newer = False                                 # the store's generation is ahead of ours
        self._seen: dict[int, tuple[str, float]] = {}       # uid -> (last counter value, local time it changed)
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._beats = 0
        self._store_error: Exception | None = None
        self._group_live = False

    # ---- position ----------------------------------------------------------------------------------
    @property
    def rank(self) -> int | None:
        return self.members.index(self.uid) if self.uid in self.members else None

    @property
    def world(self) -> int:
        return len(self.members)

    @property
    def is_leader(self) -> bool:
        return self.uid == 0

    # ---- life cycle --------------------------------------------------------------------------------
    def start(self) -> "ElasticGroup":
        """Forms generation 0 (every start-up rank is a member) and starts beating."""
        if self.is_leader:
            self.store.add("elastic/generation", 0)
        self._beat()
        self._reset_watch()
        self._thread = threading.Thread(target=self._monitor, name="bonsai-elastic", daemon=True)
        self._thread.start()
        if self.rank is not None:
            self._init_group(self._prefix(0), self.rank, self.world)
            self._group_live = True
        return self

    def close(self, shutdown: bool = False) -> None:
        """Stops beating and drops the group.  ``shutdown``: (leader) tells spares and followers that the job is over."""
        if shutdown and self.is_leader:
            try:
                self.store.set("elastic/shutdown", "1")
            except Exception:  # noqa: BLE001 - the store may be gone already
                pass
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
            self._thread = None
        self._drop_group()

    # ---- watchdog ----------------------------------------------------------------------------------
    def check(self) -> None:
        """Call before every launch that needs the peers.  Costs a lock and two reads; the store is read by the monitor
        thread, not here."""
        with self._lock:
            if self._store_error is not None:
                raise RuntimeError(f"key-value store unreachable: {self._store_error}")
            if self._lost or self._newer:
                raise RankLost(self._lost, self.generation)

    def lost(self) -> list[int]:
        with self._lock:
            return sorted(self._lost)

    def confirm_loss(self, wait: float | None = None) -> bool:
        """After a collective failed: waits up to ``wait`` seconds (default 2 x timeout) for the monitor to attribute it to
        a lost rank or a new generation.  True: rebuild; False: the failure has another cause."""
        deadline = self._clock() + (2.0 * self.timeout if wait is None else wait)
        while True:
            with self._lock:
                if self._lost or self._newer:
                    return True
            if self._clock() >= deadline:
                return False
            time.sleep(self.interval / 2)

    def wait_for_change(self, poll: float | None = None) -> str:
        """Blocks a spare until something concerns it: "rebuild" (a rank was lost or a generation opened) or "shutdown"."""
        while True:
            if self.shutdown_requested():
                return "shutdown"
            with self._lock:
                if self._lost or self._newer:
                    return "rebuild"
                if self._store_error is not None:
                    return "shutdown"
            time.sleep(self.interval if poll is None else poll)

    def shutdown_requested(self) -> bool:
        try:
            return bool(self.store.check(["elastic/shutdown"]))
        except Exception:  # noqa: BLE001
            return True

    def _beat(self) -> None:
        self._beats += 1
        self._mstore.set(f"elastic/hb/{self.uid}", str(self._beats))

    def _reset_watch(self) -> None:
        now = self._clock()
        with self._lock:
            self._lost.clear()
            self._newer = False
            # the last counter value of a known peer is kept (a peer that died during the re-formation is still caught);
            # a peer that has never been seen (value "") is not timed out: the rendezvous of the group waits for it
            self._seen = {u: (self._seen.get(u, ("", now))[0], now) for u in self.members + self.spares if u != self.uid}

    def _monitor(self) -> None:
        while not self._stop.wait(self.interval):
            try:
                self._beat()
                st = self._mstore
                gen = int(st.add("elastic/generation", 0))
                now = self._clock()
                with self._lock:
                    watched, nxt = list(self._seen), self.generation + 1
                fresh = {}
                left = False          # a peer has announced itself for the next generation: this one is broken whoever is right
                for u in watched:
                    key = f"elastic/hb/{u}"
                    fresh[u] = st.get(key).decode() if st.check([key]) else ""
                    left = left or bool(st.check([f"elastic/gen{nxt}/ready/{u}"]))
                with self._lock:
                    if nxt != self.generation + 1:
                        continue                          # a rebuild finished while the store was being read
                    if gen > self.generation or left:
                        self._newer = True
                    for u, value in fresh.items():
                        if u not in self._seen:
                            continue
                        last, since = self._seen[u]
                        if value != last:
                            self._seen[u] = (value, now)
                        elif last and now - since > self.timeout and u in self.members:
                            self._lost.add(u)
            except Exception as e:  # noqa: BLE001 - the store went away with the leader
                with self._lock:
                    self._store_error = e
                return

    # ---- re-formation ------------------------------------------------------------------------------
    def rebuild(self) -> tuple[int | None, int]:
        """Closes the current generation and joins the next one.  Returns ``(rank, world)``; rank None = spare."""
        g = self.generation + 1
        t0 = self._clock()
        self._drop_group()
        self.store.set(f"elastic/gen{g}/ready/{self.uid}", "1")
        key = f"elastic/gen{g}/members"
        if self.is_leader:
            if int(self.store.add("elastic/generation", 0)) < g:
                self.store.add("elastic/generation", 1)          # followers that have not noticed learn it from this
            with self._lock:
                believed = [u for u in self.members + self.spares if u not in self._lost]
            deadline = self._clock() + self.settle
            while True:
                ready = [u for u in self.members + self.spares if self.store.check([f"elastic/gen{g}/ready/{u}"])]
                if set(believed) <= set(ready) or self._clock() >= deadline:
                    break
                time.sleep(self.interval / 2)
            n = shrink_world(len(ready), self.supported)
            # survivors keep their order; old members come before promoted spares, so shards move as little as they can
            order = [u for u in self.members if u in ready] + [u for u in self.spares if u in ready]
            self.store.set(key, json.dumps({"active": order[:n], "spare": order[n:]}))
        deadline = self._clock() + self.settle + 4.0 * self.timeout + 5.0
        while not self.store.check([key]):
            if self._clock() >= deadline:
                raise TimeoutError(f"generation {g}: the leader published no member list")
            time.sleep(self.interval / 2)
        plan = json.loads(self.store.get(key).decode())
        if self.uid not in plan["active"] and self.uid not in plan["spare"]:
            raise Evicted(f"uid {self.uid} is not part of generation {g}")
        lost = sorted(set(self.members + self.spares) - set(plan["active"]) - set(plan["spare"]))
        self.members, self.spares, self.generation = list(plan["active"]), list(plan["spare"]), g
        self._reset_watch()
        if self.rank is not None:
            self._init_group(self._prefix(g), self.rank, self.world)
            self._group_live = True
        self.history.append({"generation": g, "lost": lost, "world": self.world, "rank": self.rank, "spares": list(self.spares),
                             "seconds": self._clock() - t0})
        return self.rank, self.world

    def run(self, serve: Callable[["ElasticGroup"], None]) -> None:
        """``serve(group)`` runs one generation: it builds what it needs for ``(group.rank, group.world)``, works until
        the job ends (returns) or a rank is lost (raises :class:`RankLost`, after releasing what it built).  Spares
        (``group.rank is None``) are parked here until a later generation promotes them."""
        while True:
            if self.rank is None:
                if self.wait_for_change() == "shutdown":
                    return
            else:
                try:
                    serve(self)
                    return
                except RankLost:
                    pass
            self.rebuild()

    # ---- communication group of a generation ---------------------------------------------------------
    def _prefix(self, g: int):
        from torch.distributed import PrefixStore
        return PrefixStore(f"elastic/pg{g}", self.store)

    def _default_init(self, store, rank: int, world: int) -> None:
        import torch.distributed as dist
        dist.init_process_group(self.backend, store=store, rank=rank, world_size=world, timeout=timedelta(seconds=self.pg_timeout))

    def _default_destroy(self) -> None:
        import torch.distributed as dist
        if dist.is_initialized():
            if self.backend == "nccl" and hasattr(dist.distributed_c10d, "_abort_process_group"):
                dist.distributed_c10d._abort_process_group()      # a communicator with a dead peer cannot be drained
            else:
                dist.destroy_process_group()

    def _drop_group(self) -> None:
        if self._group_live:
            self._group_live = False
            try:
                self._destroy_group()
            except Exception:  # noqa: BLE001 - half of the group is gone; what matters is that the handle is dropped
                pass
