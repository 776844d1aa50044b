"""Serving one model tensor-parallel over several GPUs: rank 0 decides, every rank executes.

The reference serves from one process and one device (crates/oxibonsai-runtime/src/server.rs:68,203-243).  With one process
per GPU, only rank 0 runs the HTTP front and the continuous-batching scheduler; what the scheduler asks of the engine -
open a sequence, prefill a prompt chunk, take a decode step of B sequences, move or close a slot - is broadcast as a small
command before rank 0 executes it, and every other rank executes the same call on its own engine.  All ranks hold the same
host-side state (page tables, prefix cache, sampler seeds) because they apply the same commands in the same order, so the
tensor-parallel kernels of a step always meet their peers.  Commands travel over a CPU (gloo) process group; a decode
step costs one broadcast of a small tensor holding the live positions, other commands follow as pickled tuples.
"""
from __future__ import annotations

from typing import Any, Callable

MIRRORED = ("begin_sequence", "prefill", "finish_sequence", "step_batch", "move_slot", "close_sequence", "enable_prefix_cache",
            "enable_kv_formats")
SHUTDOWN = "__shutdown__"
NOOP = "__noop__"


class CommandChannel:
    """Broadcast of (op, args) from rank ``src`` over a ``torch.distributed`` group (gloo: CPU tensors and objects).

    Every command starts with one broadcast of a fixed int64 header.  The hot command - a decode step without vocabulary
    masks - travels inside it (``[STEP, B, positions...]``), so a step costs one small tensor broadcast and no pickling;
    any other command announces itself as ``OBJECT`` and follows as a pickled tuple."""

    OBJECT, STEP = 0, 1
    MAX_INLINE = 1022            # positions that fit into the header

    def __init__(self, group=None, src: int = 0):
        import torch
        import torch.distributed as dist
        self._torch, self._dist, self.group, self.src = torch, dist, group, src
        self.rank = dist.get_rank()
        self._hdr = torch.zeros(self.MAX_INLINE + 2, dtype=torch.int64)

    def send(self, op: str, args: tuple = ()) -> None:
        assert self.rank == self.src
        h = self._hdr
        if op == "step_batch" and len(args) == 1 and len(args[0]) <= self.MAX_INLINE:
            pos = args[0]
            h[0], h[1] = self.STEP, len(pos)
            h[2:2 + len(pos)] = self._torch.as_tensor(list(pos), dtype=self._torch.int64)
            self._dist.broadcast(h, src=self.src, group=self.group)
            return
        h[0] = self.OBJECT
        self._dist.broadcast(h, src=self.src, group=self.group)
        self._dist.broadcast_object_list([(op, tuple(args))], src=self.src, group=self.group)

    def recv(self) -> tuple[str, tuple]:
        h = self._hdr
        self._dist.broadcast(h, src=self.src, group=self.group)
        if int(h[0]) == self.STEP:
            return "step_batch", (h[2:2 + int(h[1])].tolist(),)
        box: list[Any] = [None]
        self._dist.broadcast_object_list(box, src=self.src, group=self.group)
        return box[0]


class LeaderEngine:
    """Rank 0's engine as the scheduler sees it: calls that change engine state are announced on the channel first.

    ``group``: an :class:`~oxibonsai_b200.runtime.elastic.ElasticGroup`; its watchdog is asked before every announced call,
    so a call whose kernels would wait for a lost rank is never launched, and a broadcast that fails because a follower is
    gone surfaces as :class:`~oxibonsai_b200.runtime.elastic.RankLost`."""

    supports_overlap = False           # a step is one mirrored command: launch and collect are not split across ranks

    def __init__(self, engine, channel: CommandChannel, group=None):
        self._engine, self._channel, self._group = engine, channel, group

    def __getattr__(self, name: str):
        attr = getattr(self._engine, name)
        if name not in MIRRORED:
            return attr

        def mirrored(*args):
            self._send(name, _plain(args))
            if self._group is None:
                return attr(*args)
            try:
                return attr(*args)
            except (MemoryError, ValueError, KeyError):
                raise                              # refusals of the host-side bookkeeping: the same on every rank
            except Exception as e:  # noqa: BLE001 - a kernel whose bounded wait ran out, a collective that lost its peer
                _attribute(self._group, e)
        return mirrored

    def _send(self, op: str, args: tuple = ()) -> None:
        if self._group is None:
            self._channel.send(op, args)
            return
        self._group.check()
        try:
            self._channel.send(op, args)
        except Exception as e:  # noqa: BLE001 - attributed below
            _attribute(self._group, e)

    def keepalive(self) -> None:
        """An idle leader says so now and then: a follower's pending receive would otherwise run into the process group's
        time-out."""
        self._send(NOOP)

    def shutdown(self) -> None:
        self._channel.send(SHUTDOWN)


def _attribute(group, error: Exception):
    """A failed collective is either the first sign of a lost rank (the watchdog confirms it within its time-out) or
    something else (raised unchanged)."""
    from .elastic import RankLost
    if isinstance(error, RankLost):
        raise error
    if group.confirm_loss():
        raise RankLost(group.lost(), group.generation) from error
    raise error


def _plain(args: tuple) -> tuple:
    """Arguments as plain Python values (lists of ints, dataclasses) so that they pickle small and identically."""
    return tuple(list(a) if isinstance(a, (list, tuple, range)) else a for a in args)


def follower_loop(engine, channel: CommandChannel, on_error: Callable[[str, Exception], None] | None = None, group=None) -> int:
    """Runs on every rank but the leader: executes the announced calls until the leader shuts down.  An exception of a
    call is reported and the loop goes on - the leader's own call raised the same way (same state, same arguments) and its
    scheduler has already dealt with it.  Returns the number of commands executed.

    ``group``: an :class:`~oxibonsai_b200.runtime.elastic.ElasticGroup`.  With it a receive that fails because the leader
    left the generation, and a command that arrives after a peer was lost, raise
    :class:`~oxibonsai_b200.runtime.elastic.RankLost` instead of launching kernels that would wait for the lost rank."""
    n = 0
    engine.bind_thread()
    while True:
        if group is None:
            op, args = channel.recv()
        else:
            try:
                op, args = channel.recv()
            except Exception as e:  # noqa: BLE001 - attributed below
                _attribute(group, e)
            group.check()
        if op == SHUTDOWN:
            return n
        if op == NOOP:
            continue
        n += 1
        try:
            getattr(engine, op)(*args)
        except Exception as e:  # noqa: BLE001 - mirrored on the leader
            if group is not None and not isinstance(e, (MemoryError, ValueError, KeyError)) and group.confirm_loss():
                _attribute(group, e)
            if on_error is not None:
                on_error(op, e)


class Unavailable(RuntimeError):
    """The engine is being rebuilt after a lost rank; the request should be retried."""


class ElasticBackend:
    """What the HTTP front submits to while the tensor-parallel group may re-form underneath it: between generations
    ``submit`` raises :class:`Unavailable` (the server answers 503), otherwise it goes to the current generation's
    scheduler."""

    supports_on_done = True

    def __init__(self, model_name: str, max_seq_len: int):
        self.model_name, self.max_seq_len = model_name, max_seq_len
        self.s = None
        self._after_step = None
        self.generations = 0

    def attach(self, scheduler) -> None:
        scheduler.after_step = self._after_step
        self.s = scheduler
        self.generations += 1

    def set_after_step(self, fn) -> None:
        self._after_step = fn
        if self.s is not None:
            self.s.after_step = fn

    def detach(self) -> None:
        self.s = None

    def submit(self, prompt, params, max_tokens, on_token, request_id, **extra):
        s = self.s
        if s is None:
            raise Unavailable("the tensor-parallel group is re-forming after a lost rank; retry shortly")
        try:
            return s.submit(prompt, params, max_tokens, on_token=on_token, request_id=request_id, **extra)
        except Exception as e:  # noqa: BLE001
            if type(e).__name__ == "SchedulerStopped":      # the generation has just ended; the next one is not attached yet
                raise Unavailable("the tensor-parallel group is re-forming after a lost rank; retry shortly") from e
            raise

    def kv_utilization(self) -> float:
        s = self.s
        return 0.0 if s is None else s.engine.kv_utilization()


def run_elastic_rank(group, build_engine: Callable[[int, int], Any], make_channel: Callable[[], CommandChannel],
                     lead: Callable[[LeaderEngine, Any], None], on_error: Callable[[str, Exception], None] | None = None) -> list[dict]:
    """One process of an elastic tensor-parallel service.  Per generation: ``build_engine(rank, world)`` (shards for that
    degree), a command channel on the generation's process group, then the leader runs ``lead(leader_engine, group)`` -
    which returns when the job is over and raises ``RankLost`` when a rank is lost - and the others follow its commands.
    The engine of a generation is closed before the next one is built.  Returns the group's re-formation records."""
    def serve(g) -> None:
        engine = build_engine(g.rank, g.world)
        try:
            channel = make_channel()
            if g.rank == 0:
                le = LeaderEngine(engine, channel, g)
                lead(le, g)
                try:
                    le.shutdown()
                except Exception:  # noqa: BLE001 - followers that are already gone need no farewell
                    pass
            else:
                follower_loop(engine, channel, on_error, g)
        finally:
            close = getattr(engine, "close", None)
            if close is not None:
                close()

    group.start()
    try:
        group.run(serve)
    finally:
        group.close(shutdown=group.is_leader)
    return group.history


def lead_with_scheduler(make_scheduler: Callable[[LeaderEngine, Any], Any], backend: ElasticBackend, stop) -> Callable[[LeaderEngine, Any], None]:
    """The leader's part of a generation for the HTTP server: a scheduler over the leader engine is attached to
    ``backend`` until ``stop`` (a ``threading.Event``: the server is shutting down) is set or the scheduler's loop ends on
    a fatal error, which is re-raised here (``RankLost`` makes the group re-form)."""
    def lead(le: LeaderEngine, group) -> None:
        sched = make_scheduler(le, group).start()
        backend.attach(sched)
        try:
            while not stop.wait(0.05):
                if sched.fatal is not None:
                    raise sched.fatal
        finally:
            backend.detach()
            sched.stop()
    return lead
