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
    """Rank 0's engine as the scheduler sees it: calls that change engine state are announced on the channel first."""

    def __init__(self, engine, channel: CommandChannel):
        self._engine, self._channel = engine, channel

    def __getattr__(self, name: str):
        attr = getattr(self._engine, name)
        if name not in MIRRORED:
            return attr

        def mirrored(*args):
            self._channel.send(name, _plain(args))
            return attr(*args)
        return mirrored

    def shutdown(self) -> None:
        self._channel.send(SHUTDOWN)


def _plain(args: tuple) -> tuple:
    """Arguments as plain Python values (lists of ints, dataclasses) so that they pickle small and identically."""
    return tuple(list(a) if isinstance(a, (list, tuple, range)) else a for a in args)


def follower_loop(engine, channel: CommandChannel, on_error: Callable[[str, Exception], None] | None = None) -> int:
    """Runs on every rank but the leader: executes the announced calls until the leader shuts down.  An exception of a
    call is reported and the loop goes on - the leader's own call raised the same way (same state, same arguments) and its
    scheduler has already dealt with it.  Returns the number of commands executed."""
    n = 0
    engine.bind_thread()
    while True:
        op, args = channel.recv()
        if op == SHUTDOWN:
            return n
        n += 1
        try:
            getattr(engine, op)(*args)
        except Exception as e:  # noqa: BLE001 - mirrored on the leader
            if on_error is not None:
                on_error(op, e)
