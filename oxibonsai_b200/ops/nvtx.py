"""NVTX ranges around the engine's GPU phases (decode step, prompt chunk, verification pass), for timeline tools.

Off by default: a range costs two host calls per step, which is measurable next to a 1.6 ms decode step.  Set
``OXIBONSAI_NVTX=1`` in the environment, or call :func:`enable`, before the engine runs.  The reference marks the same
phases with ``tracing`` spans (crates/oxibonsai-runtime/src/tracing_setup.rs and the ``#[instrument]`` attributes of
engine.rs); spans of the host side live in :mod:`oxibonsai_b200.runtime.observability`.
"""
from __future__ import annotations

import os
from contextlib import contextmanager

_on = os.environ.get("OXIBONSAI_NVTX", "") not in ("", "0")


def enable(on: bool = True) -> None:
    global _on
    _on = bool(on)


def enabled() -> bool:
    return _on


def push(name: str) -> bool:
    """Opens a range when ranges are on; returns whether :func:`pop` must be called."""
    if not _on:
        return False
    import torch
    torch.cuda.nvtx.range_push(name)
    return True


def pop(opened: bool) -> None:
    if opened:
        import torch
        torch.cuda.nvtx.range_pop()


@contextmanager
def range(name: str):          # noqa: A001 - mirrors torch.cuda.nvtx.range
    opened = push(name)
    try:
        yield
    finally:
        pop(opened)
