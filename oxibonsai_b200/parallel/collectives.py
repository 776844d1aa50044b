"""Device mesh, collectives, weight partitioning, sharded linear layers and pipeline-parallel schedule maths.

Reference (CPU simulations there): crates/oxibonsai-model/src/multi_gpu.rs:31-320 (``DeviceMesh`` tp x pp,
``NcclCollectives::{all_reduce_sum, all_reduce_max, all_gather, reduce_scatter, broadcast}``, ``partition_weights_column`` /
``partition_weights_row`` / ``merge_column_shards``), tensor_parallel.rs:20-468 (``ShardInfo``, ``ShardedLinear``: column =
split the output rows, row = split the input columns with the bias on the last shard; ``tensor_parallel_forward``;
``ShardingPlan::standard_transformer_plan``) and pipeline_parallel.rs:21-240 (``partition_layers``, GPipe schedule, bubble
fraction, per-stage memory).

``Collectives`` has two modes with one API: given a ``torch.distributed`` process group (NCCL on GPUs, gloo on CPU) every
call is the real collective on this rank's tensor; without a group it operates on a *list* of per-rank tensors in one
process, which is what the parity tests and the planning tools use.  The latency-critical decode path does not go
through this class - it uses the fused peer-memory kernels of ``csrc/comm`` (see ``parallel/tp.py``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import torch


@dataclass(frozen=True)
class DeviceInfo:
    rank: int
    tp_rank: int
    pp_rank: int
    memory_bytes: int = 180 * 10 ** 9
    sm_count: int = 148


class DeviceMesh:
    """``tp x pp`` grid; ranks are tensor-parallel-major (consecutive ranks share a pipeline stage and NVLink domain)."""

    def __init__(self, tp: int, pp: int = 1):
        if tp < 1 or pp < 1:
            raise ValueError("mesh dimensions must be positive")
        self.tp, self.pp = tp, pp
        self.devices = [DeviceInfo(p * tp + t, t, p) for p in range(pp) for t in range(tp)]

    @classmethod
    def tensor_parallel(cls, n: int) -> "DeviceMesh":
        return cls(n, 1)

    def size(self) -> int:
        return self.tp * self.pp

    def get(self, tp_rank: int, pp_rank: int = 0) -> DeviceInfo:
        return self.devices[pp_rank * self.tp + tp_rank]

    def tp_group(self, pp_rank: int = 0) -> list[int]:
        return [d.rank for d in self.devices if d.pp_rank == pp_rank]

    def pp_group(self, tp_rank: int = 0) -> list[int]:
        return [d.rank for d in self.devices if d.tp_rank == tp_rank]


class Collectives:
    def __init__(self, group=None):
        self.group = group
        self.bytes_moved = 0

    def _dist(self):
        import torch.distributed as dist
        return dist

    def _world(self) -> int:
        return self._dist().get_world_size(self.group)

    def all_reduce_sum(self, x):
        if self.group is not None:
            self._dist().all_reduce(x, group=self.group)
            return x
        tot = torch.stack(list(x)).sum(0)
        self.bytes_moved += 2 * (len(x) - 1) * tot.numel() * tot.element_size()
        return [tot.clone() for _ in x]

    def all_reduce_max(self, x):
        if self.group is not None:
            d = self._dist()
            d.all_reduce(x, op=d.ReduceOp.MAX, group=self.group)
            return x
        m = torch.stack(list(x)).max(0).values
        return [m.clone() for _ in x]

    def all_gather(self, x, dim: int = 0):
        if self.group is not None:
            parts = [torch.empty_like(x) for _ in range(self._world())]
            self._dist().all_gather(parts, x.contiguous(), group=self.group)
            return torch.cat(parts, dim)
        g = torch.cat(list(x), dim)
        self.bytes_moved += (len(x) - 1) * g.numel() * g.element_size()
        return [g.clone() for _ in x]

    def reduce_scatter(self, x, dim: int = 0):
        if self.group is not None:
            w = self._world()
            chunks = [c.contiguous() for c in x.chunk(w, dim)]
            out = torch.empty_like(chunks[0])
            self._dist().reduce_scatter(out, chunks, group=self.group)
            return out
        tot = torch.stack(list(x)).sum(0)
        return [c.clone() for c in tot.chunk(len(x), dim)]

    def broadcast(self, x, src: int = 0):
        if self.group is not None:
            self._dist().broadcast(x, src=src, group=self.group)
            return x
        return [x[src].clone() for _ in x]


# ---- weight partitioning ----------------------------------------------------------------------------------------------------------
def partition_weights_column(w: torch.Tensor, n: int) -> list[torch.Tensor]:
    """Column parallel = split the output features (rows of a [out, in] weight)."""
    if w.shape[0] % n:
        raise ValueError(f"{w.shape[0]} output rows do not split over {n} ranks")
    return list(w.chunk(n, 0))


def partition_weights_row(w: torch.Tensor, n: int) -> list[torch.Tensor]:
    """Row parallel = split the input features (columns of a [out, in] weight)."""
    if w.shape[1] % n:
        raise ValueError(f"{w.shape[1]} input columns do not split over {n} ranks")
    return list(w.chunk(n, 1))


def merge_column_shards(shards: Sequence[torch.Tensor]) -> torch.Tensor:
    return torch.cat(list(shards), 0)


def merge_row_shards(shards: Sequence[torch.Tensor]) -> torch.Tensor:
    return torch.cat(list(shards), 1)


@dataclass
class ShardInfo:
    rank: int
    world: int
    kind: str          # "column" | "row"
    start: int
    end: int


class ShardedLinear:
    """One rank's slice of a linear layer."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None, info: ShardInfo):
        self.weight, self.bias, self.info = weight, bias, info

    @classmethod
    def shard(cls, weight: torch.Tensor, bias: torch.Tensor | None, kind: str, world: int) -> list["ShardedLinear"]:
        parts = partition_weights_column(weight, world) if kind == "column" else partition_weights_row(weight, world)
        step = (weight.shape[0] if kind == "column" else weight.shape[1]) // world
        out = []
        for r, p in enumerate(parts):
            if kind == "column":
                b = None if bias is None else bias[r * step:(r + 1) * step]
            else:
                b = bias if (bias is not None and r == world - 1) else None      # the bias is added once, on the last shard
            out.append(cls(p, b, ShardInfo(r, world, kind, r * step, (r + 1) * step)))
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xin = x if self.info.kind == "column" else x[..., self.info.start:self.info.end]
        y = xin @ self.weight.T
        return y if self.bias is None else y + self.bias


def tensor_parallel_forward(shards: Sequence[ShardedLinear], x: torch.Tensor, coll: Collectives | None = None) -> torch.Tensor:
    """Runs every shard and combines: all-gather for column parallel, all-reduce for row parallel."""
    coll = coll or Collectives()
    outs = [s.forward(x) for s in shards]
    if shards[0].info.kind == "column":
        return coll.all_gather(outs, dim=-1)[0]
    return coll.all_reduce_sum(outs)[0]


@dataclass
class ShardingPlan:
    """Layer-name suffix -> "column" / "row" / "replicated"."""
    rules: dict[str, str] = field(default_factory=dict)

    @classmethod
    def standard_transformer_plan(cls) -> "ShardingPlan":
        return cls({"attn_q": "column", "attn_k": "column", "attn_v": "column", "ffn_gate": "column", "ffn_up": "column",
                    "attn_output": "row", "ffn_down": "row", "output": "column", "token_embd": "replicated", "norm": "replicated"})

    def kind_for(self, tensor_name: str) -> str:
        for k, v in self.rules.items():
            if k in tensor_name:
                return v
        return "replicated"

    def collectives_per_layer(self) -> dict[str, int]:
        """Row-parallel outputs need one all-reduce each."""
        return {"all_reduce": sum(v == "row" for v in self.rules.values())}


# ---- pipeline parallel schedule maths ---------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class PipelineStage:
    index: int
    first_layer: int
    last_layer: int          # exclusive

    def layer_count(self) -> int:
        return self.last_layer - self.first_layer

    def contains_layer(self, layer: int) -> bool:
        return self.first_layer <= layer < self.last_layer

    def layer_range(self) -> range:
        return range(self.first_layer, self.last_layer)


def partition_layers(n_layers: int, n_stages: int) -> list[PipelineStage]:
    if n_stages < 1 or n_stages > n_layers:
        raise ValueError("need 1 <= stages <= layers")
    base, extra = divmod(n_layers, n_stages)
    out, lo = [], 0
    for s in range(n_stages):
        hi = lo + base + (1 if s < extra else 0)
        out.append(PipelineStage(s, lo, hi))
        lo = hi
    return out


@dataclass(frozen=True)
class MicroBatch:
    index: int
    tokens: int
    stage: int = 0

    def is_first_stage(self) -> bool:
        return self.stage == 0


@dataclass
class PipelineSchedule:
    n_stages: int
    n_microbatches: int
    steps: list[list[tuple[int, int]]] = field(default_factory=list)     # steps[t] = [(stage, microbatch), ...] running at time t

    @classmethod
    def gpipe_schedule(cls, n_stages: int, n_microbatches: int) -> "PipelineSchedule":
        steps = []
        for t in range(n_stages + n_microbatches - 1):
            steps.append([(s, t - s) for s in range(n_stages) if 0 <= t - s < n_microbatches])
        return cls(n_stages, n_microbatches, steps)

    def total_steps(self) -> int:
        return len(self.steps)

    def bubble_fraction(self) -> float:
        busy = sum(len(s) for s in self.steps)
        return 1.0 - busy / (self.total_steps() * self.n_stages)


def pipeline_memory_per_stage(stages: Sequence[PipelineStage], bytes_per_layer: int, embedding_bytes: int, activation_bytes_per_microbatch: int,
                              n_microbatches: int) -> list[int]:
    out = []
    for s in stages:
        m = s.layer_count() * bytes_per_layer + activation_bytes_per_microbatch * min(n_microbatches, len(stages) - s.index)
        if s.index == 0 or s.index == len(stages) - 1:
            m += embedding_bytes
        out.append(m)
    return out
