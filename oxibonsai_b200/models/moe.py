"""Mixture-of-experts routing and expert FFN layers.

Reference: crates/oxibonsai-model/src/layers/moe_router.rs:18-387 (``MoeConfig``, ``TopKRouter`` with softmax gating,
capacity-bounded ``ExpertBuffer``, auxiliary load-balance loss and z-loss, ``combine_expert_outputs``) and moe_expert.rs:16-278
(``Expert`` SwiGLU FFN, ``MoeFfnLayer`` with total / active parameter counts).  The reference keeps these single-process;
so does this module - the Qwen3 dense checkpoints served by the engine have no experts - but it runs on GPU tensors and
groups tokens per expert so each expert is one batched matmul.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class MoeConfig:
    hidden: int
    inter: int
    n_experts: int
    top_k: int = 2
    capacity_factor: float = 1.25
    normalize_top_k: bool = True
    aux_loss_weight: float = 0.01
    z_loss_weight: float = 0.001


@dataclass
class RoutingDecision:
    expert_ids: torch.Tensor        # [tokens, k]
    weights: torch.Tensor           # [tokens, k]
    probs: torch.Tensor             # [tokens, experts]
    logits: torch.Tensor
    dropped: torch.Tensor           # [tokens, k] bool: assignment exceeded the expert's capacity

    def num_tokens(self) -> int:
        return self.expert_ids.shape[0]

    def expert_loads(self, n_experts: int) -> torch.Tensor:
        return torch.bincount(self.expert_ids[~self.dropped].flatten(), minlength=n_experts)

    def max_expert_load(self, n_experts: int) -> int:
        return int(self.expert_loads(n_experts).max())

    def min_expert_load(self, n_experts: int) -> int:
        return int(self.expert_loads(n_experts).min())

    def overflow_rate(self) -> float:
        return float(self.dropped.float().mean())

    def load_balance_score(self, n_experts: int) -> float:
        """1 = perfectly even, towards 0 = everything on one expert."""
        l = self.expert_loads(n_experts).float()
        return float(l.mean() / l.max()) if l.max() > 0 else 1.0


class TopKRouter(torch.nn.Module):
    def __init__(self, cfg: MoeConfig):
        super().__init__()
        self.cfg = cfg
        self.gate = torch.nn.Linear(cfg.hidden, cfg.n_experts, bias=False)

    def capacity(self, n_tokens: int) -> int:
        c = self.cfg
        return max(1, int(c.capacity_factor * n_tokens * c.top_k / c.n_experts + 0.999))

    def route(self, x: torch.Tensor) -> RoutingDecision:
        c = self.cfg
        logits = self.gate(x).float()
        probs = torch.softmax(logits, dim=-1)
        w, ids = torch.topk(probs, c.top_k, dim=-1)
        if c.normalize_top_k:
            w = w / w.sum(-1, keepdim=True)
        # capacity: assignments are granted in token order, first choices before second choices
        cap = self.capacity(x.shape[0])
        dropped = torch.zeros_like(ids, dtype=torch.bool)
        counts = torch.zeros(c.n_experts, dtype=torch.long, device=x.device)
        for k in range(c.top_k):
            onehot = torch.nn.functional.one_hot(ids[:, k], c.n_experts)
            rank = torch.cumsum(onehot, 0) - onehot + counts[None, :]
            pos = (rank * onehot).sum(-1)
            dropped[:, k] = pos >= cap
            counts = counts + (onehot * (~dropped[:, k])[:, None]).sum(0)
        return RoutingDecision(ids, w, probs, logits, dropped)

    def aux_loss(self, d: RoutingDecision) -> torch.Tensor:
        """Switch-style balance loss: n_experts * sum_e (fraction of tokens on e) * (mean router probability of e)."""
        n = self.cfg.n_experts
        frac = torch.nn.functional.one_hot(d.expert_ids[:, 0], n).float().mean(0)
        return n * (frac * d.probs.mean(0)).sum()

    def z_loss(self, d: RoutingDecision) -> torch.Tensor:
        return (torch.logsumexp(d.logits, dim=-1) ** 2).mean()


class ExpertBuffer:
    """Host-side capacity bookkeeping (token ids per expert), mirroring the reference's buffer API."""

    def __init__(self, n_experts: int, capacity: int):
        self.capacity = capacity
        self.slots: list[list[int]] = [[] for _ in range(n_experts)]
        self.overflow = 0

    def try_assign(self, expert: int, token: int) -> bool:
        if len(self.slots[expert]) >= self.capacity:
            self.overflow += 1
            return False
        self.slots[expert].append(token)
        return True

    def tokens_for_expert(self, expert: int) -> list[int]:
        return self.slots[expert]

    def expert_utilization(self) -> list[float]:
        return [len(s) / self.capacity for s in self.slots]

    def total_assigned(self) -> int:
        return sum(len(s) for s in self.slots)

    def overflow_count(self) -> int:
        return self.overflow

    def reset(self) -> None:
        self.slots = [[] for _ in self.slots]
        self.overflow = 0


class Expert(torch.nn.Module):
    def __init__(self, hidden: int, inter: int):
        super().__init__()
        self.gate = torch.nn.Linear(hidden, inter, bias=False)
        self.up = torch.nn.Linear(hidden, inter, bias=False)
        self.down = torch.nn.Linear(inter, hidden, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down(torch.nn.functional.silu(self.gate(x)) * self.up(x))

    def param_count(self) -> int:
        return sum(p.numel() for p in self.parameters())


def combine_expert_outputs(outputs: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """outputs [tokens, k, hidden], weights [tokens, k] -> [tokens, hidden]."""
    return (outputs * weights[..., None]).sum(1)


class MoeFfnLayer(torch.nn.Module):
    def __init__(self, cfg: MoeConfig):
        super().__init__()
        self.cfg = cfg
        self.router = TopKRouter(cfg)
        self.experts = torch.nn.ModuleList([Expert(cfg.hidden, cfg.inter) for _ in range(cfg.n_experts)])
        self.last_decision: RoutingDecision | None = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        d = self.router.route(x)
        self.last_decision = d
        out = torch.zeros_like(x, dtype=torch.float32)
        for e, expert in enumerate(self.experts):
            sel = (d.expert_ids == e) & ~d.dropped
            tok, slot = torch.nonzero(sel, as_tuple=True)
            if tok.numel():
                out.index_add_(0, tok, expert(x[tok]).float() * d.weights[tok, slot][:, None])
        return out.to(x.dtype)

    def total_param_count(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def active_param_count(self) -> int:
        return self.router.gate.weight.numel() + self.cfg.top_k * self.experts[0].param_count()

    def sparsity(self) -> float:
        return 1.0 - self.active_param_count() / self.total_param_count()

    def memory_bytes(self, bytes_per_param: float = 2.0) -> int:
        return int(self.total_param_count() * bytes_per_param)


def moe_8x7b_config() -> MoeConfig:
    return MoeConfig(hidden=4096, inter=14336, n_experts=8, top_k=2)


def moe_tiny_config() -> MoeConfig:
    return MoeConfig(hidden=32, inter=64, n_experts=4, top_k=2)
