"""Fine-tuning utilities: LoRA adapters and registry, a LoRA trainer, optimizers, learning-rate schedulers, losses and
gradient checkpointing (differentiation itself is torch autograd, which stands in for the reference's hand-written
``Tensor`` with per-op backward rules).

Reference: crates/oxibonsai-model/src/lora.rs (``LoraConfig``, ``LoraAdapter::apply`` = ``(alpha / r) * B(A x)``,
``merge_into_weights``, ``LoraRegistry``, ``BonsaiLoraSet``), lora_trainer.rs (``LoraTrainer::step``), optimizer.rs (SGD
with momentum / Nesterov, Adam, AdamW, ``clip_grad_norm``, constant / warm-up / cosine schedules), lr_schedulers.rs
(one-cycle, reduce-on-plateau, linear warm-up + cosine decay, polynomial decay, cyclic), gradient.rs (scalar-graph
``Tensor`` with backward rules), losses.rs (cross-entropy, label smoothing, focal, KL, distillation, MSE, Huber,
contrastive, next-token loss) and gradient_checkpoint.rs (segments that keep only their input and recompute on demand).
Everything is written over torch tensors so it runs on the GPU next to the inference engine.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Iterable, Sequence

import torch
import torch.nn.functional as F


# ---- LoRA -------------------------------------------------------------------------------------------------------------------
@dataclass
class LoraConfig:
    rank: int = 8
    alpha: float = 16.0
    dropout: float = 0.0
    target_modules: tuple[str, ...] = ("attn_q", "attn_v")

    @property
    def scale(self) -> float:
        return self.alpha / self.rank


class LoraAdapter(torch.nn.Module):
    """``delta(x) = scale * B (A x)`` with A ~ N(0, 1/r) and B = 0, so a fresh adapter is a no-op."""

    def __init__(self, in_features: int, out_features: int, config: LoraConfig, seed: int = 0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.config = config
        self.A = torch.nn.Parameter(torch.randn(config.rank, in_features, generator=g) / math.sqrt(config.rank))
        self.B = torch.nn.Parameter(torch.zeros(out_features, config.rank))

    def apply_delta(self, x: torch.Tensor) -> torch.Tensor:
        if self.training and self.config.dropout > 0:
            x = F.dropout(x, self.config.dropout)
        return (x @ self.A.T) @ self.B.T * self.config.scale

    def forward(self, x: torch.Tensor, base_out: torch.Tensor) -> torch.Tensor:
        return base_out + self.apply_delta(x)

    def param_count(self) -> int:
        return self.A.numel() + self.B.numel()

    def memory_bytes(self) -> int:
        return self.param_count() * self.A.element_size()

    def delta_weight(self) -> torch.Tensor:
        return (self.B @ self.A) * self.config.scale

    def merge_into_weights(self, weight: torch.Tensor) -> torch.Tensor:
        """``W + scale * B A`` (a dense matrix: merged adapters lose the packed sub-2-bit storage of W)."""
        return weight + self.delta_weight().to(weight.dtype)


class LoraRegistry:
    def __init__(self, config: LoraConfig | None = None):
        self.config = config or LoraConfig()
        self.adapters: dict[str, LoraAdapter] = {}

    def add(self, module: str, in_features: int, out_features: int, seed: int = 0) -> LoraAdapter:
        a = LoraAdapter(in_features, out_features, self.config, seed)
        self.adapters[module] = a
        return a

    def get(self, module: str) -> LoraAdapter | None:
        return self.adapters.get(module)

    def apply_adapter(self, module: str, x: torch.Tensor, base_out: torch.Tensor) -> torch.Tensor:
        a = self.adapters.get(module)
        return base_out if a is None else a(x, base_out)

    def adapter_count(self) -> int:
        return len(self.adapters)

    def total_param_count(self) -> int:
        return sum(a.param_count() for a in self.adapters.values())

    def total_memory_bytes(self) -> int:
        return sum(a.memory_bytes() for a in self.adapters.values())

    def is_empty(self) -> bool:
        return not self.adapters

    def module_names(self) -> list[str]:
        return sorted(self.adapters)

    def parameters(self) -> list[torch.nn.Parameter]:
        return [p for a in self.adapters.values() for p in a.parameters()]

    @staticmethod
    def estimate_adapters_for_budget(budget_bytes: int, in_features: int, out_features: int, rank: int, bytes_per_param: int = 4) -> int:
        return budget_bytes // (rank * (in_features + out_features) * bytes_per_param)


class BonsaiLoraSet:
    """Adapters for every layer of a Qwen3-shaped model."""

    def __init__(self, cfg, config: LoraConfig | None = None):
        self.cfg, self.registry = cfg, LoraRegistry(config)

    def add_attention_adapters(self) -> "BonsaiLoraSet":
        c = self.cfg
        for l in range(c.layers):
            self.registry.add(f"blk.{l}.attn_q", c.hidden, c.heads * c.head_dim, seed=4 * l)
            self.registry.add(f"blk.{l}.attn_v", c.hidden, c.kv_heads * c.head_dim, seed=4 * l + 1)
        return self

    def add_mlp_adapters(self) -> "BonsaiLoraSet":
        c = self.cfg
        for l in range(c.layers):
            self.registry.add(f"blk.{l}.ffn_up", c.hidden, c.inter, seed=4 * l + 2)
            self.registry.add(f"blk.{l}.ffn_down", c.inter, c.hidden, seed=4 * l + 3)
        return self

    def total_trainable_params(self) -> int:
        return self.registry.total_param_count()

    def efficiency_ratio(self, base_params: int) -> float:
        return self.total_trainable_params() / base_params


# ---- optimizers ----------------------------------------------------------------------------------------------------------------
def grad_norm(params: Iterable[torch.Tensor]) -> float:
    return math.sqrt(sum(float((p.grad.detach().float() ** 2).sum()) for p in params if p.grad is not None))


def clip_grad_norm(params: Sequence[torch.Tensor], max_norm: float) -> float:
    n = grad_norm(params)
    if n > max_norm > 0:
        for p in params:
            if p.grad is not None:
                p.grad.mul_(max_norm / (n + 1e-6))
    return n


class Sgd:
    def __init__(self, params: Sequence[torch.Tensor], lr: float, momentum: float = 0.0, weight_decay: float = 0.0, nesterov: bool = False):
        self.params, self.lr, self.momentum, self.wd, self.nesterov = list(params), lr, momentum, weight_decay, nesterov
        self.buf = [None] * len(self.params)

    @torch.no_grad()
    def step(self, lr: float | None = None) -> None:
        lr = self.lr if lr is None else lr
        for i, p in enumerate(self.params):
            if p.grad is None:
                continue
            g = p.grad + self.wd * p if self.wd else p.grad
            if self.momentum:
                self.buf[i] = g.clone() if self.buf[i] is None else self.buf[i].mul_(self.momentum).add_(g)
                g = g + self.momentum * self.buf[i] if self.nesterov else self.buf[i]
            p.add_(g, alpha=-lr)

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None


class Adam:
    decoupled = False

    def __init__(self, params: Sequence[torch.Tensor], lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0):
        self.params, self.lr, self.betas, self.eps, self.wd = list(params), lr, betas, eps, weight_decay
        self.reset()

    def reset(self) -> None:
        self.m = [torch.zeros_like(p) for p in self.params]
        self.v = [torch.zeros_like(p) for p in self.params]
        self.t = 0

    @torch.no_grad()
    def step(self, lr: float | None = None) -> None:
        lr = self.lr if lr is None else lr
        self.t += 1
        b1, b2 = self.betas
        for p, m, v in zip(self.params, self.m, self.v):
            if p.grad is None:
                continue
            g = p.grad
            if self.wd and not self.decoupled:
                g = g + self.wd * p
            if self.wd and self.decoupled:
                p.mul_(1 - lr * self.wd)
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            mh, vh = m / (1 - b1 ** self.t), v / (1 - b2 ** self.t)
            p.addcdiv_(mh, vh.sqrt().add_(self.eps), value=-lr)

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None


class AdamW(Adam):
    decoupled = True

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
        super().__init__(params, lr, betas, eps, weight_decay)


# ---- learning-rate schedules ------------------------------------------------------------------------------------------------------
@dataclass
class ConstantLr:
    lr: float

    def at(self, step: int) -> float:
        return self.lr


@dataclass
class WarmupConstantLr:
    lr: float
    warmup: int

    def at(self, step: int) -> float:
        return self.lr * min(1.0, (step + 1) / max(1, self.warmup))


@dataclass
class CosineAnnealingLr:
    lr: float
    total: int
    min_lr: float = 0.0

    def at(self, step: int) -> float:
        t = min(step, self.total) / max(1, self.total)
        return self.min_lr + 0.5 * (self.lr - self.min_lr) * (1 + math.cos(math.pi * t))


@dataclass
class LinearWarmupCosineDecay:
    lr: float
    warmup: int
    total: int
    min_lr: float = 0.0

    def at(self, step: int) -> float:
        if step < self.warmup:
            return self.lr * (step + 1) / max(1, self.warmup)
        t = min(1.0, (step - self.warmup) / max(1, self.total - self.warmup))
        return self.min_lr + 0.5 * (self.lr - self.min_lr) * (1 + math.cos(math.pi * t))


@dataclass
class PolynomialDecay:
    lr: float
    total: int
    end_lr: float = 0.0
    power: float = 1.0

    def at(self, step: int) -> float:
        t = min(step, self.total) / max(1, self.total)
        return (self.lr - self.end_lr) * (1 - t) ** self.power + self.end_lr


@dataclass
class OneCycleLr:
    max_lr: float
    total: int
    warmup_fraction: float = 0.3
    min_lr: float = 0.0
    div_factor: float = 25.0

    def at(self, step: int) -> float:
        up = max(1, int(self.total * self.warmup_fraction))
        start = self.max_lr / self.div_factor
        if step < up:
            return start + (self.max_lr - start) * step / up
        t = min(1.0, (step - up) / max(1, self.total - up))
        return self.min_lr + 0.5 * (self.max_lr - self.min_lr) * (1 + math.cos(math.pi * t))

    def progress(self, step: int) -> float:
        return min(1.0, step / max(1, self.total))


@dataclass
class CyclicLr:
    base_lr: float
    max_lr: float
    step_size: int

    def cycle_position(self, step: int) -> float:
        return abs(step / self.step_size - 2 * math.floor(1 + step / (2 * self.step_size)) + 1)

    def at(self, step: int) -> float:
        return self.base_lr + (self.max_lr - self.base_lr) * max(0.0, 1 - self.cycle_position(step))


class ReduceOnPlateau:
    def __init__(self, lr: float, patience: int = 3, factor: float = 0.5, min_lr: float = 0.0, mode: str = "min", threshold: float = 1e-4):
        self.lr, self.patience, self.factor, self.min_lr, self.mode, self.threshold = lr, patience, factor, min_lr, mode, threshold
        self.best, self.bad, self.reduced = None, 0, 0

    def step(self, metric: float) -> float:
        better = self.best is None or (metric < self.best - self.threshold if self.mode == "min" else metric > self.best + self.threshold)
        if better:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
            if self.bad > self.patience:
                new = max(self.min_lr, self.lr * self.factor)
                self.reduced += new < self.lr
                self.lr, self.bad = new, 0
        return self.lr

    def current_lr(self) -> float:
        return self.lr

    def times_reduced(self) -> int:
        return self.reduced


# ---- losses -------------------------------------------------------------------------------------------------------------------------
def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    return F.cross_entropy(logits.float(), targets, ignore_index=ignore_index)


def label_smoothed_cross_entropy(logits: torch.Tensor, targets: torch.Tensor, smoothing: float = 0.1) -> torch.Tensor:
    lp = F.log_softmax(logits.float(), -1)
    nll = -lp.gather(-1, targets[..., None]).squeeze(-1)
    return ((1 - smoothing) * nll - smoothing * lp.mean(-1)).mean()


def focal_loss(logits: torch.Tensor, targets: torch.Tensor, gamma: float = 2.0) -> torch.Tensor:
    lp = F.log_softmax(logits.float(), -1).gather(-1, targets[..., None]).squeeze(-1)
    return (-(1 - lp.exp()) ** gamma * lp).mean()


def kl_divergence(p_logits: torch.Tensor, q_logits: torch.Tensor) -> torch.Tensor:
    """KL(P || Q) averaged over rows."""
    lp, lq = F.log_softmax(p_logits.float(), -1), F.log_softmax(q_logits.float(), -1)
    return (lp.exp() * (lp - lq)).sum(-1).mean()


def distillation_loss(student_logits, teacher_logits, targets, temperature: float = 2.0, alpha: float = 0.5) -> torch.Tensor:
    soft = kl_divergence(teacher_logits / temperature, student_logits / temperature) * temperature ** 2
    return alpha * soft + (1 - alpha) * cross_entropy(student_logits, targets)


def mse(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return ((a.float() - b.float()) ** 2).mean()


def huber_loss(a: torch.Tensor, b: torch.Tensor, delta: float = 1.0) -> torch.Tensor:
    d = (a.float() - b.float()).abs()
    return torch.where(d <= delta, 0.5 * d * d, delta * (d - 0.5 * delta)).mean()


def contrastive_loss(a: torch.Tensor, b: torch.Tensor, temperature: float = 0.07) -> torch.Tensor:
    """InfoNCE over a batch of paired embeddings (row i of ``a`` matches row i of ``b``)."""
    a, b = F.normalize(a.float(), dim=-1), F.normalize(b.float(), dim=-1)
    logits = a @ b.T / temperature
    t = torch.arange(a.shape[0], device=a.device)
    return 0.5 * (F.cross_entropy(logits, t) + F.cross_entropy(logits.T, t))


def ntp_loss(logits: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """Next-token prediction: position t predicts token t + 1."""
    return cross_entropy(logits[:-1], tokens[1:])


def cross_entropy_grad(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """d loss / d logits of the mean cross-entropy: ``(softmax - onehot) / n``."""
    p = F.softmax(logits.float(), -1)
    p[torch.arange(len(targets)), targets] -= 1.0
    return p / len(targets)


def sequence_perplexity(logits: torch.Tensor, tokens: torch.Tensor) -> float:
    return float(torch.exp(ntp_loss(logits, tokens)))


# ---- LoRA trainer ---------------------------------------------------------------------------------------------------------------------
@dataclass
class LoraTrainingConfig:
    lr: float = 1e-3
    total_steps: int = 100
    warmup_steps: int = 10
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0


@dataclass
class TrainingStep:
    step: int
    loss: float
    lr: float
    grad_norm: float


class LoraTrainer:
    """Trains the adapters of a registry; ``loss_fn()`` must build the loss from the registry's parameters."""

    def __init__(self, registry: LoraRegistry, config: LoraTrainingConfig | None = None):
        self.registry, self.config = registry, config or LoraTrainingConfig()
        self.opt = AdamW(registry.parameters(), self.config.lr, weight_decay=self.config.weight_decay)
        self.sched = LinearWarmupCosineDecay(self.config.lr, self.config.warmup_steps, self.config.total_steps)
        self.history: list[TrainingStep] = []

    def current_lr(self) -> float:
        return self.sched.at(len(self.history))

    def step(self, loss_fn: Callable[[], torch.Tensor]) -> TrainingStep:
        self.opt.zero_grad()
        loss = loss_fn()
        loss.backward()
        gn = clip_grad_norm(self.opt.params, self.config.max_grad_norm)
        lr = self.current_lr()
        self.opt.step(lr)
        s = TrainingStep(len(self.history), float(loss.detach()), lr, gn)
        self.history.append(s)
        return s

    def total_steps(self) -> int:
        return len(self.history)

    def is_complete(self) -> bool:
        return len(self.history) >= self.config.total_steps

    def average_loss(self, last: int = 10) -> float:
        h = self.history[-last:]
        return sum(s.loss for s in h) / len(h) if h else 0.0

    def last_step(self) -> TrainingStep | None:
        return self.history[-1] if self.history else None

    def convergence_rate(self) -> float:
        """Relative loss reduction from the first to the latest step."""
        if len(self.history) < 2 or self.history[0].loss == 0:
            return 0.0
        return (self.history[0].loss - self.history[-1].loss) / abs(self.history[0].loss)


# ---- gradient checkpointing ----------------------------------------------------------------------------------------------------------------
class _CheckpointFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, x):
        ctx.fn = fn
        ctx.save_for_backward(x)
        with torch.no_grad():
            return fn(x)

    @staticmethod
    def backward(ctx, grad_out):
        (x,) = ctx.saved_tensors
        x = x.detach().requires_grad_(True)
        with torch.enable_grad():
            y = ctx.fn(x)
        params = [p for p in getattr(ctx.fn, "parameters", lambda: [])() if p.requires_grad]
        grads = torch.autograd.grad(y, [x] + params, grad_out, allow_unused=True)
        for p, g in zip(params, grads[1:]):
            if g is not None:
                p.grad = g if p.grad is None else p.grad + g
        return None, grads[0]


def checkpoint(fn, x: torch.Tensor) -> torch.Tensor:
    """Runs ``fn(x)`` keeping only ``x``; the segment is recomputed during the backward pass."""
    return _CheckpointFn.apply(fn, x)


class CheckpointedPipeline(torch.nn.Module):
    """Sequential segments; activations inside a segment are not stored."""

    def __init__(self, segments: Sequence[torch.nn.Module]):
        super().__init__()
        self.segments = torch.nn.ModuleList(segments)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for s in self.segments:
            x = checkpoint(s, x) if torch.is_grad_enabled() else s(x)
        return x

    def num_segments(self) -> int:
        return len(self.segments)

    def memory_estimate(self, batch: int, width: int, inner_activations_per_segment: int, bytes_per_elem: int = 4) -> dict:
        ck = self.num_segments() * batch * width * bytes_per_elem
        full = self.num_segments() * (1 + inner_activations_per_segment) * batch * width * bytes_per_elem
        return {"checkpointed": ck, "full": full, "savings": 1 - ck / full}


class CheckpointBudget:
    def __init__(self, total_bytes: int):
        self.total, self.used = total_bytes, 0

    def remaining(self) -> int:
        return self.total - self.used

    def utilization(self) -> float:
        return self.used / self.total if self.total else 0.0

    def can_allocate(self, n: int) -> bool:
        return self.used + n <= self.total

    def allocate(self, n: int) -> bool:
        if not self.can_allocate(n):
            return False
        self.used += n
        return True

    def free(self, n: int) -> None:
        self.used = max(0, self.used - n)
