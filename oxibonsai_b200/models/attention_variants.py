"""Attention variants for long context and sparse patterns, as torch functions that run on CPU or GPU tensors.

Reference (all single-device CPU f32 there): generic masked attention (crates/oxibonsai-model/src/layers/attention.rs:18-216),
online-softmax fused attention (attention_fused.rs:28-400), flash-decode split-KV with log-sum-exp merge
(flash_decode.rs:15-350), sliding window (sliding_window.rs:11-173), StreamingLLM attention sinks with position remap
(attention_sink.rs:65-378), sparse masks local / strided / BigBird (sparse_attention.rs:33-375), cross attention
(cross_attention.rs:62-361), mixture-of-depths token routing (mixture_of_depths.rs:27-271) and the per-layer attention
configuration (attention_config.rs:16-160).  The production decode and prefill attention of the engine are the CUDA
kernels in csrc/cuda/attention_*.cu; these variants are the library surface for other architectures and the oracles for
tests.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from enum import Enum

import torch


def masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor | None = None, scale: float | None = None) -> torch.Tensor:
    """q [..., tq, d], k / v [..., tk, d]; ``mask`` is boolean (True = may attend), broadcastable to [..., tq, tk]."""
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * (scale or 1.0 / math.sqrt(q.shape[-1]))
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p)            # rows with nothing to attend to produce zeros
    return torch.matmul(p, v.float()).to(q.dtype)


def causal_mask(tq: int, tk: int, device=None) -> torch.Tensor:
    qp = torch.arange(tk - tq, tk, device=device)[:, None]
    return torch.arange(tk, device=device)[None, :] <= qp


def gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """q [hq, tq, d], k / v [hkv, tk, d] with hq a multiple of hkv."""
    g = q.shape[0] // k.shape[0]
    k, v = k.repeat_interleave(g, 0), v.repeat_interleave(g, 0)
    return masked_attention(q, k, v, causal_mask(q.shape[1], k.shape[1], q.device) if causal else None)


def online_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, block: int = 32) -> torch.Tensor:
    """One query vector per head (q [h, d]) against k / v [h, t, d], walking the keys in blocks with O(1) extra memory."""
    h, d = q.shape
    m = torch.full((h,), float("-inf"), dtype=torch.float32, device=q.device)
    l = torch.zeros(h, dtype=torch.float32, device=q.device)
    acc = torch.zeros(h, d, dtype=torch.float32, device=q.device)
    sc = 1.0 / math.sqrt(d)
    for t0 in range(0, k.shape[1], block):
        s = torch.einsum("hd,htd->ht", q.float(), k[:, t0:t0 + block].float()) * sc
        mn = torch.maximum(m, s.max(dim=1).values)
        r = torch.exp(m - mn)
        p = torch.exp(s - mn[:, None])
        l = l * r + p.sum(1)
        acc = acc * r[:, None] + torch.einsum("ht,htd->hd", p, v[:, t0:t0 + block].float())
        m = mn
    return (acc / l[:, None]).to(q.dtype)


def flash_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, n_splits: int = 4) -> torch.Tensor:
    """Split-KV decode: independent partial attentions over key ranges, merged through their log-sum-exp."""
    h, d = q.shape
    t = k.shape[1]
    step = max(1, -(-t // n_splits))
    outs, lses = [], []
    sc = 1.0 / math.sqrt(d)
    for t0 in range(0, t, step):
        s = torch.einsum("hd,htd->ht", q.float(), k[:, t0:t0 + step].float()) * sc
        lse = torch.logsumexp(s, dim=1)
        outs.append(torch.einsum("ht,htd->hd", torch.exp(s - lse[:, None]), v[:, t0:t0 + step].float()))
        lses.append(lse)
    L = torch.stack(lses)                       # [splits, h]
    w = torch.softmax(L, dim=0)
    return (torch.stack(outs) * w[..., None]).sum(0).to(q.dtype)


# ---- sliding window ---------------------------------------------------------------------------------------------------------------
@dataclass
class SlidingWindowConfig:
    window: int = 0              # 0 disables
    sinks: int = 0               # first tokens that stay visible

    def is_disabled(self) -> bool:
        return self.window <= 0


def attention_range(pos: int, cfg: SlidingWindowConfig) -> tuple[int, int]:
    """Half-open key range [lo, hi) visible from query position ``pos`` (sinks not included)."""
    return (0, pos + 1) if cfg.is_disabled() else (max(0, pos + 1 - cfg.window), pos + 1)


def is_in_window(q_pos: int, k_pos: int, cfg: SlidingWindowConfig) -> bool:
    if k_pos > q_pos:
        return False
    lo, hi = attention_range(q_pos, cfg)
    return lo <= k_pos < hi or k_pos < cfg.sinks


def sliding_window_mask(tq: int, tk: int, cfg: SlidingWindowConfig, device=None) -> torch.Tensor:
    m = causal_mask(tq, tk, device)
    if cfg.is_disabled():
        return m
    qp = torch.arange(tk - tq, tk, device=device)[:, None]
    kp = torch.arange(tk, device=device)[None, :]
    return m & ((kp > qp - cfg.window) | (kp < cfg.sinks))


def evict_outside_window(items: list, pos: int, cfg: SlidingWindowConfig) -> list:
    if cfg.is_disabled():
        return items
    lo, _ = attention_range(pos, cfg)
    return items[: cfg.sinks] + items[max(lo, cfg.sinks):]


# ---- attention sinks (StreamingLLM) ---------------------------------------------------------------------------------------------------
class AttentionSinkCache:
    """Keeps ``n_sinks`` first tokens and the ``window`` most recent ones; positions are re-numbered inside the cache
    so the rotary angles stay within the trained range however long the stream gets."""

    def __init__(self, n_sinks: int, window: int, n_heads: int, head_dim: int, device=None, dtype=torch.float32):
        if n_sinks < 0 or window <= 0:
            raise ValueError("need n_sinks >= 0 and window > 0")
        self.n_sinks, self.window = n_sinks, window
        self.k = torch.zeros((n_heads, n_sinks + window, head_dim), dtype=dtype, device=device)
        self.v = torch.zeros_like(self.k)
        self.len = 0
        self.seen = 0

    def push_step(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """k, v: [heads, head_dim] of the new token (un-rotated keys: rotation uses the remapped positions)."""
        cap = self.n_sinks + self.window
        if self.len < cap:
            self.k[:, self.len], self.v[:, self.len] = k, v
            self.len += 1
        else:
            self.k[:, self.n_sinks:-1] = self.k[:, self.n_sinks + 1:].clone()
            self.v[:, self.n_sinks:-1] = self.v[:, self.n_sinks + 1:].clone()
            self.k[:, -1], self.v[:, -1] = k, v
        self.seen += 1

    def get_keys(self) -> torch.Tensor:
        return self.k[:, : self.len]

    def get_values(self) -> torch.Tensor:
        return self.v[:, : self.len]

    def get_remapped_positions(self) -> torch.Tensor:
        return torch.arange(self.len)

    def cache_len(self) -> int:
        return self.len

    def is_streaming(self) -> bool:
        return self.seen > self.n_sinks + self.window

    def total_evicted(self) -> int:
        return max(0, self.seen - self.len)

    def memory_bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()


# ---- sparse patterns -------------------------------------------------------------------------------------------------------------------
class SparsePattern(Enum):
    LOCAL = "local"
    STRIDED = "strided"
    BIGBIRD = "bigbird"


class SparseAttentionMask:
    def __init__(self, mask: torch.Tensor):
        self.mask = mask

    @classmethod
    def build(cls, pattern: SparsePattern, seq_len: int, window: int = 64, stride: int = 64, n_global: int = 2, n_random: int = 2,
              seed: int = 0) -> "SparseAttentionMask":
        i = torch.arange(seq_len)[:, None]
        j = torch.arange(seq_len)[None, :]
        causal = j <= i
        local = (i - j) < window
        if pattern == SparsePattern.LOCAL:
            m = local
        elif pattern == SparsePattern.STRIDED:
            m = local | ((i - j) % stride == 0)
        else:
            g = torch.Generator().manual_seed(seed)
            rnd = torch.zeros(seq_len, seq_len, dtype=torch.bool)
            if n_random > 0 and seq_len > 1:
                cols = torch.randint(0, seq_len, (seq_len, n_random), generator=g)
                rnd.scatter_(1, cols, True)
            m = local | (j < n_global) | (i < n_global) | rnd
        return cls(m & causal)

    def keys_for_query(self, q: int) -> list[int]:
        return torch.nonzero(self.mask[q]).flatten().tolist()

    def nnz(self) -> int:
        return int(self.mask.sum())

    def density(self) -> float:
        n = self.mask.shape[0]
        return self.nnz() / (n * (n + 1) / 2)

    def can_attend(self, q: int, k: int) -> bool:
        return bool(self.mask[q, k])

    def to_dense(self) -> torch.Tensor:
        return self.mask


def sparse_attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: SparseAttentionMask) -> torch.Tensor:
    return masked_attention(q, k, v, mask.mask.to(q.device))


def sparse_vs_dense_error(q, k, v, mask: SparseAttentionMask) -> float:
    dense = masked_attention(q, k, v, causal_mask(q.shape[-2], k.shape[-2], q.device))
    return float((sparse_attention_forward(q, k, v, mask) - dense).abs().max())


def memory_reduction(mask: SparseAttentionMask) -> float:
    return 1.0 - mask.density()


# ---- cross attention, mixture of depths, per-layer config ----------------------------------------------------------------------------------
class CrossAttention(torch.nn.Module):
    """Queries from the decoder stream, keys / values from an encoder memory; optional memory padding mask."""

    def __init__(self, hidden: int, n_heads: int, memory_dim: int | None = None):
        super().__init__()
        self.h, self.d = n_heads, hidden // n_heads
        md = memory_dim or hidden
        self.q, self.k, self.v, self.o = (torch.nn.Linear(hidden, hidden, bias=False), torch.nn.Linear(md, hidden, bias=False),
                                          torch.nn.Linear(md, hidden, bias=False), torch.nn.Linear(hidden, hidden, bias=False))

    def forward(self, x: torch.Tensor, memory: torch.Tensor, memory_mask: torch.Tensor | None = None) -> torch.Tensor:
        t, s = x.shape[0], memory.shape[0]
        q = self.q(x).view(t, self.h, self.d).transpose(0, 1)
        k = self.k(memory).view(s, self.h, self.d).transpose(0, 1)
        v = self.v(memory).view(s, self.h, self.d).transpose(0, 1)
        m = None if memory_mask is None else memory_mask[None, None, :].expand(self.h, t, s)
        return self.o(masked_attention(q, k, v, m).transpose(0, 1).reshape(t, -1))


class MixtureOfDepthsRouter(torch.nn.Module):
    """Per-layer token router: only the top ``capacity`` fraction of tokens go through the block, the rest skip it."""

    def __init__(self, hidden: int, capacity: float = 0.5):
        super().__init__()
        self.score = torch.nn.Linear(hidden, 1, bias=False)
        self.capacity = capacity

    def route(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        w = self.score(x).squeeze(-1)
        k = max(1, int(round(self.capacity * x.shape[0])))
        idx = torch.topk(w, k).indices.sort().values
        return idx, torch.sigmoid(w[idx])

    def forward(self, x: torch.Tensor, block) -> torch.Tensor:
        idx, gate = self.route(x)
        out = x.clone()
        out[idx] = x[idx] + gate[:, None] * (block(x[idx]) - x[idx])
        return out


@dataclass
class AttentionLayerConfig:
    kind: str = "full"                  # full | sliding_window | sink | sparse
    window: int = 0
    sinks: int = 0
    pattern: SparsePattern | None = None


@dataclass
class AttentionConfig:
    """Per-layer attention kinds, e.g. alternating full and sliding-window layers."""
    layers: list[AttentionLayerConfig] = field(default_factory=list)

    @classmethod
    def uniform(cls, n_layers: int, kind: str = "full", **kw) -> "AttentionConfig":
        return cls([AttentionLayerConfig(kind, **kw) for _ in range(n_layers)])

    @classmethod
    def alternating(cls, n_layers: int, window: int, every: int = 2) -> "AttentionConfig":
        return cls([AttentionLayerConfig("full") if i % every == every - 1 else AttentionLayerConfig("sliding_window", window) for i in range(n_layers)])

    def mask_for_layer(self, layer: int, tq: int, tk: int, device=None) -> torch.Tensor:
        c = self.layers[layer]
        if c.kind in ("sliding_window", "sink"):
            return sliding_window_mask(tq, tk, SlidingWindowConfig(c.window, c.sinks), device)
        if c.kind == "sparse":
            return SparseAttentionMask.build(c.pattern or SparsePattern.LOCAL, tk, c.window or 64).mask[tk - tq:].to(device)
        return causal_mask(tq, tk, device)

    def kv_tokens_needed(self, layer: int, context: int) -> int:
        c = self.layers[layer]
        return min(context, c.window + c.sinks) if c.kind in ("sliding_window", "sink") and c.window > 0 else context
