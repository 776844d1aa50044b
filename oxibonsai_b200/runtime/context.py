"""Context window management, token budgets, token healing and the chunked-prefill planner.

Reference: crates/oxibonsai-runtime/src/context_manager.rs (``TruncationStrategy``, ``ContextWindow``,
``ConversationContext``), token_budget.rs (``BudgetPolicy``, ``BudgetConfig``, ``RequestBudget``, ``GlobalTokenBudget``,
``TokenCostEstimate``), token_healing.rs (``TokenHealer`` backs off over the last prompt tokens and lets the model
re-choose the boundary token) and crates/oxibonsai-model/src/chunked_prefill.rs:9-320 (``create_prefill_chunks``,
``PrefillScheduler`` alternating prefill chunks with decode steps, memory estimate).
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Sequence

import numpy as np


# ---- context window ----------------------------------------------------------------------------------------------------------
class TruncationStrategy(Enum):
    KEEP_LAST = "keep_last"          # drop the oldest conversation tokens
    KEEP_FIRST = "keep_first"        # drop the newest
    KEEP_BOTH_ENDS = "keep_both_ends"  # keep head and tail, drop the middle
    ERROR = "error"


class ContextError(ValueError):
    pass


class ContextWindow:
    """A system prompt that is never truncated plus a conversation buffer kept within ``max_tokens``."""

    def __init__(self, max_tokens: int, strategy: TruncationStrategy = TruncationStrategy.KEEP_LAST):
        self.max_tokens, self.strategy = max_tokens, strategy
        self.system: list[int] = []
        self.conversation: list[int] = []

    def set_system_prompt(self, tokens: Sequence[int]) -> None:
        if len(tokens) >= self.max_tokens:
            raise ContextError(f"system prompt of {len(tokens)} tokens does not fit a window of {self.max_tokens}")
        self.system = list(tokens)
        self.truncate_to_fit()

    def append(self, tokens: Sequence[int]) -> int:
        """Appends and truncates; returns how many tokens were dropped."""
        self.conversation.extend(int(t) for t in tokens)
        return self.truncate_to_fit()

    def truncate_to_fit(self) -> int:
        room = self.max_tokens - len(self.system)
        over = len(self.conversation) - room
        if over <= 0:
            return 0
        if self.strategy == TruncationStrategy.ERROR:
            raise ContextError(f"context overflow by {over} tokens")
        if self.strategy == TruncationStrategy.KEEP_LAST:
            self.conversation = self.conversation[over:]
        elif self.strategy == TruncationStrategy.KEEP_FIRST:
            self.conversation = self.conversation[:room]
        else:
            head = room // 2
            self.conversation = self.conversation[:head] + self.conversation[len(self.conversation) - (room - head):]
        return over

    def tokens(self) -> list[int]:
        return self.system + self.conversation

    def __len__(self) -> int:
        return len(self.system) + len(self.conversation)

    def remaining_capacity(self) -> int:
        return max(0, self.max_tokens - len(self))

    def is_at_limit(self) -> bool:
        return len(self) >= self.max_tokens

    def clear_conversation(self) -> None:
        self.conversation = []

    def utilization(self) -> float:
        return len(self) / self.max_tokens if self.max_tokens else 0.0


@dataclass
class ConversationTurn:
    role: str
    content: str
    token_ids: list[int]


class ConversationContext:
    """Whole turns are evicted oldest-first (system turns are kept) until the conversation fits."""

    def __init__(self, max_tokens: int):
        self.max_tokens = max_tokens
        self.turns: list[ConversationTurn] = []

    def add_turn(self, role: str, content: str, token_ids: Sequence[int]) -> None:
        self.turns.append(ConversationTurn(role, content, list(token_ids)))
        while self.total_tokens() > self.max_tokens:
            victim = next((i for i, t in enumerate(self.turns[:-1]) if t.role != "system"), None)
            if victim is None:
                break
            del self.turns[victim]

    def build_tokens(self) -> list[int]:
        return [t for turn in self.turns for t in turn.token_ids]

    def turn_count(self) -> int:
        return len(self.turns)

    def total_tokens(self) -> int:
        return sum(len(t.token_ids) for t in self.turns)

    def is_full(self) -> bool:
        return self.total_tokens() >= self.max_tokens

    def clear(self) -> None:
        self.turns = []

    def last_turn(self) -> ConversationTurn | None:
        return self.turns[-1] if self.turns else None

    def utilization(self) -> float:
        return self.total_tokens() / self.max_tokens if self.max_tokens else 0.0


# ---- budgets -----------------------------------------------------------------------------------------------------------------------
class BudgetError(RuntimeError):
    pass


class BudgetPolicy(Enum):
    HARD_STOP = "hard_stop"      # raise when the budget is exceeded
    TRUNCATE = "truncate"        # report exhaustion, the caller stops quietly
    WARN = "warn"                # keep going, remember the overrun


@dataclass
class BudgetConfig:
    max_completion: int | None = None
    max_total: int | None = None
    policy: BudgetPolicy = BudgetPolicy.TRUNCATE

    def with_max_completion(self, n: int) -> "BudgetConfig":
        return BudgetConfig(n, self.max_total, self.policy)

    def with_max_total(self, n: int) -> "BudgetConfig":
        return BudgetConfig(self.max_completion, n, self.policy)

    def with_policy(self, policy: BudgetPolicy) -> "BudgetConfig":
        return BudgetConfig(self.max_completion, self.max_total, policy)

    @classmethod
    def unlimited(cls) -> "BudgetConfig":
        return cls()


class RequestBudget:
    def __init__(self, config: BudgetConfig, prompt_tokens: int):
        if config.max_total is not None and prompt_tokens >= config.max_total and config.policy == BudgetPolicy.HARD_STOP:
            raise BudgetError(f"prompt of {prompt_tokens} tokens already exceeds the total budget {config.max_total}")
        self.config, self._prompt, self._completion, self.overrun = config, prompt_tokens, 0, 0

    def record_tokens(self, n: int) -> bool:
        """Counts ``n`` generated tokens; returns False once the budget is exhausted (or raises under HARD_STOP)."""
        self._completion += n
        if self.is_exhausted():
            if self.config.policy == BudgetPolicy.HARD_STOP and self._over() > 0:
                raise BudgetError("token budget exceeded")
            if self.config.policy == BudgetPolicy.WARN:
                self.overrun = self._over()
                return True
            return False
        return True

    def record_token(self) -> bool:
        return self.record_tokens(1)

    def _over(self) -> int:
        c = self.config
        a = self._completion - c.max_completion if c.max_completion is not None else 0
        b = self.total_tokens() - c.max_total if c.max_total is not None else 0
        return max(a, b, 0)

    def prompt_tokens(self) -> int:
        return self._prompt

    def completion_tokens(self) -> int:
        return self._completion

    def total_tokens(self) -> int:
        return self._prompt + self._completion

    def remaining_completion_tokens(self) -> int | None:
        c = self.config
        lims = [x for x in ((c.max_completion - self._completion) if c.max_completion is not None else None,
                            (c.max_total - self.total_tokens()) if c.max_total is not None else None) if x is not None]
        return max(0, min(lims)) if lims else None

    def is_exhausted(self) -> bool:
        r = self.remaining_completion_tokens()
        return r is not None and r <= 0

    def policy(self) -> BudgetPolicy:
        return self.config.policy


class GlobalTokenBudget:
    """Process-wide counter shared by all requests."""

    def __init__(self, max_tokens: int | None = None):
        self.max_tokens, self._used, self._lock = max_tokens, 0, threading.Lock()

    @classmethod
    def unlimited(cls) -> "GlobalTokenBudget":
        return cls(None)

    def record(self, tokens: int) -> None:
        with self._lock:
            self._used += tokens

    def total_used(self) -> int:
        return self._used

    def remaining(self) -> int | None:
        return None if self.max_tokens is None else max(0, self.max_tokens - self._used)

    def is_exhausted(self) -> bool:
        return self.max_tokens is not None and self._used >= self.max_tokens

    def utilization(self) -> float | None:
        return None if not self.max_tokens else self._used / self.max_tokens


@dataclass
class TokenCostEstimate:
    prompt_tokens: int
    completion_tokens: int
    prefill_seconds: float
    decode_seconds: float

    @classmethod
    def compute(cls, prompt_tokens: int, completion_tokens: int, prefill_tok_s: float, decode_tok_s: float) -> "TokenCostEstimate":
        return cls(prompt_tokens, completion_tokens, prompt_tokens / max(prefill_tok_s, 1e-9), completion_tokens / max(decode_tok_s, 1e-9))

    @property
    def total_seconds(self) -> float:
        return self.prefill_seconds + self.decode_seconds

    def summary(self) -> str:
        return (f"{self.prompt_tokens} prompt + {self.completion_tokens} completion tokens: "
                f"{self.prefill_seconds:.3f}s prefill + {self.decode_seconds:.3f}s decode = {self.total_seconds:.3f}s")


# ---- token healing ----------------------------------------------------------------------------------------------------------------
@dataclass
class TokenHealingConfig:
    lookback: int = 1                 # how many trailing prompt tokens may be re-chosen
    min_prob: float = 0.0             # a replacement must have at least this probability
    enabled: bool = True


@dataclass
class HealingResult:
    tokens: list[int]
    removed: list[int] = field(default_factory=list)
    replacement: list[int] = field(default_factory=list)

    @classmethod
    def unchanged(cls, tokens: Sequence[int]) -> "HealingResult":
        return cls(list(tokens))

    def was_healed(self) -> bool:
        return bool(self.removed)


class TokenHealer:
    """Prompts that stop in the middle of a word force the tokenizer into a boundary the model rarely saw.  Healing
    drops the trailing token(s), then lets the model pick the most likely token whose text *starts with* the removed
    text, so generation continues from a natural boundary."""

    def __init__(self, config: TokenHealingConfig | None = None):
        self.config = config or TokenHealingConfig()

    @classmethod
    def with_lookback(cls, lookback: int) -> "TokenHealer":
        return cls(TokenHealingConfig(lookback=lookback))

    @staticmethod
    def is_continuation_token(prev_token_text: str, token_text: str) -> bool:
        """True when ``token_text`` glues onto the previous token without a word boundary."""
        return bool(prev_token_text) and bool(token_text) and not prev_token_text[-1].isspace() and not token_text[0].isspace() \
            and (token_text[0].isalnum() == prev_token_text[-1].isalnum())

    @staticmethod
    def token_prob(logits: np.ndarray, token_id: int) -> float:
        x = np.asarray(logits, dtype=np.float64)
        e = np.exp(x - x.max())
        return float(e[token_id] / e.sum())

    def heal(self, tokens: Sequence[int], token_bytes: Callable[[int], bytes], vocab_size: int,
             get_logits: Callable[[list[int]], np.ndarray]) -> HealingResult:
        toks = list(tokens)
        if not self.config.enabled or len(toks) < 2:
            return HealingResult.unchanged(toks)
        for back in range(1, min(self.config.lookback, len(toks) - 1) + 1):
            removed = toks[-back:]
            prefix = b"".join(token_bytes(t) for t in removed)
            if not prefix:
                continue
            logits = np.asarray(get_logits(toks[:-back]), dtype=np.float64)
            best, best_p = None, self.config.min_prob
            p = np.exp(logits - logits.max())
            p /= p.sum()
            for cand in np.argsort(-p)[:512]:
                tb = token_bytes(int(cand))
                if len(tb) > len(prefix) and tb.startswith(prefix) and p[cand] > best_p:
                    best, best_p = int(cand), float(p[cand])
                    break
            if best is not None and best not in removed:
                return HealingResult(toks[:-back] + [best], removed, [best])
        return HealingResult.unchanged(toks)


# ---- chunked prefill planner -------------------------------------------------------------------------------------------------------
class PrefillPriority(Enum):
    PREFILL_FIRST = "prefill_first"       # finish the prompt before any decode step
    INTERLEAVED = "interleaved"           # one decode step of the running batch between chunks
    DECODE_FIRST = "decode_first"         # two decode steps between chunks


@dataclass
class ChunkedPrefillConfig:
    chunk_size: int = 1024
    overlap: int = 0
    priority: PrefillPriority = PrefillPriority.INTERLEAVED

    def with_overlap(self, overlap: int) -> "ChunkedPrefillConfig":
        return ChunkedPrefillConfig(self.chunk_size, overlap, self.priority)

    def with_priority(self, priority: PrefillPriority) -> "ChunkedPrefillConfig":
        return ChunkedPrefillConfig(self.chunk_size, self.overlap, priority)


@dataclass
class PrefillChunk:
    index: int
    start: int
    end: int
    is_last: bool

    def __len__(self) -> int:
        return self.end - self.start


def create_prefill_chunks(n_tokens: int, config: ChunkedPrefillConfig) -> list[PrefillChunk]:
    if config.chunk_size <= 0 or config.overlap >= config.chunk_size:
        raise ValueError("chunk_size must be positive and larger than the overlap")
    out, start = [], 0
    while start < n_tokens:
        end = min(n_tokens, start + config.chunk_size)
        out.append(PrefillChunk(len(out), start, end, end == n_tokens))
        if end == n_tokens:
            break
        start = end - config.overlap
    return out


@dataclass
class PrefillAction:
    kind: str                         # "prefill" | "decode" | "done"
    chunk: PrefillChunk | None = None


class PrefillScheduler:
    """Yields the order of work for one long prompt sharing the GPU with a running decode batch."""

    def __init__(self, n_prompt_tokens: int, config: ChunkedPrefillConfig | None = None):
        self.config = config or ChunkedPrefillConfig()
        self.chunks = create_prefill_chunks(n_prompt_tokens, self.config)
        self._next, self._owed = 0, 0

    def next_action(self) -> PrefillAction:
        if self._owed > 0:
            self._owed -= 1
            return PrefillAction("decode")
        if self._next >= len(self.chunks):
            return PrefillAction("done")
        c = self.chunks[self._next]
        self._next += 1
        if not c.is_last:
            self._owed = {PrefillPriority.PREFILL_FIRST: 0, PrefillPriority.INTERLEAVED: 1, PrefillPriority.DECODE_FIRST: 2}[self.config.priority]
        return PrefillAction("prefill", c)

    def decode_available(self) -> bool:
        return self._owed > 0

    def is_complete(self) -> bool:
        return self._next >= len(self.chunks) and self._owed == 0

    def progress(self) -> float:
        return self._next / len(self.chunks) if self.chunks else 1.0

    def total_chunks(self) -> int:
        return len(self.chunks)

    def memory_savings(self, hidden_dim: int) -> float:
        """Fraction of activation memory saved against prefilling the whole prompt at once."""
        total = self.chunks[-1].end if self.chunks else 0
        return 0.0 if total == 0 else 1.0 - min(self.config.chunk_size, total) / total


@dataclass
class PrefillMemoryEstimate:
    activation_bytes: int
    kv_bytes: int
    logits_bytes: int

    @property
    def total_bytes(self) -> int:
        return self.activation_bytes + self.kv_bytes + self.logits_bytes

    def summary(self) -> str:
        mb = lambda b: f"{b / 2 ** 20:.1f} MiB"
        return f"activations {mb(self.activation_bytes)} + KV {mb(self.kv_bytes)} + logits {mb(self.logits_bytes)} = {mb(self.total_bytes)}"


def peak_memory_estimate(n_tokens: int, chunk_size: int, hidden: int, inter: int, layers: int, kv_heads: int, head_dim: int,
                         vocab: int, kv_bytes_per_elem: float = 2.0) -> PrefillMemoryEstimate:
    t = min(n_tokens, chunk_size)
    act = t * (hidden * 4 + max(hidden, inter) * 2 + (hidden + 2 * kv_heads * head_dim) * 4 + inter * 2 + hidden * 4)
    kv = int(n_tokens * layers * 2 * kv_heads * head_dim * kv_bytes_per_elem)
    return PrefillMemoryEstimate(int(act), kv, vocab * 4)
