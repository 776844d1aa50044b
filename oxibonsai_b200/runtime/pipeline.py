"""Fluent generation pipeline composing context truncation, token healing, sampling chains, beam search, constraints and
stop strings over any ``logits_fn(tokens) -> logits`` (an engine, the CPU oracle, or a test double).

Reference: crates/oxibonsai-runtime/src/pipeline.rs:43-470 (``PipelineBuilder`` -> ``InferencePipeline::run`` returning a
``PipelineOutput`` with a ``StopReason``; presets ``chat_pipeline`` / ``code_pipeline`` / ``greedy_pipeline``).

With an ``InferenceEngine`` use :func:`engine_logits_fn`, which keeps the sequence resident in a KV slot and only feeds
the new token each step (the pipeline always extends the token list by one).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Callable, Sequence

import numpy as np

from .beam import BeamSearchConfig, BeamSearchEngine
from .constrained import ConstrainedSampler, ConstraintViolation, TokenConstraint
from .context import ContextWindow, TokenHealer, TokenHealingConfig, TruncationStrategy
from .sampling_advanced import SamplerChain


class GenerationStrategy(Enum):
    GREEDY = "greedy"
    SAMPLING = "sampling"
    BEAM = "beam"


class StopReason(Enum):
    MAX_TOKENS = "max_tokens"
    EOS = "eos"
    STOP_SEQUENCE = "stop_sequence"
    CONSTRAINT_COMPLETE = "constraint_complete"
    CONSTRAINT_DEAD_END = "constraint_dead_end"


@dataclass
class PipelineOutput:
    tokens: list[int]
    text: str
    stop_reason: StopReason
    prompt_tokens: int
    healed: bool = False
    truncated_tokens: int = 0


class InferencePipeline:
    def __init__(self, max_tokens, strategy, chain, beam, healing, constraint, stops, window, eos):
        self._max_tokens, self.strategy, self.chain, self.beam = max_tokens, strategy, chain, beam
        self.healing, self.constraint, self._stops, self.window, self.eos = healing, constraint, stops, window, eos

    def max_tokens(self) -> int:
        return self._max_tokens

    def has_healing(self) -> bool:
        return self.healing is not None

    def has_constraint(self) -> bool:
        return self.constraint is not None

    def stop_sequences(self) -> list[str]:
        return list(self._stops)

    def run(self, prompt: Sequence[int], logits_fn: Callable[[list[int]], np.ndarray], detokenize: Callable[[Sequence[int]], str],
            token_bytes: Callable[[int], bytes] | None = None, vocab_size: int | None = None) -> PipelineOutput:
        toks = [int(t) for t in prompt]
        dropped = 0
        if self.window is not None:
            w = ContextWindow(self.window[0], self.window[1])
            dropped = w.append(toks)
            toks = w.tokens()
        healed = False
        if self.healing is not None and token_bytes is not None and vocab_size:
            res = TokenHealer(self.healing).heal(toks, token_bytes, vocab_size, logits_fn)
            toks, healed = res.tokens, res.was_healed()
        n_prompt = len(toks)
        if self.strategy == GenerationStrategy.BEAM:
            cfg = self.beam or BeamSearchConfig()
            cfg = BeamSearchConfig(**{**cfg.__dict__, "max_length": min(cfg.max_length, self._max_tokens), "eos_token": cfg.eos_token if cfg.eos_token is not None else self.eos})
            res = BeamSearchEngine(cfg).search(toks, logits_fn)
            out = [t for t in res.best() if t != self.eos]
            reason = StopReason.EOS if res.beams and res.beams[0].finished else StopReason.MAX_TOKENS
            return PipelineOutput(out, detokenize(out), reason, n_prompt, healed, dropped)
        chain = self.chain if self.strategy == GenerationStrategy.SAMPLING and self.chain is not None else SamplerChain.greedy()
        sampler = chain.sample
        if self.constraint is not None:
            self.constraint.reset()
            cs = ConstrainedSampler(self.constraint, chain.sample, vocab_size or 0)
            sampler = cs.sample
        out: list[int] = []
        reason = StopReason.MAX_TOKENS
        for _ in range(self._max_tokens):
            logits = np.asarray(logits_fn(toks + out), dtype=np.float64)
            if self.constraint is not None and not vocab_size:
                cs.vocab = len(logits)
            try:
                tok = sampler(logits)
            except ConstraintViolation:
                reason = StopReason.CONSTRAINT_DEAD_END
                break
            if self.eos is not None and tok == self.eos:
                reason = StopReason.EOS
                break
            out.append(tok)
            if self._stops:
                text = detokenize(out)
                hit = min((text.find(s) for s in self._stops if s in text), default=-1)
                if hit >= 0:
                    # drop the tokens that only contribute to the stop string
                    while out and len(detokenize(out[:-1])) >= hit:
                        out.pop()
                    reason = StopReason.STOP_SEQUENCE
                    return PipelineOutput(out, detokenize(out)[:hit], reason, n_prompt, healed, dropped)
        else:
            if self.constraint is not None and self.constraint.is_complete():
                reason = StopReason.CONSTRAINT_COMPLETE
        return PipelineOutput(out, detokenize(out), reason, n_prompt, healed, dropped)


class PipelineBuilder:
    def __init__(self):
        self._max_tokens, self._strategy, self._chain, self._beam = 256, GenerationStrategy.GREEDY, None, None
        self._healing, self._constraint, self._stops, self._window, self._seed, self._eos = None, None, [], None, 42, None

    def max_tokens(self, n: int) -> "PipelineBuilder":
        self._max_tokens = n
        return self

    def greedy(self) -> "PipelineBuilder":
        self._strategy, self._chain = GenerationStrategy.GREEDY, None
        return self

    def with_sampling(self, chain: SamplerChain) -> "PipelineBuilder":
        self._strategy, self._chain = GenerationStrategy.SAMPLING, chain
        return self

    def with_beam_search(self, config: BeamSearchConfig) -> "PipelineBuilder":
        self._strategy, self._beam = GenerationStrategy.BEAM, config
        return self

    def with_token_healing(self, config: TokenHealingConfig | None = None) -> "PipelineBuilder":
        self._healing = config or TokenHealingConfig()
        return self

    def with_constraint(self, c: TokenConstraint) -> "PipelineBuilder":
        self._constraint = c
        return self

    def stop_on(self, sequences: Sequence[str]) -> "PipelineBuilder":
        self._stops = [s for s in sequences if s]
        return self

    def context_window(self, max_tokens: int, strategy: TruncationStrategy = TruncationStrategy.KEEP_LAST) -> "PipelineBuilder":
        self._window = (max_tokens, strategy)
        return self

    def seed(self, s: int) -> "PipelineBuilder":
        self._seed = s
        return self

    def eos(self, token: int | None) -> "PipelineBuilder":
        self._eos = token
        return self

    def build(self) -> InferencePipeline:
        chain = self._chain
        if self._strategy == GenerationStrategy.SAMPLING and chain is None:
            chain = SamplerChain.default_chat(self._seed)
        return InferencePipeline(self._max_tokens, self._strategy, chain, self._beam, self._healing, self._constraint, list(self._stops),
                                 self._window, self._eos)


def chat_pipeline(seed: int = 42, max_tokens: int = 512) -> InferencePipeline:
    return PipelineBuilder().max_tokens(max_tokens).with_sampling(SamplerChain.default_chat(seed)).stop_on(["<|im_end|>"]).build()


def code_pipeline(seed: int = 42, max_tokens: int = 1024) -> InferencePipeline:
    return PipelineBuilder().max_tokens(max_tokens).with_sampling(SamplerChain.precise(seed)).stop_on(["\n\n\n", "```\n"]).build()


def greedy_pipeline(max_tokens: int = 256) -> InferencePipeline:
    return PipelineBuilder().max_tokens(max_tokens).greedy().build()


def engine_logits_fn(engine, slot: int = 0, max_total: int | None = None) -> Callable[[list[int]], np.ndarray]:
    """``logits_fn`` over an :class:`InferenceEngine`: prefills on the first call, then feeds one new token per call as
    long as each call extends the previous token list by exactly one token; anything else starts the sequence over."""
    import torch
    if slot != 0:
        raise ValueError("single-sequence stepping runs in slot 0")
    state = {"tokens": None}

    def fn(tokens: list[int]) -> np.ndarray:
        r, prev = engine.runner, state["tokens"]
        if prev is not None and len(tokens) == len(prev) + 1 and tokens[:-1] == prev:
            engine._upload(slot, tokens[-1], len(prev))
            r.step_eager(1, sample=False)
        else:
            engine.close_sequence(slot)
            engine._start_sequence(slot, tokens, max_total or engine.max_seq_len)
        state["tokens"] = list(tokens)
        torch.cuda.synchronize(engine.device)
        return r.logits[slot].float().cpu().numpy()
    return fn
