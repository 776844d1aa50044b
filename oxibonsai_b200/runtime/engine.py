"""Inference engine: load a GGUF checkpoint, prefill, decode, sample, stream.

Reference surface: ``InferenceEngine`` (crates/oxibonsai-runtime/src/engine.rs:98-118) with ``from_gguf`` /
``from_gguf_path`` (:179-249, :1023-1045), ``generate`` (:376-445: prefill, then sample -> stop on token
151645 before emitting it -> forward), the streaming and seeded variants (:459-709) and the warm-up that
hides graph capture (:216-234).  The per-token loop here keeps the model state on the GPU: the host
uploads (token, position) from pinned memory, replays one CUDA graph and reads back one token id.
"""
from __future__ import annotations

import os

import time
from dataclasses import dataclass, field
from typing import Callable, Iterator, Sequence

import torch

from ..core.gguf import GgufFile, Qwen3Config
from ..core.oracle import EOS_TOKEN
from ..models.qwen3 import PagedKvCache, Qwen3Runner, Qwen3Weights
from ..ops import cuda_ops as K
from .presets import SamplingParams, SamplingPreset

KV_NAMES = {"f32": K.KV_F32, "fp32": K.KV_F32, "f16": K.KV_F16, "fp16": K.KV_F16, "q8": K.KV_Q8, "int8": K.KV_Q8, "q4": K.KV_Q4, "int4": K.KV_Q4}


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    token_times: list[float] = field(default_factory=list)

    @property
    def tokens_per_second(self) -> float:
        """The reference CLI's figure: generated / (prefill + decode) wall time (src/main.rs:604-621)."""
        t = self.prefill_seconds + self.decode_seconds
        return self.generated_tokens / t if t > 0 else 0.0

    @property
    def decode_tokens_per_second(self) -> float:
        return self.generated_tokens / self.decode_seconds if self.decode_seconds > 0 else 0.0


class InferenceEngine:
    """Single-process engine for one GPU (or one tensor-parallel rank)."""

    def __init__(self, model_path: str, max_seq_len: int = 4096, max_batch: int = 1, kv_dtype: str = "f16",
                 device: str | torch.device = "cuda:0", sampling: SamplingParams | None = None, page_size: int = 64,
                 kv_pages: int | None = None, tp_rank: int = 0, tp_size: int = 1, warmup: bool = True, exact: bool | None = None,
                 repack_cache: str | None = None, prefill_chunk: int | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("InferenceEngine needs a CUDA device; use oxibonsai_b200.core.Oracle for the CPU path")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        K.lib()  # fail loudly if the native kernels are missing
        self.model_path = str(model_path)
        self.gguf = GgufFile.open(self.model_path)
        self.config: Qwen3Config = self.gguf.config()
        self.max_seq_len = int(max_seq_len)
        self.max_batch = int(max_batch)
        self.sampling = (sampling or SamplingPreset.BALANCED.params()).validate()
        self.kvt = KV_NAMES[kv_dtype.lower()]
        t0 = time.perf_counter()
        # exact = f32 activations end to end (the token-stream gate); default: exact only with an f32 KV cache
        self.exact = (self.kvt == K.KV_F32) if exact is None else bool(exact)
        # directory of the repacked-weight cache (None = decode and repack the GGUF tensors on every start)
        self.repack_cache = repack_cache if repack_cache is not None else os.environ.get("OXIBONSAI_REPACK_CACHE") or None
        self.weights = Qwen3Weights(self.gguf, self.device, tp_rank, tp_size, decode_layout=not self.exact,
                                    cache_dir=self.repack_cache, source_path=self.model_path)
        pages_per_seq = (self.max_seq_len + page_size - 1) // page_size
        self.kv = PagedKvCache(self.config, self.weights.kv_heads_local, kv_pages or pages_per_seq * self.max_batch, page_size,
                               self.kvt, self.device)
        # Tokens per prompt chunk of the batched prefill path (the activation buffers are sized for it).  Larger chunks fill
        # the GPU better in the projections with few row tiles (QKV / attention output: 48 / 32 row tiles x one column block
        # per 256 tokens on 148 SMs): time to first token of a 4096-token prompt on the 8B shape 0.148 s at 1024, 0.132 s at
        # 2048, 0.122 s at 4096.
        self.prefill_chunk = int(prefill_chunk or os.environ.get("OXIBONSAI_PREFILL_CHUNK") or 4096)
        if self.prefill_chunk < 64 or self.prefill_chunk % 64:
            raise ValueError("prefill_chunk must be a multiple of 64")
        self.runner = Qwen3Runner(self.weights, self.kv, self.max_batch, self.max_seq_len, fast=not self.exact,
                                  prefill_chunk=self.prefill_chunk)
        self.load_seconds = time.perf_counter() - t0
        # pinned staging for the per-step host <-> device traffic
        self._tok_host = torch.zeros(self.max_batch, dtype=torch.int32).pin_memory()
        self._pos_host = torch.zeros(self.max_batch, dtype=torch.int32).pin_memory()
        self._out_host = torch.zeros(self.max_batch + 1, dtype=torch.int32).pin_memory()   # [status word, tokens...]
        self._slot_pages: dict[int, list[int]] = {}
        self._slot_fmt: dict[int, int] = {}       # page format of a bound slot when it is not the default one
        self._masked: set[int] = set()            # slots whose vocabulary mask is not "every token"
        self.prefill_min_tokens = 16   # the reference also switches to batch prefill above 16 tokens
        self.prefix_cache = None       # see enable_prefix_cache()
        self.last_stats = GenerationStats()
        if warmup:
            self.warmup()

    # ---- construction helpers -------------------------------------------------------------------
    @classmethod
    def from_gguf_path(cls, path: str, **kw) -> "InferenceEngine":
        return cls(path, **kw)

    def warmup(self) -> None:
        """Captures the decode graph and touches every kernel once (hidden from the first request)."""
        self._bind_slot(0, min(self.max_seq_len, 8))
        self._set_sampling(0, SamplingPreset.GREEDY.params())
        self._upload(0, 0, 0)
        self.runner.step_eager(1, sample=True)
        torch.cuda.synchronize(self.device)
        self._upload(0, 0, 1)
        self.runner.step(1, sample=True)
        torch.cuda.synchronize(self.device)
        self._release_slot(0)

    # ---- slot / page management -----------------------------------------------------------------
    def _pool_of(self, slot: int) -> PagedKvCache:
        return self.runner.kv_pools[self._slot_fmt.get(slot, self.kvt)]

    def _bind_slot(self, slot: int, n_tokens: int) -> None:
        if n_tokens > self.max_seq_len:
            raise ValueError(f"sequence of {n_tokens} tokens exceeds max_seq_len {self.max_seq_len}")
        need = (n_tokens + self.kv.page_size - 1) // self.kv.page_size
        have = self._slot_pages.setdefault(slot, [])
        if need > len(have):
            have.extend(self._pool_of(slot).alloc(need - len(have)))
            row = torch.tensor(have, dtype=torch.int32)
            self.runner.block_table[slot, : len(have)].copy_(row.to(self.device))

    def _release_slot(self, slot: int) -> None:
        pages = self._slot_pages.pop(slot, [])
        self._pool_of(slot).release(pages)
        if slot in self._masked:
            self.set_mask(slot, None)
        if self._slot_fmt.pop(slot, None) is not None:
            self.runner.set_slot_format(slot, self.kvt)

    # ---- KV page formats ---------------------------------------------------------------------------
    def enable_kv_formats(self, formats: Sequence[str] = ("q8", "q4"), pages: int | None = None) -> list[str]:
        """Adds page pools in further formats (``f16`` / ``q8`` / ``q4``; each ``pages`` pages, default: as many as the
        default pool) so that new sequences can be admitted in a denser format while running ones keep theirs - what a
        :class:`~oxibonsai_b200.runtime.kv_policy.KvCachePolicy` level change then means.  Returns the formats now
        available.  Not offered in the exact-f32 mode or under tensor parallelism of the prefix cache's shared pages."""
        for name in formats:
            kvt = KV_NAMES[name.lower()]
            if kvt in self.runner.kv_pools:
                continue
            pool = PagedKvCache(self.config, self.weights.kv_heads_local, pages or self.kv.num_pages, self.kv.page_size, kvt, self.device)
            self.runner.add_kv_pool(pool)
        return self.kv_formats()

    def kv_formats(self) -> list[str]:
        names = {K.KV_F32: "f32", K.KV_F16: "f16", K.KV_Q8: "q8", K.KV_Q4: "q4"}
        return [names[k] for k in sorted(self.runner.kv_pools)]

    def kv_utilization(self) -> float:
        """Bytes of KV pages in use over bytes of all pools (the pressure a KV-cache policy observes)."""
        pools = self.runner.kv_pools.values()
        used = sum(p.utilization * p.nbytes for p in pools)
        return used / max(1, sum(p.nbytes for p in pools))

    def _set_sampling(self, slot: int, p: SamplingParams) -> None:
        r = self.runner
        r.temps[slot] = float(p.temperature)
        r.topks[slot] = int(p.top_k)
        r.topps[slot] = float(p.top_p)
        seed = int(p.seed) & 0xFFFFFFFFFFFFFFFF
        r.rng[slot] = seed - (1 << 64) if seed >= (1 << 63) else seed

    def _upload(self, slot: int, token: int, pos: int) -> None:
        self._tok_host[slot] = token
        self._pos_host[slot] = pos
        self.runner.tokens[slot: slot + 1].copy_(self._tok_host[slot: slot + 1], non_blocking=True)
        self.runner.positions[slot: slot + 1].copy_(self._pos_host[slot: slot + 1], non_blocking=True)

    def _read_tokens(self, n: int = 1, slot0: int = 0) -> list[int]:
        """Brings the sampled tokens of slots slot0..slot0+n-1 to the host together with the step's status word (one
        device-to-host copy when slot0 == 0) and raises :class:`CudaKernelError` if a kernel recorded an expired wait -
        tokens computed from missing data are never handed out."""
        r = self.runner
        if slot0 == 0:
            self._out_host[: n + 1].copy_(r.ctl[: n + 1], non_blocking=True)
        else:
            self._out_host[:1].copy_(r.status, non_blocking=True)
            self._out_host[1: n + 1].copy_(r.tokens[slot0: slot0 + n], non_blocking=True)
        torch.cuda.synchronize(self.device)
        if int(self._out_host[0]):
            r.check_status(int(self._out_host[0]))
        return self._out_host[1: n + 1].tolist()

    # ---- prefix cache ----------------------------------------------------------------------------
    def enable_prefix_cache(self, max_pages: int | None = None):
        """Shares the KV pages of repeated prompt prefixes between sequences (full pages only).  The cache may hold up to
        ``max_pages`` pages (default: a quarter of the pool) and gives pages back when the pool runs dry."""
        from .prefix_cache import PrefixCache
        if self.exact:
            raise ValueError("the exact-f32 mode prefills token by token and does not use the prefix cache")
        self.prefix_cache = PrefixCache(self.kv.page_size, max_pages or max(1, self.kv.num_pages // 4), self.kv.retain, self.kv.release)
        self.kv.on_exhausted = lambda missing: self.prefix_cache.evict(missing)
        return self.prefix_cache

    def _start_sequence(self, slot: int, prompt: Sequence[int], total: int) -> None:
        """Binds pages for ``total`` tokens to ``slot`` and runs the prompt, reusing cached prefix pages when possible."""
        shared: list[int] = []
        pc = self.prefix_cache
        if pc is not None and len(prompt) > 1:
            shared = pc.lookup(prompt, max_tokens=len(prompt) - 1)   # the last prompt token is always recomputed
            if shared:
                self.kv.retain(shared)
                self._release_slot(slot)
                self._slot_pages[slot] = list(shared)
        try:
            self._bind_slot(slot, total)
        except MemoryError:
            self._release_slot(slot)
            raise
        if shared:
            row = torch.tensor(self._slot_pages[slot], dtype=torch.int32)
            self.runner.block_table[slot, : len(row)].copy_(row.to(self.device))
        cached = len(shared) * self.kv.page_size
        self.prefill(prompt[cached:], slot, cached)
        if pc is not None:
            pc.insert(prompt, self._slot_pages[slot])

    # ---- generation -------------------------------------------------------------------------------
    def prefill(self, prompt: Sequence[int], slot: int = 0, pos0: int = 0) -> None:
        """Runs the prompt through the model, leaving logits of the last prompt token in the runner.

        Prompts of at least ``prefill_min_tokens`` tokens go through the batched prefill kernels (tcgen05 GEMMs and
        causal attention over the paged cache) in chunks, on one GPU and on tensor-parallel ranks alike; shorter ones
        and the exact-f32 mode are fed through the decode path one token at a time.
        """
        n = len(prompt)
        toks = torch.tensor([int(t) for t in prompt], dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        r = self.runner
        if (n >= self.prefill_min_tokens or slot != 0) and not self.exact:
            r.prefill(toks, slot, pos0, self.prefill_chunk)
            return
        if slot != 0:
            raise NotImplementedError("the exact-f32 mode prefills through slot 0 only")
        # per-token feeds are device-to-device and stream ordered, so no host buffer is rewritten while a copy
        # that reads it is still queued
        pos = torch.arange(pos0, pos0 + n, dtype=torch.int32, device=self.device)
        for i in range(n):
            r.tokens[slot: slot + 1].copy_(toks[i: i + 1], non_blocking=True)
            r.positions[slot: slot + 1].copy_(pos[i: i + 1], non_blocking=True)
            r.step_eager(1, sample=False, lm_head=(i == n - 1))

    # ---- constrained decoding and log-probabilities -------------------------------------------------
    def set_mask(self, slot: int, mask) -> None:
        """Vocabulary mask of ``slot`` for the masked steps that follow: a packed uint32 array (bit set = token allowed, as
        ``TokenConstraint.allowed_mask`` returns it), or ``None`` for "every token"."""
        r = self.runner
        if mask is None:
            if slot in self._masked:
                r.allow_mask[slot].fill_(-1)
                self._masked.discard(slot)
            return
        self._masked.add(slot)
        import numpy as np
        m = np.zeros(r.mask_words, dtype=np.uint32)
        src = np.asarray(mask, dtype=np.uint32)[: r.mask_words]
        m[: src.size] = src
        r.allow_mask[slot].copy_(torch.from_numpy(m.view(np.int32)).pin_memory(), non_blocking=True)

    def token_logprobs(self, slot: int, token: int, top_n: int = 0) -> tuple[float, list[tuple[int, float]]]:
        """Log-probability of ``token`` under the logits that the last step (or prefill) left for ``slot``, and the ``top_n``
        most likely tokens with theirs (natural log, temperature 1)."""
        lp = torch.log_softmax(self.runner.logits[slot, : self.config.vocab].float(), dim=-1)
        top = []
        if top_n > 0:
            v, i = torch.topk(lp, min(top_n, lp.numel()))
            top = list(zip(i.tolist(), v.tolist()))
        return float(lp[int(token)]), top

    def generate_stream(self, prompt: Sequence[int], max_tokens: int | None = None, params: SamplingParams | None = None,
                        stop_at_eos: bool = True, on_token: Callable[[int], None] | None = None, constraint=None) -> Iterator[int]:
        """``constraint``: a :class:`~oxibonsai_b200.runtime.constrained.TokenConstraint`; its vocabulary mask goes to the
        device before every step and the sampler kernel only picks allowed tokens; generation ends when the constraint is
        complete (reference: ``ConstrainedSampler``, crates/oxibonsai-runtime/src/constrained_decoding/sampler.rs:19-94)."""
        p = (params or self.sampling).validate()
        max_new = p.max_tokens if max_tokens is None else max_tokens
        prompt = [int(t) for t in prompt]
        if not prompt:
            return
        stats = GenerationStats(prompt_tokens=len(prompt))
        self.last_stats = stats
        total = min(self.max_seq_len, len(prompt) + max_new)
        self._set_sampling(0, p)
        r = self.runner
        try:
            t0 = time.perf_counter()
            self._start_sequence(0, prompt, total)
            masked = constraint is not None
            if masked:
                constraint.reset()
                self.set_mask(0, constraint.allowed_mask())
            # first token: sample from the prefill logits on the device
            K.sample(r.logits[:1], r.temps[:1], r.topks[:1], r.topps[:1], r.rng[:1], out=r.tokens[:1],
                     allow_mask=r.allow_mask[:1] if masked else None)
            tok = self._read_tokens(1)[0]
            stats.prefill_seconds = time.perf_counter() - t0
            pos = len(prompt)
            t_dec = time.perf_counter()
            for _ in range(max_new):
                if stop_at_eos and tok == EOS_TOKEN:
                    break
                stats.generated_tokens += 1
                stats.token_times.append(time.perf_counter())
                if on_token is not None:
                    on_token(tok)
                yield tok
                if masked:
                    constraint.advance(tok)
                    if constraint.finished():
                        break
                    self.set_mask(0, constraint.allowed_mask())
                if pos >= self.max_seq_len:
                    break
                # the reference runs a forward after every emitted token, including the last
                self._upload(0, tok, pos)
                r.step(1, sample=True, masked=masked)
                tok = self._read_tokens(1)[0]
                pos += 1
            stats.decode_seconds = time.perf_counter() - t_dec
        finally:
            if constraint is not None:
                self.set_mask(0, None)
            self._release_slot(0)

    def generate(self, prompt: Sequence[int], max_tokens: int | None = None, params: SamplingParams | None = None,
                 stop_at_eos: bool = True, constraint=None) -> list[int]:
        return list(self.generate_stream(prompt, max_tokens, params, stop_at_eos, constraint=constraint))

    def generate_batch(self, prompts: Sequence[Sequence[int]], max_tokens: int, params: SamplingParams | None = None,
                       stop_at_eos: bool = True) -> list[list[int]]:
        """Generates for several prompts at once (true batched decode: one GEMM per linear layer for all of them).

        The reference's ``batch_generate`` runs the prompts one after another with a cache reset in between
        (crates/oxibonsai-runtime/src/batch_engine.rs:81-165).
        """
        B = len(prompts)
        if B == 0:
            return []
        if B > self.max_batch:
            raise ValueError(f"{B} prompts exceed max_batch {self.max_batch}")
        p = (params or self.sampling).validate()
        r = self.runner
        from dataclasses import replace
        try:
            for s, prompt in enumerate(prompts):
                n = len(prompt)
                self._set_sampling(s, replace(p, seed=p.seed + s))
                self._start_sequence(s, [int(t) for t in prompt], min(self.max_seq_len, n + max_tokens))
            lens = torch.tensor([len(q) for q in prompts], dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
            K.sample(r.logits[:B], r.temps[:B], r.topks[:B], r.topps[:B], r.rng[:B], out=r.tokens[:B])
            r.positions[:B].copy_(lens)
            out: list[list[int]] = [[] for _ in range(B)]
            done = [False] * B
            for step in range(max_tokens):
                host = self._read_tokens(B)
                for s in range(B):
                    if done[s]:
                        continue
                    tok = int(host[s])
                    if stop_at_eos and tok == EOS_TOKEN:
                        done[s] = True
                        continue
                    out[s].append(tok)
                    if len(prompts[s]) + len(out[s]) >= self.max_seq_len:
                        done[s] = True
                if all(done) or step == max_tokens - 1:
                    break
                r.step(B, sample=True)
            return out
        finally:
            for s in range(B):
                self._release_slot(s)

    # ---- single-step primitives (speculative decoding, schedulers) -------------------------------
    def open_sequence(self, prompt: Sequence[int], max_total: int, slot: int = 0, params: SamplingParams | None = None) -> int:
        """Binds ``slot``, prefills ``prompt`` and returns the first sampled token."""
        self._set_sampling(slot, params or self.sampling)
        self._start_sequence(slot, [int(t) for t in prompt], min(self.max_seq_len, max_total))
        r = self.runner
        K.sample(r.logits[slot: slot + 1], r.temps[slot: slot + 1], r.topks[slot: slot + 1], r.topps[slot: slot + 1], r.rng[slot: slot + 1],
                 out=r.tokens[slot: slot + 1])
        return self._read_tokens(1, slot)[0]

    def begin_sequence(self, prompt: Sequence[int], max_total: int, slot: int = 0, params: SamplingParams | None = None,
                       kv_format: str | None = None) -> int:
        """First half of :meth:`open_sequence` for callers that prefill in pieces (the scheduler interleaves prompt chunks
        with decode steps): binds pages for ``max_total`` tokens, attaches cached prefix pages and returns how many prompt
        tokens those pages already cover.  Continue with :meth:`prefill` over ``prompt[covered:]`` in as many pieces as
        wanted (``pos0`` = index of the piece's first token), then :meth:`finish_sequence`."""
        self._set_sampling(slot, params or self.sampling)
        prompt = [int(t) for t in prompt]
        kvt = self.kvt if kv_format is None else KV_NAMES[kv_format.lower()]
        if kvt not in self.runner.kv_pools:
            kvt = self.kvt                          # no pool in that format: the default one
        self._release_slot(slot)
        if kvt != self.kvt:
            self._slot_fmt[slot] = kvt
            self.runner.set_slot_format(slot, kvt)
        shared: list[int] = []
        pc = self.prefix_cache if kvt == self.kvt else None      # cached pages live in the default pool
        if pc is not None and len(prompt) > 1:
            shared = pc.lookup(prompt, max_tokens=len(prompt) - 1)
            if shared:
                self.kv.retain(shared)
                self._release_slot(slot)
                self._slot_pages[slot] = list(shared)
        try:
            self._bind_slot(slot, min(self.max_seq_len, max_total))
        except MemoryError:
            self._release_slot(slot)
            raise
        if shared:
            row = torch.tensor(self._slot_pages[slot], dtype=torch.int32)
            self.runner.block_table[slot, : len(row)].copy_(row.to(self.device))
        return len(shared) * self.kv.page_size

    def finish_sequence(self, prompt: Sequence[int], slot: int = 0, mask=None) -> int:
        """Second half of :meth:`open_sequence`: the whole prompt has been prefilled into ``slot``; registers its pages with
        the prefix cache and returns the first sampled token (restricted to ``mask`` when one is given)."""
        if self.prefix_cache is not None and slot not in self._slot_fmt:
            self.prefix_cache.insert([int(t) for t in prompt], self._slot_pages[slot])
        r = self.runner
        if mask is not None:
            self.set_mask(slot, mask)
        K.sample(r.logits[slot: slot + 1], r.temps[slot: slot + 1], r.topks[slot: slot + 1], r.topps[slot: slot + 1], r.rng[slot: slot + 1],
                 out=r.tokens[slot: slot + 1], allow_mask=r.allow_mask[slot: slot + 1] if mask is not None else None)
        return self._read_tokens(1, slot)[0]

    def step_batch(self, positions: Sequence[int], masks: dict | None = None) -> list[int]:
        """One decode step of the live sequences in slots 0..len(positions)-1 (slot i feeds its last sampled token at
        ``positions[i]``); returns the newly sampled token of every slot.  The positions go up from pinned memory and the
        tokens come back with the step's status word in one copy.  ``masks``: {slot: packed vocabulary mask} for the
        constrained sequences of the batch (the others may pick any token)."""
        B = len(positions)
        r = self.runner
        self._pos_host[:B] = torch.tensor(list(positions), dtype=torch.int32)
        r.positions[:B].copy_(self._pos_host[:B], non_blocking=True)
        for slot, m in (masks or {}).items():
            self.set_mask(slot, m)
        r.step(B, sample=True, masked=bool(masks))
        return self._read_tokens(B)

    supports_overlap = True

    def launch_batch(self, positions: Sequence[int]) -> None:
        """First half of :meth:`step_batch` (no masks): uploads the positions and enqueues the decode step of slots
        0..len(positions)-1 without waiting for it."""
        B = len(positions)
        r = self.runner
        self._pos_host[:B] = torch.tensor(list(positions), dtype=torch.int32)
        r.positions[:B].copy_(self._pos_host[:B], non_blocking=True)
        r.step(B, sample=True, masked=False)

    def collect_batch(self, batch: int) -> list[int]:
        """Second half: waits for the step launched last and returns its tokens (raises on an expired wait)."""
        return self._read_tokens(batch)

    def bind_thread(self) -> None:
        """Makes this engine's GPU the calling thread's current device (a scheduler thread calls it once)."""
        torch.cuda.set_device(self.device)

    def decode_one(self, token: int, pos: int) -> int:
        """Feeds ``token`` at position ``pos`` of slot 0 and returns the next sampled token."""
        self._upload(0, token, pos)
        self.runner.step(1, sample=True)
        return self._read_tokens(1)[0]

    def verify_greedy(self, tokens: Sequence[int], pos0: int, slot: int = 0) -> list[int]:
        """Greedy next-token choices of the model after each of ``tokens`` placed at positions pos0.. (one batched pass)."""
        t = torch.tensor([int(x) for x in tokens], dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        return self.runner.verify_greedy(t, slot, pos0).tolist()

    def verify_sampled(self, tokens: Sequence[int], pos0: int, draft_logits: torch.Tensor, temperature: float,
                       uniforms: Sequence[float], slot: int = 0) -> tuple[int, int]:
        """Rejection test of the drafted tokens ``tokens[1:]`` on the device: ``tokens`` (the last emitted token followed by the
        drafts) go through the model at positions pos0.. in one batched pass, and the logits of every position are compared
        with ``draft_logits`` (f32 [k, vocab], the distributions the drafts were drawn from) at ``temperature``.  Returns
        (number of accepted drafts, the token that follows them); only these two integers come back to the host."""
        t = torch.tensor([int(x) for x in tokens], dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        u = torch.tensor([float(x) for x in uniforms], dtype=torch.float32).pin_memory().to(self.device, non_blocking=True)
        logits = self.runner.verify_logits(t, slot, pos0)
        out = K.spec_verify(logits, draft_logits, t[1:], temperature, u)
        n, nxt = out.tolist()
        self.runner.check_status()
        return int(n), int(nxt)

    def move_slot(self, src: int, dst: int) -> None:
        """Moves a live sequence to another slot: block-table row, last token, position and sampler state.
        KV pages stay where they are (the block table references them)."""
        r = self.runner
        for t in (r.block_table, r.tokens, r.positions, r.temps, r.topks, r.topps, r.rng, r.allow_mask):
            t[dst].copy_(t[src], non_blocking=True)
        if src in self._masked:
            self._masked.discard(src)
            self._masked.add(dst)
            r.allow_mask[src].fill_(-1)
        else:
            self._masked.discard(dst)
        self._slot_pages[dst] = self._slot_pages.pop(src, [])
        fmt = self._slot_fmt.pop(src, None)
        if fmt is not None:
            self._slot_fmt[dst] = fmt
            r.set_slot_format(src, self.kvt)
        elif dst in self._slot_fmt:
            del self._slot_fmt[dst]
        r.set_slot_format(dst, fmt if fmt is not None else self.kvt)

    def close_sequence(self, slot: int = 0) -> None:
        self._release_slot(slot)

    def generate_seeded(self, prompt: Sequence[int], max_tokens: int, seed: int, params: SamplingParams | None = None) -> list[int]:
        from dataclasses import replace
        return self.generate(prompt, max_tokens, replace(params or self.sampling, seed=seed))

    # ---- introspection ----------------------------------------------------------------------------
    def model_info(self) -> dict:
        c = self.config
        return {"name": c.name, "arch": c.arch, "layers": c.layers, "hidden": c.hidden, "heads": c.heads, "kv_heads": c.kv_heads,
                "head_dim": c.head_dim, "intermediate": c.inter, "vocab": c.vocab, "context": c.context,
                "weight_bytes": self.weights.packed_bytes, "kv_bytes": self.kv.nbytes, "load_seconds": self.load_seconds,
                "weights_from_repack_cache": self.weights.from_cache}


def layer_weight_type(gguf: GgufFile) -> int:
    """GGUF type id of the first layer's attention projection (fused or split): what decides the GPU path of a checkpoint."""
    for name in ("blk.0.attn_q.weight", "blk.0.attn_qkv.weight", "blk.0.ffn_down.weight"):
        if gguf.has_tensor(name):
            return gguf.tensor_info(name).type
    raise ValueError("checkpoint has no blk.0 attention or FFN weights")


class GenericFormatEngine:
    """Engine for checkpoints whose layer weights are in a block format without a planar repack (Q4_0, Q8_0, FP8, the
    K-quants, 256-wide TQ2_0, F16 / BF16 / F32).

    Reference counterpart: the same ``InferenceEngine`` serves every format through per-format forward paths
    (crates/oxibonsai-model/src/model/types/forward_cuda/q_std.rs, k_quant.rs, forward_cuda_fp8.rs).  Here the
    sub-2-bit formats have their own runner (``InferenceEngine``) and everything else goes through
    ``models.qwen3_generic.GenericQwen3Engine``; this class gives it the engine surface: ``generate`` / ``generate_stream`` /
    ``generate_seeded`` / ``model_info`` / ``last_stats`` for one stream (serialised by a lock), and the sequence-slot
    interface (``begin_sequence`` ... ``step_batch``) through which the continuous-batching scheduler decodes up to
    ``max_batch`` sequences together."""

    def __init__(self, model_path: str, max_seq_len: int = 4096, max_batch: int = 1, kv_dtype: str = "f16",
                 device: str | torch.device = "cuda:0", sampling: SamplingParams | None = None, page_size: int = 64,
                 kv_pages: int | None = None, tp_rank: int = 0, tp_size: int = 1, warmup: bool = True, exact: bool | None = None,
                 repack_cache: str | None = None, prefill_chunk: int | None = None):      # the generic formats are used as stored: nothing to cache
        import threading
        from ..models.qwen3_generic import GenericQwen3Engine
        if tp_size != 1:
            raise NotImplementedError("tensor parallelism covers the Q1_0_g128 / TQ2_0_g128 runner only")
        kv = {"fp32": "f32", "fp16": "f16", "int8": "q8", "int4": "q4"}.get(kv_dtype.lower(), kv_dtype.lower())
        t0 = time.perf_counter()
        self.sampling = (sampling or SamplingPreset.BALANCED.params()).validate()
        self._eng = GenericQwen3Engine(str(model_path), max_seq_len=int(max_seq_len), kv_dtype=kv, device=str(device), page_size=page_size,
                                       sampling=self.sampling, max_batch=int(max_batch))
        self.load_seconds = time.perf_counter() - t0
        self.model_path, self.device = str(model_path), self._eng.device
        self.gguf, self.config = self._eng.gguf, self._eng.config
        self.max_seq_len, self.max_batch = int(max_seq_len), self._eng.max_batch
        self.prefill_min_tokens = self._eng.prefill_min_tokens
        self.exact = False
        self.last_stats = GenerationStats()
        self._lock = threading.Lock()
        if warmup:
            self.warmup()

    def warmup(self) -> None:
        """Captures the decode graph (one throw-away token) so that the first request does not pay for it."""
        with self._lock:
            self._eng.generate([0], 1, SamplingPreset.GREEDY.params(), stop_at_eos=False)

    # ---- sequence slots (the scheduler's interface; see InferenceEngine for the contract) -----------------------------------------
    def bind_thread(self) -> None:
        torch.cuda.set_device(self.device)

    def begin_sequence(self, prompt: Sequence[int], max_total: int, slot: int = 0, params: SamplingParams | None = None,
                       kv_format: str | None = None) -> int:
        return self._eng.begin_sequence(prompt, max_total, slot, params or self.sampling, kv_format)

    def prefill(self, prompt: Sequence[int], slot: int = 0, pos0: int = 0) -> None:
        self._eng.prefill_slot(prompt, slot, pos0)

    def finish_sequence(self, prompt: Sequence[int], slot: int = 0, mask=None) -> int:
        return self._eng.finish_sequence(prompt, slot, mask)

    def step_batch(self, positions: Sequence[int], masks: dict | None = None) -> list[int]:
        return self._eng.step_batch(positions, masks)

    def move_slot(self, src: int, dst: int) -> None:
        self._eng.move_slot(src, dst)

    def close_sequence(self, slot: int = 0) -> None:
        self._eng.close_sequence(slot)

    def kv_utilization(self) -> float:
        return self._eng.kv_utilization()

    def set_mask(self, slot: int, mask) -> None:
        self._eng.set_mask(slot, mask)

    def token_logprobs(self, slot: int, token: int, top_n: int = 0) -> tuple[float, list[tuple[int, float]]]:
        return self._eng.token_logprobs(slot, token, top_n)

    # ---- one stream ------------------------------------------------------------------------------------------------------------
    def generate_stream(self, prompt: Sequence[int], max_tokens: int | None = None, params: SamplingParams | None = None,
                        stop_at_eos: bool = True, on_token: Callable[[int], None] | None = None, constraint=None) -> Iterator[int]:
        p = (params or self.sampling).validate()
        max_new = p.max_tokens if max_tokens is None else max_tokens
        prompt = [int(t) for t in prompt]
        if not prompt:
            return
        stats = GenerationStats(prompt_tokens=len(prompt))
        self.last_stats = stats
        max_new = max(0, min(max_new, self.max_seq_len - len(prompt)))
        with self._lock:
            t0 = time.perf_counter()
            first = True
            for tok in self._eng.generate_stream(prompt, max_new, p, stop_at_eos, constraint):
                now = time.perf_counter()
                if first:
                    stats.prefill_seconds, t0, first = now - t0, now, False
                stats.generated_tokens += 1
                stats.token_times.append(now)
                if on_token is not None:
                    on_token(tok)
                yield tok
            stats.decode_seconds = time.perf_counter() - t0 if not first else 0.0

    def generate(self, prompt: Sequence[int], max_tokens: int | None = None, params: SamplingParams | None = None,
                 stop_at_eos: bool = True, constraint=None) -> list[int]:
        return list(self.generate_stream(prompt, max_tokens, params, stop_at_eos, constraint=constraint))

    def generate_seeded(self, prompt: Sequence[int], max_tokens: int, seed: int, params: SamplingParams | None = None) -> list[int]:
        from dataclasses import replace
        return self.generate(prompt, max_tokens, replace(params or self.sampling, seed=seed))

    def model_info(self) -> dict:
        from ..core import gguf as G
        from ..models.qwen3_generic import _Linear
        c, e = self.config, self._eng
        weight_bytes = sum(w.data.numel() for layer in e.layers for w in layer.values() if isinstance(w, _Linear))
        return {"name": c.name, "arch": c.arch, "layers": c.layers, "hidden": c.hidden, "heads": c.heads, "kv_heads": c.kv_heads,
                "head_dim": c.head_dim, "intermediate": c.inter, "vocab": c.vocab, "context": c.context, "weight_bytes": int(weight_bytes),
                "kv_bytes": int(e.kpool.numel() * e.kpool.element_size() * 2), "load_seconds": self.load_seconds,
                "weight_format": G.type_info(layer_weight_type(self.gguf))[0], "max_batch": self.max_batch}


def load_engine(model_path: str, **options):
    """``InferenceEngine`` for Q1_0_g128 / TQ2_0_g128 checkpoints, ``GenericFormatEngine`` for every other weight format."""
    from ..core import gguf as G
    with_type = layer_weight_type(GgufFile.open(str(model_path)))
    if with_type in (G.TQ2_0_G128, G.Q1_0_G128):
        return InferenceEngine(str(model_path), **options)
    return GenericFormatEngine(str(model_path), **options)
