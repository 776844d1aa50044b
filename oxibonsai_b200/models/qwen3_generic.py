"""Qwen3 decoder for checkpoints in block formats without a planar repack (Q4_0, Q8_0, FP8, K-quants, 256-wide TQ2_0, F16,
BF16, F32): weights stay on the device exactly as stored in the GGUF file and every linear layer is the generic
decode GEMV (csrc/cuda/quant_gemv.cu).

Reference: the per-format GPU forward paths (crates/oxibonsai-model/src/model/types/forward_cuda/q_std.rs, k_quant.rs,
forward_cuda_fp8.rs) and their prefill variants (crates/oxibonsai-kernels/src/gpu_backend/cuda_q_std_prefill.rs,
cuda_k_quant_prefill/*, cuda_fp8_prefill.rs).  Q / K / V and gate / up are stored as one matrix each where their block
types agree (rows of a block format concatenate byte for byte), so a decode step is 9 launches per layer, issued from
Python and captured once per batch size into a CUDA graph.  Up to ``max_batch`` sequences decode together: the batched
GEMV decodes every weight once and multiplies it into up to eight activation rows, and attention, KV append and the sampler
are the batch kernels of the native engine.  The engine has the slot interface the continuous-batching scheduler drives
(``begin_sequence`` / ``prefill`` / ``finish_sequence`` / ``step_batch`` / ``move_slot`` / ``close_sequence``).  Prompts of at least ``prefill_min`` tokens run in chunks through the tensor cores: each weight
matrix is decoded once per chunk into an f16 scratch matrix (csrc/cuda/quant_gemv.cu, bonsai_quant_to_f16) and multiplied
by all the chunk's tokens with the dense tcgen05 GEMM, with the prompt-attention kernel of the native engine in between;
shorter prompts go through the decode step token by token (all f32).  Attention, KV append, LM head and sampler are the
kernels of the native engine.  The sub-2-bit formats (Q1_0_g128, TQ2_0_g128) should use
``oxibonsai_b200.runtime.InferenceEngine``, which is several times faster.
"""
from __future__ import annotations

from typing import Iterator, Sequence

import numpy as np
import torch

from ..core import gguf as G
from ..core.gguf import GgufFile
from ..core.oracle import EOS_TOKEN, rope_table
from ..ops import cuda_ops as K
from ..runtime.presets import SamplingParams, SamplingPreset
from .qwen3 import _f16_matrix, _norm_vector

SUPPORTED = (G.F32, G.F16, G.BF16, G.Q4_0, G.Q8_0, G.TQ2_0, G.F8_E4M3, G.F8_E5M2, G.Q2_K, G.Q3_K, G.Q4_K, G.Q5_K, G.Q6_K, G.Q8_K)


class _Linear:
    """A matrix kept in its GGUF block format: ``data`` holds the rows byte for byte."""

    def __init__(self, type_id: int, n: int, k: int, data: torch.Tensor):
        self.type, self.n, self.k, self.data = type_id, n, k, data

    @classmethod
    def from_gguf(cls, f: GgufFile, name: str, device) -> "_Linear":
        info = f.tensor_info(name)
        if info.type not in SUPPORTED:
            raise ValueError(f"{name}: type {info.type_name} is not handled by the generic path")
        k, n = info.dims
        return cls(info.type, n, k, torch.from_numpy(np.array(f.tensor_bytes(name), copy=True)).to(device))

    @staticmethod
    def fuse(parts: Sequence["_Linear"]) -> list["_Linear"]:
        """Concatenates neighbouring matrices of one block type and width into one (their rows are independent byte
        strings, so the fused matrix is the concatenation of the bytes); parts of different types stay separate."""
        out: list[_Linear] = []
        for p in parts:
            if out and out[-1].type == p.type and out[-1].k == p.k:
                a = out[-1]
                out[-1] = _Linear(a.type, a.n + p.n, a.k, torch.cat([a.data, p.data]))
            else:
                out.append(p)
        return out

    def __call__(self, x, norm_w=None, eps=1e-6, residual=None, out=None):
        if x.dim() == 1:
            return K.quant_gemv(self.type, self.data, self.n, self.k, x, norm_w, eps, residual, out)
        return K.quant_gemv_batched(self.type, self.data, self.n, self.k, x, norm_w, eps, residual, out)


def _project(mats: Sequence[_Linear], x: torch.Tensor, norm_w, eps: float, out: torch.Tensor) -> None:
    """out[:, columns of mats[i]] = mats[i] (rmsnorm(x)) for a list of matrices that share the input."""
    c0 = 0
    for m in mats:
        m(x, norm_w, eps, out=out[:, c0:c0 + m.n])
        c0 += m.n


class GenericQwen3Engine:
    def __init__(self, model_path: str, max_seq_len: int = 2048, kv_dtype: str = "f16", device: str = "cuda:0", page_size: int = 64,
                 sampling: SamplingParams | None = None, prefill_min: int = 16, prefill_chunk: int = 512, max_batch: int = 1):
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.gguf = GgufFile.open(model_path)
        self.config = c = self.gguf.config()
        self.max_seq_len, self.max_batch = max_seq_len, max(1, int(max_batch))
        self.prefill_min, self.prefill_chunk = prefill_min, prefill_chunk
        self.prefill_min_tokens = prefill_min          # the name the scheduler reads
        self._wscratch = None
        self.sampling = sampling or SamplingPreset.GREEDY.params()
        f, dev, B = self.gguf, self.device, self.max_batch
        self.kvt = {"f32": K.KV_F32, "f16": K.KV_F16, "q8": K.KV_Q8, "q4": K.KV_Q4}[kv_dtype]
        self.embd = _f16_matrix(f, "token_embd.weight", dev)
        head = "output.weight" if f.has_tensor("output.weight") else "token_embd.weight"
        self.lm_head = self.embd if head == "token_embd.weight" else _f16_matrix(f, head, dev)
        self.out_norm = _norm_vector(f, "output_norm.weight", dev)
        self.layers = []
        for l in range(c.layers):
            p = f"blk.{l}."
            lin = lambda n: _Linear.from_gguf(f, p + n + ".weight", dev)
            q, k, v, gate, up = lin("attn_q"), lin("attn_k"), lin("attn_v"), lin("ffn_gate"), lin("ffn_up")
            self.layers.append(dict(
                q=q, k=k, v=v, gate=gate, up=up, o=lin("attn_output"), down=lin("ffn_down"),
                qkv=_Linear.fuse([q, k, v]), gate_up=_Linear.fuse([gate, up]),     # fused where the block types agree
                attn_norm=_norm_vector(f, p + "attn_norm.weight", dev), ffn_norm=_norm_vector(f, p + "ffn_norm.weight", dev),
                q_norm=_norm_vector(f, p + "attn_q_norm.weight", dev), k_norm=_norm_vector(f, p + "attn_k_norm.weight", dev)))
            lw = self.layers[-1]
            if len(lw["qkv"]) == 1:            # the fused matrix replaces its parts (the prompt path slices it by rows)
                lw["q"], lw["k"], lw["v"] = self._row_views(lw["qkv"][0], [q.n, k.n, v.n])
            if len(lw["gate_up"]) == 1:
                lw["gate"], lw["up"] = self._row_views(lw["gate_up"][0], [gate.n, up.n])
        hd, nkv = c.head_dim, c.kv_heads
        self.page = page_size
        self.n_pages = (max_seq_len + page_size - 1) // page_size       # pages of one sequence
        row = hd // 2 if self.kvt == K.KV_Q4 else hd
        shape = (c.layers, self.n_pages * B, nkv, page_size, row)
        self.kpool = torch.zeros(shape, dtype=K.KV_DTYPES[self.kvt], device=dev)
        self.vpool = torch.zeros_like(self.kpool)
        quant = self.kvt in (K.KV_Q8, K.KV_Q4)
        self.kscale = torch.zeros(shape[:-1], device=dev) if quant else None
        self.vscale = torch.zeros(shape[:-1], device=dev) if quant else None
        cos, sin = rope_table(hd, max_seq_len, c.rope_base)
        self.cos, self.sin = torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev)
        f32 = dict(dtype=torch.float32, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        # a sequence owns one range of n_pages pages; ranges move with their sequence when the scheduler compacts slots
        self._free_ranges = list(range(B - 1, -1, -1))
        self._slot_range: dict[int, int] = {}
        self.bt = torch.zeros((B, self.n_pages), **i32)
        self.token = torch.zeros(B, **i32)          # last token of every slot: input of a step, and where the sampler writes
        self.pos = torch.zeros(B, **i32)
        self.h = torch.zeros((B, c.hidden), **f32)
        self.qkv = torch.zeros((B, (c.heads + 2 * nkv) * hd), **f32)
        self.q = torch.zeros((B, c.heads, hd), **f32)
        self.attn = torch.zeros((B, c.heads, hd), **f32)
        self.gu = torch.zeros((B, 2 * c.inter), **f32)
        self.act = torch.zeros((B, c.inter), **f32)
        self.logits = torch.zeros((B, c.vocab), **f32)
        self.temps = torch.zeros(B, **f32)
        self.topks = torch.zeros(B, **i32)
        self.topps = torch.ones(B, **f32)
        self.rng = torch.zeros(B, dtype=torch.int64, device=dev)
        self.mask_words = (c.vocab + 31) // 32
        self.allow_mask = torch.full((B, self.mask_words), -1, **i32)
        self._masked: set[int] = set()
        self._graphs: dict[tuple[int, bool], torch.cuda.CUDAGraph] = {}
        self._host = torch.zeros(B, dtype=torch.int32).pin_memory()
        self._pos_host = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.nsplit = max(1, min(32, 296 // nkv))

    @staticmethod
    def _row_views(m: _Linear, rows: Sequence[int]) -> list[_Linear]:
        per_row = m.data.numel() // m.n
        out, r0 = [], 0
        for n in rows:
            out.append(_Linear(m.type, n, m.k, m.data[r0 * per_row:(r0 + n) * per_row]))
            r0 += n
        return out

    # ---- slots ---------------------------------------------------------------------------------------------------------------
    def _bind(self, slot: int) -> None:
        if slot in self._slot_range:
            return
        if not self._free_ranges:
            raise MemoryError("KV cache exhausted: every sequence range is in use")
        r = self._free_ranges.pop()
        self._slot_range[slot] = r
        self.bt[slot].copy_(torch.arange(r * self.n_pages, (r + 1) * self.n_pages, dtype=torch.int32), non_blocking=False)

    def _unbind(self, slot: int) -> None:
        r = self._slot_range.pop(slot, None)
        if r is not None:
            self._free_ranges.append(r)

    def kv_utilization(self) -> float:
        return len(self._slot_range) / self.max_batch

    def kernel_launches_per_step(self, batch: int = 1) -> int:
        lw = self.layers[0]
        groups = -(-batch // 8)          # the batched GEMV takes eight rows per launch
        per_layer = 5 + groups * (len(lw["qkv"]) + len(lw["gate_up"]) + 2)       # rope/KV store, attention (3), SwiGLU + projections
        return per_layer * self.config.layers + 3 + batch + 1                    # embedding (3), LM head per row, sampler

    # ---- forward ---------------------------------------------------------------------------------------------------------------
    def _forward(self, lo: int, hi: int, sample: bool, masked: bool = False) -> None:
        """One token for each of the slots lo .. hi-1 (token and position are read from the device buffers): writes their
        logits and, with ``sample``, their next tokens into ``self.token`` and advances their positions."""
        c, eps = self.config, self.config.eps
        s = slice(lo, hi)
        h, qkv, pos, bt = self.h[s], self.qkv[s], self.pos[s], self.bt[s]
        h.copy_(torch.index_select(self.embd, 0, self.token[s].long()).float())      # no host sync: capturable
        for l, w in enumerate(self.layers):
            _project(w["qkv"], h, w["attn_norm"], eps, qkv)
            ks = self.kscale[l] if self.kscale is not None else None
            vs = self.vscale[l] if self.vscale is not None else None
            K.qknorm_rope_kvstore(qkv, w["q_norm"], w["k_norm"], eps, self.cos, self.sin, pos, bt, self.q[s], c.heads, c.kv_heads,
                                  c.head_dim, self.kvt, self.page, self.kpool[l], self.vpool[l], ks, vs)
            K.attn_decode(self.q[s], pos, bt, c.heads, c.kv_heads, c.head_dim, self.kvt, self.page, self.kpool[l], self.vpool[l], ks, vs,
                          nsplit=self.nsplit, out=self.attn[s])
            w["o"](self.attn[s].view(hi - lo, -1), residual=h, out=h)
            _project(w["gate_up"], h, w["ffn_norm"], eps, self.gu[s])
            K.swiglu_rows(self.gu[s], c.inter, out=self.act[s])
            w["down"](self.act[s], residual=h, out=h)
        for b in range(lo, hi):
            K.f16gemv(self.lm_head, self.h[b], self.out_norm, eps, out=self.logits[b])
        if sample:
            K.sample(self.logits[s], self.temps[s], self.topks[s], self.topps[s], self.rng[s], positions=pos, advance=True,
                     allow_mask=self.allow_mask[s] if masked else None, out=self.token[s])

    # kept for callers of the single-stream engine
    def _step_eager(self) -> None:
        self._forward(0, 1, True)

    def prefill_supported(self) -> bool:
        """The tensor-core prompt path needs every matrix width to be a multiple of 128 and a head size the prompt attention has."""
        c = self.config
        return c.hidden % 128 == 0 and c.inter % 128 == 0 and (c.heads * c.head_dim) % 128 == 0 and c.head_dim in (64, 128)

    def prefill(self, tokens: torch.Tensor, pos0: int = 0, slot: int = 0) -> None:
        """Runs ``tokens`` (int32 on the device) of the sequence in ``slot`` through every layer as chunks of up to
        ``prefill_chunk`` tokens, filling the KV cache for positions pos0 .. pos0 + len - 1.  Nothing is sampled and no logits
        are left: the caller feeds the prompt's last token through ``_forward``."""
        c, eps, dev = self.config, self.config.eps, self.device
        qd, kvd = c.heads * c.head_dim, c.kv_heads * c.head_dim
        if self._wscratch is None:
            self._wscratch = torch.empty(max(c.hidden * c.inter, qd * c.hidden), dtype=torch.float16, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)

        def mm(lin: _Linear, x16: torch.Tensor, out: torch.Tensor, residual: torch.Tensor | None = None) -> None:
            w16 = K.quant_to_f16(lin.type, lin.data, lin.n, lin.k, out=self._wscratch[: lin.n * lin.k].view(lin.n, lin.k), paired=True)
            K.dense_gemm_f16(w16, x16, out=out, residual=residual)

        done = 0
        while done < tokens.numel():
            T = min(self.prefill_chunk, tokens.numel() - done)
            p0 = pos0 + done
            h = torch.index_select(self.embd, 0, tokens[done:done + T].long()).float()
            positions = torch.arange(p0, p0 + T, dtype=torch.int32, device=dev)
            bt = self.bt[slot:slot + 1].expand(T, -1).contiguous()
            qkv = torch.empty((T, qd + 2 * kvd), **f32)
            q = torch.empty((T, c.heads, c.head_dim), **f32)
            gate, up, act = (torch.empty((T, c.inter), **f32) for _ in range(3))
            for l, w in enumerate(self.layers):
                xn = K.norm_to_f16_paired(h, w["attn_norm"], eps)
                mm(w["q"], xn, qkv[:, :qd])
                mm(w["k"], xn, qkv[:, qd:qd + kvd])
                mm(w["v"], xn, qkv[:, qd + kvd:])
                ks = self.kscale[l] if self.kscale is not None else None
                vs = self.vscale[l] if self.vscale is not None else None
                K.qknorm_rope_kvstore(qkv, w["q_norm"], w["k_norm"], eps, self.cos, self.sin, positions, bt, q, c.heads, c.kv_heads, c.head_dim,
                                      self.kvt, self.page, self.kpool[l], self.vpool[l], ks, vs)
                a16 = K.attn_prefill(q, p0, self.bt[slot], c.heads, c.kv_heads, c.head_dim, self.kvt, self.page, self.kpool[l], self.vpool[l], ks, vs)
                mm(w["o"], a16, h, residual=h)
                xn = K.norm_to_f16_paired(h, w["ffn_norm"], eps)
                mm(w["gate"], xn, gate)
                mm(w["up"], xn, up)
                K.swiglu(gate, up, out=act)
                mm(w["down"], K.norm_to_f16_paired(act, None, eps), h, residual=h)
            done += T

    def step(self, batch: int = 1, masked: bool = False) -> None:
        """One token for the first ``batch`` slots (tokens and positions are read from device buffers); replays a graph
        captured once per (batch, masked)."""
        key = (batch, masked)
        g = self._graphs.get(key)
        if g is None:
            if not self._graphs:                    # the first capture: load every kernel before it, on slot 0, then undo the step
                tok0, pos0, rng0 = self.token[:1].clone(), self.pos[:1].clone(), self.rng[:1].clone()
                self._forward(0, 1, True)
                self.token[:1].copy_(tok0)
                self.pos[:1].copy_(pos0)
                self.rng[:1].copy_(rng0)
                torch.cuda.synchronize(self.device)
            g = K.capture_graph(self.device, lambda: self._forward(0, batch, True, masked))
            self._graphs[key] = g
        g.replay()

    # ---- sequence slots: the interface the continuous-batching scheduler drives ----------------------------------------------------
    def _set_sampling(self, p: SamplingParams, slot: int = 0) -> None:
        self.temps[slot] = float(p.temperature)
        self.topks[slot] = int(p.top_k)
        self.topps[slot] = float(p.top_p)
        seed = int(p.seed) & 0xFFFFFFFFFFFFFFFF
        self.rng[slot] = seed - (1 << 64) if seed >= (1 << 63) else seed

    def set_mask(self, slot: int, mask) -> None:
        """Vocabulary mask of ``slot`` (packed uint32, bit set = allowed) for the masked steps that follow; None = every token."""
        if mask is None:
            if slot in self._masked:
                self.allow_mask[slot].fill_(-1)
                self._masked.discard(slot)
            return
        self._masked.add(slot)
        m = np.zeros(self.mask_words, dtype=np.uint32)
        src = np.asarray(mask, dtype=np.uint32)[: self.mask_words]
        m[: src.size] = src
        self.allow_mask[slot].copy_(torch.from_numpy(m.view(np.int32)).pin_memory(), non_blocking=True)

    def begin_sequence(self, prompt: Sequence[int], max_total: int, slot: int = 0, params: SamplingParams | None = None,
                       kv_format: str | None = None) -> int:
        """Binds a page range to ``slot`` and sets its sampler; returns how many prompt tokens are already in the cache (none:
        this engine has no prefix cache)."""
        if not prompt or len(prompt) >= self.max_seq_len:
            raise ValueError("prompt must be non-empty and shorter than max_seq_len")
        if not 0 <= slot < self.max_batch:
            raise ValueError(f"slot {slot} outside max_batch {self.max_batch}")
        self._bind(slot)
        self._set_sampling((params or self.sampling).validate(), slot)
        return 0

    def prefill_slot(self, tokens: Sequence[int], slot: int = 0, pos0: int = 0) -> None:
        """Feeds prompt tokens at positions pos0.. of ``slot`` and leaves the logits of the last one in ``logits[slot]``: all
        but the last through the tensor-core prompt path when there are enough of them, the last through the decode kernels."""
        n = len(tokens)
        if n == 0:
            return
        toks = torch.tensor([int(t) for t in tokens], dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        first = 0
        if n - 1 >= self.prefill_min and self.prefill_supported():
            first = n - 1
            self.prefill(toks[:first], pos0, slot)
        for i in range(first, n):
            self.token[slot:slot + 1].copy_(toks[i:i + 1], non_blocking=True)
            self.pos[slot] = pos0 + i
            self._forward(slot, slot + 1, False)

    def finish_sequence(self, prompt: Sequence[int], slot: int = 0, mask=None) -> int:
        """Samples the first token of ``slot`` from the logits the prompt left; the slot is then ready for ``step_batch``."""
        if mask is not None:
            self.set_mask(slot, mask)
        s = slice(slot, slot + 1)
        K.sample(self.logits[s], self.temps[s], self.topks[s], self.topps[s], self.rng[s], out=self.token[s],
                 allow_mask=self.allow_mask[s] if mask is not None else None)
        self.pos[slot] = len(prompt)
        return int(self.token[slot].item())

    def step_batch(self, positions: Sequence[int], masks: dict | None = None) -> list[int]:
        """One decode step for slots 0 .. len(positions)-1; returns their sampled tokens."""
        b = len(positions)
        for i, p in enumerate(positions):
            self._pos_host[i] = int(p)
        self.pos[:b].copy_(self._pos_host[:b], non_blocking=True)
        masked = bool(masks) or any(s < b for s in self._masked)
        if masks:
            for s, m in masks.items():
                self.set_mask(s, m)
        self.step(b, masked)
        self._host[:b].copy_(self.token[:b], non_blocking=True)
        torch.cuda.synchronize(self.device)
        return self._host[:b].tolist()

    def move_slot(self, src: int, dst: int) -> None:
        for t in (self.bt, self.token, self.pos, self.temps, self.topks, self.topps, self.rng, self.allow_mask):
            t[dst].copy_(t[src], non_blocking=True)
        self._unbind(dst)
        if src in self._slot_range:
            self._slot_range[dst] = self._slot_range.pop(src)
        if src in self._masked:
            self._masked.discard(src)
            self._masked.add(dst)
            self.allow_mask[src].fill_(-1)

    def close_sequence(self, slot: int = 0) -> None:
        self.set_mask(slot, None)
        self._unbind(slot)

    def token_logprobs(self, slot: int, token: int, top_n: int = 0) -> tuple[float, list[tuple[int, float]]]:
        lp = torch.log_softmax(self.logits[slot, : self.config.vocab].float(), dim=-1)
        top = []
        if top_n > 0:
            v, i = torch.topk(lp, min(top_n, lp.numel()))
            top = list(zip(i.tolist(), v.tolist()))
        return float(lp[int(token)]), top

    # ---- single stream -------------------------------------------------------------------------------------------------------------
    def generate_stream(self, prompt: Sequence[int], max_tokens: int, params: SamplingParams | None = None, stop_at_eos: bool = True,
                        constraint=None) -> Iterator[int]:
        p = (params or self.sampling).validate()
        prompt = [int(t) for t in prompt]
        if (1, False) not in self._graphs:        # capture before the sampler state of this request is set
            self._bind(0)
            self.pos[:1].zero_()
            self.step(1)
        self.begin_sequence(prompt, min(self.max_seq_len, len(prompt) + max_tokens), 0, p)
        try:
            self.prefill_slot(prompt, 0, 0)
            masked = constraint is not None
            if masked:
                constraint.reset()
            tok = self.finish_sequence(prompt, 0, constraint.allowed_mask() if masked else None)
            pos = len(prompt)
            for _ in range(max_tokens):
                if stop_at_eos and tok == EOS_TOKEN:
                    break
                yield tok
                if masked:
                    constraint.advance(tok)
                    if constraint.finished():
                        break
                if pos >= self.max_seq_len:
                    break
                tok = self.step_batch([pos], {0: constraint.allowed_mask()} if masked else None)[0]
                pos += 1
        finally:
            self.close_sequence(0)

    def generate(self, prompt: Sequence[int], max_tokens: int, params: SamplingParams | None = None, stop_at_eos: bool = True,
                 constraint=None) -> list[int]:
        return list(self.generate_stream(prompt, max_tokens, params, stop_at_eos, constraint))
