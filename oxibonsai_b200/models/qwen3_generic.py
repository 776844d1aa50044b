"""Qwen3 decoder for checkpoints in block formats without a planar repack (Q4_0, Q8_0, FP8, K-quants, 256-wide TQ2_0, F16,
BF16, F32): weights stay on the device exactly as stored in the GGUF file and every linear layer is the generic
decode GEMV (csrc/cuda/quant_gemv.cu).

Reference: the per-format GPU forward paths (crates/oxibonsai-model/src/model/types/forward_cuda/q_std.rs, k_quant.rs,
forward_cuda_fp8.rs) and their prefill variants (crates/oxibonsai-kernels/src/gpu_backend/cuda_q_std_prefill.rs,
cuda_k_quant_prefill/*, cuda_fp8_prefill.rs).  A decode step is ~12 launches per layer issued from Python and captured
once into a CUDA graph.  Prompts of at least ``prefill_min`` tokens run in chunks through the tensor cores: each weight
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
    def __init__(self, f: GgufFile, name: str, device):
        info = f.tensor_info(name)
        if info.type not in SUPPORTED:
            raise ValueError(f"{name}: type {info.type_name} is not handled by the generic path")
        self.type, (self.k, self.n) = info.type, info.dims
        self.data = torch.from_numpy(np.array(f.tensor_bytes(name), copy=True)).to(device)

    def __call__(self, x, norm_w=None, eps=1e-6, residual=None, out=None):
        return K.quant_gemv(self.type, self.data, self.n, self.k, x, norm_w, eps, residual, out)


class GenericQwen3Engine:
    def __init__(self, model_path: str, max_seq_len: int = 2048, kv_dtype: str = "f16", device: str = "cuda:0", page_size: int = 64,
                 sampling: SamplingParams | None = None, prefill_min: int = 16, prefill_chunk: int = 512):
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.gguf = GgufFile.open(model_path)
        self.config = c = self.gguf.config()
        self.max_seq_len = max_seq_len
        self.prefill_min, self.prefill_chunk = prefill_min, prefill_chunk
        self._wscratch = None
        self.sampling = sampling or SamplingPreset.GREEDY.params()
        f, dev = self.gguf, self.device
        self.kvt = {"f32": K.KV_F32, "f16": K.KV_F16, "q8": K.KV_Q8, "q4": K.KV_Q4}[kv_dtype]
        self.embd = _f16_matrix(f, "token_embd.weight", dev)
        head = "output.weight" if f.has_tensor("output.weight") else "token_embd.weight"
        self.lm_head = self.embd if head == "token_embd.weight" else _f16_matrix(f, head, dev)
        self.out_norm = _norm_vector(f, "output_norm.weight", dev)
        self.layers = []
        for l in range(c.layers):
            p = f"blk.{l}."
            self.layers.append(dict(
                q=_Linear(f, p + "attn_q.weight", dev), k=_Linear(f, p + "attn_k.weight", dev), v=_Linear(f, p + "attn_v.weight", dev),
                o=_Linear(f, p + "attn_output.weight", dev), gate=_Linear(f, p + "ffn_gate.weight", dev), up=_Linear(f, p + "ffn_up.weight", dev),
                down=_Linear(f, p + "ffn_down.weight", dev), attn_norm=_norm_vector(f, p + "attn_norm.weight", dev),
                ffn_norm=_norm_vector(f, p + "ffn_norm.weight", dev), q_norm=_norm_vector(f, p + "attn_q_norm.weight", dev),
                k_norm=_norm_vector(f, p + "attn_k_norm.weight", dev)))
        hd, nkv = c.head_dim, c.kv_heads
        self.page = page_size
        self.n_pages = (max_seq_len + page_size - 1) // page_size
        row = hd // 2 if self.kvt == K.KV_Q4 else hd
        shape = (c.layers, self.n_pages, nkv, page_size, row)
        self.kpool = torch.zeros(shape, dtype=K.KV_DTYPES[self.kvt], device=dev)
        self.vpool = torch.zeros_like(self.kpool)
        quant = self.kvt in (K.KV_Q8, K.KV_Q4)
        self.kscale = torch.zeros(shape[:-1], device=dev) if quant else None
        self.vscale = torch.zeros(shape[:-1], device=dev) if quant else None
        cos, sin = rope_table(hd, max_seq_len, c.rope_base)
        self.cos, self.sin = torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev)
        f32 = dict(dtype=torch.float32, device=dev)
        self.bt = torch.arange(self.n_pages, dtype=torch.int32, device=dev).view(1, -1)
        self.token = torch.zeros(1, dtype=torch.int32, device=dev)
        self.pos = torch.zeros(1, dtype=torch.int32, device=dev)
        self.h = torch.zeros(c.hidden, **f32)
        self.qkv = torch.zeros((1, (c.heads + 2 * nkv) * hd), **f32)
        self.q = torch.zeros((1, c.heads, hd), **f32)
        self.attn = torch.zeros((1, c.heads, hd), **f32)
        self.gate, self.up, self.act = (torch.zeros(c.inter, **f32) for _ in range(3))
        self.logits = torch.zeros((1, c.vocab), **f32)
        self.out_token = torch.zeros(1, dtype=torch.int32, device=dev)
        self.temps = torch.zeros(1, **f32)
        self.topks = torch.zeros(1, dtype=torch.int32, device=dev)
        self.topps = torch.ones(1, **f32)
        self.rng = torch.zeros(1, dtype=torch.int64, device=dev)
        self._graph = None
        self._host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.nsplit = max(1, min(32, 296 // nkv))

    def kernel_launches_per_step(self) -> int:
        return 12 * self.config.layers + 3

    def _step_eager(self) -> None:
        c, eps = self.config, self.config.eps
        qd, kvd = c.heads * c.head_dim, c.kv_heads * c.head_dim
        self.h.copy_(torch.index_select(self.embd, 0, self.token.long())[0].float())      # no host sync: capturable
        qkv = self.qkv[0]
        for l, w in enumerate(self.layers):
            w["q"](self.h, w["attn_norm"], eps, out=qkv[:qd])
            w["k"](self.h, w["attn_norm"], eps, out=qkv[qd:qd + kvd])
            w["v"](self.h, w["attn_norm"], eps, out=qkv[qd + kvd:])
            ks = self.kscale[l] if self.kscale is not None else None
            vs = self.vscale[l] if self.vscale is not None else None
            K.qknorm_rope_kvstore(self.qkv, w["q_norm"], w["k_norm"], eps, self.cos, self.sin, self.pos, self.bt, self.q, c.heads, c.kv_heads,
                                  c.head_dim, self.kvt, self.page, self.kpool[l], self.vpool[l], ks, vs)
            K.attn_decode(self.q, self.pos, self.bt, c.heads, c.kv_heads, c.head_dim, self.kvt, self.page, self.kpool[l], self.vpool[l], ks, vs,
                          nsplit=self.nsplit, out=self.attn)
            w["o"](self.attn.view(-1), residual=self.h, out=self.h)
            w["gate"](self.h, w["ffn_norm"], eps, out=self.gate)
            w["up"](self.h, w["ffn_norm"], eps, out=self.up)
            K.swiglu(self.gate, self.up, out=self.act)
            w["down"](self.act, residual=self.h, out=self.h)
        K.f16gemv(self.lm_head, self.h, self.out_norm, eps, out=self.logits[0])
        K.sample(self.logits, self.temps, self.topks, self.topps, self.rng, positions=self.pos, advance=True, out=self.out_token)

    def prefill_supported(self) -> bool:
        """The tensor-core prompt path needs every matrix width to be a multiple of 128 and a head size the prompt attention has."""
        c = self.config
        return c.hidden % 128 == 0 and c.inter % 128 == 0 and (c.heads * c.head_dim) % 128 == 0 and c.head_dim in (64, 128)

    def prefill(self, tokens: torch.Tensor, pos0: int = 0) -> None:
        """Runs ``tokens`` (int32 on the device) through every layer as chunks of up to ``prefill_chunk`` tokens, filling the KV
        cache for positions pos0 .. pos0 + len - 1.  Nothing is sampled: the caller feeds the prompt's last token to ``step``."""
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
            bt = self.bt.expand(T, -1).contiguous()
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
                a16 = K.attn_prefill(q, p0, self.bt[0], c.heads, c.kv_heads, c.head_dim, self.kvt, self.page, self.kpool[l], self.vpool[l], ks, vs)
                mm(w["o"], a16, h, residual=h)
                xn = K.norm_to_f16_paired(h, w["ffn_norm"], eps)
                mm(w["gate"], xn, gate)
                mm(w["up"], xn, up)
                K.swiglu(gate, up, out=act)
                mm(w["down"], K.norm_to_f16_paired(act, None, eps), h, residual=h)
            done += T

    def step(self) -> None:
        """One token through the model (token and position are read from device buffers); replays a captured graph."""
        if self._graph is None:
            self._step_eager()                      # warm-up: loads every kernel before capture
            self.pos.sub_(1)
            torch.cuda.synchronize(self.device)
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(s):
                with torch.cuda.graph(g, stream=s):
                    self._step_eager()
            torch.cuda.current_stream(self.device).wait_stream(s)
            self._graph = g
        self._graph.replay()

    def _set_sampling(self, p: SamplingParams) -> None:
        self.temps.fill_(float(p.temperature))
        self.topks.fill_(int(p.top_k))
        self.topps.fill_(float(p.top_p))
        seed = int(p.seed) & 0xFFFFFFFFFFFFFFFF
        self.rng.fill_(seed - (1 << 64) if seed >= (1 << 63) else seed)

    def generate_stream(self, prompt: Sequence[int], max_tokens: int, params: SamplingParams | None = None, stop_at_eos: bool = True) -> Iterator[int]:
        p = (params or self.sampling).validate()
        prompt = [int(t) for t in prompt]
        if not prompt or len(prompt) >= self.max_seq_len:
            raise ValueError("prompt must be non-empty and shorter than max_seq_len")
        if self._graph is None:        # capture before the sampler state of this request is set
            self.pos.zero_()
            self.step()
        self._set_sampling(p)
        toks = torch.tensor(prompt, dtype=torch.int32).pin_memory().to(self.device, non_blocking=True)
        self.pos.zero_()
        first = 0
        if len(prompt) - 1 >= self.prefill_min and self.prefill_supported():
            first = len(prompt) - 1                      # the last prompt token goes through the decode step, which samples
            self.prefill(toks[:first])
            self.pos.fill_(first)
        for i in range(first, len(prompt)):
            self.token.copy_(toks[i:i + 1], non_blocking=True)
            self.step()
        for _ in range(max_tokens):
            self._host.copy_(self.out_token, non_blocking=True)
            torch.cuda.synchronize(self.device)
            tok = int(self._host[0])
            if stop_at_eos and tok == EOS_TOKEN:
                break
            yield tok
            if int(self.pos.item()) >= self.max_seq_len:
                break
            self.token.copy_(self.out_token)
            self.step()

    def generate(self, prompt: Sequence[int], max_tokens: int, params: SamplingParams | None = None, stop_at_eos: bool = True) -> list[int]:
        return list(self.generate_stream(prompt, max_tokens, params, stop_at_eos))
