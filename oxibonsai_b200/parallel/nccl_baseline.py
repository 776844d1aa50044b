"""Tensor-parallel decode step with library collectives: the baseline arm for the fused kernels.

Same engine, same weights, same per-layer kernels as the native tensor-parallel step, except that the two row-parallel
projections of a layer write their partial sums to local memory and ``torch.distributed.all_reduce`` (NCCL) combines them,
followed by a residual add, and the vocab-parallel LM head is gathered with ``all_gather_into_tensor``.  The whole step is
captured in one CUDA graph, like the native step.  Nothing here is on a serving path: ``bench.py`` times it beside the fused
step so that the value of fusing the exchange into the GEMV epilogue is a measured difference on the same box.

Reference counterpart: ``tensor_parallel_forward`` with ``NcclCollectives::all_reduce`` / ``all_gather``, which the
reference simulates on CPU threads (crates/oxibonsai-model/src/tensor_parallel.rs:338-386, multi_gpu.rs:159-238).
"""
from __future__ import annotations

import torch

from ..ops import cuda_ops as K


class NcclTpDecoder:
    """Batch-1 decode steps of a tensor-parallel :class:`~oxibonsai_b200.runtime.engine.InferenceEngine` (slot 0) with NCCL
    collectives in place of the fused GEMV -> all-reduce epilogues."""

    def __init__(self, engine):
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("the NCCL baseline needs an initialised process group")
        self.dist = dist
        self.eng, self.r, self.w = engine, engine.runner, engine.weights
        r, w, cfg = self.r, self.w, engine.config
        if any(lw.qkv_s16 is None for lw in w.layers):
            raise RuntimeError("the baseline uses the streamed GEMV: build the weights with decode_layout=True")
        dev = r.device
        self.rows_per_rank = (cfg.vocab + w.tp_size - 1) // w.tp_size
        self.partial = torch.zeros(cfg.hidden, dtype=torch.float32, device=dev)
        self.local_logits = torch.zeros(self.rows_per_rank, dtype=torch.float32, device=dev)
        self.all_logits = torch.zeros(w.tp_size * self.rows_per_rank, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._graph = None

    def step_eager(self) -> None:
        r, w, cfg, eng = self.r, self.w, self.eng.config, self.eng
        lib = K.lib()
        h, qkv, attn, act = r.h[0], r.qkv[:1], r.attn[:1], r.act[0]
        K.check(lib.bonsai_embed_f16(w.embd.data_ptr(), r.tokens.data_ptr(), h.data_ptr(), cfg.hidden, cfg.vocab, K.stream()), "embed")
        nq, nkv, hd = w.heads_local, w.kv_heads_local, cfg.head_dim
        for l, lw in enumerate(w.layers):
            K.bitgemv_s16(lw.qkv_s16, h, norm_w=lw.attn_norm, eps=cfg.eps, out=qkv[0], status=self.status)
            K.attn_decode_qkv(qkv, lw.q_norm, lw.k_norm, cfg.eps, r.rope_cos, r.rope_sin, r.positions[:1], r.block_table[:1], nq, nkv, hd,
                              r.kv.page_size, r.kv.k[l], r.kv.v[l], nsplit=r.nsplit, out=attn.view(1, nq, hd))
            K.bitgemv_s16(lw.o_s16, attn[0], out=self.partial, status=self.status)
            self.dist.all_reduce(self.partial)
            h.add_(self.partial)
            K.bitgemv_s16(lw.gate_up_s16, h, norm_w=lw.ffn_norm, eps=cfg.eps, epi=K.EPI_SWIGLU, out=act, status=self.status)
            K.bitgemv_s16(lw.down_s16, act, out=self.partial, status=self.status)
            self.dist.all_reduce(self.partial)
            h.add_(self.partial)
        n_local = w.lm_head.shape[0]
        if n_local:
            K.f16gemv(w.lm_head, h, w.out_norm, cfg.eps, out=self.local_logits[:n_local])
        self.dist.all_gather_into_tensor(self.all_logits, self.local_logits)
        K.sample(self.all_logits[: cfg.vocab].view(1, -1), out=r.tokens[:1], positions=r.positions[:1], advance=True)

    def step(self) -> None:
        """One decode step of slot 0, replayed from a CUDA graph after the first call."""
        if self._graph is None:
            tok0 = self.r.tokens[:1].clone()
            self.step_eager()                      # warm NCCL and the allocator outside the capture ...
            self.r.positions[:1].sub_(1)           # ... and take the step back: the replay below redoes it
            self.r.tokens[:1].copy_(tok0)
            torch.cuda.synchronize(self.r.device)
            g = K.capture_graph(self.r.device, self.step_eager)
            self._graph = g
        self._graph.replay()
