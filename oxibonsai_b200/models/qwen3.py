"""Qwen3 decoder on the GPU: weight loading / repacking and the native step runner.

Capability map to the reference: ``BonsaiModel::from_gguf`` + ``upload_weights_to_gpu``
(crates/oxibonsai-model/src/model/types/mod.rs:71-142,210), the fused QKV / gate-up weight handles
(block/types/upload.rs:8-39), the FP16 KV cache and activation buffers of the CUDA path
(crates/oxibonsai-kernels/src/gpu_backend/cuda_full_layer/mod.rs:112-205) and the captured whole-model
graph (encode_ternary.rs:546-660).  Differences by design: weights are repacked once into the
planar-SM layout, q/k/v rows are concatenated and gate/up rows interleaved so each is one launch,
the KV cache is paged, and every per-step scalar (token, position, sampler state) stays on the
device so one CUDA graph covers embed -> layers -> LM head -> sampler.
"""
from __future__ import annotations

import os

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from ..core import gguf as G
from ..core.gguf import GgufFile, Qwen3Config
from ..core.oracle import rope_table
from ..ops import cuda_ops as K
from ..ops import nvtx

_QUANT_TYPES = (G.TQ2_0_G128, G.Q1_0_G128)


@dataclass
class LayerWeights:
    qkv: K.PlanarWeight
    o: K.PlanarWeight
    gate_up: K.PlanarWeight
    down: K.PlanarWeight
    attn_norm: torch.Tensor
    ffn_norm: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    # the same four matrices in the streamed decode layout (None when not built)
    qkv_s16: "K.S16Weight | None" = None
    o_s16: "K.S16Weight | None" = None
    gate_up_s16: "K.S16Weight | None" = None
    down_s16: "K.S16Weight | None" = None


def _upload(arr: np.ndarray, device) -> torch.Tensor:
    """Host bytes -> device uint8 tensor through a pinned staging copy."""
    t = torch.from_numpy(np.array(arr, copy=True))
    if device.type == "cuda":
        t = t.pin_memory().to(device, non_blocking=True)
    return t


def _norm_vector(f: GgufFile, name: str, device) -> torch.Tensor:
    info = f.tensor_info(name)
    raw = f.tensor_bytes(name)
    if info.type == G.F32:
        v = np.frombuffer(raw, dtype=np.float32)
    elif info.type == G.F16:
        v = np.frombuffer(raw, dtype=np.float16).astype(np.float32)
    else:
        from ..core.blocks import dequantize
        v = dequantize(info.type, raw)
    return torch.from_numpy(np.array(v, copy=True)).to(device)


def _f16_matrix(f: GgufFile, name: str, device, row0: int = 0, nrows: int | None = None) -> torch.Tensor:
    """Loads an embedding / LM-head matrix as f16 [rows, cols] (dequantising other storage types on the host)."""
    info = f.tensor_info(name)
    cols, rows = info.dims
    nrows = rows - row0 if nrows is None else nrows
    raw = f.tensor_bytes(name)
    if info.type == G.F16:
        m = np.frombuffer(raw, dtype=np.float16).reshape(rows, cols)[row0:row0 + nrows]
        return _upload(m.view(np.uint8), device).view(torch.float16).reshape(nrows, cols)
    if info.type == G.F32:
        m = np.frombuffer(raw, dtype=np.float32).reshape(rows, cols)[row0:row0 + nrows].astype(np.float16)
    else:
        from ..core.blocks import dequantize
        _, be, bb = G.type_info(info.type)
        rb = cols // be * bb
        m = dequantize(info.type, raw[row0 * rb:(row0 + nrows) * rb]).reshape(nrows, cols).astype(np.float16)
    return torch.from_numpy(np.ascontiguousarray(m)).to(device)


class Qwen3Weights:
    """Device-resident weights of one tensor-parallel rank."""

    REPACK_LAYOUT = "planar-sm+s16-v1"

    def __init__(self, f: GgufFile, device, tp_rank: int = 0, tp_size: int = 1, decode_layout: bool = True,
                 cache_dir: str | None = None, source_path: str | None = None):
        """``decode_layout``: also build the S16 form of every layer matrix, which the batch-1 decode GEMV streams
        (the planar form stays: the prompt and batched GEMMs read it).

        ``cache_dir`` (with ``source_path``, the GGUF file ``f`` was opened from): directory of the repacked-weight cache.
        The device layouts of this rank's shard are written there once, under a key made of the file's identity, the
        layout version and the tensor-parallel coordinates; a later start reads them back instead of decoding and
        repacking the GGUF tensors (the counterpart of the reference's quantised-tensor disk cache,
        crates/oxibonsai-model/src/disk_cache.rs:7-19,277)."""
        cfg = f.config()
        self.cfg = cfg
        self.device = torch.device(device)
        self.tp_rank, self.tp_size = tp_rank, tp_size
        if cfg.heads % tp_size or cfg.kv_heads % tp_size:
            raise ValueError(f"tp_size {tp_size} must divide heads {cfg.heads} and kv_heads {cfg.kv_heads}")
        self.heads_local = cfg.heads // tp_size
        self.kv_heads_local = cfg.kv_heads // tp_size
        nblk_inter = cfg.inter // 128
        # split the intermediate dimension on 128-weight block boundaries (sizes may differ by one block)
        base, extra = divmod(nblk_inter, tp_size)
        counts = [base + (1 if r < extra else 0) for r in range(tp_size)]
        self.inter_blk0 = sum(counts[:tp_rank])
        self.inter_local = counts[tp_rank] * 128
        if self.inter_local == 0:
            raise ValueError("tensor-parallel degree leaves a rank without FFN rows")
        hd, hidden = cfg.head_dim, cfg.hidden
        qd_l, kvd_l = self.heads_local * hd, self.kv_heads_local * hd
        dev = self.device
        self.from_cache = False
        cache_file = None
        if cache_dir and source_path:
            from .checkpoint import repack_cache_key
            layout = self.REPACK_LAYOUT if decode_layout else self.REPACK_LAYOUT.split("+")[0]
            cache_file = os.path.join(cache_dir, repack_cache_key(source_path, tp_rank, tp_size, layout) + ".oxrp")
            if os.path.exists(cache_file) and self._load_cache(cache_file, decode_layout):
                return

        self.embd = _f16_matrix(f, "token_embd.weight", dev)
        head_name = "output.weight" if f.has_tensor("output.weight") else "token_embd.weight"
        if tp_size == 1:
            same = head_name == "token_embd.weight"
            self.lm_head = self.embd if same else _f16_matrix(f, head_name, dev)
            self.lm_row0 = 0
        else:
            rows = (cfg.vocab + tp_size - 1) // tp_size
            self.lm_row0 = tp_rank * rows
            self.lm_head = _f16_matrix(f, head_name, dev, self.lm_row0, max(0, min(rows, cfg.vocab - self.lm_row0)))
        self.out_norm = _norm_vector(f, "output_norm.weight", dev)
        self.layers: list[LayerWeights] = []
        self.weight_type = None
        for l in range(cfg.layers):
            p = f"blk.{l}."
            infos = {n: f.tensor_info(p + n + ".weight") for n in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")}
            for n, ti in infos.items():
                if ti.type not in _QUANT_TYPES:
                    raise NotImplementedError(f"{p}{n}: GPU path supports TQ2_0_g128 and Q1_0_g128 layer weights, got {ti.type_name}")
            self.weight_type = infos["attn_q"].type
            raws = {n: _upload(f.tensor_bytes(p + n + ".weight"), dev) for n in infos}
            ty = lambda n: infos[n].type
            qkv = K.PlanarWeight(qd_l + 2 * kvd_l, hidden, dev)
            qkv.fill_from_gguf(raws["attn_q"], ty("attn_q"), hidden, tp_rank * qd_l, qd_l, dst_row0=0)
            qkv.fill_from_gguf(raws["attn_k"], ty("attn_k"), hidden, tp_rank * kvd_l, kvd_l, dst_row0=qd_l)
            qkv.fill_from_gguf(raws["attn_v"], ty("attn_v"), hidden, tp_rank * kvd_l, kvd_l, dst_row0=qd_l + kvd_l)
            o = K.PlanarWeight(hidden, qd_l, dev)
            o.fill_from_gguf(raws["attn_output"], ty("attn_output"), cfg.q_dim, 0, hidden, blk0=tp_rank * qd_l // 128, nblk=qd_l // 128)
            gu = K.PlanarWeight(2 * self.inter_local, hidden, dev)
            gu.fill_from_gguf(raws["ffn_gate"], ty("ffn_gate"), hidden, self.inter_blk0 * 128, self.inter_local, dst_row0=0, dst_row_stride=2)
            gu.fill_from_gguf(raws["ffn_up"], ty("ffn_up"), hidden, self.inter_blk0 * 128, self.inter_local, dst_row0=1, dst_row_stride=2)
            down = K.PlanarWeight(hidden, self.inter_local, dev)
            down.fill_from_gguf(raws["ffn_down"], ty("ffn_down"), cfg.inter, 0, hidden, blk0=self.inter_blk0, nblk=self.inter_local // 128)
            lw = LayerWeights(qkv, o, gu, down,
                              _norm_vector(f, p + "attn_norm.weight", dev), _norm_vector(f, p + "ffn_norm.weight", dev),
                              _norm_vector(f, p + "attn_q_norm.weight", dev), _norm_vector(f, p + "attn_k_norm.weight", dev))
            if decode_layout and dev.type == "cuda":
                lw.qkv_s16, lw.o_s16, lw.gate_up_s16, lw.down_s16 = (K.S16Weight(m) for m in (qkv, o, gu, down))
            self.layers.append(lw)
            del raws
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        if cache_file is not None:
            self._save_cache(cache_file)

    _LAYER_MATS = ("qkv", "o", "gate_up", "down")
    _LAYER_VECS = ("attn_norm", "ffn_norm", "q_norm", "k_norm")

    def _save_cache(self, path: str) -> None:
        from .checkpoint import save_repacked
        t = {"embd": self.embd, "out_norm": self.out_norm}
        if self.lm_head is not self.embd:
            t["lm_head"] = self.lm_head
        for l, lw in enumerate(self.layers):
            for m in self._LAYER_MATS:
                pw = getattr(lw, m)
                t[f"{l}.{m}.codes"], t[f"{l}.{m}.scales"] = pw.codes, pw.scales
                s16 = getattr(lw, m + "_s16")
                if s16 is not None:
                    t[f"{l}.{m}.s16"] = s16.data
            for v in self._LAYER_VECS:
                t[f"{l}.{v}"] = getattr(lw, v)
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        try:
            save_repacked(path, t, {"layers": len(self.layers), "weight_type": int(self.weight_type), "lm_row0": int(self.lm_row0),
                                    "tp": f"{self.tp_rank}/{self.tp_size}"})
        except OSError:
            pass          # a read-only or full cache directory costs the next start its shortcut, nothing else

    def _load_cache(self, path: str, decode_layout: bool) -> bool:
        from .checkpoint import CheckpointError, load_repacked
        try:
            t, meta = load_repacked(path, self.device)
        except (CheckpointError, OSError, ValueError, KeyError):
            return False
        if int(meta.get("layers", -1)) != self.cfg.layers:
            return False
        self.embd, self.out_norm = t["embd"], t["out_norm"]
        self.lm_head = t.get("lm_head", self.embd)
        self.lm_row0 = int(meta.get("lm_row0", 0))
        self.weight_type = int(meta["weight_type"])
        self.layers = []
        for l in range(self.cfg.layers):
            mats = [K.PlanarWeight.from_tensors(t[f"{l}.{m}.codes"], t[f"{l}.{m}.scales"]) for m in self._LAYER_MATS]
            lw = LayerWeights(*mats, *(t[f"{l}.{v}"] for v in self._LAYER_VECS))
            if decode_layout and self.device.type == "cuda":
                for m, pw in zip(self._LAYER_MATS, mats):
                    setattr(lw, m + "_s16", K.S16Weight.from_tensor(pw.n, pw.k, t[f"{l}.{m}.s16"]))
            self.layers.append(lw)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        self.from_cache = True
        return True

    @property
    def packed_bytes(self) -> int:
        """Bytes a decode step must stream: packed layer weights + LM head."""
        n = sum(lw.qkv.nbytes + lw.o.nbytes + lw.gate_up.nbytes + lw.down.nbytes for lw in self.layers)
        return n + self.lm_head.numel() * 2


class PagedKvCache:
    """Page pool shared by all sequences of a rank; one K and one V pool per layer.

    Reference: ``PagedKvCache`` / ``BlockPool`` / ``BlockTable`` (crates/oxibonsai-model/src/paged_kv_cache.rs:33-557),
    with the storage formats of ``KvCacheFp16`` and ``QuantizedKvCache`` (kv_cache_fp16.rs, kv_cache_quant.rs) as page
    formats, plus an INT4 page format.
    """

    def __init__(self, cfg: Qwen3Config, kv_heads_local: int, num_pages: int, page_size: int, kvt: int, device):
        self.kvt, self.page_size, self.num_pages = kvt, page_size, num_pages
        hd = cfg.head_dim
        row = {K.KV_F32: hd, K.KV_F16: hd, K.KV_Q8: hd, K.KV_Q4: hd // 2}[kvt]
        dt = K.KV_DTYPES[kvt]
        shape = (cfg.layers, num_pages, kv_heads_local, page_size, row)
        self.k = torch.zeros(shape, dtype=dt, device=device)
        self.v = torch.zeros(shape, dtype=dt, device=device)
        if kvt in (K.KV_Q8, K.KV_Q4):
            self.k_scale = torch.zeros(shape[:-1], dtype=torch.float32, device=device)
            self.v_scale = torch.zeros(shape[:-1], dtype=torch.float32, device=device)
        else:
            self.k_scale = self.v_scale = None
        self.free_pages = list(range(num_pages - 1, -1, -1))
        self.refcount = [0] * num_pages        # pages may be shared between sequences and the prefix cache
        self.on_exhausted = None               # optional callback(n_missing) that may free pages (prefix-cache eviction)

    def alloc(self, n: int) -> list[int]:
        if n > len(self.free_pages) and self.on_exhausted is not None:
            self.on_exhausted(n - len(self.free_pages))
        if n > len(self.free_pages):
            raise MemoryError(f"KV cache exhausted: need {n} pages, {len(self.free_pages)} free")
        pages = [self.free_pages.pop() for _ in range(n)]
        for p in pages:
            self.refcount[p] = 1
        return pages

    def retain(self, pages: list[int]) -> None:
        for p in pages:
            self.refcount[p] += 1

    def release(self, pages: list[int]) -> None:
        for p in reversed(pages):
            self.refcount[p] -= 1
            if self.refcount[p] <= 0:
                self.refcount[p] = 0
                self.free_pages.append(p)

    @property
    def utilization(self) -> float:
        return 1.0 - len(self.free_pages) / max(1, self.num_pages)

    @property
    def nbytes(self) -> int:
        n = self.k.numel() * self.k.element_size() * 2
        if self.k_scale is not None:
            n += self.k_scale.numel() * 8
        return n


class Qwen3Runner:
    """Owns the activation buffers and the native step runner for a fixed maximum batch."""

    def __init__(self, weights: Qwen3Weights, kv: PagedKvCache, max_batch: int, max_seq: int, nsplit: int | None = None,
                 fast: bool = True, prefill_chunk: int = 1024, streamed_gemv_mask: int = 15):
        """``streamed_gemv_mask``: which linear layers of the batch-1 step use the streamed S16 GEMV (bit 0 QKV, 1 attention
        output, 2 gate/up, 3 down); the others stay on the planar-layout kernels."""
        self.streamed_gemv_mask = streamed_gemv_mask
        self.w, self.kv, self.max_batch, self.max_seq = weights, kv, max_batch, max_seq
        # rows of the prompt / decode-batch activation buffers: allocated once at this size, because the captured decode
        # graphs hold their addresses (a later, larger allocation would leave those graphs pointing at freed memory)
        self.prefill_capacity = max(int(prefill_chunk), 64, int(max_batch))
        cfg, dev = weights.cfg, weights.device
        self.cfg, self.device = cfg, dev
        hd = cfg.head_dim
        nq, nkv = weights.heads_local, weights.kv_heads_local
        self.max_pages = (max_seq + kv.page_size - 1) // kv.page_size
        # enough splits to spread one sequence's heads over the GPU; empty splits cost almost nothing
        # KV splits of one sequence's decode attention: about 128 CTAs over (kv head, split).  More splits shorten every
        # CTA's stream but lengthen the merge in the last CTA: 16 splits measured 10.9 us at 4096 tokens (8 kv heads)
        # against 13.5 us for 37 and 12.4 us for 8, and 0.53 of the HBM bandwidth at 16384 tokens.
        # With one or two local kv heads (tensor parallel) that rule would leave most SMs idle: up to 64 splits.
        # Up to 8192 tokens 16 splits measured best for every head count of a rank (4096 tokens, 32/8, 8/2 and 4/1 heads:
        # 11.0 / 10.1 / 9.9 us against 15.7 / 10.5 / 9.9 us for 32 splits), and 16 splits fit one thread-block cluster, whose
        # CTAs merge through distributed shared memory.
        self.nsplit = nsplit or (16 if max_seq <= 8192 else max(4, min(64, 128 // max(1, nkv))))
        if os.environ.get("OXIBONSAI_ATTN_CLUSTER", "1") == "0":       # A/B switch: merge the KV splits through global memory
            K.attn_decode_cluster_mode(1)
        self.nsplit_override = os.environ.get("OXIBONSAI_ATTN_SPLITS")
        if nsplit is None and self.nsplit_override:
            self.nsplit = max(1, int(self.nsplit_override))
        self.fast = fast
        B = max_batch
        f32 = dict(dtype=torch.float32, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)
        # [status word, token of slot 0, token of slot 1, ...]: one device-to-host copy brings the sampled tokens and the
        # word in which a kernel records an expired bounded wait (copy pipeline, tensor-parallel peer)
        self.ctl = torch.zeros(B + 1, **i32)
        self.status = self.ctl[:1]
        self.tokens = self.ctl[1:]
        self.positions = torch.zeros(B, **i32)
        self.block_table = torch.zeros((B, self.max_pages), **i32)
        self.h = torch.zeros((B, cfg.hidden), **f32)
        self.qkv = torch.zeros((B, (nq + 2 * nkv) * hd), **f32)
        self.q = torch.zeros((B, nq, hd), **f32)
        self.attn = torch.zeros((B, nq * hd), **f32)
        self.act = torch.zeros((B, weights.inter_local), **f32)
        self.tp = None
        if weights.tp_size > 1:
            from ..parallel.tp import TpGroup
            self.tp = TpGroup(weights.tp_rank, weights.tp_size, dev, cfg.hidden, cfg.vocab, B, prefill_chunk * cfg.hidden)
            self.logits = self.tp.logits          # this rank's gathered-logits area of the symmetric buffer
            self.partial = torch.zeros((B, max(1, weights.lm_head.shape[0])), **f32)   # local logits slice
        else:
            self.logits = torch.zeros((B, cfg.vocab), **f32)
            self.partial = torch.zeros((B, cfg.hidden), **f32)
        self.ws_acc = torch.zeros((B, nq, self.nsplit, hd), **f32)
        self.ws_ml = torch.zeros((B, nq, self.nsplit, 2), **f32)
        self.temps = torch.zeros(B, **f32)
        self.topks = torch.zeros(B, **i32)
        self.topps = torch.ones(B, **f32)
        self.rng = torch.full((B,), 42, dtype=torch.int64, device=dev)
        self.out_tokens = torch.zeros(B, **i32)
        # per-slot vocabulary masks of constrained decoding (bit set = token allowed), read by the sampler of a masked step
        self.mask_words = (cfg.vocab + 31) // 32
        self.allow_mask = torch.full((B, self.mask_words), -1, **i32)
        self.attn_counters = torch.zeros(B * max(1, nkv), **i32)
        cos, sin = rope_table(hd, max_seq, cfg.rope_base)
        self.rope_cos = torch.from_numpy(cos).to(dev)
        self.rope_sin = torch.from_numpy(sin).to(dev)
        self._graphs: dict[tuple, torch.cuda.CUDAGraph] = {}
        self.kv_pools: dict[int, PagedKvCache] = {kv.kvt: kv}      # page pools by format; kv is the default one
        self.slot_formats: list[int] = [kv.kvt] * B                # page format of the sequence in every slot
        self._build_native()

    def _build_native(self) -> None:
        lib = K.lib()
        w, kv, cfg = self.w, self.kv, self.cfg
        nlp, nsp = lib.bonsai_runner_layer_ptr_count(), lib.bonsai_runner_step_ptr_count()
        icfg = (C.c_int * 16)(cfg.hidden, w.inter_local, cfg.layers, w.heads_local, w.kv_heads_local, cfg.head_dim, cfg.vocab,
                              w.lm_head.shape[0], kv.kvt, kv.page_size, self.max_pages, self.nsplit, w.tp_size, w.tp_rank, int(self.fast), self.nsplit)
        gp = (C.c_uint64 * 5)(w.embd.data_ptr(), w.lm_head.data_ptr(), w.out_norm.data_ptr(), self.rope_cos.data_ptr(), self.rope_sin.data_ptr())
        lp = (C.c_uint64 * (nlp * cfg.layers))()
        for l, lw in enumerate(w.layers):
            ks = kv.k_scale[l].data_ptr() if kv.k_scale is not None else 0
            vs = kv.v_scale[l].data_ptr() if kv.v_scale is not None else 0
            vals = [lw.qkv.codes.data_ptr(), lw.qkv.scales.data_ptr(), lw.o.codes.data_ptr(), lw.o.scales.data_ptr(),
                    lw.gate_up.codes.data_ptr(), lw.gate_up.scales.data_ptr(), lw.down.codes.data_ptr(), lw.down.scales.data_ptr(),
                    lw.attn_norm.data_ptr(), lw.ffn_norm.data_ptr(), lw.q_norm.data_ptr(), lw.k_norm.data_ptr(),
                    kv.k[l].data_ptr(), kv.v[l].data_ptr(), ks, vs,
                    *[0 if m is None or not (self.streamed_gemv_mask >> i) & 1 else m.data.data_ptr()
                      for i, m in enumerate((lw.qkv_s16, lw.o_s16, lw.gate_up_s16, lw.down_s16))]]
            assert len(vals) == nlp
            for i, v in enumerate(vals):
                lp[l * nlp + i] = v
        self._native = lib.bonsai_runner_create(icfg, cfg.eps, gp, lp)
        sp = [self.tokens, self.positions, self.block_table, self.h, self.qkv, self.q, self.attn, self.act, self.logits, self.ws_acc,
              self.ws_ml, self.temps, self.topks, self.topps, self.rng, self.tokens, self.partial, self.allow_mask, self.attn_counters, self.status]
        assert len(sp) == nsp
        self._step_ptrs = (C.c_uint64 * nsp)(*[0 if t is None else t.data_ptr() for t in sp])
        if self.tp is not None:
            self.tp.use_status_word(self.status)     # peers that do not answer are reported in the same word
            lib.bonsai_runner_set_comm(self._native, self.tp.handle)
        self.launches_per_step = None

    def add_kv_pool(self, kv: PagedKvCache) -> None:
        """Registers a page pool in another format (same page size): sequences whose slot format is ``kv.kvt`` append to and
        attend over it.  The default pool keeps serving every other slot."""
        assert kv.page_size == self.kv.page_size and kv.kvt not in self.kv_pools
        lib = K.lib()
        for l in range(self.cfg.layers):
            ks = kv.k_scale[l].data_ptr() if kv.k_scale is not None else None
            vs = kv.v_scale[l].data_ptr() if kv.v_scale is not None else None
            K.check(lib.bonsai_runner_set_pool(self._native, kv.kvt, l, kv.k[l].data_ptr(), kv.v[l].data_ptr(), ks, vs), "runner_set_pool")
        self.kv_pools[kv.kvt] = kv

    def set_slot_format(self, slot: int, kvt: int) -> None:
        """Page format of the sequence that occupies ``slot`` from now on (its pool must have been registered)."""
        if kvt not in self.kv_pools:
            raise ValueError(f"no KV pool in page format {kvt}")
        if self.slot_formats[slot] != kvt:
            self.slot_formats[slot] = kvt
            self._push_slot_formats()

    def _push_slot_formats(self) -> None:
        arr = (C.c_int * len(self.slot_formats))(*self.slot_formats)
        K.check(K.lib().bonsai_runner_set_slot_formats(self._native, arr, len(self.slot_formats)), "runner_set_slot_formats")

    def check_status(self, value: int | None = None) -> None:
        """Raises when a kernel of an earlier step recorded an expired wait (``value``: the status word as already read by
        the caller, else it is read here)."""
        v = int(self.status.item()) if value is None else int(value)
        if v:
            self.status.zero_()
            what = {2: "a tensor-parallel peer did not deliver its partial sums", 3: "a tensor-parallel peer did not reach a barrier",
                    4: "a tensor-parallel peer did not enter an all-reduce", 5: "the weight copy pipeline of a GEMV stalled"}.get(v, "a bounded wait expired")
            raise K.CudaKernelError(f"decode step reported status {v}: {what}")

    def __del__(self):
        try:
            if getattr(self, "_native", None):
                K.lib().bonsai_runner_destroy(self._native)
                self._native = None
        except Exception:
            pass

    # ---- prefill (tcgen05 GEMMs + causal paged attention over a chunk of prompt tokens) ----
    def _prefill_buffers(self, chunk: int):
        """The activation buffers of the prompt path and of batched decode steps (``chunk``: rows the caller needs).  One
        allocation for the runner's lifetime, ``prefill_capacity`` rows: the addresses are part of every captured graph."""
        if chunk > self.prefill_capacity:
            raise ValueError(f"{chunk} rows exceed the runner's activation buffers ({self.prefill_capacity} rows)")
        if getattr(self, "_pf", None) is not None:
            return self._pf
        chunk = self.prefill_capacity
        cfg, w, dev = self.cfg, self.w, self.device
        hd, nq, nkv = cfg.head_dim, w.heads_local, w.kv_heads_local
        qd = nq * hd
        f32, f16, i32 = (dict(dtype=d, device=dev) for d in (torch.float32, torch.float16, torch.int32))
        b = {"chunk": chunk,
             "tokens": torch.zeros(chunk, **i32), "positions": torch.zeros(chunk, **i32),
             "h": torch.zeros((chunk, cfg.hidden), **f32), "xn": torch.zeros((chunk, max(cfg.hidden, qd)), **f16),
             "qkv": torch.zeros((chunk, (nq + 2 * nkv) * hd), **f32), "q": torch.zeros((chunk, nq, hd), **f32),
             "attn": torch.zeros((chunk, qd), **f16), "act": torch.zeros((chunk, w.inter_local), **f16),
             "status": torch.zeros(1, **i32), "gemm_ws": getattr(self, "_gemm_ws", None)}
        # chunks of up to `sm` tokens run like a decode batch: f32 attention rows and the split-KV workspace for them
        sm, ss = K._pf().bonsai_runner_small_chunk(), K._pf().bonsai_runner_small_splits()
        b.update({"sm_attn": torch.zeros((sm, qd), **f32), "sm_acc": torch.zeros((sm, nq, ss, hd), **f32),
                  "sm_ml": torch.zeros((sm, nq, ss, 2), **f32), "sm_ctr": torch.zeros(sm * max(1, nkv), **i32)})
        if b["gemm_ws"] is None:
            b["gemm_ws"] = self._gemm_ws = K.new_gemm_workspace(dev)
        order = ["tokens", "positions", "h", "xn", "qkv", "q", "attn", "act", "status", "sm_attn", "sm_acc", "sm_ml", "sm_ctr", "gemm_ws"]
        assert len(order) + 1 == K._pf().bonsai_runner_prefill_ptr_count()
        b["ptrs"] = (C.c_uint64 * (len(order) + 1))(*[b[k].data_ptr() for k in order], b["gemm_ws"].numel())
        self._pf = b
        return b

    def prefill(self, tokens: torch.Tensor, slot: int, pos0: int = 0, chunk: int = 1024) -> None:
        """Runs prompt ``tokens`` (int32 device tensor) of the sequence in ``slot`` starting at position ``pos0``;
        leaves the logits of the last token in ``self.logits[slot]``."""
        n = tokens.numel()
        chunk = max(1, min(chunk, self.prefill_capacity))
        b = self._prefill_buffers(min(chunk, max(n, 1)))
        lib = K._pf()
        done = 0
        while done < n:
            T = min(chunk, n - done)
            b["tokens"][:T].copy_(tokens[done:done + T], non_blocking=True)
            torch.arange(pos0 + done, pos0 + done + T, dtype=torch.int32, device=self.device, out=b["positions"][:T])
            last = done + T == n
            mark = nvtx.push(f"prefill_chunk[slot={slot},pos={pos0 + done},T={T}]")
            K.check(lib.bonsai_runner_prefill_chunk(self._native, self._step_ptrs, b["ptrs"], T, pos0 + done, slot, int(last), K.stream()),
                    "prefill_chunk")
            nvtx.pop(mark)
            done += T

    def verify_greedy(self, tokens: torch.Tensor, slot: int, pos0: int) -> torch.Tensor:
        """Feeds ``tokens`` (int32 device tensor, at most one prefill chunk) at positions pos0.. and returns the model's
        greedy next token after each of them (int32 [T]) - the batched verification pass of speculative decoding."""
        return K.sample(self.verify_logits(tokens, slot, pos0))

    def verify_logits(self, tokens: torch.Tensor, slot: int, pos0: int) -> torch.Tensor:
        """The same pass, returning the logits after each of ``tokens`` (f32 [T, vocab]; the tensor is reused by the next
        call) for the rejection test of sampled speculative decoding."""
        T = tokens.numel()
        b = self._prefill_buffers(max(64, T))
        with nvtx.range(f"verify[slot={slot},pos={pos0},T={T}]"):
            return self._verify_logits(tokens, slot, pos0, T, b)

    def _verify_logits(self, tokens: torch.Tensor, slot: int, pos0: int, T: int, b: dict) -> torch.Tensor:
        b["tokens"][:T].copy_(tokens, non_blocking=True)
        torch.arange(pos0, pos0 + T, dtype=torch.int32, device=self.device, out=b["positions"][:T])
        K.check(K._pf().bonsai_runner_prefill_chunk(self._native, self._step_ptrs, b["ptrs"], T, pos0, slot, 0, K.stream()), "prefill_chunk")
        xn = K.norm_to_f16_paired(b["h"][:T], self.w.out_norm, self.cfg.eps, natural=True)
        if self.tp is None:
            return K.dense_gemm_f16(self.w.lm_head, xn, status=b["status"])
        # vocab-parallel head: every rank computes its slice for the T positions and pushes it into all ranks' logits areas
        if T > self.max_batch:
            raise ValueError(f"tensor-parallel verification of {T} tokens needs max_batch >= {T} (the gathered logits use the batch rows)")
        rows = self.w.lm_head.shape[0]
        local = K.dense_gemm_f16(self.w.lm_head, xn, status=b["status"]) if rows else torch.empty((T, 0), dtype=torch.float32, device=self.device)
        from ..parallel import tp as _tp
        rows_per_rank = (self.cfg.vocab + self.w.tp_size - 1) // self.w.tp_size
        K.check(_tp._lib().bonsai_tp_allgather_logits(self.tp.handle, local.data_ptr() if rows else None, T, rows, self.w.tp_rank * rows_per_rank,
                                                      self.cfg.vocab, K.stream()), "tp_allgather_logits")
        return self.logits[:T]

    def prefill_launches(self, n_tokens: int, chunk: int = 1024) -> int:
        full, tail = divmod(n_tokens, chunk)
        small = K._pf().bonsai_runner_small_chunk()
        per_chunk = lambda t: 1 + (9 if t <= small else 8) * self.cfg.layers     # small chunks convert the f32 attention rows separately
        return full * per_chunk(chunk) + (per_chunk(tail) if tail else 0) + 2

    def set_comm(self, comm_handle: int) -> None:
        K.lib().bonsai_runner_set_comm(self._native, comm_handle)

    def kernel_launches(self, batch: int, sample: bool = True) -> int:
        """Number of kernel launches in one decode step (each is one of this library's kernels)."""
        # four GEMVs per sequence, then QK-norm/RoPE/append + attention: one fused launch for f16 pages with head_dim 128
        # on the packed-half path (page sizes are powers of two >= 16 there), two launches otherwise
        fused = self.fast and self.kv.kvt == K.KV_F16 and self.cfg.head_dim == 128 and self.kv.page_size >= 16 \
            and (self.kv.page_size & (self.kv.page_size - 1)) == 0
        per_layer = 4 * batch + (1 if fused else 2)
        return batch + per_layer * self.cfg.layers + batch + (1 if sample else 0) + (2 if self.w.tp_size > 1 else 0)

    def step_eager(self, batch: int, sample: bool = True, lm_head: bool = True, masked: bool = False) -> None:
        flags = (1 if sample else 0) | (0 if lm_head else 2)
        mw = self.mask_words if masked else 0      # masked: the sampler only picks tokens whose bit is set in ``allow_mask[slot]``
        if batch >= 2 and self.fast:
            # all sequences share one tcgen05 GEMM per linear layer
            b = self._prefill_buffers(max(64, batch))
            K.check(K._pf().bonsai_runner_decode_step_batched(self._native, self._step_ptrs, b["ptrs"], batch, flags, mw, K.stream()),
                    "decode_step_batched")
            return
        K.check(K.lib().bonsai_runner_decode_step(self._native, self._step_ptrs, batch, flags, mw, K.stream()), "decode_step")

    def step(self, batch: int, sample: bool = True, masked: bool = False) -> None:
        """One decode step for the first ``batch`` slots, replayed from a CUDA graph after the first call."""
        # the page formats of the live slots are baked into the launches of a captured step
        key = (batch, int(sample), tuple(self.slot_formats[:batch]) if len(self.kv_pools) > 1 else (), masked)
        g = self._graphs.get(key)
        if g is None:
            if batch >= 2 and self.fast:
                self._prefill_buffers(max(64, batch))   # allocate outside the capture
            # capture without running: the capture itself executes nothing, so state is untouched
            g = K.capture_graph(self.device, lambda: self.step_eager(batch, sample, masked=masked))
            self._graphs[key] = g
        mark = nvtx.push(f"decode_step[batch={batch}]")
        g.replay()
        nvtx.pop(mark)
