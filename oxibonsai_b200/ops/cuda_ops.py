"""Torch-facing wrappers of the sm_100a kernels in ``libbonsai_cuda.so``.

Every function launches on torch's current CUDA stream and takes/returns ``torch.Tensor``s.  There
is no PyTorch fallback: if the native library is missing the call raises.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native

EPI_STORE, EPI_RESID, EPI_SWIGLU = 0, 1, 2
KV_F32, KV_F16, KV_Q8, KV_Q4 = 0, 1, 2, 3
KV_DTYPES = {KV_F32: torch.float32, KV_F16: torch.float16, KV_Q8: torch.int8, KV_Q4: torch.uint8}

_vp, _i, _f, _u64 = C.c_void_p, C.c_int, C.c_float, C.c_uint64
_SIG = {
    "bonsai_repack_planar": [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _i, _i, _i, _vp],
    "bonsai_planar_to_f32": [_vp, _vp, _i, _i, _vp, _vp],
    "bonsai_bitgemv": [_vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _i, _vp],
    "bonsai_bitgemv_h2": [_vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _i, _vp],
    "bonsai_bitgemv_warp": [_vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _i, _vp],
    "bonsai_bitgemv_hmma": [_vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _i, _vp],
    "bonsai_f16gemv": [_vp, _vp, _vp, _f, _vp, _i, _i, _vp],
    "bonsai_embed_f16": [_vp, _vp, _vp, _i, _i, _vp],
    "bonsai_qknorm_rope_kvstore": [_vp, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp],
    "bonsai_attn_decode": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _vp],
    "bonsai_attn_decode_force_cuda_cores": [_i],
    "bonsai_attn_decode_qkv_f16": [_vp, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp],
    "bonsai_sample": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp],
    "bonsai_runner_create": [_vp, _f, _vp, _vp],
    "bonsai_runner_destroy": [_vp],
    "bonsai_runner_set_comm": [_vp, _vp],
    "bonsai_runner_set_nsplit": [_vp, _i],
    "bonsai_runner_set_pool": [_vp, _i, _i, _vp, _vp, _vp, _vp],
    "bonsai_runner_set_slot_formats": [_vp, _vp, _i],
    "bonsai_runner_set_fast": [_vp, _i],
    "bonsai_runner_layer_ptr_count": [],
    "bonsai_runner_step_ptr_count": [],
    "bonsai_runner_decode_step": [_vp, _vp, _i, _i, _i, _vp],
}
_RES = {"bonsai_runner_create": _vp, "bonsai_runner_destroy": None, "bonsai_runner_set_comm": None, "bonsai_runner_set_nsplit": None, "bonsai_runner_set_fast": None}
_lib = None


class CudaKernelError(RuntimeError):
    pass


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        l = _native.cuda()
        for name, args in _SIG.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = _RES.get(name, C.c_int)
        _lib = l
    return _lib


def declare(sig: dict, res: dict | None = None) -> C.CDLL:
    """Registers signatures of kernels added by other modules (prefill, comm, ...)."""
    l = lib()
    for name, args in sig.items():
        fn = getattr(l, name)
        fn.argtypes = args
        fn.restype = (res or {}).get(name, C.c_int)
    return l


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise CudaKernelError(f"{what} failed with code {rc}")


def _f32c(t: torch.Tensor) -> torch.Tensor:
    assert t.is_cuda and t.dtype == torch.float32 and t.is_contiguous(), "expected a contiguous CUDA float32 tensor"
    return t


class PlanarWeight:
    """A packed matrix in the planar-SM device layout: ``codes`` int32 [N][K/16], ``scales`` f16 [N][K/128]."""

    def __init__(self, n: int, k: int, device):
        assert k % 128 == 0
        self.n, self.k = n, k
        self.codes = torch.empty((n, k // 16), dtype=torch.int32, device=device)
        self.scales = torch.empty((n, k // 128), dtype=torch.float16, device=device)

    @classmethod
    def from_tensors(cls, codes: torch.Tensor, scales: torch.Tensor) -> "PlanarWeight":
        """Wraps tensors that already hold the layout (the repacked-weight cache)."""
        self = cls.__new__(cls)
        self.n, self.k = codes.shape[0], codes.shape[1] * 16
        assert codes.dtype == torch.int32 and scales.dtype == torch.float16 and tuple(scales.shape) == (self.n, self.k // 128)
        self.codes, self.scales = codes, scales
        return self

    @property
    def nbytes(self) -> int:
        return self.codes.numel() * 4 + self.scales.numel() * 2

    def fill_from_gguf(self, raw: torch.Tensor, src_type: int, src_k: int, row0: int, nrows: int, blk0: int = 0,
                       nblk: int | None = None, dst_row0: int = 0, dst_row_stride: int = 1, dst_blk0: int = 0) -> "PlanarWeight":
        """Repacks rows/blocks of a GGUF matrix (``raw``: uint8 CUDA tensor of its bytes) into this matrix."""
        nblk = src_k // 128 if nblk is None else nblk
        assert raw.is_cuda and raw.dtype == torch.uint8
        check(lib().bonsai_repack_planar(raw.data_ptr(), src_type, src_k // 128, row0, nrows, blk0, nblk, self.codes.data_ptr(),
                                         self.scales.data_ptr(), dst_row0, dst_row_stride, self.k // 16, dst_blk0, stream()),
              "repack_planar")
        return self

    def to_f32(self) -> torch.Tensor:
        out = torch.empty((self.n, self.k), dtype=torch.float32, device=self.codes.device)
        check(lib().bonsai_planar_to_f32(self.codes.data_ptr(), self.scales.data_ptr(), self.n, self.k // 16, out.data_ptr(), stream()),
              "planar_to_f32")
        return out


_S16_SIG = {
    "bonsai_s16_bytes": [_i, _i],
    "bonsai_repack_s16": [_vp, _vp, _i, _i, _vp, _vp],
    "bonsai_bitgemv_s16": [_vp, _vp, _vp, _f, _vp, _vp, _i, _i, _i, _vp, _vp, _vp],
    "bonsai_s16_tune": [_i],
}
_s16_declared = False
EPI_TP = 3


def _s16():
    global _s16_declared
    l = lib()
    if not _s16_declared:
        declare(_S16_SIG, {"bonsai_s16_bytes": C.c_size_t})
        _s16_declared = True
    return l


def s16_tune(pdl: bool = True) -> None:
    """Whether later launches (and graph captures) of the streamed GEMV use programmatic dependent launch."""
    check(_s16().bonsai_s16_tune(int(pdl)), "s16_tune")


class S16Weight:
    """A packed matrix in the streamed decode layout (csrc/cuda/bitgemv_stream.cu): tiles of 16 rows, one 544-byte block per
    (tile, 128-input group) holding the 2-bit codes in MMA-fragment order followed by the 16 group scales.  Built on the
    device from a :class:`PlanarWeight`; ``oxibonsai_b200.ops.s16_layout`` restates the layout on the host."""

    def __init__(self, planar: PlanarWeight):
        self.n, self.k = planar.n, planar.k
        nbytes = int(_s16().bonsai_s16_bytes(self.n, self.k))
        self.data = torch.empty(nbytes, dtype=torch.uint8, device=planar.codes.device)
        check(_s16().bonsai_repack_s16(planar.codes.data_ptr(), planar.scales.data_ptr(), self.n, self.k, self.data.data_ptr(), stream()),
              "repack_s16")

    @classmethod
    def from_tensor(cls, n: int, k: int, data: torch.Tensor) -> "S16Weight":
        """Wraps bytes that already hold the layout (the repacked-weight cache)."""
        self = cls.__new__(cls)
        self.n, self.k, self.data = n, k, data
        assert data.dtype == torch.uint8
        return self

    @property
    def nbytes(self) -> int:
        return self.data.numel()


def bitgemv_s16(w: S16Weight, x: torch.Tensor, norm_w: torch.Tensor | None = None, eps: float = 1e-6, epi: int = EPI_STORE,
                residual: torch.Tensor | None = None, out: torch.Tensor | None = None, comm: int | None = None,
                status: torch.Tensor | None = None) -> torch.Tensor:
    """out = W x through the streamed tensor-core GEMV (two-term int8 activations per 128-input group, exact integer sums).  ``epi``: store / residual add /
    SwiGLU over interleaved gate-up rows / ``EPI_TP`` (sum over the ranks of the communicator handle ``comm`` + residual)."""
    _f32c(x)
    n_out = w.n // 2 if epi == EPI_SWIGLU else w.n
    if out is None:
        out = torch.empty(n_out, dtype=torch.float32, device=x.device)
    check(_s16().bonsai_bitgemv_s16(w.data.data_ptr(), x.data_ptr(), ptr(norm_w), eps, out.data_ptr(), ptr(residual), w.n, w.k, epi,
                                    comm, ptr(status), stream()), "bitgemv_s16")
    return out


_MMA_SIG = {
    "bonsai_frag_sizes": [_i, _i, _vp, _vp],
    "bonsai_repack_frag": [_vp, _vp, _i, _i, _vp, _vp, _vp],
    "bonsai_bitgemv_mma": [_vp, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _i, _vp],
}
_mma_declared = False


def _mma():
    global _mma_declared
    l = lib()
    if not _mma_declared:
        declare(_MMA_SIG)
        _mma_declared = True
    return l


_QG_SIG = {
    "bonsai_quant_gemv": [_i, _vp, _vp, _vp, _f, _vp, _vp, _i, _i, _vp],
    "bonsai_swiglu": [_vp, _vp, _vp, _i, _vp],
    "bonsai_quant_gemv_batched": [_i, _vp, _vp, _i, _vp, _f, _vp, _vp, _i, _i, _i, _i, _vp],
    "bonsai_swiglu_rows": [_vp, _i, _vp, _i, _i, _i, _vp],
    "bonsai_quant_to_f16": [_i, _vp, _vp, _i, _i, _i, _vp],
}
_qg_declared = False


def _qg():
    global _qg_declared
    l = lib()
    if not _qg_declared:
        declare(_QG_SIG)
        _qg_declared = True
    return l


def quant_gemv(type_id: int, w: torch.Tensor, n: int, k: int, x: torch.Tensor, norm_w: torch.Tensor | None = None, eps: float = 1e-6,
               residual: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[n] = (residual) + W (rmsnorm(x)) for ``w`` = the raw GGUF bytes (uint8 CUDA tensor) of an [n, k] matrix of ``type_id`` blocks."""
    assert w.is_cuda and w.dtype == torch.uint8
    _f32c(x)
    if out is None:
        out = torch.empty(n, dtype=torch.float32, device=x.device)
    check(_qg().bonsai_quant_gemv(type_id, w.data_ptr(), x.data_ptr(), ptr(norm_w), eps, out.data_ptr(), ptr(residual), n, k, stream()), "quant_gemv")
    return out


_elt_declared = False


def _elt():
    global _elt_declared
    l = lib()
    if not _elt_declared:
        declare({"bonsai_rmsnorm_rows": [_vp, _i, _vp, _f, _i, _i, _vp, _i, _vp], "bonsai_residual_add": [_vp, _vp, C.c_size_t, _vp]})
        _elt_declared = True
    return l


def rmsnorm(x: torch.Tensor, w: torch.Tensor | None, eps: float = 1e-6, out: torch.Tensor | None = None) -> torch.Tensor:
    """Weighted RMSNorm over the rows of ``x`` (f32 [T, K] or [K]); the stand-alone form of what the GEMV / GEMM kernels fuse."""
    x2 = x if x.dim() == 2 else x.view(1, -1)
    assert x2.is_cuda and x2.dtype == torch.float32 and x2.stride(1) == 1
    o = torch.empty_like(x2) if out is None else (out if out.dim() == 2 else out.view(1, -1))
    check(_elt().bonsai_rmsnorm_rows(x2.data_ptr(), x2.stride(0), ptr(w), eps, x2.shape[0], x2.shape[1], o.data_ptr(), o.stride(0), stream()), "rmsnorm")
    return o if x.dim() == 2 else o.view(-1)


def residual_add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a += b in place (contiguous f32 tensors of one size)."""
    _f32c(a), _f32c(b)
    assert a.numel() == b.numel()
    check(_elt().bonsai_residual_add(a.data_ptr(), b.data_ptr(), a.numel(), stream()), "residual_add")
    return a


def quant_gemv_batched(type_id: int, w: torch.Tensor, n: int, k: int, x: torch.Tensor, norm_w: torch.Tensor | None = None, eps: float = 1e-6,
                       residual: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """:func:`quant_gemv` for a batch: ``x`` [B, k] f32 (row stride >= k), ``out`` and ``residual`` [B, n] with one common row stride."""
    assert w.is_cuda and w.dtype == torch.uint8 and x.dim() == 2 and x.dtype == torch.float32 and x.stride(1) == 1
    B = x.shape[0]
    if out is None:
        out = torch.empty((B, n), dtype=torch.float32, device=x.device)
    assert out.stride(1) == 1 and (residual is None or (residual.stride(1) == 1 and residual.stride(0) == out.stride(0)))
    check(_qg().bonsai_quant_gemv_batched(type_id, w.data_ptr(), x.data_ptr(), x.stride(0), ptr(norm_w), eps, out.data_ptr(), ptr(residual),
                                          out.stride(0), n, k, B, stream()), "quant_gemv_batched")
    return out


def swiglu_rows(gu: torch.Tensor, inter: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = silu(gu[t, :inter]) * gu[t, inter:2*inter] for every row of ``gu`` (f32, the output of a fused gate || up projection)."""
    assert gu.dim() == 2 and gu.dtype == torch.float32 and gu.stride(1) == 1
    T = gu.shape[0]
    if out is None:
        out = torch.empty((T, inter), dtype=torch.float32, device=gu.device)
    check(_qg().bonsai_swiglu_rows(gu.data_ptr(), gu.stride(0), out.data_ptr(), out.stride(0), inter, T, stream()), "swiglu_rows")
    return out


def quant_to_f16(type_id: int, w: torch.Tensor, n: int, k: int, out: torch.Tensor | None = None, paired: bool = True) -> torch.Tensor:
    """Decodes the raw GGUF bytes of an [n, k] matrix into dense f16 [n, k]; ``paired`` writes the K order of the tcgen05 GEMM's
    activation operand (``paired_k_index``) so that ``dense_gemm_f16`` can take paired-K activations."""
    assert w.is_cuda and w.dtype == torch.uint8
    if out is None:
        out = torch.empty((n, k), dtype=torch.float16, device=w.device)
    assert out.dtype == torch.float16 and out.is_contiguous() and out.numel() >= n * k
    check(_qg().bonsai_quant_to_f16(type_id, w.data_ptr(), out.data_ptr(), n, k, int(paired), stream()), "quant_to_f16")
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    if out is None:
        out = torch.empty_like(gate)
    check(_qg().bonsai_swiglu(_f32c(gate).data_ptr(), _f32c(up).data_ptr(), out.data_ptr(), gate.numel(), stream()), "swiglu")
    return out


class FragWeight:
    """A packed matrix in the tensor-core fragment layout of the batch-1 decode GEMV (see csrc/cuda/bitgemv_mma.cu):
    ``codes`` uint4 [N/16][K/128][32 lanes], ``scales`` half2 [N/16][K/128][8]."""

    def __init__(self, planar: PlanarWeight):
        self.n, self.k = planar.n, planar.k
        cb, sb = C.c_size_t(), C.c_size_t()
        _mma().bonsai_frag_sizes(self.n, self.k, C.byref(cb), C.byref(sb))
        dev = planar.codes.device
        self.codes = torch.empty(cb.value, dtype=torch.uint8, device=dev)
        self.scales = torch.empty(sb.value, dtype=torch.uint8, device=dev)
        check(_mma().bonsai_repack_frag(planar.codes.data_ptr(), planar.scales.data_ptr(), self.n, self.k, self.codes.data_ptr(),
                                        self.scales.data_ptr(), stream()), "repack_frag")

    @property
    def nbytes(self) -> int:
        return self.codes.numel() + self.scales.numel()


def bitgemv_mma(w: FragWeight, x: torch.Tensor, norm_w: torch.Tensor | None = None, eps: float = 1e-6, epi: int = EPI_STORE,
                residual: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """out = W x through warp-level fp8 tensor-core MMAs on fragment-layout weights (activations as three e4m3 terms)."""
    _f32c(x)
    n_out = w.n // 2 if epi == EPI_SWIGLU else w.n
    if out is None:
        out = torch.empty(n_out, dtype=torch.float32, device=x.device)
    check(_mma().bonsai_bitgemv_mma(w.codes.data_ptr(), w.scales.data_ptr(), x.data_ptr(), ptr(norm_w), eps, out.data_ptr(), ptr(residual),
                                    w.n, w.k, epi, stream()), "bitgemv_mma")
    return out


def bitgemv(w: PlanarWeight, x: torch.Tensor, norm_w: torch.Tensor | None = None, eps: float = 1e-6, epi: int = EPI_STORE,
            residual: torch.Tensor | None = None, out: torch.Tensor | None = None, fast: bool | str = False) -> torch.Tensor:
    """out = W x.  ``fast=False``: exact f32 path; ``fast=True`` / ``"warp"``: packed-half warp-per-row kernel
    (f16 activations); ``fast="tile"``: the packed-half tile kernel (the one the tensor-parallel epilogue builds on);
    ``fast="hmma"``: shift + mask expansion feeding ``mma.sync.m16n8k16`` (f16 activations, f32 accumulation).
    ``epi``: store / residual add / SwiGLU over interleaved gate-up rows."""
    _f32c(x)
    n_out = w.n // 2 if epi == EPI_SWIGLU else w.n
    if out is None:
        out = torch.empty(n_out, dtype=torch.float32, device=x.device)
    fn = (lib().bonsai_bitgemv if not fast else lib().bonsai_bitgemv_h2 if fast == "tile" else lib().bonsai_bitgemv_hmma if fast == "hmma"
          else lib().bonsai_bitgemv_warp)
    check(fn(w.codes.data_ptr(), w.scales.data_ptr(), x.data_ptr(), ptr(norm_w), eps, out.data_ptr(), ptr(residual),
                               w.n, w.k, epi, stream()), "bitgemv")
    return out


def f16gemv(w: torch.Tensor, x: torch.Tensor, norm_w: torch.Tensor | None = None, eps: float = 1e-6,
            out: torch.Tensor | None = None) -> torch.Tensor:
    assert w.dtype == torch.float16 and w.is_contiguous()
    n, k = w.shape
    if out is None:
        out = torch.empty(n, dtype=torch.float32, device=x.device)
    check(lib().bonsai_f16gemv(w.data_ptr(), _f32c(x).data_ptr(), ptr(norm_w), eps, out.data_ptr(), n, k, stream()), "f16gemv")
    return out


def qknorm_rope_kvstore(qkv, q_norm, k_norm, eps, rope_cos, rope_sin, positions, block_table, q_out, nq, nkv, hd, kvt, page_size,
                        kpool, vpool, kscale=None, vscale=None) -> None:
    batch = qkv.shape[0]
    check(lib().bonsai_qknorm_rope_kvstore(qkv.data_ptr(), qkv.stride(0), q_norm.data_ptr(), k_norm.data_ptr(), eps, rope_cos.data_ptr(),
                                           rope_sin.data_ptr(), positions.data_ptr(), block_table.data_ptr(), block_table.shape[1],
                                           q_out.data_ptr(), batch, nq, nkv, hd, kvt, page_size, kpool.data_ptr(), vpool.data_ptr(),
                                           ptr(kscale), ptr(vscale), stream()), "qknorm_rope_kvstore")


def attn_decode(q, positions, block_table, nq, nkv, hd, kvt, page_size, kpool, vpool, kscale=None, vscale=None, nsplit=8,
                extra_len=0, out=None) -> torch.Tensor:
    batch = q.shape[0]
    ws_acc = torch.empty((batch, nq, nsplit, hd), dtype=torch.float32, device=q.device)
    ws_ml = torch.empty((batch, nq, nsplit, 2), dtype=torch.float32, device=q.device)
    counters = torch.zeros(batch * nkv, dtype=torch.int32, device=q.device)
    if out is None:
        out = torch.empty((batch, nq, hd), dtype=torch.float32, device=q.device)
    check(lib().bonsai_attn_decode(q.data_ptr(), positions.data_ptr(), block_table.data_ptr(), block_table.shape[1], batch, nq, nkv, hd,
                                   kvt, page_size, kpool.data_ptr(), vpool.data_ptr(), ptr(kscale), ptr(vscale), nsplit,
                                   ws_acc.data_ptr(), ws_ml.data_ptr(), counters.data_ptr(), out.data_ptr(), extra_len, stream()),
          "attn_decode")
    return out


def attn_decode_qkv(qkv, q_norm, k_norm, eps, rope_cos, rope_sin, positions, block_table, nq, nkv, hd, page_size, kpool, vpool,
                    nsplit=8, out=None) -> torch.Tensor:
    """QK-norm + RoPE + KV append + attention of one new token per sequence in one launch (f16 pages, head_dim 128).
    Raises :class:`CudaKernelError` with the bad-argument code for shapes the fused kernel does not cover."""
    batch = qkv.shape[0]
    ws_acc = torch.empty((batch, nq, nsplit, hd), dtype=torch.float32, device=qkv.device)
    ws_ml = torch.empty((batch, nq, nsplit, 2), dtype=torch.float32, device=qkv.device)
    counters = torch.zeros(batch * nkv, dtype=torch.int32, device=qkv.device)
    if out is None:
        out = torch.empty((batch, nq, hd), dtype=torch.float32, device=qkv.device)
    check(lib().bonsai_attn_decode_qkv_f16(qkv.data_ptr(), qkv.stride(0), q_norm.data_ptr(), k_norm.data_ptr(), eps, rope_cos.data_ptr(),
                                           rope_sin.data_ptr(), positions.data_ptr(), block_table.data_ptr(), block_table.shape[1], batch, nq,
                                           nkv, hd, page_size, kpool.data_ptr(), vpool.data_ptr(), nsplit, ws_acc.data_ptr(), ws_ml.data_ptr(),
                                           counters.data_ptr(), out.data_ptr(), stream()), "attn_decode_qkv")
    return out


def sample(logits: torch.Tensor, temps=None, topks=None, topps=None, rng=None, positions=None, advance=False,
           allow_mask=None, out=None) -> torch.Tensor:
    """Samples one token per row of ``logits`` ([batch, vocab] f32).  ``temps=None`` means greedy."""
    batch, vocab = logits.shape
    if out is None:
        out = torch.empty(batch, dtype=torch.int32, device=logits.device)
    check(lib().bonsai_sample(logits.data_ptr(), batch, vocab, logits.stride(0), ptr(temps), ptr(topks), ptr(topps), ptr(rng),
                              out.data_ptr(), ptr(positions), int(advance and positions is not None), ptr(allow_mask),
                              0 if allow_mask is None else allow_mask.shape[1], stream()), "sample")
    return out


def attn_decode_cluster_mode(mode: int) -> None:
    """Decode attention for a few sequences merges its KV splits inside a thread-block cluster (distributed shared memory)
    where the device holds all clusters at once; ``mode`` 1 switches that off (partials through global memory, merged by the
    last CTA), 0 restores the default.  Takes effect for launches and graph captures that follow."""
    l = lib()
    l.bonsai_attn_decode_cluster_mode.argtypes = [C.c_int]
    l.bonsai_attn_decode_cluster_mode.restype = None
    l.bonsai_attn_decode_cluster_mode(int(mode))


def attn_decode_last_form() -> int:
    """How the last tensor-core decode attention was launched: 0 = splits merged through global memory, 8 or 4 = cluster
    merge with that many warps per CTA."""
    return int(lib().bonsai_attn_decode_last_form())


_capture_lock = __import__("threading").Lock()


def capture_graph(device, fn) -> "torch.cuda.CUDAGraph":
    """Captures the launches of ``fn()`` on a side stream into a CUDA graph.  One capture at a time per process, and in
    thread-local capture mode: engines of several GPUs live in one process (replica serving), and another engine's thread
    must be free to allocate, copy and synchronise while this one records."""
    with _capture_lock:
        s = torch.cuda.Stream(device=device)
        s.wait_stream(torch.cuda.current_stream(device))
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
                fn()
        torch.cuda.current_stream(device).wait_stream(s)
    return g


_spec_declared = False


def spec_verify(target_logits: torch.Tensor, draft_logits: torch.Tensor | None, draft_tokens: torch.Tensor | None, temperature: float,
                uniforms: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Rejection test of k drafted tokens on the device.  ``target_logits`` f32 [k+1, vocab] (row i: the target at the
    position of draft i; row k: after the last draft), ``draft_logits`` f32 [k, vocab] (the distributions the drafts were
    drawn from), ``draft_tokens`` int32 [k], ``uniforms`` f32 [2*(k+1)] in [0, 1).  Returns int32 [2]: the number of accepted
    drafts and the token that follows them (the replacement drawn from max(0, p - q) at the first rejection, or a sample
    of the last row when all were accepted).  Both distributions are softmax(logits / temperature)."""
    global _spec_declared
    l = lib()
    if not _spec_declared:
        declare({"bonsai_spec_verify": [_vp, _i, _vp, _i, _vp, _i, _i, _f, _vp, _vp, _vp, _vp]})
        _spec_declared = True
    k = target_logits.shape[0] - 1
    vocab = target_logits.shape[1]
    assert target_logits.dtype == torch.float32 and target_logits.stride(1) == 1 and uniforms.dtype == torch.float32 and uniforms.numel() >= 2 * (k + 1)
    if k > 0:
        assert draft_logits.dtype == torch.float32 and draft_logits.stride(1) == 1 and draft_logits.shape[0] >= k and draft_logits.shape[1] >= vocab
        assert draft_tokens.dtype == torch.int32 and draft_tokens.numel() >= k
    if out is None:
        out = torch.empty(2, dtype=torch.int32, device=target_logits.device)
    scratch = torch.empty(16 * (k + 1), dtype=torch.uint8, device=target_logits.device)
    check(l.bonsai_spec_verify(target_logits.data_ptr(), target_logits.stride(0), ptr(draft_logits), draft_logits.stride(0) if k > 0 else 0,
                               ptr(draft_tokens), k, vocab, float(temperature), uniforms.data_ptr(), scratch.data_ptr(), out.data_ptr(), stream()),
          "spec_verify")
    return out


# ---- tensor-core decode path ------------------------------------------------------------------------
_TC_SIG = {
    "bonsai_act_prep_fp8": [_vp, _i, _vp, _f, _i, _i, _i, _i, _vp, _vp, _vp],
    "bonsai_bitgemv_tc": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _f, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
    "bonsai_tc_tile": [_vp, _vp, _vp, _i, _i, _vp, _vp],
}
_tc_declared = False


def _tc():
    global _tc_declared
    l = lib()
    if not _tc_declared:
        declare(_TC_SIG)
        _tc_declared = True
    return l


def tc_columns(tokens: int, nterms: int) -> int:
    """MMA column count (16 / 32 / 64) for ``tokens`` activations split into ``nterms`` fp8 terms."""
    need = tokens * nterms
    for n in (16, 32, 64):
        if need <= n:
            return n
    raise ValueError(f"{tokens} tokens x {nterms} terms exceeds the 64 columns of the decode tensor-core kernel")


class TcActivations:
    """fp8-term operand of ``bitgemv_tc``: swizzled tiles [K/128][ncols][128 B] plus per-column factors."""

    def __init__(self, k: int, ncols: int, device):
        self.k, self.ncols = k, ncols
        self.xq = torch.zeros((k // 128) * ncols * 128, dtype=torch.uint8, device=device)
        self.colscale = torch.zeros(ncols, dtype=torch.float32, device=device)
        self.tokens = 0
        self.nterms = 0


def act_prep_fp8(x: torch.Tensor, nterms: int = 3, norm_w: torch.Tensor | None = None, eps: float = 1e-6,
                 out: TcActivations | None = None) -> TcActivations:
    """Splits rows of ``x`` ([T, K] f32, optionally RMS-normalised first) into e4m3 terms for the tensor cores."""
    x2 = x if x.dim() == 2 else x.view(1, -1)
    T, Kd = x2.shape
    ncols = tc_columns(T, nterms)
    if out is None:
        out = TcActivations(Kd, ncols, x.device)
    assert out.k == Kd and out.ncols >= T * nterms
    check(_tc().bonsai_act_prep_fp8(x2.data_ptr(), x2.stride(0), ptr(norm_w), eps, T, Kd, nterms, out.ncols, out.xq.data_ptr(),
                                    out.colscale.data_ptr(), stream()), "act_prep_fp8")
    out.tokens, out.nterms = T, nterms
    return out


class TcWorkspace:
    """Split-K scratch: partial sums, per-tile arrival counters and the error word of the tensor-core kernels."""

    def __init__(self, device, max_partial_floats: int = 1 << 22, max_tiles: int = 4096):
        self.partial = torch.empty(max_partial_floats, dtype=torch.float32, device=device)
        self.counters = torch.zeros(max_tiles, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def check(self) -> None:
        s = int(self.status.item())
        if s != 0:
            self.status.zero_()
            raise CudaKernelError(f"tensor-core kernel reported status {s} (a bounded wait expired)")


def pick_ksplit(n_rows: int, k: int, ncols: int, sms: int = 148) -> int:
    """K-split for the persistent tensor-core GEMV: the activation slab must fit in shared memory and the
    busiest CTA column should carry as few (tile, group) steps as possible."""
    tiles = (n_rows + 127) // 128
    ngroups = k // 128
    max_b_bytes = 88 * 1024
    best, best_cost = None, None
    for s in (1, 2, 3, 4, 6, 8, 12, 16):
        if s > ngroups or s > sms:
            continue
        gps = -(-ngroups // s)
        if gps * ncols * 128 > max_b_bytes:
            continue
        columns = min(sms // s, tiles)
        steps = -(-tiles // columns) * gps
        cost = steps + (3 if s > 1 else 0) * -(-tiles // columns)
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    if best is None:
        raise ValueError(f"no K-split fits: K={k}, columns={ncols}")
    return best


def bitgemv_tc(w: PlanarWeight, ws: TcWorkspace, act: TcActivations | None = None, x: torch.Tensor | None = None, nterms: int = 3,
               norm_w: torch.Tensor | None = None, eps: float = 1e-6, epi: int = EPI_STORE, residual: torch.Tensor | None = None,
               out: torch.Tensor | None = None, ksplit: int | None = None, sms: int = 148) -> torch.Tensor:
    """out[T, N] = epilogue(W x) on the tensor cores.

    Either pass ``act`` (from :func:`act_prep_fp8`) or ``x`` ([T, K] f32 with T <= 4), in which case the fp8-term
    operand - and the RMSNorm when ``norm_w`` is given - is built inside the kernel.
    """
    if act is not None:
        T, nt, ncols = act.tokens, act.nterms, act.ncols
        xq, cs, xp, xld = act.xq.data_ptr(), act.colscale.data_ptr(), None, 0
    else:
        x2 = x if x.dim() == 2 else x.view(1, -1)
        T, nt = x2.shape[0], nterms
        ncols = tc_columns(T, nt)
        xq, cs, xp, xld = None, None, x2.data_ptr(), x2.stride(0)
    n_out = w.n // 2 if epi == EPI_SWIGLU else w.n
    if out is None:
        out = torch.empty((T, n_out), dtype=torch.float32, device=w.codes.device)
    ks = ksplit or pick_ksplit(w.n, w.k, ncols, sms)
    assert ks * T * w.n <= ws.partial.numel() and (w.n + 127) // 128 <= ws.counters.numel()
    check(_tc().bonsai_bitgemv_tc(w.codes.data_ptr(), w.scales.data_ptr(), xq, cs, xp, xld, ptr(norm_w), eps, out.data_ptr(),
                                  ptr(residual), ws.partial.data_ptr(), ws.counters.data_ptr(), ws.status.data_ptr(), w.n, w.k, T,
                                  nt, ncols, ks, epi, out.stride(0) if out.dim() == 2 else n_out, sms, stream()), "bitgemv_tc")
    return out


# ---- prefill path -------------------------------------------------------------------------------------
_PF_SIG = {
    "bonsai_bitgemm_prefill": [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "bonsai_bitgemm_prefill_ws": [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, C.c_size_t, _i, _vp],
    "bonsai_bitgemm_prefill_ws_bytes": [],
    "bonsai_bitgemm_hmma": [_vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "bonsai_norm_to_f16_hmma": [_vp, _i, _vp, _f, _i, _i, _vp, _i, _vp],
    "bonsai_norm_to_f16_paired": [_vp, _i, _vp, _f, _i, _i, _vp, _i, _i, _vp],
    "bonsai_attn_prefill": [_vp, _i, _i, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp],
    "bonsai_attn_prefill_order": [_vp, _i, _i, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "bonsai_embed_rows_f16": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "bonsai_runner_prefill_ptr_count": [],
    "bonsai_runner_small_chunk": [],
    "bonsai_runner_small_splits": [],
    "bonsai_runner_prefill_chunk": [_vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "bonsai_runner_decode_step_batched": [_vp, _vp, _vp, _i, _i, _i, _vp],
}
_pf_declared = False


def _pf():
    global _pf_declared
    l = lib()
    if not _pf_declared:
        declare(_PF_SIG)
        _pf_declared = True
    return l


def paired_k_index(k: int, device=None) -> torch.Tensor:
    """Permutation ``perm`` with ``paired[..., perm[i]] = natural[..., i]`` (the K order of the prefill GEMM operand)."""
    i = torch.arange(k, device=device)
    j = i & 15
    return (i & ~15) | (j & 8) | ((j & 3) * 2 + ((j >> 2) & 1))


def norm_to_f16_paired(x: torch.Tensor, norm_w: torch.Tensor | None = None, eps: float = 1e-6, out: torch.Tensor | None = None,
                       natural: bool = False) -> torch.Tensor:
    """f32 [T, K] -> f16 [T, K] in paired-K order, optionally RMS-normalised first."""
    T, Kd = x.shape
    if out is None:
        out = torch.empty((T, Kd), dtype=torch.float16, device=x.device)
    check(_pf().bonsai_norm_to_f16_paired(x.data_ptr(), x.stride(0), ptr(norm_w), eps, T, Kd, out.data_ptr(), out.stride(0), int(natural), stream()),
          "norm_to_f16_paired")
    return out


def hmma_k_index(k: int, device=None) -> torch.Tensor:
    """Permutation ``perm`` with ``hmma[..., perm[i]] = natural[..., i]``: the K order (inside every 128-input group) of the
    activations of the decode-batch GEMM on ``mma.sync``."""
    i = torch.arange(k, device=device)
    r = i & 127
    wq, e = r >> 4, r & 15
    c, j, plane, p, h = wq >> 1, wq & 1, e >> 3, e & 3, (e >> 2) & 1
    return (i & ~127) | ((j * 4 + p) * 16 + plane * 8 + 2 * c + h)


def norm_to_f16_hmma(x: torch.Tensor, norm_w: torch.Tensor | None = None, eps: float = 1e-6, out: torch.Tensor | None = None) -> torch.Tensor:
    """f32 [T, K] -> f16 [T, K] in hmma-K order, optionally RMS-normalised first."""
    T, Kd = x.shape
    if out is None:
        out = torch.empty((T, Kd), dtype=torch.float16, device=x.device)
    check(_pf().bonsai_norm_to_f16_hmma(x.data_ptr(), x.stride(0), ptr(norm_w), eps, T, Kd, out.data_ptr(), out.stride(0), stream()),
          "norm_to_f16_hmma")
    return out


def bitgemm_hmma(w: PlanarWeight, x_hmma: torch.Tensor, epi: int = 0, residual: torch.Tensor | None = None,
                 out: torch.Tensor | None = None) -> torch.Tensor:
    """out[T, N] = epilogue(W x) for T <= 64 tokens on ``mma.sync`` with register-expanded weights.  ``epi``: 0 f32 store,
    1 f32 residual add, 2 f16 SwiGLU over interleaved gate / up rows (hmma-K order)."""
    T = x_hmma.shape[0]
    assert x_hmma.dtype == torch.float16 and x_hmma.shape[1] == w.k and T <= 64
    n_out = w.n // 2 if epi == 2 else w.n
    if out is None:
        out = torch.empty((T, n_out), dtype=torch.float32 if epi <= 1 else torch.float16, device=x_hmma.device)
    f32p = out.data_ptr() if epi <= 1 else None
    f16p = out.data_ptr() if epi == 2 else None
    check(_pf().bonsai_bitgemm_hmma(w.codes.data_ptr(), w.scales.data_ptr(), x_hmma.data_ptr(), x_hmma.stride(0), f32p, ptr(residual), f16p,
                                    w.n, w.k, T, epi, out.stride(0), stream()), "bitgemm_hmma")
    return out


_GEMM_WS: dict = {}


def gemm_workspace(device) -> torch.Tensor:
    """Zero-filled workspace that lets the tcgen05 GEMM cut its work into equal ranges per SM.  One per device, for
    launches on one stream at a time; an engine that runs GEMMs on its own stream allocates its own with
    ``new_gemm_workspace``."""
    key = torch.device(device).index or 0
    if key not in _GEMM_WS:
        _GEMM_WS[key] = new_gemm_workspace(device)
    return _GEMM_WS[key]


def _balance_mode(balanced) -> int:
    return 1 if balanced == "auto" else (2 if balanced else 0)


def new_gemm_workspace(device) -> torch.Tensor:
    fn = _pf().bonsai_bitgemm_prefill_ws_bytes
    fn.restype = C.c_size_t
    return torch.zeros(int(fn()), dtype=torch.uint8, device=device)


def dense_gemm_f16(w: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None, status: torch.Tensor | None = None,
                   sms: int = 148, balanced: bool | str = "auto", residual: torch.Tensor | None = None) -> torch.Tensor:
    """out[T, N] (f32) = (residual +) x[T, K] @ w[N, K]^T for dense f16 operands on tcgen05 (both in the same K order, natural
    or paired); used for the LM head and for the prompt path of the block formats without a planar repack.  ``residual``
    (f32 [T, N], same row stride as ``out``; may be ``out`` itself) is added in the epilogue."""
    T, n = x.shape[0], w.shape[0]
    assert w.dtype == torch.float16 and x.dtype == torch.float16 and w.is_contiguous() and x.shape[1] == w.shape[1]
    if out is None:
        out = torch.empty((T, n), dtype=torch.float32, device=x.device)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=x.device)
    ws = gemm_workspace(x.device) if balanced else None
    assert residual is None or residual.stride(0) == out.stride(0)
    check(_pf().bonsai_bitgemm_prefill_ws(None, None, x.data_ptr(), x.stride(0), out.data_ptr(), ptr(residual), None, status.data_ptr(), n,
                                          w.shape[1], T, 0 if residual is None else 1, out.stride(0), sms, w.data_ptr(), ptr(ws),
                                          ws.numel() if balanced else 0,
                                          _balance_mode(balanced), stream()), "dense_gemm_f16")
    return out


def bitgemm_prefill(w: PlanarWeight, x_paired: torch.Tensor, epi: int = 0, residual: torch.Tensor | None = None,
                    out: torch.Tensor | None = None, status: torch.Tensor | None = None, sms: int = 148,
                    balanced: bool | str = "auto") -> torch.Tensor:
    """out[T, N] = epilogue(W x) on tcgen05.  ``epi``: 0 f32 store, 1 f32 residual add, 2 f16 SwiGLU (paired-K), 3 f16 store.
    ``balanced``: "auto" = equal (tile, k) ranges per SM where that is expected to pay, True = wherever the workspace
    allows, False = whole tiles per CTA."""
    T = x_paired.shape[0]
    assert x_paired.dtype == torch.float16 and x_paired.shape[1] == w.k
    n_out = w.n // 2 if epi == 2 else w.n
    if out is None:
        out = torch.empty((T, n_out), dtype=torch.float32 if epi <= 1 else torch.float16, device=x_paired.device)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=x_paired.device)
    f32p = out.data_ptr() if epi <= 1 else None
    f16p = out.data_ptr() if epi >= 2 else None
    ws = gemm_workspace(x_paired.device) if balanced else None
    check(_pf().bonsai_bitgemm_prefill_ws(w.codes.data_ptr(), w.scales.data_ptr(), x_paired.data_ptr(), x_paired.stride(0), f32p,
                                          ptr(residual), f16p, status.data_ptr(), w.n, w.k, T, epi, out.stride(0), sms, None, ptr(ws),
                                          ws.numel() if balanced else 0, _balance_mode(balanced), stream()), "bitgemm_prefill")
    return out


def attn_prefill(q: torch.Tensor, pos0: int, block_table_row: torch.Tensor, nq, nkv, hd, kvt, page_size, kpool, vpool, kscale=None,
                 vscale=None, out: torch.Tensor | None = None, k_order: int = 0) -> torch.Tensor:
    """Causal attention of a T-token chunk (q f32 [T, nq, hd]) over the sequence's pages; returns f16 [T, nq*hd] in paired-K
    order (``k_order`` 0, the tcgen05 GEMM's operand order) or hmma-K order (1, the mma.sync GEMM's)."""
    T = q.shape[0]
    if out is None:
        out = torch.empty((T, nq * hd), dtype=torch.float16, device=q.device)
    check(_pf().bonsai_attn_prefill_order(q.data_ptr(), T, pos0, block_table_row.data_ptr(), nq, nkv, hd, kvt, page_size, kpool.data_ptr(),
                                          vpool.data_ptr(), ptr(kscale), ptr(vscale), out.data_ptr(), out.stride(0), k_order, stream()),
          "attn_prefill")
    return out
