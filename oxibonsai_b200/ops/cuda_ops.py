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
    "bonsai_f16gemv": [_vp, _vp, _vp, _f, _vp, _i, _i, _vp],
    "bonsai_embed_f16": [_vp, _vp, _vp, _i, _i, _vp],
    "bonsai_qknorm_rope_kvstore": [_vp, _i, _vp, _vp, _f, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp],
    "bonsai_attn_decode": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp],
    "bonsai_sample": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp],
    "bonsai_runner_create": [_vp, _f, _vp, _vp],
    "bonsai_runner_destroy": [_vp],
    "bonsai_runner_set_comm": [_vp, _vp],
    "bonsai_runner_set_nsplit": [_vp, _i],
    "bonsai_runner_layer_ptr_count": [],
    "bonsai_runner_step_ptr_count": [],
    "bonsai_runner_decode_step": [_vp, _vp, _i, _i, _i, _vp],
}
_RES = {"bonsai_runner_create": _vp, "bonsai_runner_destroy": None, "bonsai_runner_set_comm": None, "bonsai_runner_set_nsplit": None}
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


def bitgemv(w: PlanarWeight, x: torch.Tensor, norm_w: torch.Tensor | None = None, eps: float = 1e-6, epi: int = EPI_STORE,
            residual: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """out = W x (f32 exact path).  ``epi``: store / residual add / SwiGLU over interleaved gate-up rows."""
    _f32c(x)
    n_out = w.n // 2 if epi == EPI_SWIGLU else w.n
    if out is None:
        out = torch.empty(n_out, dtype=torch.float32, device=x.device)
    check(lib().bonsai_bitgemv(w.codes.data_ptr(), w.scales.data_ptr(), x.data_ptr(), ptr(norm_w), eps, out.data_ptr(), ptr(residual),
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
    if out is None:
        out = torch.empty((batch, nq, hd), dtype=torch.float32, device=q.device)
    check(lib().bonsai_attn_decode(q.data_ptr(), positions.data_ptr(), block_table.data_ptr(), block_table.shape[1], batch, nq, nkv, hd,
                                   kvt, page_size, kpool.data_ptr(), vpool.data_ptr(), ptr(kscale), ptr(vscale), nsplit,
                                   ws_acc.data_ptr(), ws_ml.data_ptr(), out.data_ptr(), extra_len, stream()), "attn_decode")
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
