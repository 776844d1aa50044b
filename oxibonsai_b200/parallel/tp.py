"""Tensor-parallel group over NVLink peer memory: symmetric buffer set-up and the native communicator handle.

The reference's tensor parallelism is a CPU simulation (``ShardedLinear``, ``tensor_parallel_forward``,
``NcclCollectives``; crates/oxibonsai-model/src/tensor_parallel.rs:20-468, multi_gpu.rs:31-320).  Here one process
per GPU joins a ``torch.distributed`` NCCL group (bootstrap, barriers), allocates one symmetric buffer with
``torch.distributed._symmetric_memory`` and hands the peer addresses to the CUDA kernels of ``csrc/comm``,
which move data with ordinary loads/stores to peer memory, or with multimem stores and load-reduces through the NVLink
switch where the buffer has a multicast mapping (never TMA, never a library kernel on a peer pointer).
"""
from __future__ import annotations

import os

import ctypes as C
from dataclasses import dataclass

import torch

from ..ops import cuda_ops as K

_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
_SIG = {
    "bonsai_tp_layout": [_sz, _sz, _sz, _vp],
    "bonsai_tp_set_spin_limit": [_vp, C.c_uint],
    "bonsai_tp_set_status_ptr": [_vp, _vp],
    "bonsai_tp_create": [_i, _i, _vp, _sz, _sz, _sz, _vp],
    "bonsai_tp_destroy": [_vp],
    "bonsai_tp_barrier": [_vp, _vp],
    "bonsai_tp_allgather_logits": [_vp, _vp, _i, _i, _i, _i, _vp],
    "bonsai_tp_set_multicast": [_vp, C.c_uint64],
    "bonsai_tp_logits_ptr": [_vp],
    "bonsai_tp_big_ptr": [_vp],
    "bonsai_tp_allreduce_big_add": [_vp, _vp, _sz, _vp],
    "bonsai_bitgemv_tp": [_vp, _vp, _vp, _vp, C.c_float, _vp, _vp, _i, _i, _i, _vp],
}
_RES = {"bonsai_tp_layout": _sz, "bonsai_tp_create": _vp, "bonsai_tp_destroy": None, "bonsai_tp_set_spin_limit": None, "bonsai_tp_set_multicast": None,
        "bonsai_tp_set_status_ptr": None, "bonsai_tp_logits_ptr": _vp, "bonsai_tp_big_ptr": _vp}
_declared = False


def _lib():
    global _declared
    l = K.lib()
    if not _declared:
        K.declare(_SIG, _RES)
        _declared = True
    return l


@dataclass(frozen=True)
class ShardRange:
    """Half-open ranges owned by one rank: rows for column-parallel matrices, 128-input blocks for row-parallel ones."""
    heads: tuple[int, int]
    kv_heads: tuple[int, int]
    inter_blocks: tuple[int, int]
    vocab_rows: tuple[int, int]


def shard_plan(heads: int, kv_heads: int, inter: int, vocab: int, tp_size: int) -> list[ShardRange]:
    """The standard transformer plan (q/k/v/gate/up column-parallel, o/down row-parallel, LM head vocab-parallel);
    the intermediate dimension is split on 128-weight block boundaries, sizes differing by at most one block."""
    if heads % tp_size or kv_heads % tp_size:
        raise ValueError(f"tp_size {tp_size} must divide heads {heads} and kv_heads {kv_heads}")
    nblk = inter // 128
    base, extra = divmod(nblk, tp_size)
    per = (vocab + tp_size - 1) // tp_size
    out, b0 = [], 0
    for r in range(tp_size):
        nb = base + (1 if r < extra else 0)
        h, kv = heads // tp_size, kv_heads // tp_size
        out.append(ShardRange((r * h, (r + 1) * h), (r * kv, (r + 1) * kv), (b0, b0 + nb), (min(vocab, r * per), min(vocab, (r + 1) * per))))
        b0 += nb
    return out


class TpGroup:
    """Symmetric buffer + native communicator of one rank."""

    def __init__(self, rank: int, size: int, device, hidden: int, vocab: int, max_batch: int, big_elems: int):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        if not dist.is_initialized():
            raise RuntimeError("tensor parallelism needs torch.distributed initialised with the nccl backend")
        lib = _lib()
        self.rank, self.size = rank, size
        self.recv_elems, self.logits_elems, self.big_elems = hidden, max_batch * vocab, big_elems
        offs = (C.c_size_t * 7)()
        total = lib.bonsai_tp_layout(self.recv_elems, self.logits_elems, self.big_elems, offs)
        self.buffer = symm.empty(total, dtype=torch.uint8, device=device)
        self._hdl = symm.rendezvous(self.buffer, dist.group.WORLD)
        self.buffer.zero_()
        torch.cuda.synchronize(device)
        dist.barrier()
        ptrs = list(self._hdl.buffer_ptrs)
        assert len(ptrs) == size
        self.state = torch.zeros(4, dtype=torch.int32, device=device)
        arr = (C.c_uint64 * size)(*ptrs)
        self.handle = lib.bonsai_tp_create(rank, size, arr, self.recv_elems, self.logits_elems, self.big_elems, self.state.data_ptr())
        if not self.handle:
            raise RuntimeError("bonsai_tp_create failed")
        lo = int(offs[3])
        self.logits = self.buffer[lo: lo + self.logits_elems * 4].view(torch.float32).view(max_batch, vocab)
        bo = int(offs[4])
        self.big = self.buffer[bo: bo + self.big_elems * 4].view(torch.float32)
        # NVLink-switch multicast (multimem.st / multimem.ld_reduce) when the fabric maps the buffer that way;
        # OXIBONSAI_TP_MULTIMEM=0 keeps every exchange on plain peer loads and stores
        self.multicast = False
        mc = int(getattr(self._hdl, "multicast_ptr", 0) or 0)
        if mc and os.environ.get("OXIBONSAI_TP_MULTIMEM", "1") != "0":
            self.set_multicast(True)

    def set_multicast(self, on: bool) -> bool:
        """Switches the exchanges between multimem instructions and plain peer accesses; returns whether multicast is on
        afterwards (it stays off where the symmetric buffer has no multicast mapping).  Collective: every rank must make the
        same choice before the next step."""
        mc = int(getattr(self._hdl, "multicast_ptr", 0) or 0) if self._hdl is not None else 0
        self.multicast = bool(on and mc)
        _lib().bonsai_tp_set_multicast(self.handle, mc if self.multicast else 0)
        return self.multicast

    @classmethod
    def loopback(cls, device, size: int = 2, hidden: int = 4096, vocab: int = 1024, max_batch: int = 1, big_elems: int = 4096,
                 rank: int = 0) -> "TpGroup":
        """A communicator of ``size`` ranks whose peers are plain buffers on this GPU that nothing ever writes: every wait on
        a peer runs into its limit and the kernel reports it in the status word.  For testing the failure path of the
        tensor-parallel kernels on one GPU without any fault (no process group, no symmetric memory)."""
        lib = _lib()
        self = cls.__new__(cls)
        self.rank, self.size = rank, size
        self.recv_elems, self.logits_elems, self.big_elems = hidden, max_batch * vocab, big_elems
        offs = (C.c_size_t * 7)()
        total = lib.bonsai_tp_layout(self.recv_elems, self.logits_elems, self.big_elems, offs)
        self._peers = [torch.zeros(total, dtype=torch.uint8, device=device) for _ in range(size)]
        self.buffer, self._hdl = self._peers[rank], None
        self.multicast = False
        self.state = torch.zeros(4, dtype=torch.int32, device=device)
        arr = (C.c_uint64 * size)(*[t.data_ptr() for t in self._peers])
        self.handle = lib.bonsai_tp_create(rank, size, arr, self.recv_elems, self.logits_elems, self.big_elems, self.state.data_ptr())
        if not self.handle:
            raise RuntimeError("bonsai_tp_create failed")
        lo, bo = int(offs[3]), int(offs[4])
        self.logits = self.buffer[lo: lo + self.logits_elems * 4].view(torch.float32).view(max_batch, vocab)
        self.big = self.buffer[bo: bo + self.big_elems * 4].view(torch.float32)
        return self

    def barrier(self) -> None:
        K.check(_lib().bonsai_tp_barrier(self.handle, K.stream()), "tp_barrier")

    def use_status_word(self, word: torch.Tensor) -> None:
        """Makes the kernels record expired waits in ``word`` (a device int32 the owner reads with its results) instead
        of the group's own word."""
        assert word.is_cuda and word.dtype == torch.int32 and word.numel() == 1
        self._status_word = word
        _lib().bonsai_tp_set_status_ptr(self.handle, word.data_ptr())

    def set_spin_limit(self, polls: int) -> None:
        """Number of polls a wait on a peer may take before the kernel gives up and records a status code."""
        _lib().bonsai_tp_set_spin_limit(self.handle, int(polls))

    def status(self) -> int:
        word = getattr(self, "_status_word", None)
        return int(word.item()) if word is not None else int(self.state[3].item())

    def check(self) -> None:
        s = self.status()
        if s:
            raise K.CudaKernelError(f"tensor-parallel kernel reported status {s}: a peer did not answer within the wait limit")

    def close(self) -> None:
        if getattr(self, "handle", None):
            _lib().bonsai_tp_destroy(self.handle)
            self.handle = None
