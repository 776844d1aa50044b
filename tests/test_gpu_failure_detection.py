"""Failure detection of the tensor-parallel kernels on one GPU, without any fault: a communicator whose peer never
writes makes every bounded wait run out; the kernel must return, record its status code and leave the context usable."""
import numpy as np
import pytest
import torch

from oxibonsai_b200.core import TQ2_0_G128, quantize

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


def test_barrier_wait_expires_with_status_3():
    from oxibonsai_b200.ops import cuda_ops as K
    from oxibonsai_b200.parallel.tp import TpGroup
    tp = TpGroup.loopback(_dev(), size=2)
    tp.set_spin_limit(2000)
    tp.barrier()
    torch.cuda.synchronize()
    assert tp.status() == 3
    with pytest.raises(K.CudaKernelError):
        tp.check()
    # the context is alive and other kernels still run
    assert float(torch.ones(8, device=_dev()).sum()) == 8.0
    tp.close()


@pytest.mark.parametrize("fast", [True, False])
def test_fused_gemv_allreduce_reports_a_silent_peer(fast):
    from oxibonsai_b200.ops import cuda_ops as K
    from oxibonsai_b200.parallel.tp import TpGroup, _lib
    rows, cols = 256, 512
    rng = np.random.default_rng(0)
    raw = quantize(TQ2_0_G128, (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32))
    pw = K.PlanarWeight(rows, cols, _dev()).fill_from_gguf(torch.from_numpy(raw).to(_dev()), TQ2_0_G128, cols, 0, rows)
    tp = TpGroup.loopback(_dev(), size=2, hidden=rows)
    tp.set_spin_limit(2000)
    word = torch.zeros(1, dtype=torch.int32, device=_dev())
    tp.use_status_word(word)
    x = torch.randn(cols, device=_dev())
    res = torch.randn(rows, device=_dev())
    out = torch.empty(rows, device=_dev())
    if fast:
        K.bitgemv_s16(K.S16Weight(pw), x, epi=K.EPI_TP, residual=res, out=out, comm=tp.handle, status=word)
    else:
        K.check(_lib().bonsai_bitgemv_tp(tp.handle, pw.codes.data_ptr(), pw.scales.data_ptr(), x.data_ptr(), 1e-6, out.data_ptr(),
                                         res.data_ptr(), rows, cols, 0, K.stream()), "bitgemv_tp")
    torch.cuda.synchronize()
    assert int(word.item()) == 2
    # the kernel returned: the exchange counter moved on, so a later healthy exchange would not be confused with this one
    assert int(tp.state[0].item()) == 1
    tp.close()


def test_engine_raises_when_the_status_word_is_set(tiny_gguf):
    """A non-zero status word read with the sampled token turns into CudaKernelError instead of a token."""
    from oxibonsai_b200.ops import cuda_ops as K
    from oxibonsai_b200.runtime import EngineBuilder
    eng = EngineBuilder().model_path(tiny_gguf).preset("greedy").max_seq_len(64).build()
    assert eng.generate([1, 2, 3], 2)            # healthy
    it = eng.generate_stream([1, 2, 3], 4)
    next(it)
    eng.runner.status.fill_(2)                   # what a kernel does when a peer stays silent
    with pytest.raises(K.CudaKernelError):
        for _ in it:
            pass
    assert int(eng.runner.status.item()) == 0    # cleared once reported
    assert eng.generate([1, 2, 3], 2)            # and the engine is usable again
