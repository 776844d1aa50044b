"""The allocation-free decode-attention entry point, called through its exported C symbol.

Collected last (file name) so that it also runs after every other GPU test has used the device; it must pass alone too.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ACC_FLOATS = 1 << 20


def _symbol():
    from oxibonsai_b200 import _native
    fn = _native.cuda().bonsai_attn_decode_static
    vp, i = C.c_void_p, C.c_int
    fn.restype = C.c_int
    fn.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, vp, vp, vp, vp, i, vp, i, vp, C.c_char_p, C.c_size_t]
    return fn


def _case(dev, seed, lens, nq=8, nkv=2, hd=128, page=16, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    batch = len(lens)
    pages_per_seq = (max(lens) + page - 1) // page
    npages = batch * pages_per_seq
    kpool = torch.randn((npages, nkv, page, hd), generator=g).to(dev).to(dtype)
    vpool = torch.randn((npages, nkv, page, hd), generator=g).to(dev).to(dtype)
    bt = torch.randperm(npages, generator=g).to(torch.int32).view(batch, pages_per_seq).to(dev)
    q = torch.randn((batch, nq, hd), generator=g).to(dev)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev)
    return dict(q=q, pos=pos, bt=bt, kpool=kpool, vpool=vpool, nq=nq, nkv=nkv, hd=hd, page=page, lens=lens)


def _call_static(fn, c, nsplit, batch=None, out=None):
    from oxibonsai_b200.ops import cuda_ops as K
    kvt = K.KV_F16 if c["kpool"].dtype == torch.float16 else K.KV_F32
    batch = c["q"].shape[0] if batch is None else batch      # an overridden batch is only ever used for calls that are rejected
    if out is None:
        out = torch.full((c["q"].shape[0], c["nq"], c["hd"]), float("nan"), device=c["q"].device)
    err = C.create_string_buffer(256)
    rc = fn(c["q"].data_ptr(), c["pos"].data_ptr(), c["bt"].data_ptr(), c["bt"].shape[1], batch, c["nq"], c["nkv"], c["hd"],
            kvt, c["page"], c["kpool"].data_ptr(), c["vpool"].data_ptr(), None, None, nsplit, out.data_ptr(), 0,
            K.stream(), err, len(err))
    return rc, err.value.decode(), out


def _fp32_reference(c):
    outs = []
    G = c["nq"] // c["nkv"]
    for b, L in enumerate(c["lens"]):
        Kc = c["kpool"][c["bt"][b].long()].permute(1, 0, 2, 3).reshape(c["nkv"], -1, c["hd"])[:, :L].cpu()
        Vc = c["vpool"][c["bt"][b].long()].permute(1, 0, 2, 3).reshape(c["nkv"], -1, c["hd"])[:, :L].cpu()
        sc = torch.einsum("hd,htd->ht", c["q"][b].cpu(), Kc.repeat_interleave(G, 0)) / c["hd"] ** 0.5
        outs.append(torch.einsum("ht,htd->hd", torch.softmax(sc, -1), Vc.repeat_interleave(G, 0)))
    return torch.stack(outs)


def test_static_scratch_entry_matches_buffer_entry_on_consecutive_calls():
    from oxibonsai_b200.ops import cuda_ops as K
    dev = torch.device("cuda:0")
    fn = _symbol()
    # two calls in a row with different shapes and split counts reuse the same built-in scratch
    for seed, lens, nsplit in ((11, [70, 5, 33], 8), (12, [129], 3), (13, [40, 41], 1)):
        c = _case(dev, seed, lens)
        rc, msg, got = _call_static(fn, c, nsplit)
        assert rc == 0, msg
        want = K.attn_decode(c["q"], c["pos"], c["bt"], c["nq"], c["nkv"], c["hd"], K.KV_F32, c["page"], c["kpool"], c["vpool"],
                             nsplit=nsplit)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (seed, (got - want).abs().max().item())
        assert torch.allclose(got.cpu(), _fp32_reference(c), rtol=1e-4, atol=1e-5)
    # same inputs twice in a row give the same bits (the counters were left clean)
    c = _case(dev, 14, [90, 17])
    a = _call_static(fn, c, 4)[2]
    b = _call_static(fn, c, 4)[2]
    torch.cuda.synchronize()
    assert torch.equal(a, b) and not torch.isnan(a).any()


def test_static_scratch_entry_takes_the_f16_tensor_core_path_and_allocates_nothing():
    """f16 pages with head_dim 128 and 16-token pages go to the warp-level tensor-core kernel behind the same symbol; the
    result equals the buffer entry's bit for bit, and a warm call leaves the device's free memory and torch's allocator
    counters where they were."""
    from oxibonsai_b200.ops import cuda_ops as K
    dev = torch.device("cuda:0")
    fn = _symbol()
    c = _case(dev, 21, [200, 77, 16], nq=8, nkv=2, hd=128, page=16, dtype=torch.float16)
    out = torch.full((3, 8, 128), float("nan"), device=dev)
    for nsplit in (4, 2):
        rc, msg, got = _call_static(fn, c, nsplit, out=out)
        assert rc == 0, msg
        want = K.attn_decode(c["q"], c["pos"], c["bt"], c["nq"], c["nkv"], c["hd"], K.KV_F16, c["page"], c["kpool"], c["vpool"], nsplit=nsplit)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    c32 = dict(c, kpool=c["kpool"].float(), vpool=c["vpool"].float())
    assert torch.allclose(got.cpu(), _fp32_reference(c32), rtol=2e-3, atol=2e-3)
    # warm call: nothing is allocated, by the driver or by torch
    torch.cuda.synchronize()
    free0, alloc0, reserved0 = torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)
    rc, msg, _ = _call_static(fn, c, 4, out=out)
    torch.cuda.synchronize()
    assert rc == 0, msg
    assert torch.cuda.mem_get_info(dev)[0] == free0
    assert torch.cuda.memory_allocated(dev) == alloc0 and torch.cuda.memory_reserved(dev) == reserved0


def test_static_scratch_entry_rejects_oversized_requests():
    dev = torch.device("cuda:0")
    fn = _symbol()
    c = _case(dev, 15, [8], nq=8, nkv=2, hd=128)
    nsplit = MAX_ACC_FLOATS // (8 * 128) + 1   # one split too many for the 1 Mi-float accumulator area
    rc, msg, out = _call_static(fn, c, nsplit)
    torch.cuda.synchronize()
    assert rc < 0 and "exceeds the built-in scratch" in msg
    assert torch.isnan(out).all()              # nothing was launched
    rc, msg, _ = _call_static(fn, c, 0)
    assert rc < 0 and "positive" in msg
    # one (sequence, kv head) pair more than there are arrival counters: rejected on the arguments alone
    one = _case(dev, 16, [8], nq=1, nkv=1, hd=128)
    rc, msg, out = _call_static(fn, one, 1, batch=4097)
    torch.cuda.synchronize()
    assert rc < 0 and "arrival counters" in msg and torch.isnan(out).all()
    # the max/sum area (32 Ki floats) runs out before the accumulators do when head_dim is small
    small = _case(dev, 17, [8], nq=8, nkv=2, hd=16)
    rc, msg, out = _call_static(fn, small, 2049)      # 8 * 2049 * 2 = 32784 > 32768, accumulators 262272 floats
    torch.cuda.synchronize()
    assert rc < 0 and "max/sum" in msg and torch.isnan(out).all()
