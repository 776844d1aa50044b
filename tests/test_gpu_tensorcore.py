"""tcgen05 kernels: operand encodings (single tile) and the tensor-core decode GEMV against fp32 references."""
import ctypes as C

import numpy as np
import pytest
import torch

from oxibonsai_b200.core import Q1_0_G128, TQ2_0_G128, dequantize, quantize

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tile(Ab, Bb, N, kind):
    from oxibonsai_b200.ops import cuda_ops as K
    lib = K._tc()
    out = torch.zeros((128, N), device=DEV)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    Ad, Bd = Ab.contiguous().to(DEV), Bb.contiguous().to(DEV)  # keep both alive across the launch
    K.check(lib.bonsai_tc_tile(Ad.data_ptr(), Bd.data_ptr(), out.data_ptr(), N, kind, st.data_ptr(), K.stream()), "tc_tile")
    torch.cuda.synchronize()
    assert st.item() == 0
    return out.cpu()


@pytest.mark.parametrize("N", [16, 64, 256])
def test_single_tile_f16_and_bf16(N):
    g = torch.Generator().manual_seed(0)
    for kind, dt in ((0, torch.float16), (1, torch.bfloat16)):
        A, B = torch.randn(128, 64, generator=g).to(dt), torch.randn(N, 64, generator=g).to(dt)
        out = _tile(A.view(torch.uint8).reshape(128, 128), B.view(torch.uint8).reshape(N, 128), N, kind)
        assert torch.allclose(out, A.float() @ B.float().T, rtol=1e-4, atol=1e-4)


def test_single_tile_fp4_times_fp8_is_exact():
    g = torch.Generator().manual_seed(1)
    N = 32
    B = torch.randn(N, 128, generator=g).to(torch.float8_e4m3fn)
    W = torch.randint(-1, 2, (128, 128), generator=g)
    nib = torch.where(W == 1, 2, torch.where(W == -1, 10, 0)).to(torch.uint8).view(128, 8, 16)
    enc = torch.zeros(128, 8, 16, dtype=torch.uint8)
    enc[:, :, :8] = nib[:, :, 0::2] | (nib[:, :, 1::2] << 4)  # 16 e2m1 values in 8 bytes, then 8 bytes of padding
    out = _tile(enc.view(128, 128), B.view(torch.uint8), N, 2)
    assert torch.equal(out, W.float() @ B.float().T)


def _random_quant(ty, rows, cols, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32)
    raw = quantize(ty, w)
    return raw, torch.from_numpy(dequantize(ty, raw).reshape(rows, cols))


@pytest.mark.parametrize("ty", [TQ2_0_G128, Q1_0_G128])
@pytest.mark.parametrize("rows,cols,T,nterms", [(6144, 4096, 1, 4), (4096, 12288, 1, 3), (1000, 2560, 2, 3), (24576, 4096, 1, 3),
                                                (512, 1024, 5, 3), (384, 256, 16, 2), (256, 9728, 21, 3)])
def test_bitgemv_tc_matches_fp32(ty, rows, cols, T, nterms):
    from oxibonsai_b200.ops import cuda_ops as K
    raw, wd = _random_quant(ty, rows, cols, 3)
    pw = K.PlanarWeight(rows, cols, DEV).fill_from_gguf(torch.from_numpy(raw).to(DEV), ty, cols, 0, rows)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(T, cols, generator=g) * torch.logspace(-2, 1, cols)[torch.randperm(cols, generator=g)]
    ws = K.TcWorkspace(DEV)
    act = K.act_prep_fp8(x.to(DEV), nterms)
    ref = x.double() @ wd.double().T
    tol = {2: 6e-3, 3: 5e-4, 4: 5e-5}[nterms]
    auto = K.pick_ksplit(rows, cols, act.ncols)
    outs = []
    for ks in sorted({auto, auto * 2, min(cols // 128, auto * 4)}):
        y = torch.full((T, rows), float("nan"), device=DEV)
        K.bitgemv_tc(pw, ws, act=act, ksplit=ks, out=y)
        ws.check()
        err = (y.cpu().double() - ref).abs().max().item() / ref.abs().max().item()
        assert err < tol, (ks, err)
    if T <= 4:
        # operand built inside the kernel gives the same numbers as the prepared operand
        ya = torch.full((T, rows), float("nan"), device=DEV)
        yb = torch.full((T, rows), float("nan"), device=DEV)
        K.bitgemv_tc(pw, ws, act=act, ksplit=auto, out=ya)
        K.bitgemv_tc(pw, ws, x=x.to(DEV), nterms=nterms, ksplit=auto, out=yb)
        assert torch.equal(ya, yb)
    # run-to-run determinism with a K split (outputs pre-filled with NaN: every element must be written)
    y1 = torch.full((T, rows), float("nan"), device=DEV)
    y2 = torch.full((T, rows), float("nan"), device=DEV)
    K.bitgemv_tc(pw, ws, act=act, ksplit=auto * 2, out=y1)
    K.bitgemv_tc(pw, ws, act=act, ksplit=auto * 2, out=y2)
    assert torch.equal(y1, y2) and not torch.isnan(y1).any()
    assert ws.counters.abs().sum().item() == 0
    # fewer SMs than tiles: every CTA column walks several tiles
    y3 = K.bitgemv_tc(pw, ws, act=act, ksplit=auto, sms=8 * auto)
    err = (y3.cpu().double() - ref).abs().max().item() / ref.abs().max().item()
    assert err < tol
    ws.check()


def test_bitgemv_tc_fused_norm_and_epilogues():
    from oxibonsai_b200.ops import cuda_ops as K
    rows, cols = 2048, 2048
    raw, wd = _random_quant(TQ2_0_G128, rows, cols, 5)
    pw = K.PlanarWeight(rows, cols, DEV).fill_from_gguf(torch.from_numpy(raw).to(DEV), TQ2_0_G128, cols, 0, rows)
    g = torch.Generator().manual_seed(6)
    x, nw, res = torch.randn(2, cols, generator=g) * 3, torch.rand(cols, generator=g) + 0.5, torch.randn(2, rows, generator=g)
    xn = nw * x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6)
    ref = xn.double() @ wd.double().T
    ws = K.TcWorkspace(DEV)
    act = K.act_prep_fp8(x.to(DEV), 3, norm_w=nw.to(DEV), eps=1e-6)
    xd, nwd = x.to(DEV), nw.to(DEV)
    for ks in (1, 4):
        for kw in (dict(act=act),):
            y = K.bitgemv_tc(pw, ws, ksplit=ks, **kw)
            assert torch.allclose(y.cpu().double(), ref, rtol=2e-3, atol=2e-3)
            h = res.to(DEV).clone()
            K.bitgemv_tc(pw, ws, epi=K.EPI_RESID, residual=h, out=h, ksplit=ks, **kw)
            assert torch.allclose(h.cpu().double(), ref + res.double(), rtol=2e-3, atol=2e-3)
            y = K.bitgemv_tc(pw, ws, epi=K.EPI_SWIGLU, ksplit=ks, **kw)
            assert torch.allclose(y.cpu().double(), torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2], rtol=3e-3, atol=3e-3)
    ws.check()
