"""Prefill kernels (tcgen05 GEMM with in-smem weight expansion, causal paged attention) against fp32 references."""
import numpy as np
import pytest
import torch

from oxibonsai_b200.core import Q1_0_G128, TQ2_0_G128, dequantize, quantize

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _random_quant(ty, rows, cols, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32)
    raw = quantize(ty, w)
    return raw, torch.from_numpy(dequantize(ty, raw).reshape(rows, cols))


def test_paired_k_layout_round_trip():
    from oxibonsai_b200.ops import cuda_ops as K
    x = torch.randn(3, 256, device=DEV)
    y = K.norm_to_f16_paired(x)
    perm = K.paired_k_index(256, DEV)
    assert torch.equal(y[:, perm], x.half())
    w = torch.rand(256, device=DEV) + 0.5
    yn = K.norm_to_f16_paired(x, w, 1e-6)
    ref = w * x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6)
    assert torch.allclose(yn[:, perm].float(), ref, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("ty", [TQ2_0_G128, Q1_0_G128])
@pytest.mark.parametrize("rows,cols,T", [(256, 256, 64), (6144, 4096, 300), (1000, 2560, 256), (512, 12288, 513), (4096, 1024, 1),
                                         (128, 12288, 7), (4096, 12288, 64), (24576, 4096, 33), (200, 128, 5), (640, 384, 65)])
def test_bitgemm_prefill_matches_fp32(ty, rows, cols, T):
    from oxibonsai_b200.ops import cuda_ops as K
    raw, wd = _random_quant(ty, rows, cols, 21)
    pw = K.PlanarWeight(rows, cols, DEV).fill_from_gguf(torch.from_numpy(raw).to(DEV), ty, cols, 0, rows)
    g = torch.Generator().manual_seed(22)
    x = torch.randn(T, cols, generator=g)
    xp = K.norm_to_f16_paired(x.to(DEV))
    ref = x.half().double() @ wd.double().T
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    y = K.bitgemm_prefill(pw, xp, status=st)
    assert st.item() == 0
    scale = ref.abs().max().item()
    assert (y.cpu().double() - ref).abs().max().item() <= 2e-4 * scale
    res = torch.randn(T, rows, generator=g)
    y = K.bitgemm_prefill(pw, xp, epi=1, residual=res.to(DEV), status=st)
    assert (y.cpu().double() - (ref + res.double())).abs().max().item() <= 2e-4 * scale + 1e-5
    y16 = K.bitgemm_prefill(pw, xp, epi=3, status=st)
    assert (y16.cpu().double() - ref).abs().max().item() <= 2e-3 * scale
    if rows % 32 == 0:
        ys = K.bitgemm_prefill(pw, xp, epi=2, status=st)
        want = torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2]
        perm = K.paired_k_index(rows // 2)
        got = ys.cpu()[:, perm].double()
        assert (got - want).abs().max().item() <= 3e-3 * want.abs().max().item() + 1e-4
    assert st.item() == 0
    # the balanced distribution sums partial tiles in a fixed order: repeatable bit for bit, and close to whole tiles
    y1 = K.bitgemm_prefill(pw, xp, status=st, balanced=True)
    y2 = K.bitgemm_prefill(pw, xp, status=st, balanced=True)
    y0 = K.bitgemm_prefill(pw, xp, status=st, balanced=False)
    assert torch.equal(y1, y2) and st.item() == 0
    assert (y1 - y0).abs().max().item() <= 5e-5 * scale
    assert int(K.gemm_workspace(DEV)[:65536].view(torch.int32).abs().sum().item()) == 0   # counters back to zero


@pytest.mark.parametrize("kvt,tol", [(1, 4e-3), (0, 3e-3), (2, 3e-2)])
@pytest.mark.parametrize("nq,nkv,hd,T,pos0", [(8, 2, 128, 100, 0), (4, 4, 64, 64, 37), (4, 1, 128, 200, 130)])
def test_attn_prefill_matches_reference(kvt, tol, nq, nkv, hd, T, pos0):
    from oxibonsai_b200.core.oracle import rope_table
    from oxibonsai_b200.ops import cuda_ops as K
    page, eps = 16, 1e-6
    total = pos0 + T
    npages = (total + page - 1) // page
    g = torch.Generator().manual_seed(31)
    kfull, vfull = torch.randn(total, nkv, hd, generator=g), torch.randn(total, nkv, hd, generator=g)
    q = torch.randn(T, nq, hd, generator=g)
    row = {0: hd, 1: hd, 2: hd}[kvt]
    kpool = torch.zeros((npages, nkv, page, row), dtype=K.KV_DTYPES[kvt], device=DEV)
    vpool = torch.zeros_like(kpool)
    ksc = torch.zeros((npages, nkv, page), device=DEV) if kvt >= 2 else None
    vsc = torch.zeros((npages, nkv, page), device=DEV) if kvt >= 2 else None
    perm_pages = torch.randperm(npages, generator=g)
    bt = perm_pages.to(torch.int32).to(DEV)
    kd, vd = kfull.clone(), vfull.clone()
    for t in range(total):
        pg, sl = int(perm_pages[t // page]), t % page
        for pool, sc, src, dst in ((kpool, ksc, kfull, kd), (vpool, vsc, vfull, vd)):
            if kvt == 2:
                s = src[t].abs().amax(-1) / 127
                qv = torch.round(src[t] / s[:, None]).clamp(-127, 127)
                pool[pg, :, sl] = qv.to(torch.int8).to(DEV)
                sc[pg, :, sl] = s.to(DEV)
                dst[t] = qv * s[:, None]
            else:
                pool[pg, :, sl] = src[t].to(K.KV_DTYPES[kvt]).to(DEV)
                dst[t] = src[t].to(K.KV_DTYPES[kvt]).float()
    out = K.attn_prefill(q.to(DEV), pos0, bt, nq, nkv, hd, kvt, page, kpool, vpool, ksc, vsc)
    perm = K.paired_k_index(nq * hd)
    got = out.cpu()[:, perm].float().view(T, nq, hd)
    grp = nq // nkv
    kk, vv = kd.repeat_interleave(grp, 1), vd.repeat_interleave(grp, 1)     # [total, nq, hd]
    sc_ = torch.einsum("tnd,snd->nts", q, kk) / hd ** 0.5
    mask = torch.arange(total)[None, :] <= (pos0 + torch.arange(T))[:, None]
    sc_ = sc_.masked_fill(~mask[None], float("-inf"))
    ref = torch.einsum("nts,snd->tnd", torch.softmax(sc_, -1), vv)
    assert (got - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
    if (nq * hd) % 128 == 0:        # the same rows in the K order of the mma.sync GEMM
        out_h = K.attn_prefill(q.to(DEV), pos0, bt, nq, nkv, hd, kvt, page, kpool, vpool, ksc, vsc, k_order=1)
        assert torch.equal(out_h.cpu()[:, K.hmma_k_index(nq * hd)], out.cpu()[:, perm])


@pytest.mark.parametrize("rows,cols,T", [(151936, 2048, 3), (1000, 4096, 64), (300, 256, 200)])
def test_dense_f16_gemm_on_tcgen05(rows, cols, T):
    from oxibonsai_b200.ops import cuda_ops as K
    g = torch.Generator().manual_seed(41)
    w = (torch.randn(rows, cols, generator=g) * 0.02).half().to(DEV)
    x = torch.randn(T, cols, generator=g).half().to(DEV)
    st = torch.zeros(1, dtype=torch.int32, device=DEV)
    y = K.dense_gemm_f16(w, x, status=st)
    ref = x.float() @ w.float().T
    assert st.item() == 0
    assert (y - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()


@pytest.mark.parametrize("ty", [TQ2_0_G128, Q1_0_G128])
@pytest.mark.parametrize("rows,cols,T", [(6144, 4096, 64), (4096, 4096, 33), (24576, 4096, 64), (4096, 12288, 64), (512, 2560, 5), (200, 128, 1),
                                         (1000, 384, 16), (256, 9728, 17)])
def test_bitgemm_hmma_matches_fp32(ty, rows, cols, T):
    """Decode-batch GEMM on mma.sync with register-expanded weights, against a plain fp32 matmul of the same operands."""
    from oxibonsai_b200.ops import cuda_ops as K
    raw, wd = _random_quant(ty, rows, cols, 41)
    pw = K.PlanarWeight(rows, cols, DEV).fill_from_gguf(torch.from_numpy(raw).to(DEV), ty, cols, 0, rows)
    g = torch.Generator().manual_seed(42)
    x = torch.randn(T, cols, generator=g)
    xh = K.norm_to_f16_hmma(x.to(DEV))
    perm = K.hmma_k_index(cols)
    assert torch.equal(xh.cpu()[:, perm], x.half())           # the layout is a pure permutation
    ref = x.half().double() @ wd.double().T
    scale = ref.abs().max().item()
    y = K.bitgemm_hmma(pw, xh)
    assert (y.cpu().double() - ref).abs().max().item() <= 2e-4 * scale
    res = torch.randn(T, rows, generator=g)
    y = K.bitgemm_hmma(pw, xh, epi=1, residual=res.to(DEV))
    assert (y.cpu().double() - (ref + res.double())).abs().max().item() <= 2e-4 * scale + 1e-5
    nw = torch.rand(cols, generator=g) + 0.5
    xn = nw * x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6)
    xnh = K.norm_to_f16_hmma(x.to(DEV), nw.to(DEV), 1e-6)
    assert torch.allclose(xnh.cpu()[:, perm].float(), xn, rtol=2e-3, atol=2e-3)
    if rows % 256 == 0:
        ys = K.bitgemm_hmma(pw, xh, epi=2)
        want = torch.nn.functional.silu(ref[:, 0::2]) * ref[:, 1::2]
        got = ys.cpu()[:, K.hmma_k_index(rows // 2)].double()
        assert (got - want).abs().max().item() <= 3e-3 * want.abs().max().item() + 1e-4
