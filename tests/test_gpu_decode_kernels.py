"""sm_100a decode kernels against plain PyTorch fp32 references of the same ops."""
import numpy as np
import pytest
import torch

from oxibonsai_b200.core import Q1_0_G128, TQ2_0_G128, dequantize, quantize

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda:0")


def _random_quant(ty, rows, cols, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32)
    raw = quantize(ty, w)
    wd = dequantize(ty, raw).reshape(rows, cols)
    return raw, torch.from_numpy(wd)


@pytest.mark.parametrize("ty", [TQ2_0_G128, Q1_0_G128])
def test_repack_round_trip_and_submatrix(ty):
    from oxibonsai_b200.ops import cuda_ops as K
    rows, cols = 96, 512
    raw, wd = _random_quant(ty, rows, cols, 0)
    rawd = torch.from_numpy(raw).to(_dev())
    pw = K.PlanarWeight(rows, cols, _dev()).fill_from_gguf(rawd, ty, cols, 0, rows)
    assert torch.equal(pw.to_f32().cpu(), wd)
    # rows 32..63, input blocks 1..2, interleaved into even rows of a 64-row matrix
    sub = K.PlanarWeight(64, 256, _dev())
    sub.codes.zero_(); sub.scales.zero_()
    sub.fill_from_gguf(rawd, ty, cols, 32, 32, blk0=1, nblk=2, dst_row0=0, dst_row_stride=2)
    got = sub.to_f32().cpu()
    assert torch.equal(got[0::2], wd[32:64, 128:384]) and (got[1::2] == 0).all()


@pytest.mark.parametrize("ty", [TQ2_0_G128, Q1_0_G128])
@pytest.mark.parametrize("rows,cols", [(6144, 4096), (4096, 12288), (512, 2560), (200, 128), (1000, 9728)])
def test_bitgemv_matches_fp32_matmul(ty, rows, cols):
    from oxibonsai_b200.ops import cuda_ops as K
    raw, wd = _random_quant(ty, rows, cols, 1)
    pw = K.PlanarWeight(rows, cols, _dev()).fill_from_gguf(torch.from_numpy(raw).to(_dev()), ty, cols, 0, rows)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(cols, generator=g)
    ref = wd.double() @ x.double()
    y = K.bitgemv(pw, x.to(_dev()))
    scale = ref.abs().max().item()
    assert (y.cpu().double() - ref).abs().max().item() <= 2e-5 * scale + 1e-6


@pytest.mark.parametrize("ty", [TQ2_0_G128, Q1_0_G128])
@pytest.mark.parametrize("kernel", ["warp", "tile", "hmma"])
@pytest.mark.parametrize("rows,cols", [(6144, 4096), (4096, 12288), (512, 2560), (200, 128), (24576, 4096), (1001, 9728), (300, 6144),
                                       (66, 16384), (5000, 2048)])
def test_bitgemv_half_path_is_close_to_fp32(ty, rows, cols, kernel):
    from oxibonsai_b200.ops import cuda_ops as K
    raw, wd = _random_quant(ty, rows, cols, 9)
    pw = K.PlanarWeight(rows, cols, _dev()).fill_from_gguf(torch.from_numpy(raw).to(_dev()), ty, cols, 0, rows)
    g = torch.Generator().manual_seed(10)
    x, nw, res = torch.randn(cols, generator=g), torch.rand(cols, generator=g) + 0.5, torch.randn(rows, generator=g)
    ref = wd.double() @ x.double()
    y = K.bitgemv(pw, x.to(_dev()), fast=kernel)
    # f16 activations and 8-deep f16 chains: relative to the typical magnitude of the outputs
    assert (y.cpu().double() - ref).abs().max().item() <= 4e-3 * ref.abs().mean().item() * (cols / 128) ** 0.5 + 1e-4
    xn = nw * x * torch.rsqrt((x * x).mean() + 1e-6)
    refn = wd.double() @ xn.double()
    y = K.bitgemv(pw, x.to(_dev()), norm_w=nw.to(_dev()), eps=1e-6, epi=K.EPI_RESID, residual=res.to(_dev()), fast=kernel)
    assert torch.allclose(y.cpu().double(), refn + res.double(), rtol=5e-3, atol=5e-3 * refn.abs().mean().item())
    if rows % 2 == 0:
        y = K.bitgemv(pw, xn.to(_dev()), epi=K.EPI_SWIGLU, fast=kernel)
        want = torch.nn.functional.silu(refn[0::2]) * refn[1::2]
        assert torch.allclose(y.cpu().double(), want, rtol=2e-2, atol=2e-2 * want.abs().mean().item())


@pytest.mark.parametrize("ty", [TQ2_0_G128, Q1_0_G128])
@pytest.mark.parametrize("rows,cols", [(6144, 4096), (4096, 12288), (512, 2560), (200, 128), (24576, 4096), (1001, 9728), (300, 6144),
                                       (66, 16384), (5000, 2048)])
def test_bitgemv_mma_fragment_path_is_close_to_fp32(ty, rows, cols):
    from oxibonsai_b200.ops import cuda_ops as K
    raw, wd = _random_quant(ty, rows, cols, 9)
    pw = K.PlanarWeight(rows, cols, _dev()).fill_from_gguf(torch.from_numpy(raw).to(_dev()), ty, cols, 0, rows)
    fw = K.FragWeight(pw)
    g = torch.Generator().manual_seed(10)
    x, nw, res = torch.randn(cols, generator=g), torch.rand(cols, generator=g) + 0.5, torch.randn(rows, generator=g)
    x[::97] *= 6.0   # outliers stretch the e4m3 range
    ref = wd.double() @ x.double()
    y = K.bitgemv_mma(fw, x.to(_dev()))
    # three e4m3 terms: 12 significant bits relative to the largest activation
    assert (y.cpu().double() - ref).abs().max().item() <= 2e-3 * ref.abs().mean().item() * (cols / 128) ** 0.5 + 1e-4
    xn = nw * x * torch.rsqrt((x * x).mean() + 1e-6)
    refn = wd.double() @ xn.double()
    y = K.bitgemv_mma(fw, x.to(_dev()), norm_w=nw.to(_dev()), eps=1e-6, epi=K.EPI_RESID, residual=res.to(_dev()))
    assert torch.allclose(y.cpu().double(), refn + res.double(), rtol=5e-3, atol=5e-3 * refn.abs().mean().item())
    if rows % 2 == 0:
        y = K.bitgemv_mma(fw, xn.to(_dev()), epi=K.EPI_SWIGLU)
        want = torch.nn.functional.silu(refn[0::2]) * refn[1::2]
        assert torch.allclose(y.cpu().double(), want, rtol=2e-2, atol=2e-2 * want.abs().mean().item())
    # a second call gives the same bits (no dependence on scheduling)
    assert torch.equal(y, K.bitgemv_mma(fw, xn.to(_dev()), epi=K.EPI_SWIGLU)) if rows % 2 == 0 else True


@pytest.mark.parametrize("ty", [TQ2_0_G128, Q1_0_G128])
def test_s16_device_repack_matches_host_layout(ty):
    """The device repack into the streamed decode layout equals the numpy statement of that layout byte for byte."""
    from oxibonsai_b200.ops import cuda_ops as K
    from oxibonsai_b200.ops import s16_layout as L
    rows, cols = 200, 384      # a ragged last tile (200 = 12 * 16 + 8)
    raw, wd = _random_quant(ty, rows, cols, 5)
    pw = K.PlanarWeight(rows, cols, _dev()).fill_from_gguf(torch.from_numpy(raw).to(_dev()), ty, cols, 0, rows)
    sw = K.S16Weight(pw)
    scales = pw.scales.cpu().numpy()
    dense = wd.numpy().reshape(rows, cols // 128, 128) / np.maximum(scales.astype(np.float32), 1e-30)[:, :, None]
    tern = np.rint(dense).astype(np.int8).reshape(rows, cols)
    want = L.pack(tern, scales)
    assert sw.data.cpu().numpy().tobytes() == want.tobytes()


@pytest.mark.parametrize("ty", [TQ2_0_G128, Q1_0_G128])
@pytest.mark.parametrize("rows,cols", [(6144, 4096), (4096, 12288), (512, 2560), (200, 128), (24576, 4096), (1001, 9728), (300, 6144),
                                       (66, 16384), (5000, 2048), (4096, 512), (4096, 1536), (16, 128)])
def test_bitgemv_streamed_is_close_to_fp32(ty, rows, cols):
    """Streamed tensor-core GEMV (S16 layout): activations as two int8 terms per 128-input group (sixteen bits of the
    group's largest value), exact integer products and sums, f32 scales."""
    from oxibonsai_b200.ops import cuda_ops as K
    raw, wd = _random_quant(ty, rows, cols, 9)
    pw = K.PlanarWeight(rows, cols, _dev()).fill_from_gguf(torch.from_numpy(raw).to(_dev()), ty, cols, 0, rows)
    sw = K.S16Weight(pw)
    status = torch.zeros(1, dtype=torch.int32, device=_dev())
    g = torch.Generator().manual_seed(10)
    x, nw, res = torch.randn(cols, generator=g), torch.rand(cols, generator=g) + 0.5, torch.randn(rows, generator=g)
    x[::97] *= 6.0
    ref = wd.double() @ x.double()
    y = K.bitgemv_s16(sw, x.to(_dev()), status=status)
    # the only error is the activation quantisation: <= 1.6e-5 of the group maximum per input
    assert (y.cpu().double() - ref).abs().max().item() <= 3e-4 * ref.abs().mean().item() + 1e-5
    xn = nw * x * torch.rsqrt((x * x).mean() + 1e-6)
    refn = wd.double() @ xn.double()
    y = K.bitgemv_s16(sw, x.to(_dev()), norm_w=nw.to(_dev()), eps=1e-6, epi=K.EPI_RESID, residual=res.to(_dev()), status=status)
    assert torch.allclose(y.cpu().double(), refn + res.double(), rtol=5e-3, atol=5e-3 * refn.abs().mean().item())
    if rows % 2 == 0:
        y = K.bitgemv_s16(sw, xn.to(_dev()), epi=K.EPI_SWIGLU, status=status)
        want = torch.nn.functional.silu(refn[0::2]) * refn[1::2]
        assert torch.allclose(y.cpu().double(), want, rtol=2e-2, atol=2e-2 * want.abs().mean().item())
        assert torch.equal(y, K.bitgemv_s16(sw, xn.to(_dev()), epi=K.EPI_SWIGLU, status=status))   # same bits on a second run
    assert int(status.item()) == 0


def test_bitgemv_fused_norm_residual_swiglu():
    from oxibonsai_b200.ops import cuda_ops as K
    rows, cols = 1024, 2048
    raw, wd = _random_quant(TQ2_0_G128, rows, cols, 2)
    dev = _dev()
    pw = K.PlanarWeight(rows, cols, dev).fill_from_gguf(torch.from_numpy(raw).to(dev), TQ2_0_G128, cols, 0, rows)
    g = torch.Generator().manual_seed(4)
    x, nw, res = torch.randn(cols, generator=g) * 3, torch.rand(cols, generator=g) + 0.5, torch.randn(rows, generator=g)
    eps = 1e-6
    xn = nw * x * torch.rsqrt((x * x).mean() + eps)
    ref = wd.double() @ xn.double()
    y = K.bitgemv(pw, x.to(dev), norm_w=nw.to(dev), eps=eps)
    assert torch.allclose(y.cpu().double(), ref, rtol=1e-4, atol=1e-4)
    y = K.bitgemv(pw, xn.to(dev), epi=K.EPI_RESID, residual=res.to(dev))
    assert torch.allclose(y.cpu().double(), ref + res.double(), rtol=1e-4, atol=1e-4)
    y = K.bitgemv(pw, xn.to(dev), epi=K.EPI_SWIGLU)
    gate, up = ref[0::2], ref[1::2]
    assert torch.allclose(y.cpu().double(), torch.nn.functional.silu(gate) * up, rtol=1e-4, atol=1e-4)
    # in-place residual
    h = res.to(dev).clone()
    K.bitgemv(pw, xn.to(dev), epi=K.EPI_RESID, residual=h, out=h)
    assert torch.allclose(h.cpu().double(), ref + res.double(), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("rows,cols", [(151936, 2048), (5000, 4096), (333, 2560), (64, 8192)])
def test_f16gemv_matches_fp32(rows, cols):
    from oxibonsai_b200.ops import cuda_ops as K
    dev = _dev()
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(rows, cols, generator=g) * 0.02).half()
    x, nw = torch.randn(cols, generator=g), torch.rand(cols, generator=g) + 0.5
    y = K.f16gemv(w.to(dev), x.to(dev))
    ref = w.double() @ x.double()
    assert torch.allclose(y.cpu().double(), ref, rtol=1e-4, atol=1e-4)
    xn = nw * x * torch.rsqrt((x * x).mean() + 1e-6)
    y = K.f16gemv(w.to(dev), x.to(dev), norm_w=nw.to(dev), eps=1e-6)
    assert torch.allclose(y.cpu().double(), w.double() @ xn.double(), rtol=1e-4, atol=1e-4)


def _torch_attention_reference(qkv_steps, nq, nkv, hd, qn, kn, eps, base):
    """Runs the QK-norm -> RoPE -> causal GQA of every step in fp32 and returns the last step's output."""
    ks, vs = [], []
    half = hd // 2
    out = None
    for pos, qkv in enumerate(qkv_steps):
        q = qkv[: nq * hd].view(nq, hd)
        k = qkv[nq * hd:(nq + nkv) * hd].view(nkv, hd)
        v = qkv[(nq + nkv) * hd:].view(nkv, hd)
        norm = lambda t, w: w * t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps)
        q, k = norm(q, qn), norm(k, kn)
        inv = 1.0 / (base ** (torch.arange(half, dtype=torch.float32) * 2 / hd))
        ang = pos * inv
        c, s = torch.cos(ang), torch.sin(ang)
        rope = lambda t: torch.cat([t[:, :half] * c - t[:, half:] * s, t[:, :half] * s + t[:, half:] * c], -1)
        q, k = rope(q), rope(k)
        ks.append(k); vs.append(v)
        Kc, Vc = torch.stack(ks, 1), torch.stack(vs, 1)  # [nkv, T, hd]
        g = nq // nkv
        sc = torch.einsum("hd,htd->ht", q, Kc.repeat_interleave(g, 0)) / hd ** 0.5
        out = torch.einsum("ht,htd->hd", torch.softmax(sc, -1), Vc.repeat_interleave(g, 0))
    return out


@pytest.mark.parametrize("kvt,tol", [(0, 2e-5), (1, 3e-3), (2, 3e-2), (3, 0.35)])
@pytest.mark.parametrize("nq,nkv,hd", [(8, 2, 128), (4, 4, 64), (16, 2, 128)])
def test_qknorm_rope_kvstore_and_paged_attention(kvt, tol, nq, nkv, hd):
    from oxibonsai_b200.core.oracle import rope_table
    from oxibonsai_b200.ops import cuda_ops as K
    dev = _dev()
    steps, page, base, eps = 70, 16, 1e6, 1e-6
    g = torch.Generator().manual_seed(6)
    qn, kn = torch.rand(hd, generator=g) + 0.5, torch.rand(hd, generator=g) + 0.5
    qkvs = [torch.randn((nq + 2 * nkv) * hd, generator=g) for _ in range(steps)]
    ref = _torch_attention_reference(qkvs, nq, nkv, hd, qn, kn, eps, base)
    npages = 8
    row = {0: hd, 1: hd, 2: hd, 3: hd // 2}[kvt]
    kpool = torch.zeros((npages, nkv, page, row), dtype=K.KV_DTYPES[kvt], device=dev)
    vpool = torch.zeros_like(kpool)
    ksc = torch.zeros((npages, nkv, page), device=dev) if kvt >= 2 else None
    vsc = torch.zeros((npages, nkv, page), device=dev) if kvt >= 2 else None
    # a shuffled block table exercises the page indirection
    bt = torch.tensor([[5, 2, 7, 0, 3, 1, 4, 6]], dtype=torch.int32, device=dev)
    cos, sin = rope_table(hd, 128, base)
    cos, sin = torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev)
    pos = torch.zeros(1, dtype=torch.int32, device=dev)
    q = torch.zeros((1, nq, hd), device=dev)
    for t, qkv in enumerate(qkvs):
        pos.fill_(t)
        K.qknorm_rope_kvstore(qkv.to(dev).view(1, -1), qn.to(dev), kn.to(dev), eps, cos, sin, pos, bt, q, nq, nkv, hd, kvt, page, kpool, vpool, ksc, vsc)
    for nsplit in (1, 3, 8):
        out = K.attn_decode(q, pos, bt, nq, nkv, hd, kvt, page, kpool, vpool, ksc, vsc, nsplit=nsplit)
        err = (out[0].cpu() - ref).abs().max().item()
        assert err <= tol * max(1.0, ref.abs().max().item()), (kvt, nsplit, err)


def test_attention_batch_with_different_lengths():
    from oxibonsai_b200.ops import cuda_ops as K
    dev = _dev()
    nq, nkv, hd, page = 4, 2, 64, 16
    g = torch.Generator().manual_seed(8)
    lens = [5, 37]
    kpool = torch.randn((6, nkv, page, hd), generator=g).to(dev)
    vpool = torch.randn((6, nkv, page, hd), generator=g).to(dev)
    bt = torch.tensor([[0, 1, 2], [3, 4, 5]], dtype=torch.int32, device=dev)
    q = torch.randn((2, nq, hd), generator=g).to(dev)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev)
    out = K.attn_decode(q, pos, bt, nq, nkv, hd, K.KV_F32, page, kpool, vpool, nsplit=4).cpu()
    for b, L in enumerate(lens):
        Kc = kpool[bt[b].long()].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :L].cpu()
        Vc = vpool[bt[b].long()].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :L].cpu()
        sc = torch.einsum("hd,htd->ht", q[b].cpu(), Kc.repeat_interleave(2, 0)) / hd ** 0.5
        ref = torch.einsum("ht,htd->hd", torch.softmax(sc, -1), Vc.repeat_interleave(2, 0))
        assert torch.allclose(out[b], ref, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("nq,nkv", [(8, 8), (8, 4), (32, 8), (16, 2)])
@pytest.mark.parametrize("page", [16, 64])
def test_tensor_core_decode_attention_f16(nq, nkv, page):
    """head_dim 128 over f16 pages runs on the mma.sync kernel: against a plain fp32 reference of the same op, with
    ragged lengths, shuffled pages, a draft tail (extra_len) and NaN in every cache row a sequence does not own."""
    from oxibonsai_b200.ops import cuda_ops as K
    dev = _dev()
    hd, G = 128, nq // nkv
    g = torch.Generator().manual_seed(31)
    lens = [1, 15, 16, 17, 250, 333]
    B = len(lens)
    pps = (max(lens) + 3 + page - 1) // page
    perm = torch.randperm(B * pps, generator=g)
    bt = perm.view(B, pps).to(torch.int32).to(dev)
    kf = torch.randn((B * pps, nkv, page, hd), generator=g)
    vf = torch.randn((B * pps, nkv, page, hd), generator=g)
    kpool = torch.full((B * pps, nkv, page, hd), float("nan"), dtype=torch.float16, device=dev)
    vpool = torch.full_like(kpool, float("nan"))
    q = torch.randn((B, nq, hd), generator=g).to(dev)
    for extra in (0, 3):
        pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev)
        refs = []
        for b, L in enumerate(lens):
            n = L + extra
            pages = bt[b].long().cpu()
            Kc = kf[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n].half()
            Vc = vf[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n].half()
            for t in range(n):   # only the rows the sequence owns are real numbers
                kpool[pages[t // page], :, t % page] = Kc[:, t].to(dev)
                vpool[pages[t // page], :, t % page] = Vc[:, t].to(dev)
            sc = torch.einsum("hd,htd->ht", q[b].cpu(), Kc.float().repeat_interleave(G, 0)) / hd ** 0.5
            refs.append(torch.einsum("ht,htd->hd", torch.softmax(sc, -1), Vc.float().repeat_interleave(G, 0)))
        ref = torch.stack(refs)
        for nsplit in (1, 5, 37):
            out = K.attn_decode(q, pos, bt, nq, nkv, hd, K.KV_F16, page, kpool, vpool, nsplit=nsplit, extra_len=extra)
            assert torch.isfinite(out).all()
            # q and the softmax weights are rounded to f16 for the tensor cores: ~1e-3 relative on the scores
            assert (out.cpu() - ref).abs().max().item() <= 4e-3 * max(1.0, ref.abs().max().item()), (nsplit, extra)
            if G <= 4:
                K.lib().bonsai_attn_decode_force_cuda_cores(1)
                try:
                    out2 = K.attn_decode(q, pos, bt, nq, nkv, hd, K.KV_F16, page, kpool, vpool, nsplit=nsplit, extra_len=extra)
                finally:
                    K.lib().bonsai_attn_decode_force_cuda_cores(0)
                assert (out - out2).abs().max().item() <= 4e-3 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("nq,nkv", [(8, 2), (32, 8), (8, 8)])
def test_fused_qknorm_rope_append_attention_matches_separate_kernels(nq, nkv):
    """One launch (QK-norm + RoPE + KV append + attention) against the two separate kernels on a copy of the cache."""
    from oxibonsai_b200.core.oracle import rope_table
    from oxibonsai_b200.ops import cuda_ops as K
    dev = _dev()
    hd, page, B, base, eps = 128, 16, 3, 1e6, 1e-6
    g = torch.Generator().manual_seed(77)
    lens = [1, 40, 129]                                     # context length including the new token
    pps = 10
    bt = torch.randperm(B * pps, generator=g).view(B, pps).to(torch.int32).to(dev)
    kpool = torch.randn((B * pps, nkv, page, hd), generator=g).half().to(dev)
    vpool = torch.randn((B * pps, nkv, page, hd), generator=g).half().to(dev)
    k2, v2 = kpool.clone(), vpool.clone()
    qn, kn = (torch.rand(hd, generator=g) + 0.5).to(dev), (torch.rand(hd, generator=g) + 0.5).to(dev)
    cos, sin = rope_table(hd, 256, base)
    cos, sin = torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev)
    qkv = torch.randn((B, (nq + 2 * nkv) * hd), generator=g).to(dev)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev)
    q = torch.zeros((B, nq, hd), device=dev)
    K.qknorm_rope_kvstore(qkv, qn, kn, eps, cos, sin, pos, bt, q, nq, nkv, hd, K.KV_F16, page, kpool, vpool)
    for nsplit in (1, 4, 16):
        want = K.attn_decode(q, pos, bt, nq, nkv, hd, K.KV_F16, page, kpool, vpool, nsplit=nsplit)
        ka, va = k2.clone(), v2.clone()
        got = K.attn_decode_qkv(qkv, qn, kn, eps, cos, sin, pos, bt, nq, nkv, hd, page, ka, va, nsplit=nsplit)
        # the same rows were appended (the sum of squares is reduced in another order: at most an f16 ulp apart)
        assert torch.equal(va, vpool) and (ka.float() - kpool.float()).abs().max().item() <= 4e-3 * kpool.float().abs().max().item()
        assert (got - want).abs().max().item() <= 2e-3 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("nq,nkv", [(32, 8), (8, 2), (4, 1), (4, 4)])
@pytest.mark.parametrize("nsplit", [2, 8, 16])
def test_cluster_merge_of_decode_attention_matches_the_global_merge(nq, nkv, nsplit):
    """One or two sequences: the KV splits of a (sequence, kv head) run as one thread-block cluster and meet in the first
    CTA's shared memory.  Against the same kernel with the merge through global memory, and against fp32 PyTorch; lengths
    that leave most splits empty are included."""
    from oxibonsai_b200.ops import cuda_ops as K
    dev = _dev()
    hd, page, G = 128, 64, nq // nkv
    g = torch.Generator().manual_seed(5)
    for lens in ([1], [100], [4096], [777, 3000]):
        B = len(lens)
        pps = (max(lens) + page - 1) // page
        bt = torch.randperm(B * pps, generator=g).view(B, pps).to(torch.int32).to(dev)
        kpool = torch.randn((B * pps, nkv, page, hd), generator=g).half().to(dev)
        vpool = torch.randn((B * pps, nkv, page, hd), generator=g).half().to(dev)
        q = torch.randn((B, nq, hd), generator=g).to(dev)
        pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=dev)
        try:
            K.attn_decode_cluster_mode(1)
            plain = K.attn_decode(q, pos, bt, nq, nkv, hd, K.KV_F16, page, kpool, vpool, nsplit=nsplit)
        finally:
            K.attn_decode_cluster_mode(0)
        got = K.attn_decode(q, pos, bt, nq, nkv, hd, K.KV_F16, page, kpool, vpool, nsplit=nsplit)
        again = K.attn_decode(q, pos, bt, nq, nkv, hd, K.KV_F16, page, kpool, vpool, nsplit=nsplit)
        assert torch.isfinite(got).all() and torch.equal(got, again)
        assert (got - plain).abs().max().item() <= 1e-4 * max(1.0, plain.abs().max().item()), (lens, nsplit)
        for b, L in enumerate(lens):
            pages = bt[b].long()
            Kc = kpool[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :L].float()
            Vc = vpool[pages].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :L].float()
            sc = torch.einsum("hd,htd->ht", q[b], Kc.repeat_interleave(G, 0)) / hd ** 0.5
            ref = torch.einsum("ht,htd->hd", torch.softmax(sc, -1), Vc.repeat_interleave(G, 0))
            assert (got[b] - ref).abs().max().item() <= 4e-3 * max(1.0, ref.abs().max().item()), (lens, nsplit, b)
