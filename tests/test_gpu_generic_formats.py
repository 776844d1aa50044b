"""Generic-format GPU path: the block-decoding GEMV for every GGUF type and a whole model served from Q8_0 / Q4_K / FP8."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oxibonsai_b200.core import gguf as G

TYPES = [("F32", G.F32, 1e-5), ("F16", G.F16, 1e-5), ("BF16", G.BF16, 1e-5), ("Q4_0", G.Q4_0, 1e-5), ("Q8_0", G.Q8_0, 1e-5), ("TQ2_0", G.TQ2_0, 1e-5),
         ("F8_E4M3", G.F8_E4M3, 1e-5), ("F8_E5M2", G.F8_E5M2, 1e-5), ("Q2_K", G.Q2_K, 1e-5), ("Q3_K", G.Q3_K, 1e-5), ("Q4_K", G.Q4_K, 1e-5),
         ("Q5_K", G.Q5_K, 1e-5), ("Q6_K", G.Q6_K, 1e-5), ("Q8_K", G.Q8_K, 1e-5)]


@pytest.mark.parametrize("name,tid,tol", TYPES)
def test_quant_gemv_matches_fp32_reference_of_the_decoded_matrix(name, tid, tol):
    from oxibonsai_b200.core.blocks import dequantize, quantize
    from oxibonsai_b200.ops import cuda_ops as K
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(3)
    n, k = 77, 1024
    w = rng.normal(size=(n, k)).astype(np.float32) * 0.05
    q = quantize(tid, w)
    wd = torch.from_numpy(dequantize(tid, q).reshape(n, k)).double()
    x = torch.from_numpy(rng.normal(size=k).astype(np.float32))
    nw = torch.from_numpy(rng.uniform(0.5, 1.5, k).astype(np.float32))
    res = torch.from_numpy(rng.normal(size=n).astype(np.float32))
    qd = torch.from_numpy(q).to(dev)
    y = K.quant_gemv(tid, qd, n, k, x.to(dev)).cpu().double()
    ref = wd @ x.double()
    assert (y - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item()) * 10, name
    xn = nw * x * torch.rsqrt((x * x).mean() + 1e-6)
    y2 = K.quant_gemv(tid, qd, n, k, x.to(dev), norm_w=nw.to(dev), eps=1e-6, residual=res.to(dev)).cpu().double()
    ref2 = wd @ xn.double() + res.double()
    assert torch.allclose(y2, ref2, rtol=1e-4, atol=1e-4), name


def test_swiglu_kernel():
    from oxibonsai_b200.ops import cuda_ops as K
    g, u = torch.randn(5000, device="cuda:0"), torch.randn(5000, device="cuda:0")
    assert torch.allclose(K.swiglu(g, u), torch.nn.functional.silu(g) * u, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k", "f8_e4m3"])
def test_generic_engine_follows_the_cpu_oracle(fmt, tiny_gguf, tmp_path):
    from oxibonsai_b200 import cli
    from oxibonsai_b200.core import GgufFile, Oracle
    from oxibonsai_b200.models.qwen3_generic import GenericQwen3Engine
    path = str(tmp_path / f"tiny_{fmt}.gguf")
    cli.requantize_gguf(tiny_gguf, path, fmt)
    prompt = [11, 257, 3, 999, 42, 7, 100, 5]
    want, _ = Oracle(GgufFile.open(path), 128).generate_greedy(prompt, 12)
    eng = GenericQwen3Engine(path, max_seq_len=128, kv_dtype="f32")
    got = eng.generate(prompt, 12, stop_at_eos=False)
    agree = sum(a == b for a, b in zip(got, want))
    assert len(got) == 12 and agree >= 10, (fmt, got, want)      # f32 everywhere; only the summation order differs from the CPU
    assert eng.generate(prompt, 12, stop_at_eos=False) == got     # graph replay is deterministic
    assert eng.kernel_launches_per_step() == 9 * 2 + 5       # fused Q/K/V and gate/up: 9 launches per layer


@pytest.mark.parametrize("name,tid,tol", TYPES)
def test_quant_to_f16_decodes_every_block_format(name, tid, tol):
    from oxibonsai_b200.core.blocks import dequantize, quantize
    from oxibonsai_b200.ops import cuda_ops as K
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(5)
    n, k = 37, 512
    q = quantize(tid, rng.normal(size=(n, k)).astype(np.float32) * 0.05)
    want = torch.from_numpy(dequantize(tid, q).reshape(n, k)).to(dev).half()      # the kernel rounds the same f32 value once
    qd = torch.from_numpy(q).to(dev)
    nat = K.quant_to_f16(tid, qd, n, k, paired=False)
    assert torch.allclose(nat.float(), want.float(), rtol=2e-3, atol=1e-6), name      # one f16 ulp: the device may fuse d * q - m
    paired = K.quant_to_f16(tid, qd, n, k, paired=True)
    perm = K.paired_k_index(k, dev)
    assert torch.equal(paired[:, perm], nat), name
    # dense GEMM over paired-K operands with the residual epilogue against fp32 PyTorch
    x = torch.randn(70, k, device=dev)
    res = torch.randn(70, n, device=dev)
    got = K.dense_gemm_f16(paired, K.norm_to_f16_paired(x, None), residual=res)
    ref = res + x.half().float() @ nat.float().T
    assert torch.allclose(got, ref, rtol=1e-3, atol=1e-3), name


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
def test_generic_engine_tensor_core_prompt_path_matches_token_by_token(fmt, tiny_gguf, tmp_path):
    from oxibonsai_b200 import cli
    from oxibonsai_b200.models.qwen3_generic import GenericQwen3Engine
    path = str(tmp_path / f"tiny_{fmt}.gguf")
    cli.requantize_gguf(tiny_gguf, path, fmt)
    prompt = [int(t) for t in np.random.default_rng(9).integers(0, 1000, 90)]
    slow = GenericQwen3Engine(path, max_seq_len=256, kv_dtype="f32", prefill_min=10**9)
    fast = GenericQwen3Engine(path, max_seq_len=256, kv_dtype="f32", prefill_min=16, prefill_chunk=64)   # two chunks, the second ragged
    assert fast.prefill_supported()
    a = slow.generate(prompt, 1, stop_at_eos=False)
    b = fast.generate(prompt, 1, stop_at_eos=False)
    la, lb = slow.logits[0].float(), fast.logits[0].float()
    assert torch.nn.functional.cosine_similarity(la, lb, dim=0).item() > 0.999, fmt     # f16 operands in the prompt path only
    assert (la - lb).abs().max().item() <= 0.03 * la.abs().max().item(), fmt
    n = len(prompt) - 1
    ka = slow.kpool[:, : (n + 63) // 64].float()
    kb = fast.kpool[:, : (n + 63) // 64].float()
    assert torch.allclose(ka, kb, rtol=2e-2, atol=2e-2)
    assert len(a) == 1 and len(b) == 1


def test_engine_builder_routes_checkpoints_by_weight_format(tiny_gguf, tmp_path):
    from oxibonsai_b200 import cli
    from oxibonsai_b200.models.qwen3_generic import GenericQwen3Engine
    from oxibonsai_b200.runtime import EngineBuilder, SamplingPreset
    from oxibonsai_b200.runtime.engine import GenericFormatEngine, InferenceEngine
    path = str(tmp_path / "tiny_q8_0.gguf")
    cli.requantize_gguf(tiny_gguf, path, "q8_0")
    eng = EngineBuilder().model_path(path).preset("greedy").max_seq_len(128).kv_cache("f32").build()
    assert isinstance(eng, GenericFormatEngine)
    prompt = [11, 257, 3, 999, 42, 7, 100, 5]
    got = eng.generate(prompt, 6, stop_at_eos=False)
    want = GenericQwen3Engine(path, max_seq_len=128, kv_dtype="f32").generate(prompt, 6, SamplingPreset.GREEDY.params(), stop_at_eos=False)
    assert got == want and len(got) == 6
    assert eng.last_stats.prompt_tokens == 8 and eng.last_stats.generated_tokens == 6 and eng.last_stats.decode_tokens_per_second > 0
    info = eng.model_info()
    assert info["weight_format"].upper().startswith("Q8_0") and info["weight_bytes"] > 0 and info["layers"] == 2
    assert eng.generate_seeded(prompt, 4, seed=7) == eng.generate_seeded(prompt, 4, seed=7)
    assert isinstance(EngineBuilder().model_path(tiny_gguf).max_seq_len(64).build(), InferenceEngine)


@pytest.mark.parametrize("name,tid", [("Q4_0", G.Q4_0), ("Q8_0", G.Q8_0), ("Q4_K", G.Q4_K), ("Q6_K", G.Q6_K), ("F8_E4M3", G.F8_E4M3), ("F16", G.F16)])
@pytest.mark.parametrize("batch", [2, 3, 8, 11])
def test_batched_quant_gemv_matches_fp32_reference(name, tid, batch):
    from oxibonsai_b200.core.blocks import dequantize, quantize
    from oxibonsai_b200.ops import cuda_ops as K
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(11)
    n, k = 70, 1024
    q = quantize(tid, rng.normal(size=(n, k)).astype(np.float32) * 0.05)
    wd = torch.from_numpy(dequantize(tid, q).reshape(n, k)).double()
    x = torch.from_numpy(rng.normal(size=(batch, k)).astype(np.float32))
    nw = torch.from_numpy(rng.uniform(0.5, 1.5, k).astype(np.float32))
    res = torch.from_numpy(rng.normal(size=(batch, n)).astype(np.float32))
    qd = torch.from_numpy(q).to(dev)
    y = K.quant_gemv_batched(tid, qd, n, k, x.to(dev)).cpu().double()
    assert torch.allclose(y, x.double() @ wd.T, rtol=1e-4, atol=1e-4), name
    xn = nw * x * torch.rsqrt((x * x).mean(dim=1, keepdim=True) + 1e-6)
    # output and residual as column ranges of a wider buffer, as the fused projections use them
    wide = torch.zeros((batch, n + 16), device=dev)
    wide[:, 8:8 + n] = res.to(dev)
    K.quant_gemv_batched(tid, qd, n, k, x.to(dev), norm_w=nw.to(dev), eps=1e-6, residual=wide[:, 8:8 + n], out=wide[:, 8:8 + n])
    assert torch.allclose(wide[:, 8:8 + n].cpu().double(), xn.double() @ wd.T + res.double(), rtol=1e-4, atol=1e-4), name
    assert wide[:, :8].abs().max().item() == 0.0 and wide[:, 8 + n:].abs().max().item() == 0.0


def test_swiglu_rows_kernel():
    from oxibonsai_b200.ops import cuda_ops as K
    gu = torch.randn(5, 2 * 300 + 4, device="cuda:0")[:, : 2 * 300]
    want = torch.nn.functional.silu(gu[:, :300]) * gu[:, 300:]
    assert torch.allclose(K.swiglu_rows(gu, 300), want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("fmt", ["q8_0", "q4_k"])
def test_generic_engine_batched_decode_through_the_scheduler(fmt, tiny_gguf, tmp_path):
    """Several sequences decoded together by the generic-format engine (batched GEMV, batch attention and sampler) give the
    streams of the same sequences decoded alone; slots are compacted when a sequence ends early."""
    from oxibonsai_b200 import cli
    from oxibonsai_b200.runtime import EngineBuilder, SamplingPreset
    from oxibonsai_b200.runtime.scheduler import BatchScheduler
    path = str(tmp_path / f"tiny_{fmt}.gguf")
    cli.requantize_gguf(tiny_gguf, path, fmt)
    eng = EngineBuilder().model_path(path).preset("greedy").max_seq_len(160).max_batch(4).kv_cache("f32").build()
    assert eng.max_batch == 4 and eng.model_info()["max_batch"] == 4
    rng = np.random.default_rng(4)
    prompts = [[int(t) for t in rng.integers(0, 1000, n)] for n in (9, 30, 5, 21, 12)]
    lens = [12, 6, 10, 8, 9]
    greedy = SamplingPreset.GREEDY.params()
    alone = [eng.generate(p, n, greedy, stop_at_eos=False) for p, n in zip(prompts, lens)]
    sched = BatchScheduler(eng, eos_token=-1).start()
    try:
        reqs = [sched.submit(p, greedy, n) for p, n in zip(prompts, lens)]
        got = [r.wait(timeout=120) for r in reqs]
    finally:
        sched.stop()
    assert [len(g) for g in got] == lens
    agree = sum(x == y for a, b in zip(alone, got) for x, y in zip(a, b))
    assert agree >= sum(lens) - 2, (alone, got)       # f32 everywhere; the batched GEMV only changes nothing but launch shapes
    assert eng.kv_utilization() == 0.0


def test_standalone_rmsnorm_and_residual_add():
    from oxibonsai_b200.ops import cuda_ops as K
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(3)
    x, w = torch.randn(5, 2560, generator=g).to(dev), (torch.rand(2560, generator=g) + 0.5).to(dev)
    ref = x * torch.rsqrt((x * x).mean(dim=1, keepdim=True) + 1e-6) * w
    assert torch.allclose(K.rmsnorm(x, w, 1e-6), ref, rtol=1e-5, atol=1e-6)
    assert torch.allclose(K.rmsnorm(x[0], None, 1e-6), x[0] * torch.rsqrt((x[0] * x[0]).mean() + 1e-6), rtol=1e-5, atol=1e-6)
    wide = torch.randn(3, 300, generator=g).to(dev)
    view = wide[:, :128]                                       # rows with a stride
    assert torch.allclose(K.rmsnorm(view, None), view * torch.rsqrt((view * view).mean(dim=1, keepdim=True) + 1e-6), rtol=1e-5, atol=1e-6)
    a, b = torch.randn(100003, generator=g).to(dev), torch.randn(100003, generator=g).to(dev)
    want = a + b
    assert torch.equal(K.residual_add(a, b), want)
