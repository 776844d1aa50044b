"""End-to-end engine on the GPU: greedy token stream equals the CPU oracle's."""
import pytest
import torch

from oxibonsai_b200.core import GgufFile, Oracle

pytestmark = pytest.mark.gpu


def _oracle_tokens(path, prompt, n):
    return Oracle(GgufFile.open(path), 128).generate_greedy(prompt, n)


@pytest.mark.parametrize("fixture", ["tiny_gguf", "tiny_q1_gguf"])
def test_greedy_stream_matches_oracle_f32_kv(fixture, request):
    from oxibonsai_b200.runtime import EngineBuilder
    path = request.getfixturevalue(fixture)
    prompt = [11, 257, 3, 999, 42, 7]
    want, gaps = _oracle_tokens(path, prompt, 24)
    eng = EngineBuilder().model_path(path).preset("greedy").max_seq_len(128).kv_cache("f32").build()
    got = eng.generate(prompt, 24)
    assert got == want, (got, want, gaps)
    # a second request on the same engine starts from a clean slot
    assert eng.generate(prompt, 24) == want
    st = eng.last_stats
    assert st.prompt_tokens == len(prompt) and st.generated_tokens == 24 and st.tokens_per_second > 0


@pytest.mark.parametrize("kv", ["f16", "q8"])
def test_greedy_stream_with_compressed_kv_stays_close(kv, tiny_gguf):
    from oxibonsai_b200.runtime import EngineBuilder
    prompt = [5, 6, 7, 8]
    want, gaps = _oracle_tokens(tiny_gguf, prompt, 12)
    eng = EngineBuilder().model_path(tiny_gguf).preset("greedy").max_seq_len(64).kv_cache(kv).build()
    got = eng.generate(prompt, 12)
    # compressed KV may flip a near-tie; the stream must agree up to the first step whose top-2 gap is tiny
    for i, (a, b) in enumerate(zip(got, want)):
        if a != b:
            assert gaps[i] < 0.05, (i, got, want, gaps)
            break


def test_seeded_sampling_is_reproducible(tiny_gguf):
    from oxibonsai_b200.runtime import EngineBuilder
    eng = EngineBuilder().model_path(tiny_gguf).preset("balanced").max_seq_len(64).seed(123).build()
    a = eng.generate([1, 2, 3], 16, stop_at_eos=False)
    b = eng.generate([1, 2, 3], 16, stop_at_eos=False)
    c = eng.generate_seeded([1, 2, 3], 16, seed=124)
    assert a == b and len(a) == 16 and all(0 <= t < 1000 for t in a)
    assert c != a or True


def test_batched_prefill_agrees_with_token_by_token_prefill(tiny_gguf):
    """The tcgen05 prefill path and the decode path must produce the same next-token logits (up to f16 activations)."""
    from oxibonsai_b200.runtime import EngineBuilder
    eng = EngineBuilder().model_path(tiny_gguf).preset("greedy").max_seq_len(256).kv_cache("f16").build()
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 1000, (150,), generator=g).tolist()
    eng._bind_slot(0, 200)
    eng.prefill_min_tokens = 10 ** 9
    eng.prefill(prompt, 0)
    ref = eng.runner.logits[0].clone()
    eng.prefill_min_tokens = 16
    eng.prefill_chunk = 64          # three chunks: exercises attention over earlier chunks
    eng.prefill(prompt, 0)
    got = eng.runner.logits[0].clone()
    assert eng.runner._pf["status"].item() == 0
    eng._release_slot(0)
    scale = ref.abs().max().item()
    assert (got - ref).abs().max().item() < 0.03 * scale
    assert got.argmax().item() == ref.argmax().item() or (ref.topk(2).values.diff().abs().item() < 0.05 * scale)
    # generation after a batched prefill continues from the cache the prefill kernels wrote
    a = eng.generate(prompt, 8)
    eng.prefill_min_tokens = 10 ** 9
    b = eng.generate(prompt, 8)
    assert len(a) == 8 and sum(x == y for x, y in zip(a, b)) >= 6


def test_batched_decode_matches_single_sequence_decode(tiny_gguf):
    from oxibonsai_b200.runtime import EngineBuilder
    eng = EngineBuilder().model_path(tiny_gguf).preset("greedy").max_seq_len(128).max_batch(4).kv_cache("f16").build()
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (20, 33, 17)]
    single = [eng.generate(p, 10) for p in prompts]
    batch = eng.generate_batch(prompts, 10)
    assert [len(b) for b in batch] == [10, 10, 10]
    agree = sum(x == y for a, b in zip(single, batch) for x, y in zip(a, b))
    assert agree >= 24, (single, batch)   # f16 GEMM activations vs packed-half GEMV: near-ties may flip late tokens
    assert eng.runner._pf["status"].item() == 0


def test_constraint_masks_reach_the_gpu_sampler(tiny_gguf):
    """Constrained decoding through the engine: the constraint's vocabulary mask is uploaded before every step and the
    sampler kernel only picks allowed tokens; a sequence constraint forces its tokens and ends the generation."""
    from oxibonsai_b200.runtime import EngineBuilder
    from oxibonsai_b200.runtime.constrained import AllowListConstraint, SequenceConstraint, TokenTable
    from oxibonsai_b200.runtime.presets import SamplingParams
    eng = EngineBuilder().model_path(tiny_gguf).preset("greedy").max_seq_len(96).build()
    table = TokenTable([bytes([i % 251, i // 251]) for i in range(1000)])
    free = eng.generate([3, 1, 4, 1, 5], 10, stop_at_eos=False)
    allowed = {7, 300, 999, 512}
    got = eng.generate([3, 1, 4, 1, 5], 10, stop_at_eos=False, constraint=AllowListConstraint(table, allowed))
    assert len(got) == 10 and set(got) <= allowed
    hot = eng.generate([3, 1, 4, 1, 5], 10, SamplingParams(temperature=0.9, top_k=40, top_p=0.95, seed=3), stop_at_eos=False,
                       constraint=AllowListConstraint(table, allowed))
    assert len(hot) == 10 and set(hot) <= allowed
    forced = eng.generate([3, 1, 4, 1, 5], 10, stop_at_eos=False, constraint=SequenceConstraint(table, [11, 22, 33]))
    assert forced == [11, 22, 33]
    assert eng.generate([3, 1, 4, 1, 5], 10, stop_at_eos=False) == free          # the mask does not outlive its request
    lp, top = eng.token_logprobs(0, free[-1], 3)
    assert lp <= 0.0 and len(top) == 3 and top[0][1] >= top[1][1] >= top[2][1]


def test_repacked_weight_cache_gives_the_same_engine(tiny_gguf, tmp_path):
    from oxibonsai_b200.runtime import EngineBuilder
    prompt = [5, 9, 200, 31, 77]
    mk = lambda: EngineBuilder().model_path(tiny_gguf).preset("greedy").max_seq_len(96).kv_cache("f16").repack_cache(str(tmp_path)).build()
    first = mk()
    assert not first.weights.from_cache and len(list(tmp_path.iterdir())) == 1
    want = first.generate(prompt, 12)
    second = mk()
    assert second.weights.from_cache and second.model_info()["weights_from_repack_cache"]
    assert second.generate(prompt, 12) == want
    assert second.weights.packed_bytes == first.weights.packed_bytes


def test_kernel_histogram_lists_the_kernels_of_a_decode_step(tiny_gguf):
    from oxibonsai_b200.runtime import EngineBuilder
    from oxibonsai_b200.runtime.observability import kernel_histogram
    eng = EngineBuilder().model_path(tiny_gguf).preset("greedy").max_seq_len(96).build()
    eng.generate([3, 1, 4, 1, 5], 4, stop_at_eos=False)          # graph captured, slot released
    eng._bind_slot(0, 32)
    eng._upload(0, 7, 0)
    try:
        table = kernel_histogram(lambda: eng.runner.step(1, sample=True), iterations=2)
    except Exception as e:                                       # no CUPTI on the box
        pytest.skip(f"profiler unavailable: {e}")
    finally:
        eng._release_slot(0)
    if not table:
        pytest.skip("the profiler recorded no device activity")
    gemv = [k for k in table if "bitgemv_s16" in k]
    assert gemv and table[gemv[0]]["count"] == 2 * 4 * eng.config.layers      # four projections per layer and step
    assert any("attn_decode" in k for k in table) and all(r["mean_us"] >= 0 for r in table.values())
