#!/usr/bin/env python
"""Long-context prefill and speculative decoding under tensor parallelism.

Workload: a Ternary-Bonsai-8B-shaped TQ2_0_g128 target over N GPUs (TP = N), eight prompts of 32768 random tokens prefilled
in chunks into the paged f16 KV cache, then 128 tokens of one of the sequences decoded two ways at that context length:
plain greedy decode, and speculative decode with a Ternary-Bonsai-1.7B-shaped draft model (also TP = N) whose proposals the
target verifies in one batched pass; the draft length adapts between 1 and 8 tokens to the acceptance history.  Both decoders
are greedy; the verification pass runs the prompt kernels (f16 tensor-core GEMMs) and the plain decode the single-token kernels
(two int8 terms per activation), so on a random-init model, whose top-2 logit gaps are tiny, the two streams may part ways:
the script reports the length of their common prefix (the exact-f32 mode, which the tests use, makes them equal).

    python benchmarks/long_context_spec.py                                                 # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 benchmarks/long_context_spec.py

Reference counterparts: the adaptive lookahead and the speculative decoder (crates/oxibonsai-runtime/src/adaptive_lookahead.rs:48-220,
speculative.rs:43-452), chunked prefill (crates/oxibonsai-runtime/src/prefill.rs) and the tensor-parallel forward
(crates/oxibonsai-model/src/tensor_parallel.rs:338-386).  Target and draft are random-init checkpoints of different shapes, so
the draft's proposals are accepted only by chance: the acceptance rate reported here is the floor of the mechanism, and the
``self_draft`` arm (the target drafting for itself, acceptance 1 by construction) is its ceiling.

Rank 0 prints one JSON line.  Times are host wall-clock around synchronised regions, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SHAPES = {
    "8b": dict(hidden=4096, inter=12288, layers=36, heads=32, kv_heads=8, head_dim=128, vocab=151936, name="Ternary-Bonsai-8B-shaped"),
    "1.7b": dict(hidden=2048, inter=6144, layers=28, heads=16, kv_heads=8, head_dim=128, vocab=151936, name="Ternary-Bonsai-1.7B-shaped"),
    "tiny": dict(hidden=512, inter=1024, layers=2, heads=8, kv_heads=8, head_dim=128, vocab=4096, name="tiny"),
    "tiny-draft": dict(hidden=256, inter=1024, layers=1, heads=8, kv_heads=8, head_dim=128, vocab=4096, name="tiny-draft"),
}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--target", default="8b", choices=list(SHAPES))
    ap.add_argument("--draft", default="1.7b", choices=list(SHAPES))
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=32768)
    ap.add_argument("--decode", type=int, default=128)
    ap.add_argument("--max-lookahead", type=int, default=8)
    ap.add_argument("--no-self-draft", action="store_true", help="skip the arm in which a copy of the target drafts")
    ap.add_argument("--model-dir", default=os.environ.get("BONSAI_BENCH_DIR", "/tmp/oxibonsai_b200_bench"))
    a = ap.parse_args()

    import torch
    import torch.distributed as dist
    from oxibonsai_b200.core import Qwen3Config, write_synthetic_gguf
    from oxibonsai_b200.runtime import EngineBuilder
    from oxibonsai_b200.runtime.speculative import AdaptiveLookahead, GpuSpeculativeDecoder, LookaheadConfig

    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def rmax(v: float) -> float:
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    os.makedirs(a.model_dir, exist_ok=True)
    paths = {}
    for m in (a.target, a.draft):
        paths[m] = os.path.join(a.model_dir, f"{m}_tq2_seed42.gguf")
        if rank == 0 and not os.path.exists(paths[m]):
            write_synthetic_gguf(paths[m] + ".tmp", Qwen3Config(context=65536, **SHAPES[m]), tied=m != "8b", seed=42)
            os.replace(paths[m] + ".tmp", paths[m])
    barrier()

    total = a.prompt_len + a.decode + a.max_lookahead + 16

    def build(model: str, max_batch: int):
        b = (EngineBuilder().model_path(paths[model]).preset("greedy").max_seq_len(total).max_batch(max_batch).kv_cache("f16")
             .device(f"cuda:{local}"))
        if world > 1:
            b = b.tensor_parallel(rank, world)
        return b.build()

    # the batch rows of the gathered logits hold the verified positions: lookahead + 1 of them
    target = build(a.target, max(a.seqs, a.max_lookahead + 1))
    draft = build(a.draft, 1)
    vocab = target.config.vocab
    gen = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, vocab, (a.prompt_len,), generator=gen).tolist() for _ in range(a.seqs)]

    # ---- prefill of all sequences (slot s holds sequence s) ----
    barrier()
    t0 = time.perf_counter()
    for s in range(a.seqs):
        target._bind_slot(s, total)
        target._set_sampling(s, target.sampling)
        target.prefill(prompts[s], s)
    barrier()
    prefill_s = rmax(time.perf_counter() - t0)
    for s in range(a.seqs):
        target._release_slot(s)

    # ---- plain greedy decode of sequence 0 at that context ----
    barrier()
    t0 = time.perf_counter()
    it = target.generate_stream(prompts[0], max_tokens=a.decode, stop_at_eos=False)
    plain, t_first = [], None
    for tok in it:
        plain.append(tok)
        if t_first is None:
            t_first = time.perf_counter()
    barrier()
    plain_decode_s = rmax(time.perf_counter() - t_first)
    plain_prefill_s = rmax(t_first - t0)

    def spec_run(draft_engine) -> dict:
        dec = GpuSpeculativeDecoder(target, draft_engine,
                                    AdaptiveLookahead(LookaheadConfig(min_lookahead=1, max_lookahead=a.max_lookahead, initial=min(4, a.max_lookahead))),
                                    eos_token=None)
        barrier()
        out = dec.generate(prompts[0], a.decode)
        barrier()
        st = dec.stats
        dsec = rmax(st.decode_seconds)
        return {"tokens": len(out), "common_prefix_with_plain_greedy": next((i for i, (x, y) in enumerate(zip(out, plain)) if x != y), min(len(out), len(plain))), "decode_s": round(dsec, 4),
                "tokens_per_s": round((len(out) - 1) / dsec, 2), "prefill_s_target_plus_draft": round(rmax(st.prefill_seconds), 3),
                "acceptance_rate": round(st.acceptance_rate, 4), "mean_lookahead": round(st.drafted / max(1, st.steps), 3),
                "tokens_per_target_pass": round(st.tokens_per_target_pass, 3), "verify_passes": st.target_passes}

    spec = spec_run(draft)
    res = {
        "metric": "long-context prefill + speculative decode", "target": SHAPES[a.target]["name"], "draft": SHAPES[a.draft]["name"],
        "parallelism": f"tp{world}" if world > 1 else "single GPU", "sequences": a.seqs, "prompt_len": a.prompt_len, "kv_cache": "f16",
        "prefill_s": round(prefill_s, 3), "prefill_tokens_per_s": round(a.seqs * a.prompt_len / prefill_s, 1),
        "plain_decode": {"tokens_per_s": round((len(plain) - 1) / plain_decode_s, 2), "prefill_s_one_sequence": round(plain_prefill_s, 3)},
        "speculative": spec,
        "data": "synthetic (seeded random-init GGUFs of both shapes, random prompt tokens): unrelated models agree only by chance",
    }
    if not a.no_self_draft:
        # ceiling of the mechanism: a second engine over the target's own checkpoint drafts, so nearly every proposal is
        # accepted (the draft runs the decode kernels, the verification the prompt kernels); it costs as much as the target,
        # so this arm shows tokens per verification pass, not a speed-up
        del draft
        torch.cuda.empty_cache()
        twin = build(a.target, 1)
        res["self_draft"] = spec_run(twin)
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
