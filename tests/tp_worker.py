"""Worker of the multi-GPU tensor-parallel tests: run as one process per GPU under torch.distributed.run."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main():
    path, mode, out_dir = sys.argv[1], sys.argv[2], sys.argv[3]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from oxibonsai_b200.core import GgufFile, Oracle
    from oxibonsai_b200.runtime import EngineBuilder

    prompt = [11, 257, 3, 999, 42, 7]
    out = {"rank": rank}
    if mode == "exact":
        want, gaps = Oracle(GgufFile.open(path), 128).generate_greedy(prompt, 16)
        eng = EngineBuilder().model_path(path).preset("greedy").max_seq_len(128).kv_cache("f32").device(f"cuda:{local}").tensor_parallel(rank, world).build()
        got = eng.generate(prompt, 16)
        out.update(ok=(got == want), got=got, want=want, status=eng.runner.tp.status())
    elif mode == "fast":
        eng = EngineBuilder().model_path(path).preset("greedy").max_seq_len(256).kv_cache("f16").device(f"cuda:{local}").tensor_parallel(rank, world).build()
        g = torch.Generator().manual_seed(5)
        long_prompt = torch.randint(0, 1000, (90,), generator=g).tolist()
        a = eng.generate(long_prompt, 8)               # batched prefill (tcgen05 GEMMs + two-shot all-reduce)
        eng.prefill_min_tokens = 10 ** 9
        b = eng.generate(long_prompt, 8)               # token-by-token prefill through the fused GEMV all-reduce
        toks = torch.tensor(a, device=f"cuda:{local}")
        gathered = [torch.zeros_like(toks) for _ in range(world)]
        dist.all_gather(gathered, toks)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        out.update(ok=(len(a) == 8 and same and sum(x == y for x, y in zip(a, b)) >= 6), a=a, b=b, same=same, status=eng.runner.tp.status())
    elif mode == "batched":
        # four sequences decoded together: tcgen05 GEMMs + one-shot all-reduce kernels + vocab-parallel dense LM head
        eng = (EngineBuilder().model_path(path).preset("greedy").max_seq_len(160).max_batch(4).kv_cache("f16").device(f"cuda:{local}")
               .tensor_parallel(rank, world).build())
        g = torch.Generator().manual_seed(9)
        prompts = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (20, 33, 17, 41)]
        single = [eng.generate(p, 10) for p in prompts]
        batch = eng.generate_batch(prompts, 10)
        again = eng.generate_batch(prompts, 10)        # graph replay after the capture, halves keep alternating
        toks = torch.tensor(batch, device=f"cuda:{local}")
        gathered = [torch.zeros_like(toks) for _ in range(world)]
        dist.all_gather(gathered, toks)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        agree = sum(x == y for a, b in zip(single, batch) for x, y in zip(a, b))
        out.update(ok=(same and batch == again and agree >= 32 and all(len(b) == 10 for b in batch)), agree=agree, same=same,
                   single=single, batch=batch, again=again, status=eng.runner.tp.status(), pf_status=int(eng.runner._pf["status"].item()))
    elif mode == "speculative":
        # exact mode on both sides: the batched verification (vocab-parallel head gathered for every verified position)
        # picks the target's own greedy tokens, and a draft with the same weights is accepted every time
        from oxibonsai_b200.runtime.speculative import GpuSpeculativeDecoder
        mk = lambda nb: (EngineBuilder().model_path(path).preset("greedy").max_seq_len(128).max_batch(nb).kv_cache("f32").device(f"cuda:{local}")
                         .tensor_parallel(rank, world).build())
        target, draft = mk(9), mk(1)
        want = target.generate(prompt, 20)
        dec = GpuSpeculativeDecoder(target, draft)
        got = dec.generate(prompt, 20)
        out.update(ok=(got[:len(want)] == want[:len(got)] and len(got) >= len(want) - 1 and dec.stats.acceptance_rate > 0.9),
                   got=got, want=want, acceptance=dec.stats.acceptance_rate, status=target.runner.tp.status() | draft.runner.tp.status())
    dist.barrier()
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(out, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
