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
    elif mode == "multimem":
        # the exchanges through the NVLink switch (multimem.st / multimem.ld_reduce) against the plain peer accesses and
        # against NCCL; reported as skipped where the symmetric buffer has no multicast mapping
        import ctypes as C
        from oxibonsai_b200.ops import cuda_ops as K
        from oxibonsai_b200.parallel import tp as TP
        eng = (EngineBuilder().model_path(path).preset("greedy").max_seq_len(256).max_batch(4).kv_cache("f16").device(f"cuda:{local}")
               .tensor_parallel(rank, world).build())
        tp = eng.runner.tp
        if not tp.multicast:
            out.update(ok=True, skipped="no multicast mapping on this fabric", status=tp.status())
        else:
            lib = TP._lib()
            K.declare({"bonsai_tp_allreduce_oneshot_add": [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p],
                       "bonsai_tp_big_half_ptr": [C.c_void_p, C.c_int]}, {"bonsai_tp_big_half_ptr": C.c_void_p})
            dev = torch.device("cuda", local)
            n = 4096 * 6
            g = torch.Generator(device=dev).manual_seed(100 + rank)
            checks = {}
            for mc in (True, False):
                tp.set_multicast(mc)
                for half in (0, 1):
                    part = torch.randn(n, device=dev, generator=g)
                    base = lib.bonsai_tp_big_half_ptr(tp.handle, half) - tp.big.data_ptr()
                    tp.big[base // 4: base // 4 + n].copy_(part)
                    h = torch.full((n,), 0.5, device=dev)
                    K.check(lib.bonsai_tp_allreduce_oneshot_add(tp.handle, h.data_ptr(), n, half, K.stream()), "oneshot")
                    ref = part.clone()
                    dist.all_reduce(ref)
                    checks[f"oneshot mc={mc} half={half}"] = bool(torch.allclose(h, ref + 0.5, rtol=1e-5, atol=1e-5))
                part = torch.randn(n, device=dev, generator=g)
                tp.big[:n].copy_(part)
                h = torch.zeros(n, device=dev)
                K.check(lib.bonsai_tp_allreduce_big_add(tp.handle, h.data_ptr(), n, K.stream()), "twoshot")
                ref = part.clone()
                dist.all_reduce(ref)
                checks[f"twoshot mc={mc}"] = bool(torch.allclose(h, ref, rtol=1e-5, atol=1e-5))
            long_prompt = torch.randint(0, 1000, (90,), generator=torch.Generator().manual_seed(5)).tolist()
            tp.set_multicast(True)
            a = eng.generate(long_prompt, 8)         # prompt: two-shot all-reduce through the switch; decode: multicast {value, tag} stores
            tp.set_multicast(False)
            b = eng.generate(long_prompt, 8)
            out.update(ok=all(checks.values()) and len(a) == 8 and sum(x == y for x, y in zip(a, b)) >= 6, checks=checks, a=a, b=b,
                       status=tp.status())
    dist.barrier()
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(out, f)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
