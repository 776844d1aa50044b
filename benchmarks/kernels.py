#!/usr/bin/env python
"""Kernel micro-benchmarks on Qwen3-8B-shaped matrices (the counterpart of the reference's ``benches/*.rs`` and its
``gemv_benchmark`` example, crates/oxibonsai-kernels/examples/).

    python benchmarks/kernels.py gemv   [--fast s16|0|warp|tile|hmma|mma]    packed-bit GEMV, batch 1 (s16 = the streamed kernel)
    python benchmarks/kernels.py gemm   [--tokens 64]         packed-bit tcgen05 GEMM (prefill / batched decode)
    python benchmarks/kernels.py lmhead [--tokens 64]         dense f16 tcgen05 GEMM of the LM head
    python benchmarks/kernels.py attn   [--ctx 4096 --batch 1 --kv f16]   split-KV decode attention

Every case cycles through enough weight copies that successive launches never hit L2 (the working set is > 400 MB);
timing is CUDA events around a graph of ``--iters`` launches after warm-up.  ``--profile`` runs each case exactly
``--iters`` times eagerly without the graph, for captures under a profiler (use a small ``--iters``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

SHAPES = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (24576, 4096), "down": (4096, 12288)}


def peaks() -> dict:
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except Exception:
        return {}


def time_us(fn, iters: int, profile: bool) -> float:
    if profile:
        for _ in range(iters):
            fn()
        torch.cuda.synchronize()
        return float("nan")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, g = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for _ in range(iters):
                fn()
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1000.0


def weight_copies(K, rows, cols, dev, budget=400e6, copies=0):
    n = copies if copies > 0 else max(2, int(budget // (rows * cols // 4)))
    out = []
    for _ in range(n):
        w = K.PlanarWeight(rows, cols, dev)
        w.codes.random_(-2 ** 31, 2 ** 31 - 1)
        w.scales.fill_(0.02)
        out.append(w)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemv", "gemm", "lmhead", "attn", "attn_prefill"])
    ap.add_argument("--fast", default="s16", help="s16 (streamed tensor-core GEMV), 0 (exact f32), warp, tile, hmma or mma")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--kv", default="f16")
    ap.add_argument("--nsplit", type=int, default=16)
    ap.add_argument("--no-cluster", action="store_true", help="attn: merge the KV splits through global memory instead of a thread-block cluster")
    ap.add_argument("--heads", type=int, default=32, help="attn: query heads (a tensor-parallel rank of the 8B model has 32 / N)")
    ap.add_argument("--kv-heads", type=int, default=8, help="attn: KV heads (8 / N on a tensor-parallel rank)")
    ap.add_argument("--iters", type=int, default=40)
    ap.add_argument("--shapes", default=",".join(SHAPES))
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--copies", type=int, default=0, help="gemv / gemm: weight copies to cycle through (default: enough to miss L2; 1 = L2-resident weights)")
    ap.add_argument("--balanced", action="store_true", help="gemm: equal (tile, k) ranges per SM wherever possible")
    ap.add_argument("--whole-tiles", action="store_true", help="gemm: whole tiles per CTA instead of equal (tile, k) ranges")
    a = ap.parse_args()
    from oxibonsai_b200.ops import cuda_ops as K
    dev = torch.device("cuda:0")
    pk = peaks()
    hbm, tf = pk.get("hbm_gbs", 6650.0) * 1e9, pk.get("bf16_tflops", 1590.0) * 1e12
    tag = "of measured" if pk else "of fallback"
    rows_out = []
    it = [0]
    if a.case in ("gemv", "gemm"):
        for name in a.shapes.split(","):
            n, k = SHAPES[name]
            ws = weight_copies(K, n, k, dev, copies=a.copies)
            byts = n * k / 4 + n * k / 64
            if a.case == "gemv":
                x = torch.randn(k, device=dev)

                if a.fast == "mma":
                    fws = [K.FragWeight(w) for w in ws]
                if a.fast == "s16":
                    sws = [K.S16Weight(w) for w in ws]
                out = torch.empty(n, device=dev)

                def fn():
                    it[0] += 1
                    if a.fast == "mma":
                        K.bitgemv_mma(fws[it[0] % len(ws)], x, out=out)
                    elif a.fast == "s16":
                        K.bitgemv_s16(sws[it[0] % len(ws)], x, out=out)
                    else:
                        K.bitgemv(ws[it[0] % len(ws)], x, out=out, fast=(False if a.fast == "0" else a.fast))
                us = time_us(fn, a.iters, a.profile)
                rows_out.append({"case": f"gemv/{name}", "n": n, "k": k, "us": round(us, 2), "GB/s": round(byts / us / 1e3, 1),
                                 f"hbm_frac_{tag.replace(' ', '_')}": round(byts / (us * 1e-6) / hbm, 3)})
            else:
                T = a.tokens
                hm = a.fast == "hmma" and T <= 64            # decode-batch GEMM on mma.sync instead of tcgen05
                x = (K.norm_to_f16_hmma if hm else K.norm_to_f16_paired)(torch.randn(T, k, device=dev), None, 1e-6)
                out = torch.empty((T, n), device=dev)
                status = torch.zeros(1, dtype=torch.int32, device=dev)

                def fn():
                    it[0] += 1
                    if hm:
                        K.bitgemm_hmma(ws[it[0] % len(ws)], x, out=out)
                        return
                    K.bitgemm_prefill(ws[it[0] % len(ws)], x, out=out, status=status, balanced=(False if a.whole_tiles else (True if a.balanced else "auto")))
                us = time_us(fn, a.iters, a.profile)
                fl = 2.0 * n * k * T
                rows_out.append({"case": f"gemm/{name}", "n": n, "k": k, "tokens": T, "us": round(us, 2), "TFLOP/s": round(fl / us / 1e6, 1),
                                 f"tensor_frac_{tag.replace(' ', '_')}": round(fl / (us * 1e-6) / tf, 3),
                                 f"hbm_frac_{tag.replace(' ', '_')}": round(byts / (us * 1e-6) / hbm, 3), "status": int(status.item())})
    elif a.case == "lmhead":
        n, k, T = 151936, 4096, a.tokens
        ws = [torch.randn(n, k, device=dev, dtype=torch.float16) * 0.02 for _ in range(2)]
        x = K.norm_to_f16_paired(torch.randn(T, k, device=dev), None, 1e-6, natural=True)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        out = torch.empty((T, n), device=dev)

        def fn():
            it[0] += 1
            K.dense_gemm_f16(ws[it[0] % 2], x, out=out, status=status)
        us = time_us(fn, a.iters, a.profile)
        byts, fl = n * k * 2.0, 2.0 * n * k * T
        rows_out.append({"case": "lmhead", "tokens": T, "us": round(us, 2), "TFLOP/s": round(fl / us / 1e6, 1),
                         f"hbm_frac_{tag.replace(' ', '_')}": round(byts / (us * 1e-6) / hbm, 3), "status": int(status.item())})
    elif a.case == "attn":
        nq, nkv, hd, page = a.heads, a.kv_heads, 128, 64
        kvt = {"f32": K.KV_F32, "f16": K.KV_F16, "q8": K.KV_Q8, "q4": K.KV_Q4}[a.kv]
        B, ctx = a.batch, a.ctx
        pps = (ctx + page - 1) // page
        layers = max(2, int(400e6 // max(1, B * pps * page * nkv * hd * 4)))   # distinct pools so launches miss L2
        row = hd // 2 if kvt == K.KV_Q4 else hd
        pools = []
        for _ in range(layers):
            kp = torch.empty((B * pps, nkv, page, row), dtype=K.KV_DTYPES[kvt], device=dev)
            vp = torch.empty_like(kp)
            if kp.dtype.is_floating_point:
                kp.normal_()
                vp.normal_()
            else:
                kp.random_(0, 127)
                vp.random_(0, 127)
            sc = (torch.rand((B * pps, nkv, page), device=dev) * 0.01, torch.rand((B * pps, nkv, page), device=dev) * 0.01) if kvt >= 2 else (None, None)
            pools.append((kp, vp, *sc))
        bt = torch.arange(B * pps, dtype=torch.int32, device=dev).view(B, pps)
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
        q = torch.randn((B, nq, hd), device=dev)
        out = torch.empty_like(q)
        K.attn_decode_cluster_mode(1 if a.no_cluster else 0)

        def fn():
            it[0] += 1
            kp, vp, ks, vs = pools[it[0] % layers]
            K.attn_decode(q, pos, bt, nq, nkv, hd, kvt, page, kp, vp, ks, vs, nsplit=a.nsplit, out=out)
        us = time_us(fn, a.iters, a.profile)
        elt = {K.KV_F32: 4, K.KV_F16: 2, K.KV_Q8: 1, K.KV_Q4: 0.5}[kvt]
        byts = 2.0 * B * ctx * nkv * hd * elt
        rows_out.append({"case": f"attn_decode/{a.kv}", "batch": B, "ctx": ctx, "heads": f"{nq}/{nkv}", "nsplit": a.nsplit, "launch_form": K.attn_decode_last_form(), "us": round(us, 2),
                         "GB/s": round(byts / us / 1e3, 1), f"hbm_frac_{tag.replace(' ', '_')}": round(byts / (us * 1e-6) / hbm, 3)})
    elif a.case == "attn_prefill":
        # one prompt chunk of --tokens queries whose first token sits at position --ctx (8B head layout, f16 / --kv pages)
        nq, nkv, hd, page = 32, 8, 128, 64
        kvt = {"f32": K.KV_F32, "f16": K.KV_F16, "q8": K.KV_Q8, "q4": K.KV_Q4}[a.kv]
        T, pos0 = a.tokens, a.ctx
        pps = (pos0 + T + page - 1) // page
        row = hd // 2 if kvt == K.KV_Q4 else hd
        kp = torch.empty((pps, nkv, page, row), dtype=K.KV_DTYPES[kvt], device=dev)
        vp = torch.empty_like(kp)
        if kp.dtype.is_floating_point:
            kp.normal_()
            vp.normal_()
        else:
            kp.random_(0, 127)
            vp.random_(0, 127)
        ks, vs = ((torch.rand((pps, nkv, page), device=dev) * 0.01, torch.rand((pps, nkv, page), device=dev) * 0.01) if kvt >= 2 else (None, None))
        bt = torch.arange(pps, dtype=torch.int32, device=dev)
        q = torch.randn((T, nq, hd), device=dev)
        out = torch.empty((T, nq * hd), dtype=torch.float16, device=dev)

        def fn():
            K.attn_prefill(q, pos0, bt, nq, nkv, hd, kvt, page, kp, vp, ks, vs, out=out)
        us = time_us(fn, a.iters, a.profile)
        flops = 4.0 * T * (pos0 + (T + 1) / 2.0) * hd * nq            # QK^T and PV over the causal part
        rows_out.append({"case": f"attn_prefill/{a.kv}", "tokens": T, "pos0": pos0, "us": round(us, 2), "TFLOP/s": round(flops / us / 1e6, 1)})
    for r in rows_out:
        print(json.dumps(r))


if __name__ == "__main__":
    main()
