"""Command line: ``python -m oxibonsai_b200 <run|chat|serve|info|benchmark|quantize|validate|convert|tokenizer> ...``.

Reference: the ``oxibonsai`` binary (src/main.rs:37-240 subcommands, :254-420 tokenizer auto-discovery next to the
model, :420-625 run / chat loops, :604-621 the summary line ``"{p} prompt + {g} generated = {t} tokens in {s}s
({tok/s} tok/s)"`` where tok/s counts generated tokens over prefill + decode wall time).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
import time
from pathlib import Path

_QUANT_SUFFIX = re.compile(r"[-_.](Q\d+(_[A-Z0-9]+)*|TQ\d+(_[A-Z0-9]+)*|F16|BF16|F32|FP8)$", re.IGNORECASE)


def strip_quant_suffix(stem: str) -> str:
    return _QUANT_SUFFIX.sub("", stem)


def tokenizer_candidates(model_path: str) -> list[Path]:
    """Conventional places for ``tokenizer.json``: beside the model, one directory up, sibling directories named after
    the model (with ``-unpacked`` / ``-ONNX``), and the enclosing ``models/`` directory."""
    p = Path(model_path)
    parent = p.parent if str(p.parent) else Path(".")
    out: list[Path] = []

    def push(c: Path):
        if c not in out:
            out.append(c)
    push(parent / "tokenizer.json")
    push(parent / ".." / "tokenizer.json")
    base = strip_quant_suffix(p.stem)
    for v in (base, f"{base}-unpacked", f"{base}-ONNX"):
        push(parent / v / "tokenizer.json")
    for anc in list(p.parents):
        if anc.name == "models":
            push(anc / "tokenizer.json")
            break
    return out


def resolve_tokenizer(model_path: str, explicit: str | None) -> tuple[str | None, list[Path]]:
    if explicit:
        return explicit, []
    cands = tokenizer_candidates(model_path)
    for c in cands:
        if c.exists():
            return str(c), cands
    return None, cands


def no_tokenizer_warning(searched: list[Path]) -> str:
    lines = ["warning: no tokenizer.json found; falling back to raw byte tokens.", "  searched:"]
    lines += [f"    {c}" for c in searched]
    lines.append("  pass --tokenizer PATH (or run `tokenizer download`) to use the model's vocabulary.")
    return "\n".join(lines)


def summary_line(n_prompt: int, n_gen: int, seconds: float) -> str:
    tps = n_gen / seconds if seconds > 0 else 0.0
    return f"{n_prompt} prompt + {n_gen} generated = {n_prompt + n_gen} tokens in {seconds:.2f}s ({tps:.1f} tok/s)"


def _load_tokenizer(model: str, explicit: str | None, quiet: bool = False):
    from .tokenizer import load_tokenizer
    path, searched = resolve_tokenizer(model, explicit)
    tok = load_tokenizer(path, model_path=model)
    if path is None and not quiet:
        if type(tok).__name__ == "BpeTokenizer":
            print(f"no tokenizer.json found; using the vocabulary embedded in {model} ({tok.vocab_size} tokens)", file=sys.stderr)
        else:
            print(no_tokenizer_warning(searched), file=sys.stderr)
    return tok


def _engine(args, max_batch: int = 1):
    from .runtime import EngineBuilder
    from .runtime.presets import SamplingParams
    sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=args.seed, max_tokens=args.max_tokens)
    b = EngineBuilder().model_path(args.model).sampler(sp).max_seq_len(args.max_seq_len).max_batch(max_batch).kv_cache(getattr(args, "kv_cache", "f16"))
    return b.build()


def cmd_run(args) -> int:
    from .tokenizer import StreamingDecoder
    prompt = sys.stdin.read() if args.prompt == "-" else args.prompt
    tok = _load_tokenizer(args.model, args.tokenizer)
    eng = _engine(args)
    ids = tok.encode(prompt) or [151644]
    dec = StreamingDecoder()
    t0 = time.perf_counter()
    n = 0
    for t in eng.generate_stream(ids, args.max_tokens):
        sys.stdout.write(dec.push(tok.token_bytes(t)))
        sys.stdout.flush()
        n += 1
    sys.stdout.write(dec.flush() + "\n")
    print(summary_line(len(ids), n, time.perf_counter() - t0), file=sys.stderr)
    return 0


def cmd_chat(args) -> int:
    from .tokenizer import StreamingDecoder, chat_prompt
    tok = _load_tokenizer(args.model, args.tokenizer)
    eng = _engine(args)
    messages: list[dict] = []
    if args.system:
        messages.append({"role": "system", "content": args.system})
    print("type /exit to quit, /reset to clear the conversation", file=sys.stderr)
    while True:
        try:
            line = input("> ")
        except EOFError:
            break
        if line.strip() == "/exit":
            break
        if line.strip() == "/reset":
            messages = messages[:1] if args.system else []
            continue
        messages.append({"role": "user", "content": line})
        ids = tok.encode(chat_prompt(messages, args.template))
        if len(ids) + args.max_tokens > args.max_seq_len:      # drop the oldest turns until the prompt fits
            while len(messages) > 2 and len(ids) + args.max_tokens > args.max_seq_len:
                del messages[1 if args.system else 0]
                ids = tok.encode(chat_prompt(messages, args.template))
        dec, reply, t0, n = StreamingDecoder(), [], time.perf_counter(), 0
        for t in eng.generate_stream(ids, args.max_tokens):
            piece = dec.push(tok.token_bytes(t))
            reply.append(piece)
            sys.stdout.write(piece)
            sys.stdout.flush()
            n += 1
        sys.stdout.write(dec.flush() + "\n")
        messages.append({"role": "assistant", "content": "".join(reply)})
        print(summary_line(len(ids), n, time.perf_counter() - t0), file=sys.stderr)
    return 0


def cmd_serve(args) -> int:
    from .server.__main__ import main as serve_main
    argv = ["--model-path", args.model, "--host", args.host, "--port", str(args.port), "--max-seq-len", str(args.max_seq_len)]
    if args.tokenizer:
        argv += ["--tokenizer-path", args.tokenizer]
    return serve_main(argv)


def model_info(path: str) -> dict:
    from .core import GgufFile
    from .core.compat import build_compat_report, extract_model_card
    from .models.registry import validate_gguf
    f = GgufFile.open(path)
    cfg = f.config()
    v = validate_gguf(f)
    card = extract_model_card(f, os.path.getsize(path))
    from .core import gguf as G
    # which GPU engine EngineBuilder would pick: decided by the storage format of the layer weights
    lw = next((f.tensor_info(n).type for n in ("blk.0.attn_q.weight", "blk.0.attn_qkv.weight", "blk.0.ffn_down.weight") if f.has_tensor(n)), None)
    gpu_engine = "none" if lw is None else ("sub-2-bit runner" if lw in (G.TQ2_0_G128, G.Q1_0_G128) else "generic-format engine")
    return {"path": path, "gpu_engine": gpu_engine, "gguf_version": f.version, "tensors": len(f.tensors), "metadata_entries": len(f.metadata), "variant": v.variant.value,
            "architecture": card.architecture, "name": card.name, "quantization": card.quantization, "bits_per_weight": card.bits_per_weight,
            "estimated_parameters": card.estimated_param_count(), "file_size_bytes": os.path.getsize(path),
            "config": {"layers": cfg.layers, "hidden": cfg.hidden, "heads": cfg.heads, "kv_heads": cfg.kv_heads, "head_dim": cfg.head_dim,
                       "intermediate": cfg.inter, "vocab": cfg.vocab, "context": cfg.context, "rope_base": cfg.rope_base, "rms_eps": cfg.eps},
            "embedded_tokenizer": ({"model": f.metadata.get("tokenizer.ggml.model"), "tokens": len(f.metadata.get("tokenizer.ggml.tokens") or []),
                                    "merges": len(f.metadata.get("tokenizer.ggml.merges") or [])} if f.metadata.get("tokenizer.ggml.tokens") else None),
            "valid": v.ok, "errors": v.errors, "warnings": v.warnings, "compat": build_compat_report(f).summary()}


def cmd_info(args) -> int:
    info = model_info(args.model)
    if args.json:
        print(json.dumps(info, indent=2))
    else:
        from .core import GgufFile
        from .core.compat import extract_model_card
        print(extract_model_card(GgufFile.open(args.model), info["file_size_bytes"]).to_markdown())
        et = info["embedded_tokenizer"]
        print(f"variant: {info['variant']}\nGPU engine: {info['gpu_engine']}\n"
              f"embedded tokenizer: {'none' if et is None else '%s, %d tokens, %d merges' % (et['model'], et['tokens'], et['merges'])}\n{info['compat']}")
    return 0


def cmd_validate(args) -> int:
    info = model_info(args.model)
    for w in info["warnings"]:
        print(f"warning: {w}")
    for e in info["errors"]:
        print(f"error: {e}")
    print(f"{args.model}: {'OK' if info['valid'] else 'INVALID'} - GGUF v{info['gguf_version']}, {info['tensors']} tensors, {info['quantization']}, "
          f"{info['config']['layers']} layers x {info['config']['hidden']}")
    return 0 if info["valid"] else 1


def cmd_benchmark(args) -> int:
    """Throughput of a model file, or of a synthetic random-init checkpoint of a named shape when no file is given."""
    import tempfile
    from .core import Qwen3Config, write_synthetic_gguf
    path = args.model
    tmp = None
    if path is None:
        shapes = {"tiny": dict(hidden=512, inter=1024, layers=2, heads=4, kv_heads=2, head_dim=128, vocab=4096),
                  "1.7b": dict(hidden=2048, inter=6144, layers=28, heads=16, kv_heads=8, head_dim=128, vocab=151936),
                  "8b": dict(hidden=4096, inter=12288, layers=36, heads=32, kv_heads=8, head_dim=128, vocab=151936)}
        tmp = tempfile.NamedTemporaryFile(suffix=".gguf", delete=False)
        tmp.close()
        write_synthetic_gguf(tmp.name, Qwen3Config(context=65536, name=args.shape, **shapes[args.shape]), seed=args.seed)
        path = tmp.name
    try:
        args.model, args.max_seq_len, args.top_k, args.top_p, args.max_tokens = path, args.prompt_len + args.tokens + args.warmup + 8, 40, 0.9, args.tokens
        eng = _engine(args)
        import torch
        prompt = torch.randint(0, eng.config.vocab, (args.prompt_len,), generator=torch.Generator().manual_seed(args.seed)).tolist()
        eng.generate(prompt, args.warmup, stop_at_eos=False)
        t0 = time.perf_counter()
        out = eng.generate(prompt, args.tokens, stop_at_eos=False)
        dt = time.perf_counter() - t0
        st = eng.last_stats
        print(json.dumps({"model": os.path.basename(path), "prompt_tokens": len(prompt), "generated": len(out), "seconds": round(dt, 4),
                          "tokens_per_second": round(len(out) / dt, 2), "decode_tokens_per_second": round(st.decode_tokens_per_second, 2),
                          "prefill_seconds": round(st.prefill_seconds, 4)}))
        print(summary_line(len(prompt), len(out), dt), file=sys.stderr)
    finally:
        if tmp is not None:
            os.unlink(tmp.name)
    return 0


def requantize_gguf(src: str, dst: str, fmt: str) -> dict:
    """Re-encodes every 2-D tensor of a GGUF file into ``fmt`` (norm vectors stay as they are)."""
    import numpy as np
    from .convert import QUANT_TYPES
    from .core import GgufFile, GgufWriter, dequantize, quantize, gguf as G
    aliases = {"q1_0": "q1_0_g128", "tq2_0": "tq2_0_g128", "ternary": "tq2_0_g128"}
    fmt = aliases.get(fmt.lower(), fmt.lower())
    kq = {"q2_k": G.Q2_K, "q3_k": G.Q3_K, "q4_k": G.Q4_K, "q5_k": G.Q5_K, "q6_k": G.Q6_K, "q8_k": G.Q8_K}
    types = {**QUANT_TYPES, **kq}
    if fmt not in types:
        raise SystemExit(f"unknown format {fmt!r}; choose from {sorted(types)}")
    tid = types[fmt]
    _, be, _ = G.type_info(tid)
    f = GgufFile.open(src)
    w = GgufWriter()
    for k, v in f.metadata.items():
        w.add(k, v)
    n_in = n_out = changed = 0
    for t in f.tensors:
        raw = f.tensor_bytes(t.name)
        n_in += len(raw)
        if len(t.dims) == 2 and t.dims[0] % be == 0 and t.type != tid and not t.name.endswith("norm.weight"):
            vals = dequantize(t.type, raw) if t.type not in (G.F32,) else np.frombuffer(raw, dtype=np.float32)
            blob = quantize(tid, vals)
            w.add_tensor(t.name, t.dims, tid, blob)
            n_out += blob.size
            changed += 1
        else:
            w.add_tensor(t.name, t.dims, t.type, np.frombuffer(raw, dtype=np.uint8))
            n_out += len(raw)
    w.write(dst)
    return {"tensors": len(f.tensors), "requantized": changed, "bytes_in": n_in, "bytes_out": n_out, "format": fmt}


def cmd_quantize(args) -> int:
    r = requantize_gguf(args.input, args.output, args.format)
    print(f"{r['requantized']} of {r['tensors']} tensors -> {r['format']}: {r['bytes_in'] / 1e6:.1f} MB -> {r['bytes_out'] / 1e6:.1f} MB")
    return 0


def cmd_convert(args) -> int:
    if args.onnx:
        from .convert.onnx import convert_onnx_to_gguf
        st = convert_onnx_to_gguf(args.from_, args.to, args.quant)
    else:
        from .convert import convert_safetensors_to_gguf
        st = convert_safetensors_to_gguf(args.from_, args.to, args.quant, quantize_embeddings=not args.f16_embeddings)
    print(f"wrote {args.to}: {st.tensors} tensors, {st.bytes_in / 1e6:.1f} MB -> {st.bytes_out / 1e6:.1f} MB" + (" (tied embeddings duplicated)" if st.tied else ""))
    return 0


def cmd_tokenizer(args) -> int:
    if args.action == "download":
        print("downloading needs network access; fetch tokenizer.json of the Qwen3 repository with any HTTP client and place it at "
              f"{args.output}", file=sys.stderr)
        return 2
    from .tokenizer import load_tokenizer
    with open(args.path, encoding="utf-8") as f:
        j = json.load(f)
    tok = load_tokenizer(args.path)
    print(json.dumps({"path": args.path, "model_type": j.get("model", {}).get("type"), "vocab_size": tok.vocab_size,
                      "added_tokens": len(j.get("added_tokens", [])), "merges": len(j.get("model", {}).get("merges", []))}))
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="oxibonsai_b200", description="Sub-2-bit Qwen3 inference on B200")
    ap.add_argument("--config", help="TOML configuration file (see server/config.py)")
    sub = ap.add_subparsers(dest="command", required=True)

    def sampling(p, max_tokens):
        p.add_argument("--max-tokens", type=int, default=max_tokens)
        p.add_argument("--temperature", type=float, default=0.7)
        p.add_argument("--top-k", type=int, default=40)
        p.add_argument("--top-p", type=float, default=0.9)
        p.add_argument("--seed", type=int, default=42)
        p.add_argument("--max-seq-len", type=int, default=4096)
        p.add_argument("--tokenizer")
        p.add_argument("--kv-cache", default="f16", choices=["f32", "f16", "q8", "q4"])
    r = sub.add_parser("run", help="run inference on a GGUF model")
    r.add_argument("-m", "--model", required=True)
    r.add_argument("-p", "--prompt", required=True, help='prompt text, "-" for stdin')
    sampling(r, 256)
    r.set_defaults(fn=cmd_run)
    c = sub.add_parser("chat", help="interactive multi-turn conversation")
    c.add_argument("-m", "--model", required=True)
    c.add_argument("--system")
    c.add_argument("--template", default="chatml")
    sampling(c, 512)
    c.set_defaults(fn=cmd_chat)
    s = sub.add_parser("serve", help="start the OpenAI-compatible server")
    s.add_argument("-m", "--model", required=True)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8080)
    s.add_argument("--max-seq-len", type=int, default=4096)
    s.add_argument("--tokenizer")
    s.set_defaults(fn=cmd_serve)
    i = sub.add_parser("info", help="display model info from a GGUF file")
    i.add_argument("-m", "--model", required=True)
    i.add_argument("--json", action="store_true")
    i.set_defaults(fn=cmd_info)
    b = sub.add_parser("benchmark", help="quick throughput benchmark")
    b.add_argument("-m", "--model")
    b.add_argument("--shape", default="tiny", choices=["tiny", "1.7b", "8b"])
    b.add_argument("--tokens", type=int, default=100)
    b.add_argument("--warmup", type=int, default=10)
    b.add_argument("--prompt-len", type=int, default=32)
    b.add_argument("--temperature", type=float, default=0.7)
    b.add_argument("--seed", type=int, default=42)
    b.set_defaults(fn=cmd_benchmark)
    q = sub.add_parser("quantize", help="re-encode a GGUF model in another block format")
    q.add_argument("-i", "--input", required=True)
    q.add_argument("-o", "--output", required=True)
    q.add_argument("--format", default="q1_0")
    q.set_defaults(fn=cmd_quantize)
    v = sub.add_parser("validate", help="check that a GGUF file is well formed and complete")
    v.add_argument("-m", "--model", required=True)
    v.set_defaults(fn=cmd_validate)
    cv = sub.add_parser("convert", help="convert a Hugging Face safetensors (or ONNX MatMulNBits) model to GGUF")
    cv.add_argument("--from", dest="from_", required=True)
    cv.add_argument("--to", required=True)
    cv.add_argument("--quant", default="tq2_0_g128")
    cv.add_argument("--onnx", action="store_true")
    cv.add_argument("--f16-embeddings", action="store_true", help="keep the embedding table and LM head in F16")
    cv.set_defaults(fn=cmd_convert)
    t = sub.add_parser("tokenizer", help="manage the tokenizer")
    t.add_argument("action", choices=["download", "info"])
    t.add_argument("--path", default="models/tokenizer.json")
    t.add_argument("--output", default="models/tokenizer.json")
    t.set_defaults(fn=cmd_tokenizer)
    return ap


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    return int(args.fn(args) or 0)


if __name__ == "__main__":
    sys.exit(main())
