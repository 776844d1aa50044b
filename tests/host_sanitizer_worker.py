"""Worker of tests/test_host_sanitizers.py: drives the native host library (loaded from OXIBONSAI_HOST_LIB, an ASan + UBSan
build) through its codecs, GGUF reader / writer, CPU kernels, tokenizer merges, vocabulary masks and the HTTP / SSE front."""
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np

from oxibonsai_b200.core import GgufFile, Oracle, Qwen3Config, write_synthetic_gguf
from oxibonsai_b200.core import gguf as G
from oxibonsai_b200.core.blocks import dequantize, quantize
from oxibonsai_b200.ops import cpu_ops as CK


def main() -> None:
    rng = np.random.default_rng(0)
    # every block codec, both directions, including a ragged tail of the float side
    for ty in (G.Q1_0_G128, G.TQ2_0_G128, G.TQ2_0, G.Q4_0, G.Q8_0, G.F8_E4M3, G.F8_E5M2, G.Q2_K, G.Q3_K, G.Q4_K, G.Q5_K, G.Q6_K, G.Q8_K):
        w = rng.normal(size=(3, 512)).astype(np.float32)
        q = quantize(ty, w)
        assert dequantize(ty, q).size == w.size
    # GGUF writer -> reader -> oracle forward on a tiny model
    cfg = Qwen3Config(hidden=256, inter=512, layers=1, heads=2, kv_heads=1, head_dim=128, vocab=300, context=64, name="san")
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        write_synthetic_gguf(path, cfg, tied=False, seed=3)
        f = GgufFile.open(path)
        toks, _ = Oracle(f, 32).generate_greedy([1, 2, 3], 4)
        assert len(toks) == 4
        blob = open(path, "rb").read()
        GgufFile.parse(blob)
        for cut in (10, 100, len(blob) // 2):       # truncated files must be refused, not read past their end
            try:
                GgufFile.parse(blob[:cut])
            except Exception:
                pass
    # CPU tiers, tiled and adaptive products, packing
    for ty in (G.TQ2_0_G128, G.Q1_0_G128, G.F8_E4M3):
        rows, cols = 77, 384
        q = quantize(ty, rng.normal(size=(rows, cols)).astype(np.float32) * 0.05)
        x = rng.normal(size=cols).astype(np.float32)
        for tier in (0, 1, 2):
            CK.gemv(ty, q, rows, cols, x, tier, threads=2)
        CK.gemv_tiled(ty, q, rows, cols, x, tile_rows=5, threads=3)
        CK.gemm_tiled(ty, q, rows, cols, rng.normal(size=(4, cols)).astype(np.float32), tile_rows=9, tile_batch=3, threads=2)
        CK.pack_rows_tiled(ty, q, rows, cols, tile=32)
    CK.rms_norm(rng.normal(size=300).astype(np.float32), np.ones(300, np.float32))
    # tokenizer merges and vocabulary masks
    from oxibonsai_b200.tokenizer import train_bpe
    tok = train_bpe(["the quick brown fox jumps over the lazy dog " * 4, "pack my box with five dozen liquor jugs"], 300)
    ids = tok.encode("the quick dog jumps")
    assert tok.decode(ids) == "the quick dog jumps"
    # long pieces (the heap and its linked list), empty and non-ASCII segments, bytes the vocabulary lacks
    for text in ("thethe" * 700, "", " ", "wörd ☃ " * 90, "q" * 513 + " the " * 40):
        assert tok.decode(tok.encode(text)) == text
    gap = type(tok)({k: v for k, v in tok.vocab.items() if k != "q"}, [], {})
    assert gap.decode(gap.encode("quick")) == "uick"
    from oxibonsai_b200.runtime.constrained import DfaConstraint, TokenTable
    table = TokenTable([bytes([b]) for b in range(256)] + [b"true", b"false"])
    c = DfaConstraint.from_regex(table, r"(true|false)+", eos_token=None)
    assert c.allowed_mask().any() and c.advance(256) and c.is_complete()
    # the Earley matcher and the trie walk behind grammar constraints
    from oxibonsai_b200.runtime.constrained import json_constraint, json_schema_constraint, mask_to_bool
    for gc in (json_constraint(table, None), json_schema_constraint(table, {"type": "object", "required": ["a"], "properties": {"a": {"type": "array", "items": {"type": "number"}}}}, None)):
        for b in b'{"a": [1, 2.5e3, -7]}':
            m = gc.allowed_mask()
            assert mask_to_bool(m, table.n)[b]
            assert gc.advance(b)
        assert gc.is_complete() and not gc.advance(ord("x"))
        gc.reset()
        assert gc.allowed_mask().any()
    # malformed grammar blobs are refused by the compiler, never read past their end
    import ctypes as C
    from oxibonsai_b200.runtime.grammar.compilers import json_grammar
    from oxibonsai_b200.runtime.grammar import native as GN
    lib = GN._lib()
    good = GN.serialize(json_grammar())
    noise = np.random.default_rng(9)
    for trial in range(300):
        blob = good.copy()
        if trial % 3 == 0:
            blob = blob[: int(noise.integers(0, blob.size))]
        elif trial % 3 == 1:
            for _ in range(int(noise.integers(1, 6))):
                blob[int(noise.integers(0, blob.size))] = int(noise.integers(-5000, 5000))
        else:
            blob = noise.integers(-300, 300, size=int(noise.integers(0, 200))).astype(np.int32)
        blob = np.ascontiguousarray(blob, dtype=np.int32)
        hg = lib.bgram_compile(blob.ctypes.data if blob.size else None, blob.size)
        if hg:                                          # still a well-formed grammar: it must also run
            hm = lib.bgram_matcher_new(hg)
            lib.bgram_matcher_feed(hm, b'{"a": [1, "x"]}', 15)
            lib.bgram_matcher_free(hm)
            lib.bgram_free(hg)
    # HTTP / SSE front: requests (whole, split, malformed), a token stream with stop sequences and broken UTF-8, a client
    # that leaves in mid-stream, shutdown with open connections
    import http.client
    import socket
    import threading
    from oxibonsai_b200.server.native_front import NativeFront, StreamClosed
    from oxibonsai_b200.tokenizer import ByteTokenizer
    front = NativeFront("127.0.0.1", 0)
    front.set_vocab(ByteTokenizer(), 300)
    front.start()

    def answer():
        while True:
            try:
                ev = front.next_event(100)
            except EOFError:
                return
            if ev is None or ev[0] != 1:
                continue
            conn, target = ev[1], ev[3]
            if target == "/stream":
                st = front.open_stream(conn, '{"choices": [{"index": 0, ', True, ["END", "é!"], 'data: {"first": 1}\n\n', 0)
                st.begin([(b"content-type", b"text/event-stream")])
                try:
                    for t in list("héllo \"wörld\" 日本".encode()) + [0xE6, 0x97, 0xFF, 299, 7] + list(b"the END never"):
                        st.push(t)
                except StreamClosed:
                    pass
                st.finish("length")
            else:
                front.respond(conn, 200, [(b"content-type", b"text/plain")], b"x" * 100000)

    threading.Thread(target=answer, daemon=True).start()
    hc = http.client.HTTPConnection("127.0.0.1", front.port, timeout=10)
    for target in ("/a", "/stream", "/b"):
        hc.request("GET", target)
        assert hc.getresponse().read()
    for raw in (b"GET / HTTP/1.1\r\nHost: x\r\n\r\nGET /2 HTTP/1.1\r\n\r\n", b"BROKEN\r\n\r\n", b"POST / HTTP/1.1\r\nContent-Length: 10\r\n\r\nabc"):
        sk = socket.create_connection(("127.0.0.1", front.port))
        sk.sendall(raw)
        sk.settimeout(0.3)
        try:
            sk.recv(1 << 20)
        except OSError:
            pass
        sk.close()
    sk = socket.create_connection(("127.0.0.1", front.port))
    sk.sendall(b"GET /stream HTTP/1.1\r\n\r\n")
    sk.close()
    # the parser against noise: random bytes, and valid requests with random mutations (a byte changed, cut short, doubled)
    import random
    fuzz = random.Random(5)
    valid = b"POST /v1/x?y=1 HTTP/1.1\r\nHost: a\r\nContent-Length: 12\r\nExpect: 100-continue\r\nConnection: keep-alive\r\n\r\nhello world!"
    chunky = b"POST /c HTTP/1.1\r\nTransfer-Encoding: chunked\r\n\r\n5;x=y\r\nhello\r\n1a\r\nabcdefghijklmnopqrstuvwxyz\r\n0\r\nT: v\r\n\r\n"
    for i in range(240):
        if i >= 150:
            valid = chunky
        kind = i % 4
        if kind == 0:
            payload = bytes(fuzz.randrange(256) for _ in range(fuzz.randint(1, 400)))
        elif kind == 1:
            b = bytearray(valid)
            for _ in range(fuzz.randint(1, 4)):
                b[fuzz.randrange(len(b))] = fuzz.randrange(256)
            payload = bytes(b)
        elif kind == 2:
            payload = valid[:fuzz.randrange(len(valid))]
        else:
            cut = fuzz.randrange(len(valid))
            payload = valid[:cut] + valid[cut:] * 2 + b"\r\n" * fuzz.randint(0, 3)
        sk = socket.create_connection(("127.0.0.1", front.port))
        sk.sendall(payload)
        sk.settimeout(0.02)
        try:
            sk.recv(1 << 16)
        except OSError:
            pass
        sk.close()
    dangling = socket.create_connection(("127.0.0.1", front.port))      # still open when the front shuts down
    import time
    time.sleep(0.3)
    front.close()
    dangling.close()
    print("sanitizer worker ok")


if __name__ == "__main__":
    main()
