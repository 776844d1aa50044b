"""GGUF container: round trips, layout facts, malformed input (reference test strategy: synthetic fixtures
written by the project's own writer, fuzzing that must never crash)."""
import struct

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from oxibonsai_b200 import _native
from oxibonsai_b200.core import (GgufFile, GgufStreamParser, GgufWriter, Oracle, Q1_0_G128, TQ2_0_G128, F32, F16, data_size,
                                 type_info, write_synthetic_gguf)
from oxibonsai_b200.core import gguf as G


def _sample_writer():
    w = GgufWriter()
    w.add("general.architecture", "qwen3").add("general.name", "unit").add("qwen3.block_count", 2)
    w.add("qwen3.rope.freq_base", 1e6).add("flag", True).add("neg", -5).add("big", 2**40)
    w.add("tokens", ["a", "bc", "d\n\"e"]).add("ints", [1, 2, 3]).add("floats", [0.5, 1.5])
    w.add_tensor("a.weight", [128, 2], TQ2_0_G128, np.arange(68, dtype=np.uint8))
    w.add_tensor("b.weight", [3], F32, np.array([1, 2, 3], dtype=np.float32))
    return w


def test_type_table_matches_block_layouts():
    assert type_info(Q1_0_G128) == ("Q1_0_g128", 128, 18)
    assert type_info(TQ2_0_G128) == ("TQ2_0_g128", 128, 34)
    assert type_info(G.TQ2_0) == ("TQ2_0", 256, 66)
    assert type_info(G.Q4_0)[1:] == (32, 18) and type_info(G.Q8_0)[1:] == (32, 34)
    assert [type_info(t)[2] for t in (10, 11, 12, 13, 14, 15)] == [84, 110, 144, 176, 210, 292]
    assert type_info(9) == ("Q8_1", 32, 40)      # sized as the reference sizes it (crates/oxibonsai-core/src/gguf/types.rs:96)
    assert data_size(TQ2_0_G128, 4096 * 4096) == 4096 * 32 * 34
    with pytest.raises(_native.NativeError):
        type_info(99)


def test_writer_reader_round_trip():
    data = _sample_writer().to_bytes()
    f = GgufFile.parse(data)
    assert f.version == 3 and f.alignment == 32 and f.data_offset % 32 == 0
    m = f.metadata
    assert m["general.name"] == "unit" and m["qwen3.block_count"] == 2 and m["flag"] is True
    assert m["neg"] == -5 and m["big"] == 2**40 and m["tokens"] == ["a", "bc", "d\n\"e"]
    assert m["ints"] == [1, 2, 3] and m["floats"] == [0.5, 1.5]
    a, b = f.tensors
    assert (a.name, a.dims, a.type, a.offset, a.nbytes) == ("a.weight", (128, 2), TQ2_0_G128, 0, 68)
    # offsets are a running sum with no per-tensor padding
    assert b.offset == 68 and b.nbytes == 12
    assert bytes(f.tensor_bytes("a.weight")) == bytes(range(68))
    assert np.frombuffer(f.tensor_bytes("b.weight"), dtype=np.float32).tolist() == [1, 2, 3]


def test_header_bytes_are_as_specified():
    data = _sample_writer().to_bytes()
    magic, version, nt, nkv = struct.unpack_from("<IIQQ", data, 0)
    assert magic == 0x46554747 and version == 3 and nt == 2 and nkv == 10


def test_alignment_key_and_v2():
    w = GgufWriter(version=2, alignment=64)
    w.add_tensor("t", [4], F32, np.zeros(4, dtype=np.float32))
    f = GgufFile.parse(w.to_bytes())
    assert f.version == 2 and f.alignment == 64 and f.data_offset % 64 == 0


def test_errors_have_stable_codes():
    with pytest.raises(_native.NativeError) as e:
        GgufFile.parse(b"NOPE" + b"\0" * 40)
    assert e.value.name == "invalid_magic" and not e.value.retryable
    good = _sample_writer().to_bytes()
    with pytest.raises(_native.NativeError) as e:
        GgufFile.parse(good[:40])
    assert e.value.name == "unexpected_eof"
    bad_version = good[:4] + struct.pack("<I", 7) + good[8:]
    with pytest.raises(_native.NativeError) as e:
        GgufFile.parse(bad_version)
    assert e.value.name == "unsupported_version"
    # tensor data past the end of the file
    f = GgufFile.parse(good[:-4])
    with pytest.raises(_native.NativeError):
        f.tensor_bytes("b.weight")
    with pytest.raises(_native.NativeError) as e:
        GgufWriter().add_tensor("x", [128], TQ2_0_G128, np.zeros(10, dtype=np.uint8))
    assert e.value.name == "shape_mismatch"


def test_streaming_parser_matches_full_parse():
    data = _sample_writer().to_bytes()
    for chunk in (1, 7, 64, len(data)):
        p = GgufStreamParser()
        state = 0
        for i in range(0, len(data), chunk):
            state = p.feed(data[i:i + chunk])
        assert state == GgufStreamParser.HEADER_COMPLETE
        f = p.file
        assert [t.name for t in f.tensors] == ["a.weight", "b.weight"]
        assert p.bytes_consumed == len(data)
        assert p.data_bytes_expected == 80 and p.data_bytes_seen == len(data) - f.data_offset
    p = GgufStreamParser()
    assert p.feed(b"XXXXXXXXXXXXXXXXXXXXXXXXXXXX") == GgufStreamParser.FAILED and "magic" in p.error


@settings(max_examples=200, deadline=None)
@given(st.binary(min_size=0, max_size=300))
def test_fuzz_random_bytes_never_crash(blob):
    try:
        GgufFile.parse(blob)
    except _native.NativeError:
        pass


@settings(max_examples=200, deadline=None)
@given(st.integers(0, 400), st.integers(0, 255), st.integers(0, 2000))
def test_fuzz_mutated_header_never_crashes(pos, val, cut):
    data = bytearray(_sample_writer().to_bytes())
    data[pos % len(data)] = val
    data = bytes(data[: max(0, len(data) - cut % len(data))])
    try:
        f = GgufFile.parse(data)
        _ = f.metadata
        for t in f.tensors:
            try:
                f.tensor_bytes(t.name)
            except (_native.NativeError, KeyError):
                pass
    except _native.NativeError:
        pass


def test_config_keys_fallbacks_and_key_length(tmp_path, tiny_cfg):
    p = str(tmp_path / "llm.gguf")
    write_synthetic_gguf(p, tiny_cfg, llm_keys=True)
    c = GgufFile.open(p).config()
    assert (c.hidden, c.inter, c.layers, c.heads, c.kv_heads, c.head_dim, c.vocab) == (256, 512, 2, 4, 2, 64, 1000)
    # head_dim comes from attention.key_length when present, else hidden / heads
    w = GgufWriter().add("general.architecture", "qwen3").add("qwen3.embedding_length", 2560).add("qwen3.attention.head_count", 32)
    w.add("qwen3.attention.key_length", 128)
    assert GgufFile.parse(w.to_bytes()).config().head_dim == 128
    w = GgufWriter().add("qwen3.embedding_length", 2560).add("qwen3.attention.head_count", 32)
    assert GgufFile.parse(w.to_bytes()).config().head_dim == 80
    d = GgufFile.parse(GgufWriter().to_bytes()).config()
    assert (d.hidden, d.layers, d.heads, d.kv_heads, d.inter, d.vocab, d.context) == (4096, 36, 32, 8, 14336, 151936, 65536)


def test_synthetic_gguf_is_seeded_and_loadable(tmp_path, tiny_cfg):
    a, b, c = (str(tmp_path / n) for n in ("a.gguf", "b.gguf", "c.gguf"))
    write_synthetic_gguf(a, tiny_cfg, seed=42)
    write_synthetic_gguf(b, tiny_cfg, seed=42)
    write_synthetic_gguf(c, tiny_cfg, seed=43)
    assert open(a, "rb").read() == open(b, "rb").read() != open(c, "rb").read()
    f = GgufFile.open(a)
    names = {t.name for t in f.tensors}
    assert {"token_embd.weight", "output.weight", "output_norm.weight", "blk.1.ffn_down.weight", "blk.0.attn_q_norm.weight"} <= names
    ti = f.tensor_info("blk.0.ffn_down.weight")
    assert ti.dims == (512, 256) and ti.type == TQ2_0_G128
    assert f.tensor_info("token_embd.weight").type == F16
    o = Oracle(f, 32)
    toks, gaps = o.generate_greedy([1, 2, 3], 4)
    assert len(toks) == 4 and all(0 <= t < 1000 for t in toks) and all(g >= 0 for g in gaps)
