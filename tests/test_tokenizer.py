"""Tokenizers on CPU: byte-level BPE with the C++ merge engine, HF json loading, trainer, streaming decoder, chat
templates, Unigram / WordPiece / char models, byte fallback and text serialisation."""
import json

import pytest

from oxibonsai_b200 import tokenizer as T
from oxibonsai_b200.tokenizer import extras as X

CORPUS = ["the quick brown fox jumps over the lazy dog", "the quicker the better", "lazy dogs and quick foxes", "héllo wörld, the end"] * 4


def test_bpe_train_encode_decode_roundtrip_and_merges_run_in_native_code():
    tok = T.train_bpe(CORPUS, vocab_size=320, special_tokens=["<|im_start|>", "<|im_end|>"])
    assert 256 < len(tok.vocab) <= 318 and tok.merges and tok.vocab_size == max(tok.special.values()) + 1
    for text in CORPUS + ["unseen wörds ☃ too", ""]:
        ids = tok.encode(text)
        assert tok.decode(ids) == text
    ids = tok.encode("the the the")
    assert len(ids) < len("the the the")                                   # merges were applied
    assert tok.encode("the") == tok.encode("the")                           # cache hit path gives the same ids
    sp = tok.encode("<|im_start|>user\nhi<|im_end|>")
    assert sp[0] == tok.special["<|im_start|>"] and sp[-1] == tok.special["<|im_end|>"]
    assert tok.decode(sp, skip_special=True) == "user\nhi" and tok.encode("<|im_end|>", allow_special=False) != [tok.special["<|im_end|>"]]
    assert b"".join(tok.token_bytes(i) for i in tok.encode("héllo")) == "héllo".encode()
    assert tok.encode_batch(["a", "b"]) == [tok.encode("a"), tok.encode("b")]


def test_hf_json_loading_and_text_serialisation(tmp_path):
    tok = T.train_bpe(CORPUS, vocab_size=300, special_tokens=["<eos>"])
    inv = {i: t for t, i in tok.vocab.items()}
    j = {"model": {"type": "BPE", "vocab": tok.vocab, "merges": [f"{inv[a]} {inv[b]}" for a, b, _ in tok.merges]},
         "added_tokens": [{"id": i, "content": t} for t, i in tok.special.items()]}
    p = tmp_path / "tokenizer.json"
    p.write_text(json.dumps(j))
    again = T.BpeTokenizer.from_hf_json(str(p))
    text = "the quick brown fox<eos>"
    assert again.encode(text) == tok.encode(text) and isinstance(T.load_tokenizer(str(p)), T.BpeTokenizer)
    assert isinstance(T.load_tokenizer(None), T.ByteTokenizer) and T.load_tokenizer(str(p), "bytes").vocab_size == 256
    pairs = tmp_path / "pairs.json"
    j["model"]["merges"] = [[inv[a], inv[b]] for a, b, _ in tok.merges]       # the list-of-pairs form of newer files
    pairs.write_text(json.dumps(j))
    assert T.BpeTokenizer.from_hf_json(str(pairs)).encode(text) == tok.encode(text)
    j["model"]["type"] = "Unigram"
    p.write_text(json.dumps(j))
    with pytest.raises(ValueError):
        T.BpeTokenizer.from_hf_json(str(p))
    txt = tmp_path / "bpe.txt"
    X.save_bpe_text(tok, str(txt))
    assert X.load_bpe_text(str(txt)).encode(text) == tok.encode(text)


def test_streaming_decoder_never_splits_utf8():
    d = T.StreamingDecoder()
    data = "añ☃😀z".encode()
    out = [d.push(bytes([b])) for b in data]
    assert "".join(out) + d.flush() == "añ☃😀z" and all("�" not in o for o in out)
    assert out[1] == "" and out[2] == "ñ"
    d2 = T.StreamingDecoder()
    assert d2.push(b"\xe2\x98") == "" and d2.flush() == "�"


def test_chat_templates():
    msgs = [{"role": "system", "content": "S"}, {"role": "user", "content": "U"}, {"role": "assistant", "content": "A"}, {"role": "user", "content": "Q"}]
    assert T.chat_prompt(msgs, "chatml") == "<|im_start|>system\nS<|im_end|>\n<|im_start|>user\nU<|im_end|>\n<|im_start|>assistant\nA<|im_end|>\n<|im_start|>user\nQ<|im_end|>\n<|im_start|>assistant\n"
    assert T.chat_prompt(msgs, "qwen") == T.chat_prompt(msgs, "chatml") and not T.chat_prompt(msgs, "chatml", add_generation_prompt=False).endswith("assistant\n")
    l3 = T.chat_prompt(msgs, "llama3")
    assert l3.startswith("<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\nS<|eot_id|>") and l3.endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")
    assert T.chat_prompt(msgs, "mistral") == "<s>[INST] S\n\nU [/INST] A</s>[INST] Q [/INST]"
    assert T.chat_prompt(msgs[1:2], "gemma") == "<bos><start_of_turn>user\nU<end_of_turn>\n<start_of_turn>model\n"
    with pytest.raises(ValueError):
        T.chat_prompt(msgs, "nope")


def test_unigram_wordpiece_char_and_byte_fallback():
    u = X.UnigramTokenizer([("<unk>", 0.0), ("▁", -2.0), ("▁the", -1.0), ("▁th", -3.0), ("e", -2.5), ("▁c", -3.0), ("a", -2.0), ("t", -2.0), ("at", -1.5), ("▁cat", -6.5)])
    ids = u.encode(" the cat")
    assert [u.pieces[i] for i in ids] == ["▁the", "▁c", "at"] and u.decode(ids) == " the cat"      # -1 -3 -1.5 beats -1 -6.5
    assert u.encode("x") == [0] and u.token_bytes(2) == b" the"
    w = X.WordPieceTokenizer(["[UNK]", "un", "##aff", "##able", "play", "##ing", ",", "aff"], lowercase=True)
    assert [w.tokens[i] for i in w.encode("Unaffable, playing xyz")] == ["un", "##aff", "##able", ",", "play", "##ing", "[UNK]"]
    assert w.decode(w.encode("unaffable playing")) == "unaffable playing"
    c = X.CharTokenizer("hello")
    assert c.decode(c.encode("hello")) == "hello" and c.encode("z") == [0] and c.vocab_size == 5
    vocab = {"a": 1, "b": 2, **{X.byte_fallback_token(b): 10 + b for b in range(256)}}
    ids = X.encode_with_byte_fallback("aé", vocab)
    assert ids == [1, 10 + 0xC3, 10 + 0xA9] and X.decode_with_byte_fallback(ids, {v: k for k, v in vocab.items()}) == "aé"
    assert X.parse_byte_fallback("<0x0A>") == 10 and X.parse_byte_fallback("<0xZZ>") is None and X.parse_byte_fallback("abc") is None


def test_hf_bridge_gives_the_real_bytes_of_byte_level_tokens(tmp_path):
    """A byte-level BPE token may be a fragment of a UTF-8 character; ``decode`` turns that into U+FFFD, the bridge must
    not: streaming joins fragments of several tokens into one character."""
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=400, special_tokens=["<|endoftext|>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(["héllo wörld 日本語 " * 20, "the quick brown fox 🙂 " * 20], trainer)
    path = str(tmp_path / "tokenizer.json")
    tok.save(path)
    hf, native = T.HfTokenizerBridge(path), T.BpeTokenizer.from_hf_json(path)
    text = "héllo 日本語 🙂 fox"
    assert hf.encode(text) == native.encode(text)
    assert all(hf.token_bytes(i) == native.token_bytes(i) for i in range(1, hf.vocab_size))           # (id 0 is the special token)
    assert hf.token_bytes(0) == b"<|endoftext|>"
    dec = T.StreamingDecoder()
    assert "".join(dec.push(hf.token_bytes(i)) for i in hf.encode(text)) + dec.flush() == text


def test_native_bpe_uses_the_files_own_split_pattern(tmp_path):
    """Qwen-style files carry their pre-tokenizer's regular expression (digits one by one, contractions case-insensitive);
    the native tokenizer takes it from the file and agrees with the ``tokenizers`` library on text where the GPT-2 pattern
    would split differently."""
    pytest.importorskip("tokenizers")
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    qwen = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(qwen), behavior="isolated"),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|endoftext|>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(["call 911 or 1234567 now, it's 12:30pm!! " * 30, "the quick brown fox's 42 jumps\n\nnew line " * 30, "IT'S DONE, I'LL go.  ok\t\tthen" * 30], trainer)
    path = str(tmp_path / "tokenizer.json")
    tok.save(path)
    native = T.BpeTokenizer.from_hf_json(path)
    assert native._split.pattern == qwen
    for text in ("call 911 or 1234567 now", "it's 12:30pm!!\n\nnew", "fox's  42   jumps", "IT'S DONE, I'LL go.", "a\t\tb  \n c", "x=3.14159;y=-2"):
        assert native.encode(text) == tok.encode(text, add_special_tokens=False).ids, text
        assert native.decode(native.encode(text)) == text


def test_tokenizer_embedded_in_a_gguf_file(tmp_path):
    """``tokenizer.ggml.*`` metadata (tokens, merges, token types, eos) make a working tokenizer; ``load_tokenizer`` falls
    back to it when no tokenizer file is given, and to raw bytes when the checkpoint embeds nothing."""
    from oxibonsai_b200.core import GgufWriter, Qwen3Config, write_synthetic_gguf
    tok = T.train_bpe(["the quick brown fox jumps over the lazy dog " * 10, "héllo wörld 日本 12345 " * 10], 420, special_tokens=["<|endoftext|>", "<|im_start|>"])
    tokens = [tok.id_to_token[i] for i in range(tok.vocab_size)]
    w = GgufWriter()
    w.add("general.architecture", "qwen3").add("tokenizer.ggml.model", "gpt2").add("tokenizer.ggml.pre", "qwen2")
    w.add("tokenizer.ggml.tokens", tokens).add("tokenizer.ggml.merges", [f"{tok.id_to_token[a]} {tok.id_to_token[b]}" for a, b, _ in tok.merges])
    w.add("tokenizer.ggml.token_type", [3 if t in tok.special else 1 for t in tokens]).add("tokenizer.ggml.eos_token_id", tok.special["<|endoftext|>"])
    path = str(tmp_path / "with_vocab.gguf")
    w.write(path)
    emb = T.BpeTokenizer.from_gguf(path)
    text = "the quick dog says héllo 日本<|im_start|>ok"
    assert emb.vocab_size == tok.vocab_size and emb.special == tok.special and emb.eos_token_id == tok.special["<|endoftext|>"]
    ids = emb.encode(text)
    assert tok.special["<|im_start|>"] in ids and emb.decode(ids) == text and emb.normal_form == "NFC"
    assert emb.encode("abc 12345") != [] and all(emb.decode([i]) in "12345" for i in emb.encode("12345"))     # the Qwen pattern isolates digits
    assert isinstance(T.load_tokenizer(None, model_path=path), T.BpeTokenizer) and isinstance(T.load_tokenizer(path), T.BpeTokenizer)
    plain = str(tmp_path / "no_vocab.gguf")
    write_synthetic_gguf(plain, Qwen3Config(hidden=256, inter=512, layers=1, heads=2, kv_heads=1, head_dim=128, vocab=300, context=64, name="t"), seed=1)
    assert isinstance(T.load_tokenizer(None, model_path=plain), T.ByteTokenizer)
    with pytest.raises(ValueError, match="embeds no"):
        T.BpeTokenizer.from_gguf(plain)


def _greedy_reference(ids: list[int], table: dict) -> list[int]:
    """Lowest rank first, leftmost among equals, one merge at a time: the definition the native heap has to reproduce."""
    ids = list(ids)
    while len(ids) > 1:
        best = min(((table[(a, b)][0], i) for i, (a, b) in enumerate(zip(ids, ids[1:])) if (a, b) in table), default=None)
        if best is None:
            break
        i = best[1]
        ids[i:i + 2] = [table[(ids[i], ids[i + 1])][1]]
    return ids


def test_native_merge_equals_the_one_merge_at_a_time_definition_on_long_pieces():
    import random
    rng = random.Random(7)
    corpus = ["".join(rng.choice("abcd") for _ in range(rng.randint(1, 12))) for _ in range(400)]
    tok = T.train_bpe([" ".join(corpus)], vocab_size=330)
    table = {(a, b): (r, m) for r, (a, b, m) in enumerate(tok.merges)}
    assert len(table) > 30
    for n in (1, 2, 3, 17, 200, 3000):
        for _ in range(5):
            piece = "".join(rng.choice("abcd") for _ in range(n))            # no split point: one piece of n bytes
            want = _greedy_reference([tok._byte_id[b] for b in piece.encode()], table)
            assert tok.encode(piece) == want == tok._encode_piece(piece)
    assert tok.encode("a" * 1001) == _greedy_reference([tok._byte_id[ord("a")]] * 1001, table)


def test_encode_of_a_long_text_is_one_native_call_and_matches_piecewise_encoding():
    import random
    import time
    rng = random.Random(3)
    words = ["".join(rng.choice("abcdefghij") for _ in range(rng.randint(2, 8))) for _ in range(300)]
    tok = T.train_bpe([" ".join(rng.choice(words) for _ in range(2000))], vocab_size=500, special_tokens=["<|sep|>"])
    text = " ".join(rng.choice(words) for _ in range(40000)) + "<|sep|>" + "wörd ☃ 日本 " * 500 + "\n\n  tail"
    t0 = time.perf_counter()
    ids = tok.encode(text)
    dt = time.perf_counter() - t0
    piecewise = []
    for seg in text.split("<|sep|>"):
        for p in tok._split.findall(seg):
            piecewise.extend(tok._encode_piece(p))
        piecewise.append(tok.special["<|sep|>"])
    assert ids == piecewise[:-1] and tok.decode(ids) == text
    assert dt < 1.0                                                          # ~25 ms here; the per-piece path took ~0.3 s
    # a piece without any split point, as long as a request can be: n log n, not n^2 (2 s at 200k characters before)
    blob = "".join(rng.choice("abcdefghij") for _ in range(200000))
    t0 = time.perf_counter()
    out = tok.encode(blob)
    assert time.perf_counter() - t0 < 1.0 and tok.decode(out) == blob
