"""Tokenizer toolkit: vocabulary, chat-template families, normaliser, batch encoder, BPE trainer + state, streaming decoder."""
import pytest

from oxibonsai_b200.tokenizer import ByteTokenizer, chat_prompt
from oxibonsai_b200.tokenizer import toolkit as T


def test_vocabulary():
    v = T.Vocabulary()
    assert v.is_empty()
    v.insert("hello", 5)
    v.insert("world", 6)
    v.add_special("<eos>", 2)
    assert v.size() == 3 and v.get_id("world") == 6 and v.get_token(5) == "hello" and v.get_id("nope") is None and v.get_token(9) is None
    assert v.is_special_token("<eos>") and v.is_special_id(2) and not v.is_special_token("hello") and not v.is_special_id(5)
    assert list(v) == [("<eos>", 2), ("hello", 5), ("world", 6)]
    v.insert("hello", 7)                                       # re-inserting moves the token to the new id
    assert v.get_id("hello") == 7 and v.get_token(5) is None
    back = T.Vocabulary.from_json(v.to_json())
    assert list(back) == list(v) and back.is_special_id(2)
    assert T.Vocabulary.from_json('{"a": 0, "b": 1}').size() == 2


def test_chat_template_families():
    msgs = [T.ChatMessage.system("be brief"), T.ChatMessage.user("hi {{ role }}"), T.ChatMessage.assistant("hello"), T.ChatMessage.user("bye")]
    K = T.ChatTemplateKind
    chatml = K.CHATML.render_with_generation_prompt(msgs)
    assert chatml == ("<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi {{ role }}<|im_end|>\n<|im_start|>assistant\nhello<|im_end|>\n"
                      "<|im_start|>user\nbye<|im_end|>\n<|im_start|>assistant\n")
    # the evaluator agrees with the hand-written renderer of the package
    plain = [{"role": m.role, "content": m.content} for m in msgs]
    assert chatml == chat_prompt(plain, "chatml") and K.QWEN.render(msgs) == chat_prompt(plain, "qwen", add_generation_prompt=False)
    assert K.LLAMA3.render_with_generation_prompt(msgs) == chat_prompt(plain, "llama3")
    llama = K.LLAMA3.render(msgs[1:2])
    assert llama == "<|begin_of_text|><|start_header_id|>user<|end_header_id|>\n\nhi {{ role }}<|eot_id|>"
    mistral = K.MISTRAL.render([T.ChatMessage.user("q1"), T.ChatMessage.assistant("a1"), T.ChatMessage.user("q2")])
    assert mistral == "<s>[INST] q1 [/INST] a1</s><s>[INST] q2 [/INST]" and K.MISTRAL.generation_prompt() == ""
    assert K.GEMMA.render_with_generation_prompt([T.ChatMessage.user("x")]) == "<start_of_turn>user\nx<end_of_turn>\n<start_of_turn>model\n"
    assert len(K.all()) == 5 and all(k.template() for k in K.all())
    assert [K.infer_from_name(n) for n in ("Meta-Llama-3-8B", "Qwen3-8B", "mistral-7b", "gemma-2b", "my-chatml", "gpt2")] == \
        [K.LLAMA3, K.QWEN, K.MISTRAL, K.GEMMA, K.CHATML, None]
    assert K.CHATML.encode(ByteTokenizer(), [T.ChatMessage.user("a")]) == list(b"<|im_start|>user\na<|im_end|>\n<|im_start|>assistant\n")
    custom = T.ChatTemplate('[{% for message in messages %}{% if role != "system" %}<{{ role }}:{{ content }}>{% endif %}{% endfor %}]')
    assert custom.format([("system", "s"), ("user", "u"), ("assistant", "a")]) == "[<user:u><assistant:a>]"
    assert T.ChatTemplate.chatml().format([("user", "x")]) == "<|im_start|>user\nx<|im_end|>\n"
    assert T.ChatTemplate.extract_user_message(chatml) == "bye" and T.ChatTemplate.extract_user_message("no markers") is None
    assert T.ChatTemplate.llama3().format([]) == "<|begin_of_text|>"


def test_normalizer_and_batch_encoder():
    n = T.TextNormalizer(lowercase=True, strip_accents=True)
    assert n.normalize("  Crème   BRÛLÉE\t\n now ") == "creme brulee now"
    assert T.TextNormalizer.lowercase_only().normalize("  ÀB  c ") == "  àb  c "          # nothing but the case is touched
    assert T.TextNormalizer.whitespace_only().normalize("  A   b ") == "A b"
    tok = ByteTokenizer()
    texts = ["abcdef", "xy", ""]
    plain = T.BatchEncoder(tok).encode_batch(texts)
    assert plain.lengths == [6, 2, 0] and not plain.is_padded() and plain.batch_size() == 3 and plain.max_seq_len() == 6
    right = T.BatchEncoder(tok, pad_id=0).with_max_length(4).with_padding(T.PaddingStrategy.longest()).encode_batch(texts)
    assert right.input_ids == [list(b"abcd"), list(b"xy") + [0, 0], [0] * 4] and right.attention_mask == [[1] * 4, [1, 1, 0, 0], [0] * 4]
    assert right.lengths == [4, 2, 0] and right.is_padded()
    left = T.BatchEncoder(tok, pad_id=9).with_max_length(4).with_truncation(T.TruncationSide.LEFT).with_padding(T.PaddingStrategy.to(5), left=True).encode_batch(texts)
    assert left.input_ids[0] == [9] + list(b"cdef") and left.input_ids[1] == [9, 9, 9] + list(b"xy") and left.attention_mask[1] == [0, 0, 0, 1, 1]
    assert T.BatchEncoder(tok).with_padding(T.PaddingStrategy.to(3)).encode_batch(["abcdef"]).input_ids == [list(b"abc")]


def test_trainer_state_and_roundtrip(tmp_path):
    corpus = ["the quick brown fox jumps over the lazy dog " * 3, "the quicker the better", "pack my box with five dozen liquor jugs"]
    trainer = T.BpeTrainer(T.TrainerConfig(vocab_size=300).with_special_tokens())
    trained = trainer.train(corpus)
    st = trained.stats
    assert st.initial_vocab_size == 260 and st.final_vocab_size == 260 + st.num_merges_performed and 0 < st.num_merges_performed <= 40
    assert trained.special_tokens == {"<BOS>": 0, "<EOS>": 1, "<PAD>": 2, "<UNK>": 3} and trained.vocab[4] == b"\x00" and trained.vocab_size() == st.final_vocab_size + 0
    assert st.corpus_size_chars == sum(len(c) for c in corpus) and st.unique_words > 10 and "merges applied" in st.summary()
    first = trained.merges[0]
    assert trained.vocab[first.merged] == trained.vocab[first.left] + trained.vocab[first.right] and first.frequency >= trained.merges[-1].frequency
    text = trained.merges_to_text()
    assert len(text.splitlines()) == len(trained.merges) and all(len(l.split(" ")) == 2 for l in text.splitlines())
    tok = trained.to_tokenizer()
    sample = "the quick dog jumps"
    ids = tok.encode(sample)
    assert tok.decode(ids) == sample and len(ids) < len(sample)                     # merges shorten the sequence
    # a high frequency floor stops the training early and says how many candidates fell below it
    strict = T.BpeTrainer(T.TrainerConfig(vocab_size=400).with_min_frequency(1000)).train(corpus)
    assert strict.stats.num_merges_performed == 0 and strict.stats.num_merges_skipped > 0 and strict.special_tokens == {}
    with pytest.raises(T.TrainerError):
        T.BpeTrainer(T.TrainerConfig(vocab_size=100)).train(corpus)
    with pytest.raises(T.TrainerError):
        T.BpeTrainer.default_config().train([])
    state = T.TokenizerState.from_trained(trained)
    path = str(tmp_path / "tok.state")
    state.save_to(path)
    again = T.TokenizerState.load_from(path)
    assert again.vocab == state.vocab and again.merges == state.merges and again.special_tokens == state.special_tokens and again.vocab_size() == trained.vocab_size()
    assert again.to_tokenizer().encode(sample) == ids
    assert T.base64_decode(T.base64_encode(b"\x00\xff\x10abc")) == b"\x00\xff\x10abc"
    for bad in ("", "wrong header\n", T.TokenizerState.MAGIC + "\nvocab 2\n0 AA==\n", T.TokenizerState.MAGIC + "\nvocab 1\n0 !!!\nmerges 0\nspecial 0\n",
                T.TokenizerState.MAGIC + "\nvocab 0\nmerges 1\n1 2\nspecial 0\n"):
        with pytest.raises(T.SerializationError):
            T.TokenizerState.load(bad)


def test_token_stream_decoder():
    d = T.TokenStreamDecoder(ByteTokenizer())
    euro = "€".encode()                                    # three bytes
    assert d.push_token(ord("a")) == "a" and d.push_token(euro[0]) == "" and d.pending_len() == 1
    assert d.push_token(euro[1]) == "" and d.pending_len() == 2 and d.push_token(euro[2]) == "€" and d.pending_len() == 0
    assert d.push_tokens("héllo 日本".encode()) == "héllo 日本" and d.total_tokens() == 4 + len("héllo 日本".encode()) and d.total_bytes() == d.total_tokens()
    assert d.finish() == ""
    d.push_token(euro[0])
    with pytest.raises(T.IncompleteUtf8):
        d.finish()
    d.push_token(euro[0])
    assert d.finish_lossy() == "�" and d.pending_len() == 0
    d.reset()
    assert d.total_tokens() == 0 and d.total_bytes() == 0


def test_incremental_merge_learning_equals_a_full_recount_per_merge():
    import random
    from collections import Counter
    from oxibonsai_b200.tokenizer._merge_learner import MergeLearner
    rng = random.Random(11)
    words = Counter()
    for _ in range(300):
        words[tuple(rng.choice("abc") for _ in range(rng.randint(1, 10)))] += rng.randint(1, 5)
    words[tuple("aaaaaaa")] += 3                                           # overlapping occurrences of one pair

    def naive(words, n):
        words, out = Counter(words), []
        for k in range(n):
            pairs = Counter()
            for w, c in words.items():
                for p in zip(w, w[1:]):
                    pairs[p] += c
            if not pairs:
                break
            (a, b), cnt = max(pairs.items(), key=lambda kv: (kv[1], kv[0]))
            new = f"<{k}>"
            out.append(((a, b), cnt, new))
            merged = Counter()
            for w, c in words.items():
                o, i = [], 0
                while i < len(w):
                    if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                        o.append(new)
                        i += 2
                    else:
                        o.append(w[i])
                        i += 1
                merged[tuple(o)] += c
            words = merged
        return out
    learner = MergeLearner(dict(words), make=lambda a, b, i: f"<{i}>", tie=lambda p: p)
    got = list(learner.run(60, 1))
    assert got == naive(words, 60) and len(got) == 60
    # min_count ends the run early, and the counts that are left are those of the rewritten words
    learner = MergeLearner(dict(words), make=lambda a, b, i: f"<{i}>", tie=lambda p: p)
    early = list(learner.run(1000, 20))
    assert early == [m for m in naive(words, 1000) if m[1] >= 20][:len(early)] and all(c >= 20 for _, c, _ in early)
    assert learner.best() is None or learner.best()[1] < 20
