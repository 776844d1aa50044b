"""RAG and evaluation packages (CPU)."""
import json

import numpy as np
import pytest

from oxibonsai_b200 import eval as EV
from oxibonsai_b200 import rag as RG

DOC = """# Bonsai

Bonsai trees are grown in small pots. They need careful watering. Pruning keeps them small!

## Tools

Concave cutters and wire are the classic tools. Wire shapes the branches over months.

## Species

Juniper, maple and pine are popular species. Pines like full sun.
"""


def test_chunkers_cover_the_text_and_respect_limits():
    for chunks in (RG.chunk_chars(DOC, 80, 10), RG.chunk_sentences(DOC, 100), RG.chunk_paragraphs(DOC, 120), RG.chunk_recursive(DOC, 90),
                   RG.chunk_sliding(DOC, 100, 50)):
        assert chunks and all(c.text == DOC[c.start:c.end] for c in chunks) and [c.index for c in chunks] == list(range(len(chunks)))
    assert max(len(c.text) for c in RG.chunk_chars(DOC, 80, 10)) <= 80 and max(len(c.text) for c in RG.chunk_recursive(DOC, 90)) <= 90
    cc = RG.chunk_chars("abcdefghij", 4, 1)
    assert [c.text for c in cc] == ["abcd", "defg", "ghij", "j"]
    s = RG.chunk_sentences("One. Two! Three? Four.", 12)
    assert [c.text.strip() for c in s] == ["One. Two!", "Three? Four."]
    md = RG.chunk_markdown(DOC)
    assert [c.metadata["heading_path"] for c in md] == ["Bonsai", "Bonsai > Tools", "Bonsai > Species"]
    code = RG.chunk_code("import os\n\ndef a():\n    return 1\n\nclass B:\n    def m(self):\n        pass\n")
    assert any(c.text.startswith("def a") for c in code) and any(c.text.startswith("class B") for c in code)
    emb = RG.IdentityEmbedder(64)
    sem = RG.chunk_semantic("Cats purr. Cats meow. Stocks fell today. Stocks rose later.", emb.embed, threshold=0.2)
    assert len(sem) == 2 and "Stocks" in sem[1].text and "Cats" in sem[0].text
    with pytest.raises(ValueError):
        RG.chunk_chars("x", 4, 4)


def test_embedders_store_filters_and_snapshots(tmp_path):
    e = RG.IdentityEmbedder(128)
    a, b, c = e.embed("bonsai trees need water"), e.embed("bonsai trees need careful water"), e.embed("stock markets fell")
    assert abs(np.linalg.norm(a) - 1) < 1e-6 and a @ b > 0.7 > a @ c and not e.embed("").any()
    t = RG.TfIdfEmbedder(128).fit(["the cat sat", "the dog sat", "the bird flew"])
    assert t.idf("the") < t.idf("cat") < t.idf("zebra") and t.embed("the cat").shape == (128,)
    st = RG.VectorStore(128)
    for i, (txt, lang) in enumerate([("bonsai trees need water", "en"), ("pines like full sun", "en"), ("les bonsais aiment l'eau", "fr")]):
        st.add(e.embed(txt), txt, {"lang": lang, "n": i})
    hits = st.search(e.embed("water for bonsai trees"), k=2)
    assert hits[0].text == "bonsai trees need water" and hits[0].score > hits[1].score
    fr = st.search(e.embed("bonsai"), k=3, flt=RG.MetadataFilter.eq("lang", "fr"))
    assert [h.metadata["lang"] for h in fr] == ["fr"]
    f = RG.MetadataFilter.all_of(RG.MetadataFilter("gt", "n", 0), RG.MetadataFilter.any_of(RG.MetadataFilter.eq("lang", "en"), RG.MetadataFilter("exists", "zz")))
    assert [h.metadata["n"] for h in st.search(e.embed("sun"), 3, f)] == [1]
    assert RG.MetadataFilter("not", children=[RG.MetadataFilter("in", "lang", ["en"])]).matches({"lang": "fr"}) and not RG.MetadataFilter("contains", "lang", "x").matches({})
    q = e.embed("pines sun")
    for d in RG.Distance:
        s2 = RG.VectorStore(128, d)
        for txt in ("pines like full sun", "stock markets fell"):
            s2.add(e.embed(txt), txt)
        assert s2.search(q, 1)[0].text == "pines like full sun", d
    p = tmp_path / "store.json"
    st.save(str(p))
    back = RG.VectorStore.load(str(p))
    assert len(back) == 3 and back.search(e.embed("water for bonsai trees"), 1)[0].text == hits[0].text
    with pytest.raises(ValueError):
        st.add([1.0], "bad")
    st.remove(0)
    assert len(st) == 2 and st.search(e.embed("water"), 1)[0].text != "bonsai trees need water"


def test_rag_pipeline_builds_prompt_from_best_chunks():
    for chunker in ("markdown", "recursive", "sentence", "paragraph", "char", "sliding", "code", "semantic"):
        pipe = RG.RagPipeline(config=RG.RagConfig(chunker=chunker, chunk_chars=160, top_k=2))
        assert pipe.index_document(DOC, {"source": "bonsai.md"}) >= 1
    pipe = RG.RagPipeline(config=RG.RagConfig(chunker="markdown", top_k=2))
    pipe.index_document(DOC, {"source": "bonsai.md"})
    pipe.index_document("Stock markets fell sharply on Monday.", {"source": "news"})
    hits = pipe.query("which tools shape the branches with wire?")
    assert "wire" in hits[0].text.lower() and hits[0].metadata["source"] == "bonsai.md"
    prompt = pipe.build_prompt("which tools shape the branches with wire?")
    assert prompt.startswith("Use the following context") and "[1]" in prompt and prompt.endswith("Answer:") and "Question: which tools" in prompt
    only_news = pipe.query("markets", flt=RG.MetadataFilter.eq("source", "news"))
    assert len(only_news) == 1 and pipe.stats()["documents"] == 2
    with pytest.raises(ValueError):
        RG.RagPipeline(config=RG.RagConfig(chunker="nope")).index_document("x")


# ---- eval ---------------------------------------------------------------------------------------------------------------------------
def test_perplexity_matches_closed_form_and_windows_do_not_double_count():
    V = 8
    uniform = lambda toks: np.zeros((len(toks), V))
    r = EV.PerplexityEvaluator().evaluate(list(range(8)) * 4, uniform)
    assert r.perplexity == pytest.approx(V) and r.tokens == 31 and r.bits_per_token == pytest.approx(3.0)
    # a model that always predicts "previous + 1" is perfect on a counting sequence
    def counting(toks):
        out = np.full((len(toks), V), -50.0)
        for i, t in enumerate(toks):
            out[i, (t + 1) % V] = 50.0
        return out
    seq = [i % V for i in range(40)]
    assert EV.PerplexityEvaluator().evaluate(seq, counting).perplexity == pytest.approx(1.0, abs=1e-6)
    w = EV.PerplexityEvaluator(stride=8, max_len=16).evaluate(seq, uniform)
    assert w.tokens == 39 and w.perplexity == pytest.approx(V)


def test_multiple_choice_evaluators_and_item_adapters():
    items = [EV.McItem("2+2=", ["3", "4", "5"], 1, "math"), EV.McItem("capital of France?", ["Paris", "Rome"], 0, "geo"), EV.McItem("sky colour?", ["green", "blue"], 1, "geo")]
    truth = {"2+2=": " 4", "capital of France?": " Paris", "sky colour?": " green"}
    lp = lambda ctx, cont: 0.0 if truth.get(ctx) == cont else -5.0
    r = EV.MultipleChoiceEvaluator().evaluate(items, lp)
    assert r.correct == 2 and r.accuracy == pytest.approx(2 / 3) and r.group_accuracy() == {"math": 1.0, "geo": 0.5} and len(r.confidences) == 3
    letter = EV.mmlu_evaluator()
    seen = []
    letter.evaluate(items[:1], lambda c, k: seen.append((c, k)) or -1.0)
    assert seen[0][0].endswith("A. 3\nB. 4\nC. 5\nAnswer:") and [k for _, k in seen] == [" A", " B", " C"] and "about math" in seen[0][0]
    assert EV.hellaswag_evaluator().scores(EV.McItem("x", ["ab", "abcd"], 0), lambda c, k: -4.0) == [-2.0, -1.0]
    assert EV.mmlu_item({"question": "q", "choices": ["a", "b", "c", "d"], "answer": "C", "subject": "s"}).answer == 2
    assert EV.arc_item({"question": "q", "choices": {"label": ["A", "B"], "text": ["x", "y"]}, "answerKey": "B"}).answer == 1
    assert EV.hellaswag_item({"ctx": "c", "endings": ["a", "b"], "label": "1"}).answer == 1
    wg = EV.winogrande_item({"sentence": "The trophy didn't fit in the case because _ was too big.", "option1": "the trophy", "option2": "the case", "answer": "1"})
    assert wg.answer == 0 and wg.choices[0] == "the trophy was too big." and wg.question.endswith("because")
    assert EV.boolq_item({"passage": "p", "question": "is it", "answer": True}).answer == 1
    assert EV.truthfulqa_item({"question": "q", "mc1_targets": {"choices": ["a", "b"], "labels": [0, 1]}}).answer == 1


def test_generative_and_overlap_metrics():
    assert EV.extract_final_number("so 3 + 4 = 7.\n#### 1,234") == "1234" and EV.extract_final_number("the answer is 42.") == "42" and EV.extract_final_number("none") is None
    rows = [{"question": "1+1", "answer": "#### 2"}, {"question": "2+2", "answer": "#### 4"}]
    r = EV.Gsm8kEvaluator().evaluate(rows, lambda p: "it is 2" if "1+1" in p else "maybe 5")
    assert r.correct == 1 and r.total == 2
    assert EV.exact_match("The Eiffel Tower!", ["eiffel tower"]) == 1.0 and EV.qa_f1("the big red dog", ["big dog"]) == pytest.approx(0.8)
    assert EV.bleu("the cat sat on the mat", ["the cat sat on the mat"]) == pytest.approx(1.0) and EV.bleu("dog", ["the cat"]) == 0.0
    assert 0 < EV.bleu("the cat sat on a mat", ["the cat sat on the mat"]) < 1
    assert EV.chrf("hello world", "hello world") == pytest.approx(1.0) and 0 < EV.chrf("hello word", "hello world") < 1
    rg = EV.rouge("the cat sat", "the cat sat down")
    assert rg["rouge1"] == pytest.approx(2 * 1.0 * 0.75 / 1.75) and rg["rougeL"] == rg["rouge1"] and rg["rouge2"] > 0
    assert EV.meteor("the cat sat", "the cat sat") > 0.9 and EV.meteor("sat cat the", "the cat sat") < EV.meteor("the cat sat", "the cat sat") and EV.meteor("x", "y") == 0.0


def test_calibration_bootstrap_streaming_throughput_report(tmp_path):
    assert EV.expected_calibration_error([0.9] * 10, [1] * 9 + [0]) == pytest.approx(0.0, abs=1e-9)
    assert EV.expected_calibration_error([0.9] * 10, [0] * 10) == pytest.approx(0.9)
    assert EV.brier_score([1.0, 0.0], [1, 0]) == 0.0 and EV.negative_log_likelihood([0.5, 0.5]) == pytest.approx(np.log(2))
    m, lo, hi = EV.bootstrap_ci([0, 1] * 50, 500)
    assert m == 0.5 and lo < 0.5 < hi and hi - lo < 0.3
    s = EV.StreamingAccuracy()
    for v in (1.0, 2.0, 3.0, 4.0):
        s.update(v, v > 2)
    assert s.mean == 2.5 and s.variance == pytest.approx(np.var([1, 2, 3, 4], ddof=1)) and s.accuracy == 0.5 and s.stderr() > 0
    calls = []
    tr = EV.ThroughputBenchmark(1, 3).run(lambda: calls.append(1) or 10)
    assert len(calls) == 4 and tr.tokens == 30 and tr.tokens_per_second > 0 and set(tr.summary()) >= {"p50_ms", "p99_ms"}
    rep = EV.EvalReport("tiny").add("mmlu", accuracy=0.5, n=10).add("ppl", perplexity=12.3)
    assert json.loads(rep.to_json())["results"]["mmlu"]["n"] == 10 and "| mmlu | accuracy | 0.5000 |" in rep.to_markdown()
    p = tmp_path / "d.jsonl"
    EV.save_jsonl(str(p), [{"a": 1}, {"b": "é"}])
    assert EV.load_jsonl(str(p)) == [{"a": 1}, {"b": "é"}]
    p.write_text('{"a": 1}\nnot json\n')
    with pytest.raises(ValueError):
        EV.load_jsonl(str(p))
