"""RAG extras: chunking strategies and registry, language-aware code chunks, validated filters, configured retriever with
re-ranking, snapshots that survive a restart."""
import json

import numpy as np
import pytest

from oxibonsai_b200.rag import Distance, IdentityEmbedder, MetadataFilter, RagPipeline, TfIdfEmbedder, VectorStore
from oxibonsai_b200.rag import extras as X

TEXT = ("Bonsai trees are grown in shallow pots. They need regular pruning! Do they need sun? Yes, most species do.\n\n"
        "# Watering\nWater when the soil feels dry. Never let the roots stand in water.\n\n# Wiring\nWire branches in autumn.")


def test_strategies_registry_and_rich_chunks():
    reg = X.ChunkerRegistry.default_registry()
    assert reg.available_strategies() == ["markdown", "recursive", "sentence", "sliding"]
    for name in reg.available_strategies():
        chunks = reg.chunk(name, TEXT)
        assert chunks and all(c.metadata["strategy"] == name and TEXT[c.char_start:c.char_end] == c.text and not c.is_empty() for c in chunks)
        assert [c.chunk_index for c in chunks] == list(range(len(chunks)))
    with pytest.raises(KeyError, match="available"):
        reg.chunk("nope", TEXT)
    sent = X.SentenceChunker(60).chunk(TEXT)
    lap = X.SentenceChunker(60).with_overlap(1).chunk(TEXT)
    assert len(lap) >= len(sent) and any(a.char_end > b.char_start for a, b in zip(lap, lap[1:]))      # consecutive chunks share a sentence
    assert sent[0].word_count() == len(sent[0].text.split()) and len(sent[0]) == len(sent[0].text)
    win = X.SlidingWindowChunker.with_50pct_overlap(40).chunk(TEXT)
    assert win[1].char_start == 20 and X.SlidingWindowChunker.non_overlapping(40).chunk(TEXT)[1].char_start == 40
    with pytest.raises(ValueError):
        X.SlidingWindowChunker(10, 20)
    rec = X.RecursiveCharSplitter(80).with_overlap(10).chunk(TEXT)
    assert all(len(c.text) <= 80 + 10 for c in rec) and rec[1].char_start < rec[0].char_end
    assert X.RecursiveCharSplitter.default_separators()[0] == "\n\n" and X.RecursiveCharSplitter(50).with_separators(["\n", ""]).chunk("a\nb") 
    md = X.MarkdownChunker(200).chunk(TEXT)
    assert any(c.text.lstrip().startswith("# Wiring") for c in md)


def test_code_chunker_by_language():
    assert [X.Language.from_extension(e) for e in ("rs", ".PY", "json", "txt")] == [X.Language.RUST, X.Language.PYTHON, X.Language.JSON, X.Language.PLAIN]
    py = "import os\n\nclass A:\n    def m(self):\n        return 1\n\ndef free(x):\n    return x * 2\n\nasync def co():\n    pass\n"
    chunks = X.CodeChunker(X.Language.PYTHON).with_min_chunk_chars(12).chunk(py)
    heads = [c.text.lstrip().split("\n")[0] for c in chunks]
    assert heads == ["import os", "def free(x):", "async def co():"] and "class A:" in chunks[0].text          # the short import line joined the class
    assert all(py[c.char_start:c.char_end] == c.text and c.metadata["language"] == "python" for c in chunks)
    rs = "use std::fmt;\n\npub struct P { x: i32 }\n\nimpl P {\n    pub fn new() -> Self { P { x: 0 } }\n}\n\npub(crate) fn helper() {}\n\nmod tests {}\n"
    r = X.CodeChunker(X.Language.RUST).with_min_chunk_chars(1).chunk(rs)
    assert [c.text.split("\n")[0] for c in r] == ["use std::fmt;", "pub struct P { x: i32 }", "impl P {", "pub(crate) fn helper() {}", "mod tests {}"]
    js = json.dumps({"name": "bonsai", "tags": ["a", "b,c"], "nested": {"k": [1, 2]}, "n": 3}, indent=1)
    j = X.CodeChunker(X.Language.JSON).with_min_chunk_chars(1).chunk(js)
    assert [c.text.split(":")[0] for c in j] == ['"name"', '"tags"', '"nested"', '"n"'] and '"b,c"' in j[1].text
    arr = X.CodeChunker(X.Language.JSON).with_min_chunk_chars(1).chunk('[{"a": 1}, {"b": [2, 3]}, 4]')
    assert [c.text for c in arr] == ['{"a": 1}', '{"b": [2, 3]}', "4"]
    broken = X.CodeChunker(X.Language.JSON).with_fallback_window(20).chunk('{"a": 1, "b": ' + "x" * 50)
    assert len(broken) > 1 and X.CodeChunker().language() is X.Language.PLAIN and X.CodeChunker().chunk("just text")[0].text == "just text"


def test_filters_and_distances():
    ok = MetadataFilter.all_of(MetadataFilter.eq("lang", "en"), MetadataFilter.any_of(X.filter_exists("year"), X.filter_neq("kind", "draft")))
    X.validate_filter(ok)
    assert ok.matches({"lang": "en", "kind": "final"}) and not ok.matches({"lang": "en", "kind": "draft"}) and ok.matches({"lang": "en", "kind": "draft", "year": 2020})
    for bad in (MetadataFilter("like", "k", 1), MetadataFilter("eq", "", 1), MetadataFilter("and"), MetadataFilter("not", children=[ok, ok]),
                MetadataFilter("in", "k", 5), MetadataFilter("gt", "k", "x")):
        with pytest.raises(ValueError):
            X.validate_filter(bad)
    deep = MetadataFilter.eq("a", 1)
    for _ in range(40):
        deep = MetadataFilter("not", children=[deep])
    with pytest.raises(ValueError, match="deeper"):
        X.validate_filter(deep)
    assert X.is_similarity(Distance.COSINE) and X.is_similarity(Distance.DOT) and X.is_distance(Distance.EUCLIDEAN) and X.is_distance(Distance.MANHATTAN)
    assert X.compute_distance(Distance.EUCLIDEAN, [0, 0], [3, 4]) == 5.0 and X.compute_distance(Distance.MANHATTAN, [0, 0], [3, 4]) == 7.0
    assert X.compute_distance(Distance.COSINE, [1, 0], [1, 0]) == pytest.approx(1.0) and X.compute_distance(Distance.COSINE, [0, 0], [1, 0]) == 0.0
    assert X.to_score(Distance.EUCLIDEAN, 5.0) == -5.0 and X.to_score(Distance.DOT, 5.0) == 5.0
    with pytest.raises(ValueError):
        X.compute_distance(Distance.DOT, [1, 2], [1])
    with pytest.raises(ValueError):
        X.compute_distance(Distance.DOT, [1e308, 1e308], [1e308, 1e308])


def test_configured_retriever_rerank_and_snapshot(tmp_path):
    docs = ["Prune the maple bonsai in early spring before the buds open.", "Water the juniper when the top soil is dry to the touch.",
            "Repot every two years and trim a third of the roots.", "Maple leaves scorch in strong summer sun, so give shade."]
    emb = TfIdfEmbedder(2048).fit(docs)
    r = X.ConfiguredRetriever(emb, X.RetrieverConfig().with_top_k(2))
    assert r.add_documents(docs) == 4 and r.document_count() == 4 and r.chunk_count() == 4
    r.add_document("Fertilise monthly in the growing season.", {"topic": "feeding"})
    plain = r.retrieve("when should I prune a maple")
    assert len(plain) == 2 and "Prune the maple" in plain[0].text
    assert r.retrieve_text("how often to repot", 1) == [docs[2]]
    only = r.retrieve_filtered("anything at all", MetadataFilter.eq("topic", "feeding"), 3)
    assert [h.metadata.get("topic") for h in only] == ["feeding"]
    with pytest.raises(ValueError):
        r.retrieve_filtered("x", MetadataFilter("bogus", "k"))
    # re-ranking: a lexical match is lifted above a slightly closer dense neighbour
    hits = [X.SearchHit(0, 0.50, "nothing shared here", {}), X.SearchHit(1, 0.47, "maple pruning in spring", {}), X.SearchHit(2, 0.99, "maple maple maple prune spring when", {})]
    rr = X.rerank(hits, "when to prune maple in spring")
    assert [h.id for h in rr] == [2, 1, 0] and rr[0].score == 1.0 and rr[1].score == pytest.approx(0.47 + 0.06) and rr[2].score == 0.50
    strict = X.ConfiguredRetriever(emb, X.RetrieverConfig().with_top_k(3).with_min_score(0.99).with_rerank())
    strict.add_documents(docs)
    assert strict.retrieve("completely unrelated words zebra quartz") == []
    snap = X.RetrieverSnapshot.to_snapshot(r)
    path = str(tmp_path / "retriever.json")
    snap.save(path)
    back = X.RetrieverSnapshot.load(path).from_snapshot()
    assert back.document_count() == 5 and back.chunk_count() == 5 and back.config.top_k == 2
    again = back.retrieve("when should I prune a maple")
    assert [h.text for h in again] == [h.text for h in plain] and again[0].score == pytest.approx(plain[0].score, abs=1e-6)
    doc = json.loads(snap.save_json())
    doc["version"] = 99
    with pytest.raises(ValueError, match="version"):
        X.RetrieverSnapshot.load_json(json.dumps(doc))

    class Custom:
        dim = 4

        def embed(self, text):
            return np.ones(4, dtype=np.float32)
    with pytest.raises(ValueError, match="cannot be snapshotted"):
        X.RetrieverSnapshot.to_snapshot(X.ConfiguredRetriever(Custom()))
    st = X.pipeline_stats(r)
    assert (st.documents_indexed, st.chunks_indexed, st.embedding_dim) == (5, 5, 2048) and st.store_memory_bytes > 5 * 2048 * 4
    p = RagPipeline(IdentityEmbedder(64))
    p.index_document(TEXT)
    assert X.pipeline_stats(p).documents_indexed == 1 and X.pipeline_stats(p).embedding_dim == 64
    s = VectorStore(2)
    s.add([1, 0], "a")
    s.add([0, 1], "b")
    assert [h.text for h in X.search_with_threshold(s, [1, 0], 5, 0.5)] == ["a"]
    X.clear_store(s)
    assert len(s) == 0 and s.search([1, 0]) == []
