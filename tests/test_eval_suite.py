"""The evaluation suite's scored-object forms against hand-computed values and the benchmark evaluators' protocols."""
import json
import math

import pytest

from oxibonsai_b200.eval import benchmarks as B
from oxibonsai_b200.eval import suite as S


def test_tokenize_and_bleu_variants():
    assert S.tokenize("The cat, (the) CAT!  -- sat.") == ["the", "cat", "the", "cat", "sat"]
    ref = "the cat is on the mat"
    perfect = S.sentence_bleu(ref, [ref])
    assert perfect.bleu == pytest.approx(1.0) and perfect.brevity_penalty == 1.0 and perfect.length_ratio == 1.0
    # clipped unigram precision: "the" x7 against a reference with two "the" -> 2/7 (Papineni's example)
    s = S.sentence_bleu("the the the the the the the", ["the cat is on the mat"], S.BleuConfig(1))
    assert s.precisions == [pytest.approx(2 / 7)]
    # no 4-gram match: zero without smoothing, positive with either smoothing
    cand = "the cat sat on a mat"
    none = S.sentence_bleu(cand, [ref])
    add1 = S.sentence_bleu(cand, [ref], S.BleuConfig(4, S.SmoothingMethod.ADD_ONE))
    decay = S.sentence_bleu(cand, [ref], S.BleuConfig(4, S.SmoothingMethod.EXP_DECAY))
    assert none.bleu == 0.0 and none.precisions[0] == pytest.approx(4 / 6) and none.precisions[3] == 0.0
    assert none.precisions[1] == pytest.approx(1 / 5) and none.precisions[2] == 0.0              # one shared bigram, no trigram
    assert 0 < decay.bleu < add1.bleu < 1
    assert decay.precisions[2] == pytest.approx(1 / (2 * 6)) and decay.precisions[3] == pytest.approx(1 / (4 * 6))   # first and second zero
    assert add1.precisions[1] == pytest.approx((1 + 1) / (5 + 1)) and add1.precisions[0] == pytest.approx(4 / 6)
    # brevity penalty: candidate of 3 words against 6 -> exp(1 - 6/3); closest reference length with ties to the shorter one
    short = S.sentence_bleu("the cat is", [ref], S.BleuConfig(1))
    assert short.brevity_penalty == pytest.approx(math.exp(1 - 2)) and short.bleu == pytest.approx(math.exp(-1))
    tie = S.sentence_bleu_tokens(["a"] * 4, [["a"] * 3, ["a"] * 5], S.BleuConfig(1))
    assert tie.length_ratio == pytest.approx(4 / 3) and tie.brevity_penalty == 1.0
    assert S.sentence_bleu("", [ref]).bleu == 0.0 and S.sentence_bleu("", [ref]).brevity_penalty == 0.0
    # corpus BLEU pools the counts: two sentences, 3/4 + 2/2 unigrams -> 5/6
    c = S.corpus_bleu(["a b c d", "x y"], [["a b c z"], ["x y"]], S.BleuConfig(1))
    assert c.precisions[0] == pytest.approx(5 / 6) and c.bleu == pytest.approx(5 / 6)


def test_rouge_family():
    cand, ref = "the cat sat on the mat", "the cat lay on the mat today"
    r1 = S.RougeNScore.compute(cand, ref, 1)
    assert (r1.precision, r1.recall) == (pytest.approx(5 / 6), pytest.approx(5 / 7)) and r1.f1 == pytest.approx(2 * (5 / 6) * (5 / 7) / (5 / 6 + 5 / 7))
    r2 = S.RougeNScore.compute(cand, ref, 2)
    assert r2.precision == pytest.approx(3 / 5) and r2.recall == pytest.approx(3 / 6)          # the cat, on the, the mat
    rl = S.RougeLScore.compute(cand, ref)
    assert rl.lcs_length == 5 and rl.recall == pytest.approx(5 / 7)
    assert S.lcs_length("ABCBDAB", "BDCABA") == 4
    rs = S.RougeSScore.compute("a b c", "a c b")
    # skip-bigrams {ab, ac, bc} vs {ac, ab, cb}: two shared of three
    assert rs.precision == rs.recall == pytest.approx(2 / 3)
    multi = S.RougeNScore.compute_multi_ref("a b c d", ["a x y z w", "a b c q"], 1)
    assert multi.recall == pytest.approx(3 / 4)
    empty = S.RougeNScore.compute("", ref, 1)
    assert (empty.precision, empty.recall, empty.f1) == (0.0, 0.0, 0.0) and S.RougeSScore.compute("a", "a").f1 == 0.0
    corpus = S.CorpusRouge.compute([(cand, ref), ("x", "x")])
    assert corpus.num_samples == 2 and corpus.rouge_1.f1 == pytest.approx((r1.f1 + 1.0) / 2) and "ROUGE-1 F1" in corpus.summary()
    assert S.CorpusRouge.compute([]).num_samples == 0 and S.CorpusRouge.compute([]).rouge_1 is None


def test_chrf_meteor_qa():
    assert S.chrf_score("abc", "abc").score == pytest.approx(1.0) and S.chrf_score("abc", "xyz").score == 0.0
    plain, plus = S.chrf_score("the cat sat", "the cat sits"), S.chrf_plus_plus("the cat sat", "the cat sits")
    assert 0 < plain.score < 1 and plus.word_order == 2 and plus.score != plain.score and plus.order == 6
    # order-1 characters only, beta 1: candidate "aab" vs "ab": overlap 2, p 2/3, r 1 -> F1 0.8
    assert S.chrf_with("aab", "ab", order=1, beta=1.0).score == pytest.approx(0.8)
    m = S.meteor_score("the cat sat on the mat", "the cat sat on the mat")
    assert m.precision == m.recall == 1.0 and m.fragmentation == pytest.approx(1 / 6) and m.score == pytest.approx(1 - 0.5 * (1 / 6) ** 3)
    assert S.align_tokens(["b", "a", "a"], ["a", "b", "a"]) == [(0, 1), (1, 0), (2, 2)]
    scattered = S.meteor_tokens(["c", "b", "a"], ["a", "b", "c"])
    assert scattered.fragmentation == 1.0 and scattered.score == pytest.approx(0.5)
    assert S.meteor_multi("a b", ["x y", "a b"]).score > 0.9 and S.meteor_score("", "a").score == 0.0
    assert S.normalize_tokens("The  Eiffel-Tower, in a Paris!") == ["eiffeltower", "in", "paris"]
    assert S.f1_score("Paris France", "paris") == pytest.approx(2 / 3) and S.f1_score("", "") == 1.0 and S.f1_score("x", "") == 0.0
    sc = S.score_multi("the Paris", ["London", "Paris"])
    assert sc.exact_match == 1.0 and sc.f1 == 1.0
    corpus = S.corpus_em_f1(["Paris", "Rome Italy"], [["Paris"], ["Rome"]])
    assert corpus.exact_match == 0.5 and corpus.f1 == pytest.approx((1 + 2 / 3) / 2)


def test_calibration_bootstrap_and_online_counters():
    r = S.calibration_all([0.95, 0.9, 0.55, 0.6], [1, 1, 0, 1], n_bins=10)
    assert len(r.bin_stats) == 10 and [b.count for b in r.bin_stats] == [0, 0, 0, 0, 0, 1, 1, 0, 0, 2]
    nine = r.bin_stats[9]
    assert nine.lo == pytest.approx(0.9) and nine.avg_confidence == pytest.approx(0.925) and nine.avg_accuracy == 1.0
    assert r.ece == pytest.approx(0.25 * 0.55 + 0.25 * 0.4 + 0.5 * 0.075)
    assert r.brier == pytest.approx((0.05 ** 2 + 0.1 ** 2 + 0.55 ** 2 + 0.4 ** 2) / 4)
    assert r.nll == pytest.approx(-(math.log(0.95) + math.log(0.9) + math.log(0.45) + math.log(0.6)) / 4)
    assert S.nll_from_logits([[0.0, 0.0], [2.0, 0.0]], [0, 0]) == pytest.approx((math.log(2) + math.log(1 + math.exp(-2))) / 2)
    assert S.calibration_all([], []).ece == 0.0
    ci = S.bootstrap_interval([0, 1, 1, 1, 0, 1, 1, 0, 1, 1], n_resamples=500, seed=7)
    again = S.bootstrap_interval([0, 1, 1, 1, 0, 1, 1, 0, 1, 1], n_resamples=500, seed=7)
    assert ci.mean == pytest.approx(0.7) and ci.lo < 0.7 < ci.hi and ci.contains(0.7) and (ci.lo, ci.hi) == (again.lo, again.hi) and ci.width > 0
    assert S.bootstrap_interval([]).mean == 0.0
    op = S.OnlinePerplexity()
    assert op.current() == float("inf")
    op.push_chunk([math.log(0.5)] * 4)
    assert op.tokens() == 4 and op.current() == pytest.approx(2.0)
    op.reset()
    assert op.tokens() == 0
    oa = S.OnlineAccuracy()
    oa.push_many([True, False, True, True])
    assert oa.counts() == (3, 4) and oa.current() == 0.75


def test_datasets_sampling_and_splits():
    text = "\n".join(json.dumps({"id": f"e{i}", "input": f"q{i}", "expected_output": str(i), "metadata": {"k": i}}) for i in range(10)) + "\n\n"
    ds = B.EvalDataset.from_jsonl("toy", text)
    assert len(ds) == 10 and not ds.is_empty() and ds.examples[3].metadata == {"k": 3}
    assert B.EvalDataset.from_jsonl("toy", ds.to_jsonl()).to_jsonl() == ds.to_jsonl()
    a, b = ds.sample(4, seed=1), ds.sample_with_seed(4, seed=1)
    assert [e.id for e in a.examples] == [e.id for e in b.examples] and len(a) == 4 and len({e.id for e in a.examples}) == 4
    assert [e.id for e in ds.sample(4, seed=2).examples] != [e.id for e in a.examples]
    assert sorted(e.id for e in ds.sample(99, seed=3).examples) == sorted(e.id for e in ds.examples)
    tr, te = ds.split(0.75)
    assert [len(tr), len(te)] == [7, 3] and tr.examples[0].id == "e0" and te.examples[0].id == "e7"
    with pytest.raises(ValueError, match="line 2"):
        B.EvalDataset.from_jsonl("bad", '{"input": "x"}\n{broken\n')
    mc = B.McDataset.from_jsonl("mc", "\n".join(json.dumps({"question": f"q{i}", "choices": ["A: w", "B: x", "C: y", "D: z"], "answer": "ABCD"[i % 4],
                                                            "subject": ["bio", "law"][i % 2]}) for i in range(6)))
    assert mc.subjects() == ["bio", "law"] and len(mc.filter_by_subject("law")) == 3 and mc.questions[2].correct_answer == 2
    assert len(mc.sample_with_seed(2, 5)) == 2


def test_multiple_choice_evaluators_and_benchmarks():
    q = B.MultipleChoiceQuestion("1", "2 + 2 = ?", ["A: 3", "B: 4", "C: 5"], 1, "math")
    ev = B.McEvaluator()
    assert ev.format_question(q) == "2 + 2 = ?\nA) 3\nB) 4\nC) 5\nD) \nAnswer:"
    assert [ev.extract_answer(s) for s in (" b) four", "D", "4", "")] == [1, 3, None, None]
    assert B.McEvaluator.with_template("Q: {question} [{a}|{b}]").format_question(q) == "Q: 2 + 2 = ? [3|4]"
    ds = B.McDataset("m", [q, B.MultipleChoiceQuestion("2", "x", ["a", "b"], 0, "law")])
    r = ev.evaluate_dataset(ds, ["B", "B"])
    assert (r.correct, r.total) == (1, 2) and r.by_group == {"math": (1, 1), "law": (0, 1)} and B.accuracy_pct(r) == 50.0
    lr = B.McLogitEvaluator.score([-3.0, -1.0, -2.5], 1)
    assert lr.predicted == 1 and lr.correct and lr.margin == pytest.approx(1.5)
    assert B.McLogitEvaluator().evaluate_dataset(ds, [[0, 1, 0], [0, 1]]).correct == 1
    mm = B.MmluEvaluator().evaluate_by_subject_completions(ds, ["B", "A"])
    assert mm.accuracy_pct == 100.0 and mm.by_subject["math"].total == 1 and B.MmluEvaluator().evaluate_by_subject_logits(ds, [[1, 0, 0], [1, 0]]).correct == 1
    arc = B.ArcEvaluator.challenge().evaluate_completions(ds, ["b", "b"])
    assert arc.split_name() == "ARC-Challenge" and arc.accuracy_pct() == 50.0 and B.ArcEvaluator.easy().split() == "ARC-Easy"
    em = B.ExactMatchEvaluator()
    assert em.score("  Paris ", "paris") and not B.ExactMatchEvaluator(case_sensitive=True).score("Paris", "paris")
    eds = B.EvalDataset("e", [B.EvalExample("1", "capital?", "Paris"), B.EvalExample("2", "x", None)])
    assert em.evaluate_dataset(eds, ["paris", "anything"]).correct == 1
    hs = B.HellaSwagDataset.from_jsonl(json.dumps({"ind": 7, "activity_label": "cooking", "ctx_a": "She takes a pan", "ctx_b": "and", "endings": ["a", "bbbb", "c", "d"], "label": 1}))
    he = B.HellaSwagEvaluator()
    assert hs.items[0].ctx == "She takes a pan and" and he.evaluate_completions(hs, ["B."]).correct == 1
    assert he.evaluate_logits(hs, [[-1.0, -2.0, -3.0, -4.0]]).correct == 0 and he.evaluate_logits(hs, [[-1.0, -2.0, -3.0, -4.0]], length_normalize=True).correct == 1
    wg = B.WinoGrandeDataset.from_items([B.WinoGrandeItem("The trophy did not fit the case because _ was too big.", "the trophy", "the case", 1)])
    we = B.WinoGrandeEvaluator()
    assert we.build_prompt(wg.items[0]).endswith("A) the trophy\nB) the case\nAnswer:") and "because the case was" in we.fill(wg.items[0], 2)
    assert we.evaluate_completions(wg, ["A"]).correct == 1 and we.evaluate_logits(wg, [[0.1, 0.9]]).correct == 0
    bq = B.BoolQDataset.from_items([B.BoolQItem("p", "is it", True), B.BoolQItem("p", "is it", False), B.BoolQItem("p", "q", True)])
    be = B.BoolQEvaluator()
    assert be.build_prompt(bq.items[0]) == "Passage: p\nQuestion: is it\nAnswer:"
    assert [be.extract_answer(s) for s in ("Yes, it is", "  NO.", "nope", "y", "maybe")] == [True, False, False, None, None]
    res = be.evaluate_completions(bq, ["yes", "No", "unsure"])
    assert (res.correct, res.total, res.yes_predicted, res.no_predicted) == (2, 3, 1, 1)
    assert be.evaluate_logits(bq, [(1.0, 0.0), (0.0, 1.0), (0.0, 1.0)]).correct == 2
    tq = B.TruthfulQaDataset.from_jsonl(json.dumps({"question": "q", "mc1_targets": {"choices": ["t", "f1", "f2"], "labels": [1, 0, 0]},
                                                    "mc2_targets": {"choices": ["t1", "t2", "f"], "labels": [1, 1, 0]}}))
    assert B.TruthfulQaEvaluator.mc1().evaluate_logits(tq, [[2.0, 1.0, 0.0]]).accuracy == 1.0
    mc2 = B.TruthfulQaEvaluator.mc2().evaluate_logits(tq, [[0.0, 0.0, 0.0]])
    assert mc2.accuracy == pytest.approx(2 / 3) and mc2.correct == 1 and mc2.mode == "mc2"
    assert B.TruthfulQaEvaluator.mc2().evaluate_logits(tq, [[0.0]]).accuracy == 0.0                   # wrong row length scores nothing
    g = B.Gsm8kAnswerEvaluator()
    assert [g.extract_final_answer(s) for s in ("so #### 1,234", "#### 3 then #### -5.5 apples", "no marker", "#### x")] == [1234.0, -5.5, None, None]
    gd = B.EvalDataset("g", [B.gsm8k_example("q", "think", 42), B.gsm8k_example("q", "think", 7), B.gsm8k_example("q", "t", 1)])
    gr = g.evaluate_dataset(gd, ["#### 42", "#### 8", "I do not know"])
    assert (gr.correct, gr.total, gr.no_answer_extracted) == (1, 3, 1) and gr.no_answer_rate() == pytest.approx(1 / 3) and gr.accuracy_pct() == pytest.approx(100 / 3)


def test_throughput_perplexity_and_report():
    assert B.percentile([1, 2, 3, 4], 50) == 2.5 and B.percentile([], 50) == 0.0 and B.percentile([5], 99) == 5 and B.percentile([1, 2, 3, 4], 200) == 4
    out, dt = B.time_fn(lambda: 7)
    assert out == 7 and dt >= 0
    st = B.ThroughputRuns.from_timings([(10.0, 1000.0, 100), (14.0, 500.0, 100)])
    assert st.tokens_per_second == pytest.approx(200 / 1.5) and st.prefill_ms == 12.0 and st.decode_ms_per_token == 7.5 and st.runs == 2
    assert (st.min_tps, st.max_tps, st.p50_tps) == (100.0, 200.0, 150.0) and st.meets_target(130) and not st.meets_target(140)
    assert st.summary().startswith("Throughput: 133.3 t/s") and st.latency_breakdown() == "Prefill: 12.00 ms | Decode: 7.500 ms/token"
    assert B.ThroughputRuns.from_timings([]).runs == 0
    calls = []
    m = B.ThroughputRuns().with_warmup(2).with_runs(3).measure(lambda: calls.append(1) or (1.0, 10.0, 10))
    assert len(calls) == 5 and m.runs == 3 and m.tokens_per_second == pytest.approx(1000.0)
    lp = [math.log(0.25)] * 8
    assert B.perplexity_from_log_probs(lp) == pytest.approx(4.0) and B.perplexity_from_log_probs([]) == float("inf")
    assert B.perplexity_from_log_probs([math.log(0.5)] * 2 + [math.log(0.01)] * 9, max_length=2) == pytest.approx(2.0)
    assert B.bits_per_byte(lp, 4) == pytest.approx(8 * 2 / 4) and B.bits_per_byte(lp, 0) == float("inf")
    assert B.perplexity_batch([[math.log(0.5)] * 3, [math.log(0.125)]]) == pytest.approx(2 ** 1.5)
    assert B.perplexity_from_logits([[0.0, 0.0], [0.0, 0.0, 0.0, 0.0]], [1, 2]) == pytest.approx(math.sqrt(8))
    rep = B.EvalSuiteReport("bonsai").add_perplexity("wikitext", 12.5, tokens=1000).add_throughput("decode", st)
    from oxibonsai_b200.eval import AccuracyResult
    rep.add_accuracy("mmlu", AccuracyResult(3, 4))
    doc = json.loads(rep.to_json())
    assert doc["model"] == "bonsai" and [r["task"] for r in doc["results"]] == ["wikitext", "decode", "mmlu"] and doc["results"][2]["value"] == 0.75
    assert "| mmlu | accuracy | 0.7500 |" in rep.to_markdown() and "wikitext perplexity 12.5" in rep.summary()
    assert B.EvalSuiteReport("x").summary() == "x: no results"


def test_bit_parallel_lcs_equals_the_dynamic_programme():
    import random
    from oxibonsai_b200.eval import _lcs
    from oxibonsai_b200.eval.suite import lcs_length

    def table(a, b):
        row = [0] * (len(b) + 1)
        for x in a:
            prev = 0
            for j, y in enumerate(b, 1):
                cur = row[j]
                row[j] = prev + 1 if x == y else max(row[j], row[j - 1])
                prev = cur
        return row[-1]
    rng = random.Random(2)
    for _ in range(200):
        a = [rng.choice("abcde") for _ in range(rng.randrange(0, 70))]
        b = [rng.choice("abcdef") for _ in range(rng.randrange(0, 130))]          # past one machine word
        assert _lcs(a, b) == table(a, b) == lcs_length(a, b)
    assert _lcs([], ["a"]) == 0 and _lcs(["a"], ["a"]) == 1 and _lcs("abc", "xyz") == 0
