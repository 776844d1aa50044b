"""Host-side decoding machinery: advanced samplers, beam / n-best search, constrained decoding, grammars, JSON schema."""
import json

import numpy as np
import pytest

from oxibonsai_b200.runtime import sampling_advanced as SA
from oxibonsai_b200.runtime.presets import SamplingParams


def _logits(seed=0, n=64):
    return np.random.default_rng(seed).normal(size=n) * 3.0


def test_basic_probability_helpers():
    x = _logits()
    p = SA.softmax(x)
    assert abs(p.sum() - 1.0) < 1e-12 and np.allclose(np.exp(SA.log_softmax(x)), p)
    assert SA.entropy(np.full(8, 1 / 8)) == pytest.approx(np.log(8))
    assert SA.perplexity([np.log(0.25)] * 5) == pytest.approx(4.0)
    assert list(SA.top_k_indices(np.array([0.1, 5.0, 3.0, 4.0]), 2)) == [1, 3]
    y = SA.apply_repetition_penalty(np.array([2.0, -2.0, 1.0]), [0, 1], 2.0)
    assert list(y) == [1.0, -4.0, 1.0]
    z = SA.apply_frequency_presence_penalty(np.zeros(3), [1, 1, 2], frequency=0.5, presence=1.0)
    assert list(z) == [0.0, -2.0, -1.5]
    a, b = SA.LcgRng(7), SA.LcgRng(7)
    assert [a.next_u64() for _ in range(4)] == [b.next_u64() for _ in range(4)] and 0.0 <= a.next_f32() < 1.0


def test_filters_keep_expected_sets():
    x = np.log(np.array([0.5, 0.25, 0.125, 0.0625, 0.0625]))
    assert list(SA.MinPSampler(0.3).filter(x)) == [True, True, False, False, False]
    assert SA.TypicalSampler(0.5).filter(x).sum() >= 1
    assert SA.EtaSampler(0.2).filter(x)[0]
    rng = SA.LcgRng(1)
    draws = [SA.MinPSampler(0.3).sample(x, rng) for _ in range(200)]
    assert set(draws) <= {0, 1} and 0 in draws and 1 in draws


def test_mirostat_tracks_target_surprise():
    rng = SA.LcgRng(3)
    for sampler in (SA.MirostatV2(tau=2.0, eta=0.2), SA.MirostatV1(tau=2.0, eta=0.2, m=32)):
        surprises = []
        for i in range(300):
            x = _logits(i, 128)
            t = sampler.sample(x, rng)
            surprises.append(-np.log2(SA.softmax(x)[t]))
        assert 0.5 < np.mean(surprises[100:]) < 4.5
        sampler.reset()
        assert sampler.mu == pytest.approx(4.0)


def test_sampler_chain_presets_and_greedy_tie_rule():
    assert SA.SamplerChain.greedy().sample(np.array([1.0, 3.0, 3.0, 0.0])) == 2      # last index among ties
    c1, c2 = SA.SamplerChain.default_chat(5), SA.SamplerChain.default_chat(5)
    xs = [_logits(i) for i in range(20)]
    assert [c1.sample(x) for x in xs] == [c2.sample(x) for x in xs]
    top1 = SA.SamplerChain(0).add("top_k", 1)
    assert all(top1.sample(x) == int(np.argmax(x)) for x in xs)
    assert len(SA.SamplerChain.creative().steps) == 3 and SA.SamplerChain.precise().steps[0].kind == "repetition_penalty"


def test_adaptive_strategies():
    st = SA.GenerationState()
    for i in range(40):
        st.update(i % 3, 4.0)
    assert st.recent_repetition_rate(30) > 0.8 and st.mean_recent_entropy() == pytest.approx(4.0)
    base = SamplingParams(temperature=0.8, repetition_penalty=1.1)
    chain = SA.AdaptiveSamplerChain().add(SA.EntropyCooling(target_entropy=2.0)).add(SA.RepetitionAdaptation())
    p = chain.adjust(st, base)
    assert p.temperature != base.temperature and p.repetition_penalty > base.repetition_penalty and len(chain) == 2
    d = SA.ScheduledDecay(1.0, 0.2, 100)
    assert d.temperature_at_step(0) == 1.0 and d.temperature_at_step(50) == pytest.approx(0.6) and d.temperature_at_step(500) == 0.2


# ---- beam / n-best -----------------------------------------------------------------------------------------------------------------
def _markov(n=6, seed=1):
    T = np.random.default_rng(seed).normal(size=(n, n)) * 2.0
    return lambda toks: T[toks[-1] % n]


def test_beam_search_beats_greedy_and_respects_ngram_ban():
    from oxibonsai_b200.runtime.beam import BeamSearchConfig, BeamSearchEngine, apply_no_repeat_ngram, top_k_log_probs
    fn = _markov()
    cfg = BeamSearchConfig(beam_width=4, max_length=6, length_penalty=0.0, early_stopping=False)
    res = BeamSearchEngine(cfg).search([0], fn)
    greedy = BeamSearchEngine(BeamSearchConfig(beam_width=1, max_length=6, length_penalty=0.0)).search([0], fn)
    assert len(res.best()) == 6 and res.best_score() >= greedy.best_score() - 1e-9
    assert len(res.beams) == 4 and res.beams[0].log_prob >= res.beams[-1].log_prob
    banned = apply_no_repeat_ngram(np.zeros(6), [1, 2, 3, 1, 2], 3)
    assert banned[3] == -np.inf and np.isfinite(banned[0])
    lp = top_k_log_probs(np.array([0.0, 1.0, 2.0]), 2)
    assert [t for t, _ in lp] == [2, 1] and lp[0][1] < 0
    eos = BeamSearchEngine(BeamSearchConfig(beam_width=2, max_length=8, eos_token=int(np.argmax(fn([0]))))).search([0], fn)
    assert eos.beams[0].finished or len(eos.best()) <= 8


def test_nbest_list_and_decoder():
    from oxibonsai_b200.runtime.beam import Hypothesis, NBestDecoder, NBestList
    l = NBestList(2)
    for lp in (-3.0, -1.0, -2.0, -5.0):
        l.push(Hypothesis([1], lp))
    assert [h.log_prob for h in l.into_sorted()] == [-1.0, -2.0] and l.is_full() and l.worst_score() == -2.0 and l.top().log_prob == -1.0
    hyps = NBestDecoder(3, eos_id=5, max_len=5).decode([0], _markov())
    assert len(hyps) == 3 and hyps[0].score() >= hyps[1].score() >= hyps[2].score()
    done, live = NBestDecoder.partition(hyps)
    assert len(done) + len(live) == 3


# ---- regex / grammar -----------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("pattern,good,bad", [
    (r"[a-z]+@[a-z]+\.(com|org)", ["ab@cd.com", "x@y.org"], ["ab@cd.net", "@cd.com", "ab@cd.co"]),
    (r"\d{3}-\d{4}", ["555-1234"], ["5555-1234", "555-123", "abc-defg"]),
    (r"(ab|cd)*e?", ["", "ab", "abcde", "e"], ["a", "abce e", "ea"]),
    (r"[^0-9]{2,3}", ["ab", "abc"], ["a", "abcd", "a1"]),
    (r"h.llo\x21", ["hello!", "hxllo!"], ["h\nllo!", "hello"]),
    ("é+", ["é", "éé"], ["e", "è"]),
])
def test_regex_compiler(pattern, good, bad):
    from oxibonsai_b200.runtime.grammar import compile_regex, regex_to_grammar, EarleyRecognizer
    dfa = compile_regex(pattern)
    g = EarleyRecognizer(regex_to_grammar(pattern))
    for s in good:
        assert dfa.matches(s.encode()) and g.accepts(s.encode()), s
    for s in bad:
        assert not dfa.matches(s.encode()) and not g.accepts(s.encode()), s


def test_regex_errors_and_state_bound():
    from oxibonsai_b200.runtime.grammar import RegexError, compile_regex
    for bad in ("(ab", "a{3,2}", "*a", "[a-"):
        with pytest.raises(RegexError):
            compile_regex(bad)
    with pytest.raises(RegexError):
        compile_regex("(a|b)*a(a|b){14}", max_states=256)     # classic exponential blow-up


def test_gbnf_json_grammar_and_next_bytes():
    from oxibonsai_b200.runtime.grammar import EarleyRecognizer, json_grammar, arithmetic_grammar, parse_gbnf, GrammarError
    rec = EarleyRecognizer(json_grammar())
    for doc in ('{"a": [1, 2.5e3, true, null], "b": {"c": "x\\n\\u00e9"}}', "[]", ' "s" ', "-0.5"):
        assert rec.accepts(doc.encode()), doc
    for doc in ('{"a": }', "[1,]", "01", '{"a" 1}', '"unterminated'):
        assert not rec.accepts(doc.encode()), doc
    r = EarleyRecognizer(json_grammar())
    assert r.feed_bytes(b'{"k"')
    assert r.next_bytes() == frozenset(b" \t\n\r:")
    f = r.fork()
    assert f.feed_bytes(b': 1}') and f.is_complete() and not r.is_complete() and r.position == 4
    assert not r.feed(ord("x")) and r.dead
    ar = EarleyRecognizer(arithmetic_grammar())
    assert ar.accepts(b"(1 + 2.5) * 3") and not ar.accepts(b"(1 + ) * 3")
    with pytest.raises(GrammarError):
        parse_gbnf('root ::= missing "a"')
    g = parse_gbnf('root ::= item{2,3}\nitem ::= [a-c] | "zz"\n# trailing comment\n')
    r2 = EarleyRecognizer(g)
    assert r2.accepts(b"ab") and r2.accepts(b"azzc") and not r2.accepts(b"a") and not r2.accepts(b"abcd")
    assert g.first_sets()["root"] == frozenset(b"abcz")


def test_bnf_parser():
    from oxibonsai_b200.runtime.grammar import EarleyRecognizer, parse_bnf
    g = parse_bnf('<expr> ::= <term> "+" <expr> | <term>\n<term> ::= "x" | "y" | "(" <expr> ")"\n')
    r = EarleyRecognizer(g)
    assert r.accepts(b"x+(y+x)") and not r.accepts(b"x+") and g.start == "expr"


def test_json_schema_grammar_validator_and_generators():
    from oxibonsai_b200.runtime.grammar import EarleyRecognizer, json_schema_to_grammar
    from oxibonsai_b200.runtime import json_schema as JS
    schema = {"type": "object", "required": ["name", "age"],
              "properties": {"name": {"type": "string", "minLength": 1}, "age": {"type": "integer", "minimum": 0},
                             "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "maxItems": 2},
                             "id": {"type": "string", "pattern": "[A-Z]{2}[0-9]+"}}}
    rec = EarleyRecognizer(json_schema_to_grammar(schema))
    good = ['{"name": "bo", "age": 3}', '{"name":"x","age":10,"tags":["a","b"]}', '{"name": "x", "age": 0, "id": "AB12"}']
    bad = ['{"age": 3, "name": "bo"}', '{"name": "", "age": 3}', '{"name": "x", "age": 1.5}', '{"name": "x", "age": 1, "tags": ["c"]}',
           '{"name": "x", "age": 1, "tags": ["a","a","a"]}', '{"name": "x"}']
    for d in good:
        assert rec.accepts(d.encode()), d
        assert JS.validate_against_schema(d, schema)
    for d in bad:
        assert not rec.accepts(d.encode()), d
    assert not JS.validate_against_schema('{"name": "x", "age": -1}', schema)
    s = JS.parse_schema(schema)
    assert s.is_required_property("age") and not s.is_required_property("tags") and s.type_name() == "object"
    ex = JS.schema_example(s)
    assert not JS.validate_value(ex, s), ex
    assert '"name": <string>' in JS.schema_template(s)
    st = JS.SchemaState(schema)
    assert st.feed('{"name": "a') and '"' in st.valid_next_chars() and st.depth() == 1 and not st.is_complete()
    assert st.feed('", "age": 7}') and st.is_complete() and st.buffer().endswith("7}")
    with pytest.raises(JS.SchemaError):
        JS.parse_schema({"type": "object", "required": ["zz"], "properties": {}})


# ---- token-level constraints ---------------------------------------------------------------------------------------------------------
def _table():
    from oxibonsai_b200.runtime.constrained import TokenTable
    toks = [bytes([b]) for b in range(256)] + [b"true", b"false", b"null", b'{"', b'":', b", ", b"12", b"ab", b"", b"\xc3\xa9"]
    return TokenTable(toks)


def test_dfa_constraint_masks_and_cache():
    from oxibonsai_b200.runtime.constrained import DfaConstraint, mask_to_bool
    t = _table()
    eos = 264          # the empty token doubles as EOS here
    c = DfaConstraint.from_regex(t, r"(true|false)(, (true|false))*", eos_token=eos)
    allowed = mask_to_bool(c.allowed_mask(), t.n)
    assert set(np.flatnonzero(allowed)) == {ord("t"), ord("f"), 256, 257}
    assert c.advance(256) and c.is_complete()
    allowed = mask_to_bool(c.allowed_mask(), t.n)
    assert set(np.flatnonzero(allowed)) == {ord(","), 261, eos}
    assert c.advance(261) and not c.is_complete() and c.advance(ord("f")) and not c.advance(ord("x"))
    c.reset()
    c.allowed_mask()
    assert c.cache_hits >= 1


def test_grammar_constraint_drives_sampler_to_valid_json():
    from oxibonsai_b200.runtime.constrained import ConstrainedSampler, GrammarConstraint, json_schema_constraint
    t = _table()
    eos = 264
    schema = {"type": "object", "required": ["ok", "n"], "properties": {"ok": {"type": "boolean"}, "n": {"type": "integer", "maximum": 99}}}
    c = json_schema_constraint(t, schema, eos_token=eos)
    rng = np.random.default_rng(0)
    out = bytearray()

    def pick(logits):
        ok = np.flatnonzero(np.isfinite(logits))
        # prefer EOS once the document is complete, otherwise a random allowed token
        return eos if eos in ok and rng.random() < 0.5 else int(rng.choice(ok[ok != eos]) if (ok != eos).any() else eos)
    s = ConstrainedSampler(c, pick, t.n)
    for _ in range(200):
        tok = s.sample(np.zeros(t.n))
        if tok == eos:
            break
        out += t.tokens[tok]
    doc = json.loads(out.decode())
    assert isinstance(doc["ok"], bool) and isinstance(doc["n"], int) and s.masked_steps > 0
    assert isinstance(s.gpu_mask(), np.ndarray) and s.gpu_mask().dtype == np.uint32


def test_simple_constraints_and_intersection():
    from oxibonsai_b200.runtime.constrained import (AllOf, AllowListConstraint, ConstrainedSampler, ConstraintViolation, LengthConstraint,
                                                     NoConstraint, SequenceConstraint, mask_to_bool)
    t = _table()
    assert NoConstraint().allowed_mask() is None and NoConstraint().is_complete()
    al = AllowListConstraint(t, [1, 5, 300])        # 300 is outside the table and ignored by the mask
    assert set(np.flatnonzero(mask_to_bool(al.allowed_mask(), t.n))) == {1, 5}
    sq = SequenceConstraint(t, [7, 8])
    assert not sq.is_complete() and sq.advance(7) and not sq.advance(9) and sq.advance(8) and sq.is_complete() and sq.allowed_mask() is None
    ln = LengthConstraint(t, eos_token=264, min_tokens=2, max_tokens=3)
    assert not mask_to_bool(ln.allowed_mask(), t.n)[264]
    ln.advance(1), ln.advance(1)
    assert ln.allowed_mask() is None and ln.is_complete()
    ln.advance(1)
    assert set(np.flatnonzero(mask_to_bool(ln.allowed_mask(), t.n))) == {264}
    both = AllOf(AllowListConstraint(t, [1, 2, 3]), AllowListConstraint(t, [3, 4]))
    assert set(np.flatnonzero(mask_to_bool(both.allowed_mask(), t.n))) == {3}
    s = ConstrainedSampler(AllOf(AllowListConstraint(t, [1]), AllowListConstraint(t, [2])), lambda x: 0, t.n)
    with pytest.raises(ConstraintViolation):
        s.sample(np.zeros(t.n))


def test_finished_is_asked_for_by_bounded_constraints_only():
    """``is_complete`` says a stop is valid, ``finished`` says the generation has to end: engines end a sequence on the
    latter, so an always-terminal constraint (allow-list, length window) must never report it."""
    from oxibonsai_b200.runtime.constrained import AllOf, AllowListConstraint, DfaConstraint, LengthConstraint, NoConstraint, SequenceConstraint
    t = _table()
    assert not NoConstraint().finished()
    al = AllowListConstraint(t, [1, 5])
    assert al.is_complete() and not al.finished() and al.advance(5) and not al.finished()
    ln = LengthConstraint(t, eos_token=264, min_tokens=0, max_tokens=2)
    assert ln.is_complete() and not ln.finished()
    sq = SequenceConstraint(t, [7, 8])
    assert not sq.finished() and sq.advance(7) and not sq.finished() and sq.advance(8) and sq.finished()
    # "true" can be followed by ", true": accepting but extendable; "(ab)" has nothing after its match
    ext = DfaConstraint.from_regex(t, r"(true|false)(, (true|false))*", eos_token=264)
    assert ext.advance(256) and ext.is_complete() and not ext.finished()
    end = DfaConstraint.from_regex(t, r"ab", eos_token=264)
    assert not end.finished() and end.advance(263) and end.is_complete() and end.finished()
    both = AllOf(AllowListConstraint(t, [7, 8]), SequenceConstraint(t, [7]))
    assert not both.finished() and both.advance(7) and both.finished()


WEATHER = {"type": "function", "function": {"name": "get_weather", "description": "current weather",
                                            "parameters": {"type": "object", "required": ["city"],
                                                           "properties": {"city": {"type": "string", "maxLength": 12}, "celsius": {"type": "boolean"}}}}}
CLOCK = {"type": "function", "function": {"name": "get_time", "parameters": {"type": "object", "properties": {"tz": {"enum": ["UTC", "JST"]}}}}}


def test_tool_selection_validation_and_errors():
    from oxibonsai_b200.runtime import tools as T
    call = T.select_tool('I will check. {"name": "get_weather", "arguments": {"city": "Kyoto"}}', [WEATHER, CLOCK])
    assert call["id"].startswith("call_") and len(call["id"]) == 29 and call["type"] == "function"
    assert call["function"]["name"] == "get_weather" and json.loads(call["function"]["arguments"]) == {"city": "Kyoto"}
    assert T.make_tool_call("call_x", "f", {"a": 1}) == {"id": "call_x", "type": "function", "function": {"name": "f", "arguments": '{"a": 1}'}}
    with pytest.raises(T.NoToolCallFound):
        T.select_tool("no call here", [WEATHER])
    with pytest.raises(T.UnknownTool, match="unknown tool: 'launch'"):
        T.select_tool('{"name": "launch", "arguments": {}}', [WEATHER])
    assert T.select_tool('{"name": "launch", "arguments": {}}', [])["function"]["name"] == "launch"      # no list: any name passes
    with pytest.raises(T.MalformedArguments):
        T.select_tool('{"name": "get_weather", "arguments": "{not json"}', [WEATHER])
    reg = T.ToolRegistry([WEATHER, CLOCK])
    assert len(reg) == 2 and set(reg.names()) == {"get_weather", "get_time"} and reg.get("get_time") is CLOCK and reg.get("x") is None
    assert not reg.is_empty() and T.ToolRegistry([]).is_empty() and "get_time" in reg
    assert T.validate_tool_arguments('{"city": "Nara", "extra": 1}', WEATHER) == {"city": "Nara", "extra": 1}
    for bad, why in (('{"celsius": true}', "missing required field 'city'"), ("[1]", "must be a JSON object"), ("{", "malformed")):
        with pytest.raises(T.MalformedArguments, match=why):
            T.validate_tool_arguments(bad, WEATHER)
    with pytest.raises(T.MalformedArguments):
        T.validate_tool_arguments('{"city": 5}', WEATHER, strict=True)                                      # wrong type: only the strict check sees it
    assert T.validate_tool_arguments('{"city": 5}', WEATHER) == {"city": 5}
    assert [e.kind for e in (T.NoToolCallFound(), T.UnknownTool("x"), T.MalformedArguments("r"), T.GrammarCompileError("r"), T.EmptyToolList())] == \
        ["NoToolCallFound", "UnknownTool", "MalformedArguments", "GrammarCompileError", "EmptyToolList"]
    assert T.tool_choice_names("auto", [WEATHER]) is None and T.tool_choice_names(None, [WEATHER]) is None
    assert T.tool_choice_names("required", [WEATHER, CLOCK]) == ["get_weather", "get_time"]
    assert T.tool_choice_names({"type": "function", "function": {"name": "get_time"}}, [WEATHER, CLOCK]) == ["get_time"]
    with pytest.raises(T.UnknownTool):
        T.tool_choice_names({"type": "function", "function": {"name": "nope"}}, [WEATHER])


def test_tool_constraint_only_admits_well_formed_calls():
    from oxibonsai_b200.runtime import tools as T
    from oxibonsai_b200.runtime.constrained import ConstrainedSampler
    with pytest.raises(T.EmptyToolList):
        T.build_tool_grammar([])
    t = _table()
    eos = 264
    rng = np.random.default_rng(1)
    seen = set()
    for trial in range(6):
        c = T.build_tool_constraint(t, [WEATHER, CLOCK], None if trial < 4 else ["get_time"], eos_token=eos)
        out = bytearray()

        def pick(logits):
            ok = np.flatnonzero(np.isfinite(logits))
            if eos in ok:
                return eos
            printable = [i for i in ok if i >= 256 or 32 <= i < 127]      # keep the random strings short and readable
            return int(rng.choice(printable if printable else ok))
        s = ConstrainedSampler(c, pick, t.n)
        for _ in range(400):
            tok = s.sample(np.zeros(t.n))
            if tok == eos:
                break
            out += t.tokens[tok]
        text = out.decode("utf-8", errors="replace")
        assert text.startswith('<tool_call>{"name":"get_') and text.endswith("}</tool_call>"), text
        call = T.select_tool(text, [WEATHER, CLOCK])
        tool = T.ToolRegistry([WEATHER, CLOCK]).get(call["function"]["name"])
        T.validate_tool_arguments(call["function"]["arguments"], tool, strict=True)
        seen.add(call["function"]["name"])
        if trial >= 4:
            assert call["function"]["name"] == "get_time"
    assert seen <= {"get_weather", "get_time"} and seen
    # the constraint refuses a call of a tool that is not in the list, byte by byte
    c = T.build_tool_constraint(t, [WEATHER], eos_token=eos)
    for b in b'<tool_call>{"name":"get_':
        assert c.advance(b)
    from oxibonsai_b200.runtime.constrained import mask_to_bool
    allowed = mask_to_bool(c.allowed_mask(), t.n)
    assert allowed[ord("w")] and not allowed[ord("t")] and allowed.sum() == 1
