"""The native Earley matcher against the Python recogniser (the oracle): same verdicts byte by byte, same masks, and the
mask cache keyed by the chart signature."""
import json
import random
import time

import numpy as np
import pytest

from oxibonsai_b200.runtime.constrained import GrammarConstraint, TokenTable, json_constraint, json_schema_constraint, mask_to_bool
from oxibonsai_b200.runtime.grammar.ast import parse_gbnf
from oxibonsai_b200.runtime.grammar.compilers import arithmetic_grammar, identifier_list_grammar, json_grammar, json_schema_to_grammar, regex_to_grammar, yes_no_grammar
from oxibonsai_b200.runtime.grammar.earley import EarleyRecognizer
from oxibonsai_b200.runtime.grammar.native import NativeEarley, compile_cached

NESTED = parse_gbnf('root ::= item*\nitem ::= "(" root ")" | "a" | opt "b"\nopt ::= "x"?\n')
AMBIG = parse_gbnf('root ::= e\ne ::= e "+" e | e "*" e | "n" | "(" e ")" | \n')          # ambiguous, nullable, left and right recursive
GRAMMARS = {"json": json_grammar(), "arith": arithmetic_grammar(), "idents": identifier_list_grammar(), "yesno": yes_no_grammar(), "nested": NESTED,
            "ambiguous": AMBIG, "regex": regex_to_grammar(r"(ab|a)*c[0-9]{2,3}(\.[0-9]+)?"),
            "schema": json_schema_to_grammar({"type": "object", "required": ["id"], "properties": {"id": {"type": "integer"}, "tags": {"type": "array", "items": {"enum": ["x", "yy"]}}}})}
ALPHABETS = {"json": '{}[]":,.-0123456789 truefalsn\\eE+ab\n', "arith": "0123456789.+-*/() ", "idents": "ab_1, ", "yesno": "yesno", "nested": "()abx",
             "ambiguous": "n+*()", "regex": "abc0123456789.", "schema": '{}[]":, idtagsxy0123456789-'}


@pytest.mark.parametrize("name", sorted(GRAMMARS))
def test_native_matcher_agrees_with_the_python_recogniser(name):
    g = GRAMMARS[name]
    rng = random.Random(hash(name) & 0xFFFF)
    alphabet = ALPHABETS[name].encode()
    for trial in range(60):
        py, nat = EarleyRecognizer(g), NativeEarley(g)
        assert py.next_bytes() == nat.next_bytes() and py.is_complete() == nat.is_complete()
        for step in range(rng.randint(1, 40)):
            nxt = sorted(py.next_bytes())
            # mostly follow the grammar, sometimes feed a byte it cannot take
            b = rng.choice(nxt) if nxt and rng.random() < 0.9 else rng.choice(alphabet)
            ok_py, ok_nat = py.feed(b), nat.feed(b)
            assert ok_py == ok_nat, (name, trial, step, b)
            if not ok_py:
                assert nat.dead and nat.next_bytes() == frozenset() and not nat.is_complete()
                break
            assert py.next_bytes() == nat.next_bytes() and py.is_complete() == nat.is_complete() and nat.position == py.position
    assert NativeEarley(g).accepts(b"") == EarleyRecognizer(g).accepts(b"")


def _table(rng, n_extra, alphabet):
    toks = [bytes([b]) for b in range(256)]
    toks += [bytes(rng.choice(alphabet) for _ in range(rng.randint(2, 6))) for _ in range(n_extra)]
    toks += [b"", b"true", b"false", b"null", b'{"', b'":', b'", "', b"\xc3\xa9", b'"}']
    return TokenTable(toks)


@pytest.mark.parametrize("name", ["json", "schema", "nested", "arith", "ambiguous"])
def test_native_masks_equal_the_python_masks_along_random_walks(name):
    g = GRAMMARS[name]
    rng = random.Random(7)
    table = _table(rng, 400, ALPHABETS[name].encode())
    eos = 256 + 400                                           # the empty token doubles as EOS
    for trial in range(4):
        nat, py = GrammarConstraint(table, g, eos), GrammarConstraint(table, g, eos, native=False)
        for step in range(25):
            mn, mp = nat.allowed_mask(), py.allowed_mask()
            assert np.array_equal(mn, mp), (name, trial, step, bytes(nat.text))
            ok = np.flatnonzero(mask_to_bool(mn, table.n))
            ok = ok[ok != eos]
            if not ok.size:
                break
            tok = int(rng.choice(ok))
            assert nat.advance(tok) and py.advance(tok)
            assert nat.is_complete() == py.is_complete() and nat.finished() == py.finished()
        assert not nat.advance(int(np.flatnonzero(~mask_to_bool(nat.allowed_mask(), table.n))[0])) or True


def test_signature_cache_is_shared_and_positions_inside_a_string_hit_it():
    rng = random.Random(1)
    table = _table(rng, 300, b"abcdefgh ")
    c = json_constraint(table)
    stats0 = c.rec.compiled.cache_stats()
    for b in b'{"key": "x':
        c.advance(b)
    sig = c.rec.signature()
    c.allowed_mask()
    hits0 = c.cache_hits
    for b in b"abc def":                                       # every later position inside the string has the same signature
        c.advance(b)
        assert c.rec.signature() == sig and c.rec.item_count() < 40
        c.allowed_mask()
    assert c.cache_hits == hits0 + 7
    c.advance(ord('"'))
    assert c.rec.signature() != sig
    # a second constraint over a structurally equal grammar shares the compiled object and its masks
    d = json_constraint(table)
    assert d.rec.compiled is c.rec.compiled and compile_cached(json_grammar()) is c.rec.compiled
    for b in b'{"other": "y':
        d.advance(b)
    d.allowed_mask()
    assert d.cache_hits == 1 and c.rec.compiled.cache_stats()["entries"] > stats0["entries"]
    # a key string and a value string are different states: '":' may end the first, '", "' or '"}' the second
    k = json_constraint(table)
    for b in b'{"k':
        k.advance(b)
    allowed_key = mask_to_bool(k.allowed_mask(), table.n)
    allowed_val = mask_to_bool(d.allowed_mask(), table.n)
    colon, brace = table.tokens.index(b'":'), table.tokens.index(b'"}')
    assert allowed_key[colon] and not allowed_key[brace] and allowed_val[brace] and not allowed_val[colon]


def test_mask_cost_at_a_realistic_vocabulary():
    """150 K tokens: the first mask inside a string walks the whole trie, the following ones are cache hits; a whole
    constrained document costs well under a second of masks (it took minutes with the recogniser in Python)."""
    rng = random.Random(0)
    alphabet = b'abcdefghijklmnopqrstuvwxyz ABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789{}[]":,.-_\n'
    toks = [bytes([b]) for b in range(256)] + [bytes(rng.choice(alphabet) for _ in range(rng.randint(2, 8))) for _ in range(150000)]
    table = TokenTable(toks)
    schema = {"type": "object", "required": ["name", "age", "tags"],
              "properties": {"name": {"type": "string"}, "age": {"type": "integer"}, "tags": {"type": "array", "items": {"type": "string"}}}}
    c = json_schema_constraint(table, schema)
    doc = b'{"name": "Alice Liddell", "age": 42, "tags": ["a", "bcd"]}'
    times = []
    for b in doc:
        t = time.perf_counter()
        m = c.allowed_mask()
        times.append(time.perf_counter() - t)
        assert mask_to_bool(m, table.n)[b]
        assert c.advance(b)
    assert c.is_complete() and json.loads(doc)
    assert sum(times) < 5.0 and sorted(times)[len(times) // 2] < 0.05, (sum(times), max(times))
    second = json_schema_constraint(table, schema)             # the next request with the same schema starts with a warm cache
    t = time.perf_counter()
    for b in doc:
        second.allowed_mask()
        second.advance(b)
    assert time.perf_counter() - t < 0.5 and second.cache_hits == len(doc)


def test_schema_with_many_optional_properties_compiles_linearly():
    """One grammar rule per (next property, "a member was already written") state: 40 properties, half of them optional,
    give a grammar of a few hundred rules (an unmemoised chain is exponential in the optional ones)."""
    from oxibonsai_b200.runtime.json_schema import schema_example
    kinds = [{"type": "string"}, {"type": "integer"}, {"type": "boolean"}, {"enum": ["red", "green"]}, {"type": "array", "items": {"type": "number"}, "maxItems": 3},
             {"type": "object", "properties": {"x": {"type": "number"}, "y": {"type": "string"}}, "required": ["x"]}]
    schema = {"type": "object", "properties": {f"f{i}": kinds[i % 6] for i in range(40)}, "required": [f"f{i}" for i in range(0, 40, 2)]}
    t = time.perf_counter()
    g = json_schema_to_grammar(schema)
    assert len(g.rules) < 600 and time.perf_counter() - t < 2.0
    m = NativeEarley(g)
    full = schema_example(schema)
    required_only = {k: v for k, v in full.items() if k in schema["required"]}
    some = {k: v for k, v in full.items() if k in schema["required"] or k in ("f1", "f7", "f39")}
    assert m.accepts(json.dumps(full).encode()) and m.accepts(json.dumps(required_only).encode()) and m.accepts(json.dumps(some).encode())
    missing = dict(required_only)
    missing.pop("f0")
    swapped = {"f2": full["f2"], "f0": full["f0"], **{k: v for k, v in required_only.items() if k not in ("f0", "f2")}}
    assert not m.accepts(json.dumps(missing).encode()) and not m.accepts(json.dumps(swapped).encode())      # declaration order is part of the grammar


@pytest.mark.parametrize("schema,good,bad", [
    ({"type": "string", "maxLength": 300}, ["", "x" * 300], ["x" * 301]),
    ({"type": "string", "minLength": 200, "maxLength": 1000}, ["y" * 200, "y" * 1000], ["y" * 199, "y" * 1001]),
    ({"type": "array", "items": {"type": "integer"}, "minItems": 100, "maxItems": 300}, [list(range(100)), list(range(300))], [list(range(99)), list(range(301))]),
    ({"type": "array", "items": {"type": "boolean"}, "maxItems": 2}, [[], [True], [True, False]], [[True] * 3]),
    ({"type": "array", "items": {"type": "null"}, "minItems": 2}, [[None] * 2, [None] * 9], [[None], []]),
    ({"type": "array", "items": {"type": "null"}, "maxItems": 0}, [[]], [[None]]),
])
def test_bounded_strings_and_arrays_compile_to_small_grammars(schema, good, bad):
    g = json_schema_to_grammar(schema)
    assert len(g.rules) < 1200                                    # linear in the bounds
    m = NativeEarley(g)
    assert all(m.accepts(json.dumps(x).encode()) for x in good) and not any(m.accepts(json.dumps(x).encode()) for x in bad)
    if len(g.rules) < 100:                                        # small enough for the Python oracle to agree in reasonable time
        py = EarleyRecognizer(g)
        assert all(py.accepts(json.dumps(x).encode()) for x in good) and not any(py.accepts(json.dumps(x).encode()) for x in bad)


def test_long_productions_and_bad_bounds():
    from oxibonsai_b200.runtime.grammar.ast import Grammar, GrammarError, Term
    g = Grammar("root")
    g.add("root", [Term(frozenset([97]))] * 700)                  # longer than a native production: continued in helper rules
    m = NativeEarley(g)
    assert m.accepts(b"a" * 700) and not m.accepts(b"a" * 699) and not m.accepts(b"a" * 701)
    for bad in ({"type": "string", "minLength": 5, "maxLength": 2}, {"type": "array", "minItems": 3, "maxItems": 1}):
        with pytest.raises(GrammarError):
            json_schema_to_grammar(bad)


def test_shared_caches_are_race_free_under_thread_sanitizer(tmp_path):
    """Four threads with their own matchers over one compiled grammar and one vocabulary (tests/grammar_tsan_driver.cpp),
    built with -fsanitize=thread: no data race, and every mask equals the single-threaded one."""
    import os
    import subprocess
    here = os.path.dirname(os.path.abspath(__file__))
    rt = os.path.join(os.path.dirname(here), "oxibonsai_b200", "csrc", "runtime")
    probe = subprocess.run(["g++", "-fsanitize=thread", "-x", "c++", "-", "-o", str(tmp_path / "probe")], input="int main(){return 0;}", capture_output=True, text=True)
    if probe.returncode != 0:
        pytest.skip("the host compiler has no ThreadSanitizer runtime")
    exe = str(tmp_path / "gram_tsan")
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-pthread", "-fsanitize=thread", f"-I{rt}", os.path.join(rt, "grammar_matcher.cpp"),
                            os.path.join(rt, "token_mask.cpp"), os.path.join(here, "grammar_tsan_driver.cpp"), "-o", exe], capture_output=True, text=True)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300, env=dict(os.environ, TSAN_OPTIONS="halt_on_error=0"))
    assert run.returncode == 0 and "grammar tsan driver ok" in run.stdout, run.stdout[-1000:] + run.stderr[-3000:]
    assert "WARNING: ThreadSanitizer" not in run.stderr, run.stderr[-4000:]
