"""Cost of the allowed-token mask of grammar constraints at a realistic vocabulary size (no GPU needed).

    python benchmarks/grammar_mask.py [--vocab 152000] [--python-oracle]

A synthetic vocabulary (256 byte tokens + random 2-8 character tokens) stands in for a 152 K-entry BPE table.  A JSON
document is pushed byte by byte through a JSON-schema constraint and a free-form JSON constraint; before every byte the
mask of allowed tokens is computed, as the engine does before every sampled token.  Reported per constraint: the first
pass over the document (cold cache) and a second constraint over the same schema (the masks of every grammar state are
cached in the compiled grammar).  ``--python-oracle`` also times the Python recogniser on the first bytes (it needs
seconds per mask at this size).  Prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np

from oxibonsai_b200.runtime.constrained import GrammarConstraint, TokenTable, json_constraint, json_schema_constraint, mask_to_bool
from oxibonsai_b200.runtime.grammar.compilers import json_schema_to_grammar

SCHEMA = {"type": "object", "required": ["name", "age", "tags"],
          "properties": {"name": {"type": "string"}, "age": {"type": "integer"}, "tags": {"type": "array", "items": {"type": "string"}}}}
DOC = b'{"name": "Alice Liddell", "age": 42, "tags": ["a", "bcd"]}'


def run(c, doc: bytes, n: int) -> dict:
    times = []
    for b in doc:
        t = time.perf_counter()
        m = c.allowed_mask()
        times.append(time.perf_counter() - t)
        assert mask_to_bool(m, n)[b]
        assert c.advance(b)
    ms = np.asarray(times) * 1e3
    return {"total_ms": round(float(ms.sum()), 2), "mean_ms": round(float(ms.mean()), 3), "p50_ms": round(float(np.median(ms)), 3), "max_ms": round(float(ms.max()), 2),
            "cache_hits": int(getattr(c, "cache_hits", 0)), "masks": len(doc)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--vocab", type=int, default=152000)
    ap.add_argument("--python-oracle", action="store_true")
    a = ap.parse_args()
    rng = random.Random(0)
    alphabet = 'abcdefghijklmnopqrstuvwxyz ABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789{}[]":,.-_\n'
    toks = [bytes([b]) for b in range(256)] + ["".join(rng.choice(alphabet) for _ in range(rng.randint(2, 8))).encode() for _ in range(a.vocab - 256)]
    t = time.perf_counter()
    table = TokenTable(toks)
    out = {"vocab": table.n, "table_build_s": round(time.perf_counter() - t, 3), "document_bytes": len(DOC)}
    for label, make in (("json_schema", lambda: json_schema_constraint(table, SCHEMA)), ("json_object", lambda: json_constraint(table))):
        out[label] = {"first_request": run(make(), DOC, table.n), "second_request": run(make(), DOC, table.n)}
    if a.python_oracle:
        py = GrammarConstraint(table, json_schema_to_grammar(SCHEMA), native=False)
        out["python_recogniser_first_12_bytes"] = run(py, DOC[:12], table.n)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
