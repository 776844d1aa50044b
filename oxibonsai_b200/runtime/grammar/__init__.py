"""Grammar engine: AST, BNF / GBNF parsers, Earley recogniser, regex and JSON-Schema compilers, canned grammars.

Reference: crates/oxibonsai-runtime/src/grammar/ (ast.rs, bnf_parser.rs, gbnf_parser.rs, earley.rs, regex_compiler.rs,
json_schema_compiler.rs, constraint.rs, cache.rs, examples.rs).  The token-level constraint built on top of it is
``oxibonsai_b200.runtime.constrained.GrammarConstraint``.
"""
from .ast import Grammar, GrammarError, NonTerm, Rule, Term, parse_bnf, parse_gbnf
from .compilers import (arithmetic_grammar, identifier_list_grammar, json_grammar, json_schema_to_grammar, regex_to_grammar,
                        yes_no_grammar)
from .earley import EarleyRecognizer
from .regex_compiler import Dfa, RegexError, compile_regex, regex_to_nfa, nfa_to_dfa
