"""Constrained decoding: the sampler kernel only picks tokens that keep the output inside a JSON schema (needs a GPU).

    python examples/constrained_json.py model.gguf
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.runtime import EngineBuilder
from oxibonsai_b200.runtime.constrained import TokenTable, json_schema_constraint
from oxibonsai_b200.tokenizer import ByteTokenizer

engine = EngineBuilder().model_path(sys.argv[1]).preset("balanced").max_seq_len(512).build()
tok = ByteTokenizer()                                       # ids 0..255 are bytes; use the model's tokenizer for a real checkpoint
vocab = engine.config.vocab                                 # ids above 255 get bytes no JSON text contains, so the mask never allows them
table = TokenTable([tok.token_bytes(i) if i < 256 else b"\xff" for i in range(vocab)])
schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"}}, "required": ["name", "age"]}
constraint = json_schema_constraint(table, schema)
out = engine.generate(tok.encode("Describe a person as JSON: "), 96, constraint=constraint)
print(tok.decode(out))
