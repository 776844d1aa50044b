"""Summarise an ONNX graph: operator counts and the MatMulNBits nodes a ternary export consists of
(reference: crates/oxibonsai-model/examples/onnx_inspect.rs)."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.convert.onnx import inspect_onnx

info = inspect_onnx(sys.argv[1])
print(f"graph {info['graph']!r}: {info['nodes']} nodes, {info['initializers']} initializers")
for op, n in sorted(info["ops"].items(), key=lambda kv: -kv[1]):
    print(f"  {op:<24} {n}")
print(json.dumps(info["matmul_nbits"][:8], indent=1))
