"""Print a model card and a compatibility report for a GGUF file (reference: examples/model_info.rs, gguf_dump)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.core import GgufFile
from oxibonsai_b200.core.compat import build_compat_report, extract_model_card

path = sys.argv[1]
f = GgufFile.open(path)
print(extract_model_card(f, os.path.getsize(path)).to_markdown())
print(build_compat_report(f).summary())
for t in f.tensors[:12]:
    print(f"{t.name:<40} {t.type_name:<12} {tuple(t.dims)}")
