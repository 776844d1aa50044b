"""Dump the header, metadata and tensor table of a GGUF file (reference: crates/oxibonsai-model/examples/gguf_dump.rs)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.core import GgufFile

path = sys.argv[1]
f = GgufFile.open(path)
print(f"{path}: GGUF v{f.version}, alignment {f.alignment}, {len(f.tensors)} tensors, {len(f.metadata)} metadata keys, "
      f"data at byte {f.data_offset} of {os.path.getsize(path)}")
for key, value in sorted(f.metadata.items()):
    text = repr(value)
    print(f"  {key} = {text if len(text) <= 90 else text[:87] + '...'}")
total = 0
for t in f.tensors:
    total += t.nbytes
    print(f"  {t.name:<44} {t.type_name:<12} {str(tuple(t.dims)):<22} {t.nbytes:>12} B at +{t.offset}")
print(f"tensor bytes: {total}")
