"""Convert an ONNX export with MatMulNBits(bits=2) weights into a GGUF checkpoint this engine loads
(reference: crates/oxibonsai-model/examples/onnx_convert.rs).

    python examples/onnx_convert.py model.onnx model.gguf [tq2_0_g128 | q1_0_g128]
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from oxibonsai_b200.convert.onnx import convert_onnx_to_gguf

src, dst = sys.argv[1], sys.argv[2]
quant = sys.argv[3] if len(sys.argv) > 3 else "tq2_0_g128"
st = convert_onnx_to_gguf(src, dst, quant)
print(f"{st.tensors} tensors written ({st.skipped} skipped), {st.bytes_in} -> {st.bytes_out} bytes, tied embeddings: {st.tied}")
