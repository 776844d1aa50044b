"""Core layer: GGUF container, block codecs, model config, CPU oracle."""
from .gguf import (GgufFile, GgufWriter, GgufStreamParser, Qwen3Config, TensorInfo, type_info, data_size,
                   F32, F16, BF16, Q4_0, Q8_0, TQ2_0, Q1_0_G128, TQ2_0_G128, F8_E4M3, F8_E5M2)
from .blocks import dequantize, quantize
from .oracle import Oracle, write_synthetic_gguf, EOS_TOKEN
