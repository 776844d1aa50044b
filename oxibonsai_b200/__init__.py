"""oxibonsai_b200: a Blackwell-native sub-2-bit LLM inference engine.

PyTorch is the tensor/stream/allocator layer; every hot op is a hand-written sm_100a CUDA kernel
in ``csrc/cuda`` and ``csrc/comm``; the host runtime is C++ in ``csrc/core``, ``csrc/cpu`` and
``csrc/runtime``.
"""
__version__ = "0.1.0"
