"""The example scripts that need no GPU run to completion on small inputs."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, *args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script), *args], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    return r.stdout


def test_metrics_demo():
    out = _run("metrics_demo.py")
    assert "requests 3" in out and "oxibonsai_tokens_generated_total 48" in out


def test_gguf_dump(tmp_path):
    from oxibonsai_b200.core import Qwen3Config, write_synthetic_gguf
    path = str(tmp_path / "m.gguf")
    write_synthetic_gguf(path, Qwen3Config(hidden=256, inter=512, layers=1, heads=2, kv_heads=1, head_dim=128, vocab=300, context=64, name="ex"), seed=1)
    out = _run("gguf_dump.py", path)
    assert "GGUF v3" in out and "general.architecture = 'qwen3'" in out and "token_embd.weight" in out


def test_every_example_compiles():
    import py_compile
    for name in sorted(os.listdir(os.path.join(ROOT, "examples"))):
        if name.endswith(".py"):
            py_compile.compile(os.path.join(ROOT, "examples", name), doraise=True)


def test_onnx_inspect_and_convert(tmp_path):
    import numpy as np
    from test_cli_convert import _attr_i, _ld, _node, _tensor, _vi
    rng = np.random.default_rng(0)
    K, N, bs = 256, 128, 128
    q = rng.integers(1, 4, size=(N, K // bs, bs)).astype(np.uint8)
    packed = (q[:, :, 0::4] | (q[:, :, 1::4] << 2) | (q[:, :, 2::4] << 4) | (q[:, :, 3::4] << 6)).astype(np.uint8)
    scales = rng.uniform(0.01, 0.03, size=N * K // bs).astype(np.float32)
    nm = "/model/layers.0/attn/q_proj/MatMulNBits"
    graph = _ld(1, _node(nm, "MatMulNBits", ["x", nm + ".B", nm + ".scales"], ["y"], _attr_i("K", K) + _attr_i("N", N) + _attr_i("bits", 2) + _attr_i("block_size", bs)))
    graph += _ld(5, _tensor(nm + ".B", packed, 2)) + _ld(5, _tensor(nm + ".scales", scales, 1)) + _ld(2, b"example-graph")
    graph += _ld(5, _tensor("model.embed_tokens.weight", rng.normal(size=(50, K)).astype(np.float16), 10))
    src = tmp_path / "m.onnx"
    src.write_bytes(_vi((1 << 3) | 0) + _vi(8) + _ld(7, graph))
    out = _run("onnx_inspect.py", str(src))
    assert "example-graph" in out and "MatMulNBits" in out
    dst = tmp_path / "m.gguf"
    out = _run("onnx_convert.py", str(src), str(dst))
    assert "tensors written" in out and dst.stat().st_size > 0
