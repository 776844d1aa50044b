"""Command line helpers and the ONNX importer (CPU)."""
import json
import struct

import numpy as np
import pytest


def test_tokenizer_discovery_and_summary_line(tmp_path):
    from oxibonsai_b200 import cli
    assert cli.strip_quant_suffix("Ternary-Bonsai-8B-Q2_0") == "Ternary-Bonsai-8B" and cli.strip_quant_suffix("model-Q4_K_M") == "model"
    assert cli.strip_quant_suffix("model-F16") == "model" and cli.strip_quant_suffix("plain") == "plain"
    d = tmp_path / "models" / "x"
    d.mkdir(parents=True)
    m = d / "bonsai-8b-TQ2_0.gguf"
    m.write_bytes(b"")
    cands = cli.tokenizer_candidates(str(m))
    assert cands[0] == d / "tokenizer.json" and d / "bonsai-8b-unpacked" / "tokenizer.json" in cands and tmp_path / "models" / "tokenizer.json" in cands
    assert cli.resolve_tokenizer(str(m), None)[0] is None and "searched" in cli.no_tokenizer_warning(cands)
    (tmp_path / "models" / "tokenizer.json").write_text("{}")
    import os
    assert os.path.realpath(cli.resolve_tokenizer(str(m), None)[0]).endswith("models/tokenizer.json") and cli.resolve_tokenizer(str(m), "/x/t.json") == ("/x/t.json", [])
    assert cli.summary_line(16, 32, 2.0) == "16 prompt + 32 generated = 48 tokens in 2.00s (16.0 tok/s)"
    args = cli.build_parser().parse_args(["run", "-m", "a.gguf", "-p", "hi", "--temperature", "0"])
    assert args.max_tokens == 256 and args.top_k == 40 and args.seed == 42 and args.fn is cli.cmd_run
    assert cli.build_parser().parse_args(["serve", "-m", "a.gguf"]).port == 8080


def test_info_validate_quantize_commands(tiny_gguf, tmp_path, capsys):
    from oxibonsai_b200 import cli
    from oxibonsai_b200.core import GgufFile, gguf as G
    info = cli.model_info(tiny_gguf)
    assert info["valid"] and info["config"]["layers"] == 2 and info["quantization"] == "TQ2_0_g128" and info["variant"] == "Custom"
    assert info["gpu_engine"] == "sub-2-bit runner"
    q8 = str(tmp_path / "q8.gguf")
    cli.requantize_gguf(tiny_gguf, q8, "q8_0")
    assert cli.model_info(q8)["gpu_engine"] == "generic-format engine"
    assert cli.main(["info", "-m", tiny_gguf, "--json"]) == 0
    assert json.loads(capsys.readouterr().out)["tensors"] == info["tensors"]
    assert cli.main(["info", "-m", tiny_gguf]) == 0 and "Architecture Details" in capsys.readouterr().out
    assert cli.main(["validate", "-m", tiny_gguf]) == 0 and ": OK" in capsys.readouterr().out
    out = str(tmp_path / "q.gguf")
    assert cli.main(["quantize", "-i", tiny_gguf, "-o", out, "--format", "q1_0"]) == 0
    g = GgufFile.open(out)
    assert g.tensor_info("blk.0.attn_q.weight").type == G.Q1_0_G128 and g.tensor_info("blk.0.attn_norm.weight").type == G.F32
    assert g.config().layers == 2 and cli.model_info(out)["quantization"] == "Q1_0_g128"
    r = cli.requantize_gguf(tiny_gguf, str(tmp_path / "k.gguf"), "q4_k")
    assert r["requantized"] == 16 and r["format"] == "q4_k"      # 14 linear layers + embedding table + LM head
    with pytest.raises(SystemExit):
        cli.requantize_gguf(tiny_gguf, out, "q9")
    assert cli.main(["tokenizer", "download"]) == 2


# ---- a minimal protobuf writer to fabricate ONNX files ---------------------------------------------------------------------
def _vi(v):
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _ld(fn, payload):
    return _vi((fn << 3) | 2) + _vi(len(payload)) + payload


def _tensor(name, arr, dtype_id):
    p = b"".join(_vi((1 << 3) | 0) + _vi(d) for d in arr.shape) + _vi((2 << 3) | 0) + _vi(dtype_id) + _ld(8, name.encode()) + _ld(9, arr.tobytes())
    return p


def _attr_i(name, v):
    return _ld(5, _ld(1, name.encode()) + _vi((3 << 3) | 0) + _vi(v))


def _node(name, op, inputs, outputs, attrs=b""):
    return b"".join(_ld(1, i.encode()) for i in inputs) + b"".join(_ld(2, o.encode()) for o in outputs) + _ld(3, name.encode()) + _ld(4, op.encode()) + attrs


def test_onnx_matmulnbits_import(tmp_path):
    from oxibonsai_b200.convert import onnx as OX
    from oxibonsai_b200.core import GgufFile, dequantize, gguf as G
    rng = np.random.default_rng(0)
    K, N, bs = 256, 128, 128
    tern = rng.integers(-1, 2, size=(N, K)).astype(np.float32)
    scales = rng.uniform(0.01, 0.03, size=(N, K // bs)).astype(np.float32)
    q = (tern + 2).astype(np.uint8).reshape(N, K // bs, bs)                    # zero point 2 (the default for 2 bits)
    packed = (q[:, :, 0::4] | (q[:, :, 1::4] << 2) | (q[:, :, 2::4] << 4) | (q[:, :, 3::4] << 6)).astype(np.uint8)
    want = tern.reshape(N, K // bs, bs) * scales[:, :, None]
    assert np.allclose(OX.dequant_matmul_nbits(packed, scales, None, K, N, 2, bs), want.reshape(N, K))
    zp = np.full((N, 1), 2 | (2 << 2), dtype=np.uint8)
    assert np.allclose(OX.dequant_matmul_nbits(packed, scales, zp, K, N, 2, bs), want.reshape(N, K))
    graph = b""
    for l in range(2):
        for role in ("q_proj", "down_proj"):
            nm = f"/model/layers.{l}/{'attn' if role == 'q_proj' else 'mlp'}/{role}/MatMulNBits"
            graph += _ld(1, _node(nm, "MatMulNBits", ["x", nm + ".B", nm + ".scales"], ["y"],
                                  _attr_i("K", K) + _attr_i("N", N) + _attr_i("bits", 2) + _attr_i("block_size", bs)))
            graph += _ld(5, _tensor(nm + ".B", packed, 2)) + _ld(5, _tensor(nm + ".scales", scales.reshape(-1), 1))
        graph += _ld(5, _tensor(f"model.layers.{l}.input_layernorm.weight", np.ones(K, np.float32), 1))
    graph += _ld(1, _node("/model/Add", "Add", ["a", "b"], ["c"])) + _ld(2, b"tiny-onnx")
    graph += _ld(5, _tensor("model.embed_tokens.weight", rng.normal(size=(50, K)).astype(np.float16), 10))
    graph += _ld(5, _tensor("model.norm.weight", np.ones(K, np.float32), 1))
    path = tmp_path / "m.onnx"
    path.write_bytes(_vi((1 << 3) | 0) + _vi(8) + _ld(7, graph))
    info = OX.inspect_onnx(str(path))
    assert info["ops"] == {"MatMulNBits": 4, "Add": 1} and info["matmul_nbits"][0]["bits"] == 2 and info["graph"] == "tiny-onnx"
    assert OX.role_for("/model/layers.3/mlp/up_proj/MatMulNBits") == "blk.3.ffn_up.weight" and OX.role_for("/lm_head/MatMulNBits") == "output.weight"
    assert OX.role_for("model.layers.0.self_attn.k_norm.weight") == "blk.0.attn_k_norm.weight" and OX.role_for("random.thing") is None
    out = str(tmp_path / "m.gguf")
    st = OX.convert_onnx_to_gguf(str(path), out)
    f = GgufFile.open(out)
    assert st.tensors == 4 + 2 + 2 + 1 and st.tied and f.tensor_info("blk.1.ffn_down.weight").type == G.TQ2_0_G128
    deq = dequantize(G.TQ2_0_G128, f.tensor_bytes("blk.0.attn_q.weight")).reshape(N, K)
    rows = np.abs(want.reshape(N, K)).max(1) > 0
    # ternary data survives exactly up to the f16 rounding of the scale (rows whose groups contain a +-1)
    full = np.array([np.abs(tern[r].reshape(-1, bs)).max(1).min() > 0 for r in range(N)])
    assert np.allclose(deq[full], want.reshape(N, K)[full], rtol=2e-3) and rows.any()
    assert f.metadata["qwen3.block_count"] == 2 and f.tensor_info("token_embd.weight").type in (G.TQ2_0_G128, G.F16)
