"""Tensor parallelism on real GPUs: fused GEMV -> all-reduce over peer memory, vocab-parallel LM head, TP prefill.
Runs child processes (one per GPU) with NVLS off; skipped on boxes with fewer than two GPUs."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(path, mode, nproc, out_dir):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "tp_worker.py"), path, mode, str(out_dir)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    res = [json.load(open(os.path.join(out_dir, f"rank{r}.json"))) for r in range(nproc)]
    return res


@pytest.mark.parametrize("mode", ["exact", "fast", "batched", "speculative", "multimem"])
def test_tensor_parallel_two_gpus(mode, tiny_gguf, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    for r in _run(tiny_gguf, mode, 2, tmp_path):
        assert r["ok"] and r["status"] == 0, r
