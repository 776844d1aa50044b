"""The native host library under AddressSanitizer + UndefinedBehaviorSanitizer (the race / memory-error check of the C++ side
that needs no GPU): an instrumented build is loaded in a child process with the sanitizer runtimes preloaded."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def test_host_library_is_clean_under_asan_and_ubsan(tmp_path):
    from oxibonsai_b200 import _build
    runtimes = _build.sanitizer_runtimes()
    if len(runtimes) < 2:
        pytest.skip("the host compiler ships no sanitizer runtimes")
    so = _build.build_sanitized(tmp_path / "san")
    env = dict(os.environ, OXIBONSAI_HOST_LIB=str(so), LD_PRELOAD=":".join(runtimes), CUDA_VISIBLE_DEVICES="",
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:halt_on_error=1", UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1",
               OMP_NUM_THREADS="1")
    p = subprocess.run([sys.executable, os.path.join(HERE, "host_sanitizer_worker.py")], capture_output=True, text=True, timeout=900, env=env)
    report = p.stdout[-1500:] + p.stderr[-4000:]
    assert p.returncode == 0 and "sanitizer worker ok" in p.stdout, report
    assert "ERROR: AddressSanitizer" not in p.stderr and "runtime error:" not in p.stderr, report
