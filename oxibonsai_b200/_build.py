"""In-tree native builds.

Two shared libraries are produced under ``oxibonsai_b200/_lib``:

* ``libbonsai_host.so`` - C++17 host library (GGUF, codecs, CPU oracle, runtime data structures),
  compiled with g++.
* ``libbonsai_cuda.so`` - every CUDA kernel and native launcher, compiled by nvcc for
  ``sm_100a`` only (``-gencode arch=compute_100a,code=sm_100a``); nvcc cross-compiles without a GPU.

Both expose a plain C ABI and are loaded with ctypes (``oxibonsai_b200._native``), so neither the
build nor the import depends on torch's extension machinery.  A content hash of the sources is
stored beside each library; a library is rebuilt only when its hash is stale.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "_lib"

HOST_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-shared", "-pthread", "-ffp-contract=off", "-fno-fast-math",
              "-Wall", "-Wno-unused-function"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
              "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr",
              "-Xcompiler", "-pthread"]


def _sources(kind: str) -> list[Path]:
    if kind == "host":
        pats = ["capi_*.cpp", "core/*.cpp", "cpu/*.cpp", "runtime/*.cpp"]
    else:
        pats = ["cuda/*.cu", "comm/*.cu"]
    out: list[Path] = []
    for p in pats:
        out += sorted(CSRC.glob(p))
    return out


def _digest(kind: str, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".cpp", ".hpp", ".h", ".cu", ".cuh"):
            if kind == "host" and p.suffix in (".cu", ".cuh"):
                continue
            h.update(p.relative_to(CSRC).as_posix().encode())
            h.update(p.read_bytes())
    return h.hexdigest()


def lib_path(kind: str) -> Path:
    return LIB / ("libbonsai_host.so" if kind == "host" else "libbonsai_cuda.so")


def is_stale(kind: str) -> bool:
    flags = HOST_FLAGS if kind == "host" else NVCC_FLAGS
    so, stamp = lib_path(kind), LIB / f".{kind}.sha256"
    return not (so.exists() and stamp.exists() and stamp.read_text().strip() == _digest(kind, flags))


def _nvcc() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def _headers_digest(kind: str, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    for p in sorted(CSRC.rglob("*")):
        if p.suffix in (".hpp", ".h", ".cuh"):
            h.update(p.relative_to(CSRC).as_posix().encode())
            h.update(p.read_bytes())
    return h.hexdigest()


def build(kind: str, force: bool = False, verbose: bool = False) -> Path:
    """Builds one library (``"host"`` or ``"cuda"``) if its sources changed; returns its path.

    Each translation unit is compiled to an object under ``_lib/obj`` (skipped when neither it nor
    any header changed) and the objects are linked into the shared library.
    """
    from concurrent.futures import ThreadPoolExecutor

    LIB.mkdir(exist_ok=True)
    obj_dir = LIB / "obj"
    obj_dir.mkdir(exist_ok=True)
    flags = HOST_FLAGS if kind == "host" else NVCC_FLAGS
    so, stamp = lib_path(kind), LIB / f".{kind}.sha256"
    if not force and not is_stale(kind):
        return so
    srcs = _sources(kind)
    if not srcs:
        raise RuntimeError(f"no sources for the {kind} library")
    if kind == "host":
        cc = "g++"
    else:
        cc = _nvcc()
        if cc is None:
            raise RuntimeError("nvcc not found; cannot build the CUDA library")
    cflags = [f for f in flags if f != "-shared"]
    if kind == "cuda" and verbose:
        cflags += ["-Xptxas", "-v"]
    hd = _headers_digest(kind, cflags)

    def compile_one(src: Path) -> tuple[Path, str]:
        tag = hashlib.sha256((hd + src.as_posix()).encode() + src.read_bytes()).hexdigest()
        obj = obj_dir / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        st = obj.with_suffix(".o.sha")
        if not force and obj.exists() and st.exists() and st.read_text() == tag:
            return obj, ""
        cmd = [cc, *cflags, f"-I{CSRC}", "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"native build failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
        st.write_text(tag)
        return obj, proc.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(compile_one, srcs))
    if verbose:
        for _, err in results:
            sys.stderr.write(err)
    objs = [str(o) for o, _ in results]
    tmp = so.with_suffix(f".tmp{os.getpid()}.so")
    if kind == "host":
        cmd = ["g++", "-shared", "-pthread", *objs, "-o", str(tmp)]
    else:
        cmd = [cc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *objs, "-o", str(tmp), "-lcuda"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f"native link failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, so)
    stamp.write_text(_digest(kind, flags))
    return so


def build_sanitized(out_dir: str | os.PathLike) -> Path:
    """Builds the host library with AddressSanitizer and UndefinedBehaviorSanitizer into ``out_dir`` (the regular library is
    left alone) and returns its path.  Load it through ``OXIBONSAI_HOST_LIB=<path>`` in a process started with the sanitizer
    runtimes preloaded (``sanitizer_runtimes()``); ``tests/test_host_sanitizers.py`` runs the codecs, the GGUF reader and
    writer, the CPU kernels and the tokenizer / constraint helpers that way."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    flags = [f for f in HOST_FLAGS if f not in ("-shared", "-O2")] + ["-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
                                                                     "-fno-sanitize-recover=undefined"]
    objs = []
    for src in _sources("host"):
        obj = out / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        cmd = ["g++", *flags, f"-I{CSRC}", "-c", str(src), "-o", str(obj)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"sanitized build failed: {' '.join(cmd)}\n{proc.stderr}")
        objs.append(str(obj))
    so = out / "libbonsai_host_san.so"
    proc = subprocess.run(["g++", "-shared", "-pthread", "-fsanitize=address,undefined", *objs, "-o", str(so)], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"sanitized link failed:\n{proc.stderr}")
    return so


def sanitizer_runtimes() -> list[str]:
    """Paths of libasan / libubsan of the host compiler, for ``LD_PRELOAD`` (empty when the compiler has none)."""
    libs = []
    for name in ("libasan.so", "libubsan.so"):
        p = subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True).stdout.strip()
        if p and os.path.isabs(p) and os.path.exists(p):
            libs.append(os.path.realpath(p))
    return libs


def build_all(force: bool = False, verbose: bool = False) -> dict[str, Path]:
    return {k: build(k, force=force, verbose=verbose) for k in ("host", "cuda")}


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "-v" in sys.argv
    kinds = [a for a in sys.argv[1:] if a in ("host", "cuda")] or ["host", "cuda"]
    for k in kinds:
        print(k, "->", build(k, force=force, verbose=verbose))
