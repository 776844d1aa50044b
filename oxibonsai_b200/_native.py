"""ctypes loaders for the two in-tree native libraries.

``host()`` returns ``libbonsai_host.so`` (C++: GGUF, codecs, CPU oracle, runtime structures) and
``cuda()`` returns ``libbonsai_cuda.so`` (sm_100a kernels and native launchers).  Libraries are
built on first use when missing or stale and a compiler is present.  ``cuda()`` raises when the
library cannot be loaded: GPU code paths never fall back silently to PyTorch ops.
"""
from __future__ import annotations

import ctypes as C
import threading

from . import _build

_lock = threading.Lock()
_host = None
_cuda = None


class NativeError(RuntimeError):
    """Error raised by the native host library; carries the stable code and retryable flag."""

    def __init__(self, code: int, name: str, message: str, retryable: bool):
        super().__init__(f"[{name}] {message}")
        self.code = code
        self.name = name
        self.retryable = retryable


def _load(kind: str) -> C.CDLL:
    import os
    override = os.environ.get("OXIBONSAI_HOST_LIB") if kind == "host" else None
    if override:            # an instrumented build of the host library (see _build.build_sanitized)
        return C.CDLL(override, mode=C.RTLD_GLOBAL)
    path = _build.lib_path(kind)
    try:
        if _build.is_stale(kind):
            # Every rank of a torchrun job imports this module at the same time.  One process rebuilds; the others wait
            # on the file lock and find the library fresh when they get it.
            import fcntl
            _build.LIB.mkdir(exist_ok=True)
            with open(_build.LIB / f".{kind}.lock", "w") as lock:
                fcntl.flock(lock, fcntl.LOCK_EX)
                try:
                    if _build.is_stale(kind):
                        _build.build(kind)
                finally:
                    fcntl.flock(lock, fcntl.LOCK_UN)
    except Exception:
        if not path.exists():
            raise
    return C.CDLL(str(path), mode=C.RTLD_GLOBAL if kind == "host" else C.RTLD_LOCAL)


def host() -> C.CDLL:
    global _host
    if _host is None:
        with _lock:
            if _host is None:
                lib = _load("host")
                _declare_host(lib)
                _host = lib
    return _host


def cuda() -> C.CDLL:
    global _cuda
    if _cuda is None:
        with _lock:
            if _cuda is None:
                lib = _load("cuda")
                _cuda = lib
    return _cuda


def check(rc: int) -> int:
    """Raises NativeError for a negative return code of a host-library call."""
    if rc < 0:
        raise last_error()
    return rc


def last_error() -> NativeError:
    lib = host()
    code = lib.bonsai_last_error_code()
    return NativeError(code, lib.bonsai_error_name(code).decode(), lib.bonsai_last_error().decode(errors="replace"),
                       bool(lib.bonsai_error_retryable(code)))


def _declare_host(lib: C.CDLL) -> None:
    vp, u8p, u32p, u64p, f32p, cp = C.c_void_p, C.POINTER(C.c_uint8), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.POINTER(C.c_float), C.c_char_p
    sig = {
        "bonsai_last_error": (cp, []),
        "bonsai_last_error_code": (C.c_int, []),
        "bonsai_error_name": (cp, [C.c_int]),
        "bonsai_error_retryable": (C.c_int, [C.c_int]),
        "bonsai_free": (None, [vp]),
        "bonsai_type_info": (C.c_int, [C.c_uint32, u32p, u32p, C.c_char_p, C.c_size_t]),
        "bgguf_open": (vp, [cp]),
        "bgguf_parse": (vp, [vp, C.c_size_t]),
        "bgguf_close": (None, [vp]),
        "bgguf_version": (C.c_uint32, [vp]),
        "bgguf_alignment": (C.c_uint32, [vp]),
        "bgguf_data_offset": (C.c_uint64, [vp]),
        "bgguf_n_tensors": (C.c_uint64, [vp]),
        "bgguf_n_kv": (C.c_uint64, [vp]),
        "bgguf_file_size": (C.c_uint64, [vp]),
        "bgguf_metadata_json": (vp, [vp, C.c_uint64]),
        "bgguf_find_tensor": (C.c_int, [vp, cp]),
        "bgguf_tensor_info": (C.c_int, [vp, C.c_uint64, C.c_char_p, C.c_size_t, u64p, u32p, u32p, u64p, u64p]),
        "bgguf_tensor_data": (vp, [vp, C.c_uint64, u64p]),
        "bgguf_config": (C.c_int, [vp, u32p, f32p, C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t]),
        "bggufw_new": (vp, [C.c_uint32, C.c_uint32]),
        "bggufw_free": (None, [vp]),
        "bggufw_add_u32": (None, [vp, cp, C.c_uint32]),
        "bggufw_add_u64": (None, [vp, cp, C.c_uint64]),
        "bggufw_add_i32": (None, [vp, cp, C.c_int32]),
        "bggufw_add_f32": (None, [vp, cp, C.c_float]),
        "bggufw_add_f64": (None, [vp, cp, C.c_double]),
        "bggufw_add_bool": (None, [vp, cp, C.c_int]),
        "bggufw_add_str": (None, [vp, cp, cp]),
        "bggufw_add_scalar": (None, [vp, cp, C.c_uint32, C.c_int64, C.c_double]),
        "bggufw_add_str_array": (None, [vp, cp, C.POINTER(cp), u64p, C.c_uint64]),
        "bggufw_add_num_array": (None, [vp, cp, C.c_uint32, C.POINTER(C.c_int64), C.POINTER(C.c_double), C.c_uint64]),
        "bggufw_add_tensor": (C.c_int, [vp, cp, u64p, C.c_uint32, C.c_uint32, vp, C.c_uint64, C.c_int]),
        "bggufw_write": (C.c_int, [vp, cp]),
        "bggufw_to_bytes": (vp, [vp, u64p]),
        "bggufs_new": (vp, []),
        "bggufs_free": (None, [vp]),
        "bggufs_feed": (C.c_int, [vp, vp, C.c_size_t]),
        "bggufs_file": (vp, [vp]),
        "bggufs_bytes_consumed": (C.c_uint64, [vp]),
        "bggufs_data_seen": (C.c_uint64, [vp]),
        "bggufs_data_expected": (C.c_uint64, [vp]),
        "bggufs_error": (cp, [vp]),
        "bonsai_dequant": (C.c_int, [C.c_uint32, vp, C.c_uint64, vp]),
        "bonsai_quant": (C.c_int, [C.c_uint32, vp, C.c_uint64, vp, C.c_uint32]),
        "bonsai_fp8_encode": (C.c_uint8, [C.c_float, C.c_int]),
        "bonsai_fp8_decode": (C.c_float, [C.c_uint8, C.c_int]),
        "bonsai_f32_to_f16": (C.c_uint16, [C.c_float]),
        "bonsai_f16_to_f32": (C.c_float, [C.c_uint16]),
        "bcpu_gemv": (C.c_int, [C.c_uint32, vp, C.c_uint64, C.c_uint64, vp, vp]),
        "bcpu_rmsnorm": (None, [vp, vp, vp, C.c_uint64, C.c_float]),
        "bcpu_rope": (None, [vp, C.c_uint64, C.c_uint32, C.c_float]),
        "bcpu_swiglu": (None, [vp, vp, vp, C.c_uint64]),
        "bcpu_argmax_last": (C.c_int, [vp, C.c_uint64]),
        "bcpu_rope_table": (None, [C.c_uint32, C.c_uint32, C.c_float, vp, vp]),
        "boracle_new": (vp, [vp, C.c_uint32]),
        "boracle_free": (None, [vp]),
        "boracle_forward": (C.c_int, [vp, C.c_uint32, C.c_uint32, vp]),
        "boracle_last_hidden": (C.c_int, [vp, vp, C.c_uint64]),
        "boracle_generate": (C.c_int, [vp, vp, C.c_uint32, C.c_uint32, vp, vp, C.c_int]),
        "bonsai_write_synthetic": (C.c_int, [cp, u32p, f32p, cp, C.c_uint32, C.c_int, C.c_uint64, C.c_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    # optional symbol groups declared by the modules that use them
    lib._declared = set(sig)


def declare(lib: C.CDLL, sig: dict) -> None:
    """Declares extra function signatures (used by modules that wrap later additions)."""
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
