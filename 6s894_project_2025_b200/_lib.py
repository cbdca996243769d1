"""ctypes binding of libb200ht.so (the C ABI declared in include/b200ht.h).

There is no CPU fallback: if the shared library is missing or stale it is built
with nvcc, and if that is impossible the import of an op raises.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libb200ht.so"

F16, BF16, F32 = 0, 1, 2
OUT_MN, OUT_NM = 0, 1
STATIC_SCRATCH_BYTES = 32 << 20

# every symbol include/b200ht.h declares
EXPORTS = (
    "b200ht_version",
    "b200ht_error_string",
    "b200ht_fwht",
    "b200ht_fwht_signed",
    "b200ht_fused_gemm_workspace_bytes",
    "b200ht_fused_gemm_tc_workspace_bytes",
    "b200ht_fused_gemm",
    "b200ht_fused_gemm_signed",
    "b200ht_fused_gemm_scaled",
    "b200ht_fused_gemm_static",
    "b200ht_fused_gemv",
    "b200ht_fused_gemv_max_batch",
    "b200ht_fused_gemv_peers",
    "b200ht_ipc_export",
    "b200ht_ipc_open",
    "b200ht_ipc_close",
    "b200ht_device_status",
    "b200ht_launch_count",
    "b200ht_selftest_wait_timeout",
)

_lock = threading.Lock()
_lib = None


def _declare(lib: ctypes.CDLL) -> None:
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.b200ht_version.restype = i
    lib.b200ht_version.argtypes = []
    lib.b200ht_error_string.restype = ctypes.c_char_p
    lib.b200ht_error_string.argtypes = [i]
    lib.b200ht_fwht.restype = i
    lib.b200ht_fwht.argtypes = [vp, vp, ctypes.c_uint64, ctypes.c_uint32, i, f, vp]
    lib.b200ht_fwht_signed.restype = i
    lib.b200ht_fwht_signed.argtypes = [vp, vp, ctypes.c_uint64, ctypes.c_uint32, i, f, vp, vp]
    lib.b200ht_fused_gemm_signed.restype = i
    lib.b200ht_fused_gemm_signed.argtypes = [vp, vp, vp, i, i, i, i, i, i, f, vp, vp, ctypes.c_size_t, vp]
    lib.b200ht_fused_gemm_scaled.restype = i
    lib.b200ht_fused_gemm_scaled.argtypes = [vp, vp, vp, i, i, i, i, i, i, f, vp, vp, vp, vp, ctypes.c_size_t, vp]
    lib.b200ht_fused_gemm_workspace_bytes.restype = ctypes.c_size_t
    lib.b200ht_fused_gemm_workspace_bytes.argtypes = [i, i, i, i]
    lib.b200ht_fused_gemm_tc_workspace_bytes.restype = ctypes.c_size_t
    lib.b200ht_fused_gemm_tc_workspace_bytes.argtypes = [i, i, i, i]
    lib.b200ht_fused_gemm.restype = i
    lib.b200ht_fused_gemm.argtypes = [vp, vp, vp, i, i, i, i, i, i, f, vp, ctypes.c_size_t, vp]
    lib.b200ht_fused_gemm_static.restype = i
    lib.b200ht_fused_gemm_static.argtypes = [vp, vp, vp, i, i, i, i, i, i, f, vp]
    lib.b200ht_fused_gemv.restype = i
    lib.b200ht_fused_gemv.argtypes = [vp, vp, vp, i, i, i, i, i, f, vp]
    lib.b200ht_fused_gemv_max_batch.restype = i
    lib.b200ht_fused_gemv_max_batch.argtypes = [i, i]
    lib.b200ht_fused_gemv_peers.restype = i
    lib.b200ht_fused_gemv_peers.argtypes = [vp, vp, vp, i, i, i, i, i, f, i, i, i, ctypes.POINTER(vp), vp, vp,
                                            ctypes.c_uint, vp]
    lib.b200ht_ipc_export.restype = i
    lib.b200ht_ipc_export.argtypes = [vp, ctypes.c_char_p, ctypes.POINTER(ctypes.c_ulonglong)]
    lib.b200ht_ipc_open.restype = i
    lib.b200ht_ipc_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
    lib.b200ht_ipc_close.restype = i
    lib.b200ht_ipc_close.argtypes = [vp]
    lib.b200ht_selftest_wait_timeout.restype = i
    lib.b200ht_selftest_wait_timeout.argtypes = [ctypes.c_uint, vp]
    lib.b200ht_launch_count.restype = ctypes.c_ulonglong
    lib.b200ht_launch_count.argtypes = []
    lib.b200ht_device_status.restype = i
    lib.b200ht_device_status.argtypes = [i]


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Load the shared library; raises if impossible.

    The library is (re)built first when it is missing or was built from other sources than the ones on disk (a
    digest of sources, headers and flags is stored beside it), so a stale binary is never loaded against a newer
    header.  The build takes a file lock: ranks started together do not compile the same objects twice.
    """
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        from . import build as _build

        if not _build.is_current():
            if not build_if_missing:
                raise RuntimeError(f"{LIB_PATH} is missing or stale and there is no fallback implementation")
            _build.build()
        lib = ctypes.CDLL(str(LIB_PATH))
        for name in EXPORTS:
            if not hasattr(lib, name):
                raise RuntimeError(f"{LIB_PATH} does not export {name}")
        _declare(lib)
        _lib = lib
        return lib


def error_string(code: int) -> str:
    return load().b200ht_error_string(int(code)).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed: {error_string(code)} (code {code})")
