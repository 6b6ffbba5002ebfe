"""ctypes binding of the C ABI in include/fp8mm_b200.h (libfp8mm_b200.so).

This is the only place that touches the native library.  It stands where the
reference's lazy kernel import stood (fp8_gemm_h20/engine.py:13-16): loaded on the
first GEMM call, so importing the package and routing stay GPU-free
(docs/configuration.md:36).  There is no fallback: a missing library is an error.
"""
import ctypes
import os
import threading
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_NAME = "libfp8mm_b200.so"
LIB_PATH = _PKG / LIB_NAME

IMPL_UMMA = 0
IMPL_UMMA_SWAP = 1
IMPL_UMMA_2CTA = 2
IMPL_GEMV = 3
IMPL_UMMA_MX = 4
E_DEVICE_TIMEOUT = -8
E_TOO_LARGE = -9

# every symbol include/fp8mm_b200.h declares
SYMBOLS = (
    "fp8mm_b200_validate",
    "fp8mm_b200_workspace_bytes",
    "fp8mm_b200_workspace_init",
    "fp8mm_b200_gemm",
    "fp8mm_b200_gemm_bcast",
    "fp8mm_b200_gemm_static_scratch",
    "fp8mm_b200_quantize_act",
    "fp8mm_b200_quantize_act_ue8m0",
    "fp8mm_b200_expand_ue8m0",
    "fp8mm_b200_static_scratch_bytes",
    "fp8mm_b200_static_scratch_status",
    "fp8mm_b200_last_status",
    "fp8mm_b200_strerror",
    "fp8mm_b200_version",
)


class Args(ctypes.Structure):
    _fields_ = [
        ("A", ctypes.c_void_p), ("B", ctypes.c_void_p),
        ("As", ctypes.c_void_p), ("Bs", ctypes.c_void_p), ("C", ctypes.c_void_p),
        ("M", ctypes.c_int32), ("N", ctypes.c_int32), ("K", ctypes.c_int32),
        ("reserved0", ctypes.c_int32),
        ("as_stride_m", ctypes.c_int64), ("as_stride_k", ctypes.c_int64),
        ("bs_stride_n", ctypes.c_int64), ("bs_stride_k", ctypes.c_int64),
        ("ldc", ctypes.c_int64),
    ]


class Cfg(ctypes.Structure):
    _fields_ = [
        ("impl", ctypes.c_int32), ("block_t", ctypes.c_int32), ("block_w", ctypes.c_int32),
        ("stages", ctypes.c_int32), ("split", ctypes.c_int32), ("group_m", ctypes.c_int32),
        ("max_ctas", ctypes.c_int32), ("flags", ctypes.c_int32),
    ]


class NativeLibraryMissing(RuntimeError):
    pass


_lock = threading.Lock()
_lib = None


def load():
    """Return the loaded library; raise NativeLibraryMissing when it was never built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = Path(os.environ.get("FP8MM_LIB", LIB_PATH))
        if not path.is_file():
            raise NativeLibraryMissing(
                f"{path} not found: build it with `python -m fp8_gemm_h20_b200.build` "
                "(nvcc, sm_100a). There is no CPU or Triton fallback.")
        lib = ctypes.CDLL(str(path))
        lib.fp8mm_b200_validate.argtypes = [ctypes.c_int32] * 3 + [ctypes.POINTER(Cfg)]
        lib.fp8mm_b200_validate.restype = ctypes.c_int
        lib.fp8mm_b200_workspace_bytes.argtypes = [ctypes.c_int32] * 3 + [ctypes.POINTER(Cfg)]
        lib.fp8mm_b200_workspace_bytes.restype = ctypes.c_size_t
        lib.fp8mm_b200_workspace_init.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
        lib.fp8mm_b200_workspace_init.restype = ctypes.c_int
        lib.fp8mm_b200_gemm.argtypes = [ctypes.POINTER(Args), ctypes.POINTER(Cfg), ctypes.c_void_p,
                                        ctypes.c_size_t, ctypes.c_void_p]
        lib.fp8mm_b200_gemm.restype = ctypes.c_int
        lib.fp8mm_b200_gemm_bcast.argtypes = [ctypes.POINTER(Args), ctypes.POINTER(Cfg), ctypes.c_void_p,
                                              ctypes.c_size_t, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                              ctypes.c_int32]
        lib.fp8mm_b200_gemm_bcast.restype = ctypes.c_int
        lib.fp8mm_b200_gemm_static_scratch.argtypes = [ctypes.POINTER(Args), ctypes.POINTER(Cfg), ctypes.c_void_p]
        lib.fp8mm_b200_gemm_static_scratch.restype = ctypes.c_int
        lib.fp8mm_b200_quantize_act.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                                ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                                ctypes.c_float, ctypes.c_void_p]
        lib.fp8mm_b200_quantize_act.restype = ctypes.c_int
        lib.fp8mm_b200_quantize_act_ue8m0.argtypes = lib.fp8mm_b200_quantize_act.argtypes
        lib.fp8mm_b200_quantize_act_ue8m0.restype = ctypes.c_int
        lib.fp8mm_b200_expand_ue8m0.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                                ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p]
        lib.fp8mm_b200_expand_ue8m0.restype = ctypes.c_int
        lib.fp8mm_b200_static_scratch_bytes.argtypes = []
        lib.fp8mm_b200_static_scratch_bytes.restype = ctypes.c_size_t
        lib.fp8mm_b200_static_scratch_status.argtypes = [ctypes.POINTER(ctypes.c_int32)]
        lib.fp8mm_b200_static_scratch_status.restype = ctypes.c_int
        lib.fp8mm_b200_last_status.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]
        lib.fp8mm_b200_last_status.restype = ctypes.c_int
        lib.fp8mm_b200_strerror.argtypes = [ctypes.c_int]
        lib.fp8mm_b200_strerror.restype = ctypes.c_char_p
        lib.fp8mm_b200_version.argtypes = []
        lib.fp8mm_b200_version.restype = ctypes.c_int
        _lib = lib
    return _lib


def strerror(code):
    return load().fp8mm_b200_strerror(int(code)).decode()
