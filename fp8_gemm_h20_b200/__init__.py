"""Block-scaled FP8 GEMM for NVIDIA B200 (sm_100a) behind the fp8_gemm_h20 operator API.

    from fp8_gemm_h20_b200 import matmul, select, supports, available_profiles

Importing this package and calling `select`/`supports` never touches CUDA; the native
library is loaded on the first `matmul`.
"""
from .config import available_profiles, select, supports
from .dispatch import matmul

__all__ = ["matmul", "available_profiles", "select", "supports"]
