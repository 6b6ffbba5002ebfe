"""Block-scaled FP8 GEMM for NVIDIA B200 (sm_100a) behind the fp8_gemm_h20 operator API.

    from fp8_gemm_h20_b200 import matmul, select, supports, available_profiles

Importing this package and calling `select`/`supports` never touches CUDA; the native
library is loaded on the first `matmul`.
"""
from .config import available_profiles, select, supports
from .dispatch import matmul


def matmul_ue8m0(A, B, As, Bs, *, profile="35b_tp1"):
    """`matmul` for power-of-two (UE8M0) scales given as bytes, packed words or float32 (quant.py)."""
    from .quant import matmul_ue8m0 as impl
    return impl(A, B, As, Bs, profile=profile)


__all__ = ["matmul", "matmul_ue8m0", "available_profiles", "select", "supports"]
