"""Validated public entry point (same contract as fp8_gemm_h20/dispatch.py:5-30)."""
from .config import _select
from .engine import run


def matmul(A, B, As, Bs, *, profile="35b_tp1"):
    """FP8 A[M,K], B[N,K], FP32 block scales -> BF16 C[M,N] on A's device.

    C[m,n] = sum_kb (A[m,128kb:128kb+128] . B[n,128kb:128kb+128]) * As[m,kb] * Bs[n//128,kb]

    Every contract violation raises ValueError before any GPU work, in the order the
    reference checks them (dispatch.py:12-27): rank, matching/aligned dimensions, fp8
    dtype, one CUDA device, contiguous A and B, float32 scales, scale shapes.  Scale
    strides are free.  Shapes the profile does not list and M outside 1..16384 raise
    ValueError from the selector; nothing falls back to another backend.
    """
    import torch
    if A.ndim != 2 or B.ndim != 2:
        raise ValueError("A and B must be rank-2 tensors")
    m, k = A.shape
    n, k_b = B.shape
    if k != k_b or k % 128 != 0 or n % 128 != 0:
        raise ValueError("A/B dimensions must match and N,K must be multiples of 128")
    fp8 = torch.float8_e4m3fn
    if A.dtype != fp8 or B.dtype != fp8:
        raise ValueError("A and B must be float8_e4m3fn")
    if not A.is_cuda or B.device != A.device or As.device != A.device or Bs.device != A.device:
        raise ValueError("All tensors must reside on the same CUDA device")
    if not (A.is_contiguous() and B.is_contiguous()):
        raise ValueError("A and B must be contiguous row-major tensors")
    if As.dtype != torch.float32 or Bs.dtype != torch.float32:
        raise ValueError("Scales must be float32")
    if tuple(As.shape) != (m, k // 128) or tuple(Bs.shape) != (n // 128, k // 128):
        raise ValueError("Expected As[M,K/128] and Bs[N/128,K/128]")
    entry, _ = _select(profile, m, n, k)
    with torch.cuda.device(A.device):
        return run(entry, (A, B, As, Bs))
