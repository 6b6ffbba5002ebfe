"""The reference's CPU path, restated with the same torch ops — TEST/BENCH INFRASTRUCTURE.

`reference_cpu` is scripts/validate.py:32-34 (dequantise, one FP32 matmul) followed by the
bf16 cast of bench.py:30, on CPU tensors.  bench.py times it on the host cores as the CPU
baseline and as its `--impl reference` arm; tests use it as a second checker next to the
numpy oracle.  The product never imports this module.
"""
import torch


def dequantize_cpu(A, B, As, Bs):
    m, k = A.shape
    n = B.shape[0]
    a = (A.float().view(m, k // 128, 128) * As[..., None]).reshape(m, k)
    b = (B.float().view(n // 128, 128, k // 128, 128) * Bs[:, None, :, None]).reshape(n, k)
    return a, b


def reference_cpu(A, B, As, Bs, out_dtype=torch.bfloat16):
    a, b = dequantize_cpu(A, B, As, Bs)
    c = a @ b.T
    return c if out_dtype is None else c.to(out_dtype)
