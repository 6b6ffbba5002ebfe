"""Activation quantiser on the GPU (bf16 -> e4m3 + fp32 1x128 scales), the step before `matmul`.

The reference's adapter delegates this to SGLang (sgl_patch/fp8mm_sglang_patch.py:53); callers
without SGLang can use this kernel instead.  Output layout is what `matmul` expects: A [M,K]
float8_e4m3fn contiguous, As [M,K/128] float32 row-major."""
from . import _lib


def quantize_activations(x, floor=1e-10):
    """x: CUDA bfloat16 [M, K] (K a multiple of 128, unit column stride) -> (A, As)."""
    import torch
    if x.ndim != 2 or x.dtype != torch.bfloat16 or not x.is_cuda or x.stride(1) != 1:
        raise ValueError("x must be a CUDA bfloat16 [M,K] tensor with unit column stride")
    m, k = x.shape
    if k % 128 or m < 1:
        raise ValueError("K must be a multiple of 128 and M >= 1")
    lib = _lib.load()
    A = torch.empty((m, k), dtype=torch.float8_e4m3fn, device=x.device)
    As = torch.empty((m, k // 128), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.fp8mm_b200_quantize_act(x.data_ptr(), A.data_ptr(), As.data_ptr(), m, k, x.stride(0),
                                         As.stride(0), As.stride(1), float(floor),
                                         torch.cuda.current_stream(x.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"fp8mm_b200_quantize_act failed: {_lib.strerror(rc)}")
    return A, As


def expand_ue8m0(scales):
    """UE8M0 scales -> float32 [rows, kblocks] (contiguous), exactly: value = 2^(e - 127).

    `scales` is a CUDA tensor of either uint8 [rows, kblocks] (any strides), or int32
    [rows, ceil(kblocks/4)] with four consecutive K blocks per word (the packed MN-major form
    DeepGEMM uses on sm_100; any strides) - then every byte of every word is expanded, i.e.
    kblocks = 4 * words per row."""
    import torch
    if scales.ndim != 2 or not scales.is_cuda:
        raise ValueError("scales must be a 2-D CUDA tensor")
    if scales.dtype == torch.uint8:
        rows, kblocks, packed = scales.shape[0], scales.shape[1], 0
    elif scales.dtype == torch.int32:
        rows, kblocks, packed = scales.shape[0], scales.shape[1] * 4, 1
    else:
        raise ValueError("UE8M0 scales come as uint8 exponents or as int32 words of four exponents")
    out = torch.empty((rows, kblocks), dtype=torch.float32, device=scales.device)
    lib = _lib.load()
    with torch.cuda.device(scales.device):
        rc = lib.fp8mm_b200_expand_ue8m0(scales.data_ptr(), out.data_ptr(), rows, kblocks, scales.stride(0),
                                         scales.stride(1), packed,
                                         torch.cuda.current_stream(scales.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"fp8mm_b200_expand_ue8m0 failed: {_lib.strerror(rc)}")
    return out
