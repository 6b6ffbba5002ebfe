"""Activation quantiser on the GPU (bf16 -> e4m3 + fp32 1x128 scales), the step before `matmul`.

The reference's adapter delegates this to SGLang (sgl_patch/fp8mm_sglang_patch.py:53); callers
without SGLang can use this kernel instead.  Output layout is what `matmul` expects: A [M,K]
float8_e4m3fn contiguous, As [M,K/128] float32 row-major."""
from . import _lib


def quantize_activations(x, floor=1e-10, ue8m0=False):
    """x: CUDA bfloat16 [M, K] (K a multiple of 128, unit column stride) -> (A, As).

    ue8m0=True rounds every group's scale UP to a power of two and returns As as uint8 exponents
    (value 2^(b-127)), what `matmul_ue8m0` and the block-scaled kernels take."""
    import torch
    if x.ndim != 2 or x.dtype != torch.bfloat16 or not x.is_cuda or x.stride(1) != 1:
        raise ValueError("x must be a CUDA bfloat16 [M,K] tensor with unit column stride")
    m, k = x.shape
    if k % 128 or m < 1:
        raise ValueError("K must be a multiple of 128 and M >= 1")
    if not floor > 0:
        raise ValueError("floor must be positive")
    lib = _lib.load()
    A = torch.empty((m, k), dtype=torch.float8_e4m3fn, device=x.device)
    As = torch.empty((m, k // 128), dtype=torch.uint8 if ue8m0 else torch.float32, device=x.device)
    fn = lib.fp8mm_b200_quantize_act_ue8m0 if ue8m0 else lib.fp8mm_b200_quantize_act
    with torch.cuda.device(x.device):
        rc = fn(x.data_ptr(), A.data_ptr(), As.data_ptr(), m, k, x.stride(0), As.stride(0), As.stride(1),
                float(floor), torch.cuda.current_stream(x.device).cuda_stream)
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


def ue8m0_bytes(scales):
    """Scales that are powers of two -> their UE8M0 exponent bytes as a uint8 view/tensor [rows, kblocks].

    Accepts uint8 [rows, kblocks] (returned as is), int32 words of four consecutive K blocks
    [rows, ceil(kblocks/4)] (the packed form DeepGEMM uses on sm_100: reinterpreted, no copy; the row
    stride must be in whole words), or float32 powers of two (exponent field taken; one small kernel)."""
    import torch
    if scales.dtype == torch.uint8:
        return scales
    if scales.dtype == torch.int32:
        if scales.stride(1) != 1:
            scales = scales.contiguous()
        return scales.view(torch.uint8)
    if scales.dtype == torch.float32:
        return ((scales.contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.uint8)
    raise ValueError("UE8M0 scales come as uint8 exponents, int32 words of four exponents, or float32 powers of two")


MX_MIN_TOKENS = 256       # from here on the token-major block-scaled kernels (128x256, 256x224 tiles);
GEMV_MAX_TOKENS = 4       # up to here the decode kernel, reading the exponent bytes itself; between the two the
                          # swap-AB block-scaled kernel.  (Expanding the scales to float32 for the table
                          # kernels costs two more launches per call, more than those kernels are ahead
                          # anywhere in that range.)


def _mxs_tile(m, n, k=2048, sms=148):
    """Token tile (16..128) of the swap-AB block-scaled kernel by a cost model fitted to measurements on
    a B200: waves of (weight tile, token tile) units over the SMs x K blocks x the time of a K block,
    which is what its 16 KB of weights + T x 128 bytes of tokens cost on the ~65 B/clk path from L2, and
    never less than ~300 cycles.  Small tiles spread a narrow layer over more SMs; large ones read the
    weights fewer times."""
    best = None
    for t in (16, 32, 64, 128):
        units = (n // 128) * -(-m // t)
        cost = -(-units // sms) * max(300.0, (16384 + t * 128) / 65.0)
        if best is None or cost < best[0] - 1e-9:
            best = (cost, t)
    return best[1]


def _mx_tile(m, n, k=2048, sms=148):
    """128x256 or 256x224 tiles, by a cost model fitted to measurements on a B200: waves of tiles over
    the SMs times the time of one tile = K blocks x block period + the accumulator drain
    (128x256: ~790 cycles per K block + ~1500; 256x224: ~1200 + ~2600 for 1.75 x the work)."""
    kb = max(1, k // 128)

    def cost(t, w, period, drain):
        units = -(-m // t) * -(-n // w)
        return -(-units // sms) * (kb * period + drain)
    return (256, 224) if cost(256, 224, 1200, 2600) < cost(128, 256, 790, 1500) else (128, 256)


def matmul_ue8m0(A, B, As, Bs, *, profile="35b_tp1"):
    """`matmul` for power-of-two scales: A[M,K], B[N,K] float8_e4m3fn, As[M,K/128] and Bs[N/128,K/128]
    in any of the forms `ue8m0_bytes` takes -> bfloat16 C[M,N].

    The scales stay bytes all the way: up to GEMV_MAX_TOKENS tokens the decode kernel reads them, from
    MX_MIN_TOKENS on the token-major and in between the swap-AB block-scaled kernels hand them to the
    tensor cores (`umma_mx`, tcgen05.mma kind::mxf8f6f4.block_scale).  No shape table is involved, so any
    N and K that are multiples of 128 work; `profile` is accepted for symmetry with `matmul`."""
    import torch
    from . import engine
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
    kb = k // 128
    with torch.cuda.device(A.device):
        # float32 activation scales (what a quantiser with power-of-two scales returns as floats) go to the
        # kernels as they are: they take the exponent field themselves, no conversion launch in front
        act_f32 = As.dtype == torch.float32
        a8, b8 = (As if act_f32 else ue8m0_bytes(As)), ue8m0_bytes(Bs)
        if a8.shape[0] != m or a8.shape[1] < kb or b8.shape[0] != n // 128 or b8.shape[1] < kb:
            raise ValueError("Expected As[M,K/128] and Bs[N/128,K/128] (packed words may pad K/128 up to a multiple of 4)")
        extra = {"ACT_SCALES_F32": True} if act_f32 else {}
        if m >= MX_MIN_TOKENS:
            bt, bw = _mx_tile(m, n, k)
            return engine.launch(A, B, a8, b8, "umma_mx", {"BLOCK_T": bt, "BLOCK_W": bw, **extra})
        if m <= GEMV_MAX_TOKENS:
            # one token per warp pass up to two tokens, else four
            return engine.launch(A, B, a8, b8, "gemv", {"BLOCK_T": 1 if m <= 2 else 4, "SCALES_UE8M0": True, **extra})
        return engine.launch(A, B, a8, b8, "umma_mx", {"BLOCK_T": _mxs_tile(m, n, k), "BLOCK_W": 128,
                                                       "NUM_STAGES": 4, "GROUP_SIZE_M": 1, **extra})
