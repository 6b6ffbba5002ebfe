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


GEMV_MAX_TOKENS_SHORT = 8   # the decode kernel (it reads the exponent bytes itself) is considered up to here (_gemv_wins)

# Cycles measured on a B200.  Swap-AB block-scaled tiles by token tile: one K block (bound by the issue of
# tensor-core instructions up to 64 tokens, by the copies at 128).  Token-major tiles: one K block (bound by
# shared-memory bandwidth), the accumulator drain per tile, and what a launch pays once (set-up, first
# copies in flight, last drain).
_MXS_PERIOD = {16: 300.0, 32: 315.0, 64: 380.0, 128: 880.0}
_MX_TILES = {(128, 256): (790.0, 1500.0, 4000.0), (256, 224): (1200.0, 2600.0, 5000.0)}


def _mxs_cost(m, n, k, t, sms=148):
    units = (n // 128) * -(-m // t)
    kb = max(1, k // 128)
    drain = 24.0 * t + 300.0        # an epilogue of t two-byte stores per thread
    period = _MXS_PERIOD[t] * (1.2 if t == 16 and m > 16 else 1.0)   # 16-token tiles sharing a weight tile: measured
    return -(-units // sms) * (kb * period + drain)


def _mx_cost(m, n, k, tile, sms=148):
    period, drain, once = _MX_TILES[tile]
    units = -(-m // tile[0]) * -(-n // tile[1])
    return once + -(-units // sms) * (max(1, k // 128) * period + drain)


def _gemv_block_t(m, n, k):
    """Tokens per pass of the decode kernel (1, 2 or 4; every pass of ceil(m / that) streams the weights again,
    from L2, with its own CTAs): the smallest that keeps the row-passes under ~4700 and their work under
    ~8.5 M multiply-adds x K, which is where the tuned tables of both profiles change over (512 x 3072: one
    token per pass up to 5 tokens, two from 6; 2048 x 512: 1 / 2 / 4 from 1 / 3 / 5 tokens; 3072 x 256 and
    3072 x 2048: two tokens in one pass)."""
    for bt in (1, 2, 4):
        passes = -(-m // bt)
        if passes == 1 or (n * passes <= 4700 and n * passes * k <= 8.5e6):
            return bt
    return 4


def _gemv_wins(m, n, k):
    """The decode kernel against the 16-token swap-AB tile, from timings of both on a B200: always for one
    token; for two up to ~15 M weights (2 x 4608 x 3072 5.5 us against 5.8, but 2 x 9216 x 2048 6.4 against 5.3);
    up to 8 tokens where the layer is at most 2048 rows (one wave of the decode kernel's CTAs; 4096 rows while
    one pass of four tokens does it) and the work, in passes of four tokens, stays under what the tile kernel
    needs for its K blocks (4 x 2048 x 2048 4.0 us against 5.3, 8 x 1024 x 2048 3.3 against 4.2, 4 x 3072 x 256 2.4
    against 3.0, but 8 x 2048 x 2048 6.9 against 5.0 and 4 x 3072 x 2048 6.6 against 4.5)."""
    if m == 1:
        return True
    if m == 2:
        return n * k <= 15e6
    rows_max = 4096 if m <= 4 else 2048
    return m <= GEMV_MAX_TOKENS_SHORT and n <= rows_max and 4 * -(-m // 4) * n * k <= 17e6


_MXS_CLUSTER_MAX_CTAS = {2: 148, 4: 128, 8: 64}     # clusters of 8 need eight free SMs in one GPC
_MXS_STREAM_BYTES_PER_CLK = 3800.0                   # what all CTAs together pull when every weight tile is read once
_MXS_REDUCE_BASE = 1300.0                           # cycles: two cluster barriers and the first round trip of the reduction


def _mxs_split_cost(m, n, k, t, s):
    """Cycles of the swap-AB block-scaled kernel with s CTAs per tile in a cluster, or None where that is not
    offered: one wave of clusters; at least three K blocks per CTA; per K block the longer of the kernel's own
    period and the CTAs' share of the stream; plus the reduction over distributed shared memory, which grows
    with the token tile (~14 bytes per clock and SM)."""
    kb = max(1, k // 128)
    units = (n // 128) * -(-m // t)
    if kb % s or kb // s < 3 or units * s > _MXS_CLUSTER_MAX_CTAS[s]:
        return None
    period = max(_MXS_PERIOD[t], units * s * 128.0 * (128 + t) / _MXS_STREAM_BYTES_PER_CLK)
    return (kb // s) * period + 24.0 * t + 300.0 + _MXS_REDUCE_BASE + 40.0 * t


# The half-size form of the 32- and 64-token tiles (two issuing threads, two CTAs per SM): cycles of a K block
# for each of the two CTAs of an SM, and what their unit pays on top of the accumulator drain.
_MXS_HALF = {32: (600.0, 0.0), 64: (720.0, 0.0)}


def _mxs_half_cost(m, n, k, t, sms=148):
    """Cycles with two CTAs per SM, or None where that cannot pay: with no more units than SMs every CTA has an
    SM to itself anyway and four issuing threads are faster than two (timed: 384 x 3072 x 2048, 144 units, 7.3 us
    against 7.0; 256 x 9216 x 2048, 288 units, 9.8 against 11.6)."""
    units = (n // 128) * -(-m // t)
    if t not in _MXS_HALF or units <= sms:
        return None
    period, extra = _MXS_HALF[t]
    return -(-units // (2 * sms)) * (max(1, k // 128) * period + 24.0 * t + 300.0 + extra)


def _mxs_choice(m, n, k, sms=148):
    """(cycles, token tile, split, half-size form) of the swap-AB block-scaled kernel: the cheapest of the token
    tiles 16..128, each unsplit (waves of (weight tile, token tile) units over the SMs x K blocks x the time of a K block:
    small tiles spread a narrow layer over more SMs, large ones read the weights fewer times) or split 2, 4 or
    8 ways along K, or in its half-size form with two CTAs per SM.  Measured on a B200 (us, best split against unsplit): 4 x 512 x 3072 4.2 / 6.1,
    8 x 2048 x 4096 4.9 / 7.4, 32 x 2048 x 4096 5.7 / 7.6, 16 x 2048 x 2048 4.3 / 5.1, 16 x 3072 x 2048 4.6 / 5.2;
    no gain at 64 x 2048 x 2048 (5.5 / 5.2) or 16 x 5120 x 3072 (6.5 / 6.4): enough tiles already."""
    best = None
    for t in (16, 32, 64, 128):
        cands = [(_mxs_cost(m, n, k, t, sms), t, 1, False)]
        for s in (2, 4, 8):
            c = _mxs_split_cost(m, n, k, t, s)
            if c is not None:
                cands.append((1.1 * c, t, s, False))       # a split has to promise 10 % to be taken
        c = _mxs_half_cost(m, n, k, t, sms)
        if c is not None:
            cands.append((c, t, 1, True))
        for cand in cands:
            if best is None or cand < best:
                best = cand
    return best


def _mxs_tile(m, n, k=2048, sms=148):
    """Token tile (16..128) of the unsplit swap-AB block-scaled kernel by the cost model of `_mxs_choice`."""
    return min((16, 32, 64, 128), key=lambda t: (_mxs_cost(m, n, k, t, sms), t))


def _mx_tile(m, n, k=2048, sms=148):
    """128x256 or 256x224 token-major tiles: the cheaper by waves of tiles x (K blocks x period + drain)."""
    return min(_MX_TILES, key=lambda tile: (_mx_cost(m, n, k, tile, sms), tile))


def plan_ue8m0(m, n, k, sms=148):
    """(impl, config) of `matmul_ue8m0` for one problem: the decode kernel for one token, for two on all but the largest layers (up to 8
    where the layer is narrow or K short), else the cheaper of the swap-AB and the token-major block-scaled tiles by the cost
    models above (the swap-AB tiles win wherever the token-major ones would leave most SMs without a tile:
    up to ~1000 tokens on layers of a few thousand rows)."""
    if _gemv_wins(m, n, k):
        return "gemv", {"BLOCK_T": _gemv_block_t(m, n, k), "SCALES_UE8M0": True}
    cost, t, split, half = _mxs_choice(m, n, k, sms)
    tile = _mx_tile(m, n, k, sms)
    if cost <= _mx_cost(m, n, k, tile, sms):
        conf = {"BLOCK_T": t, "BLOCK_W": 128, "NUM_STAGES": 2 if half else 4, "GROUP_SIZE_M": 1, "SPLIT": split}
        if half:
            conf["HALF_FORM"] = True
        return "umma_mx", conf
    return "umma_mx", {"BLOCK_T": tile[0], "BLOCK_W": tile[1]}


def matmul_ue8m0(A, B, As, Bs, *, profile="35b_tp1"):
    """`matmul` for power-of-two scales: A[M,K], B[N,K] float8_e4m3fn, As[M,K/128] and Bs[N/128,K/128]
    in any of the forms `ue8m0_bytes` takes -> bfloat16 C[M,N].

    The scales stay bytes all the way: the decode kernel reads them for a few tokens, the swap-AB
    and token-major block-scaled kernels hand them to the tensor cores (`umma_mx`, tcgen05.mma
    kind::mxf8f6f4.block_scale); `plan_ue8m0` picks by measured cost models.  No shape table is involved, so
    any N and K that are multiples of 128 work; `profile` is accepted for symmetry with `matmul`."""
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
        impl, conf = plan_ue8m0(m, n, k)
        if act_f32:
            conf = dict(conf, ACT_SCALES_F32=True)
        return engine.launch(A, B, a8, b8, impl, conf)
