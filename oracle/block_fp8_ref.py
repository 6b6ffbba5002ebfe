"""CPU oracle for the block-scaled FP8 GEMM — TEST INFRASTRUCTURE, not product code.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may
import this module; the product (fp8_gemm_h20_b200) never does and has no CPU path.

It restates, in numpy, the reference project's own definition of the result:
  * dequantise-then-FP32-matmul      scripts/validate.py:32-34 (`reference`)
  * the same followed by a bf16 cast bench.py:25-30 (`ref`)
  * the error metric                 scripts/validate.py:36-37 (`error`)
  * the synthetic-input quantiser    scripts/validate.py:26-29, bench.py:17-21
  * the per-K-block promote order of the kernels (for diagnosis only)
                                     fp8_gemm_h20/kernels/kernel_v2.py:86-91,164-174
FP8 values are handled as raw bytes with an explicit e4m3fn decode/encode, so the
oracle does not depend on torch's float8 support.

Pinned: tests/test_oracle.py checks it bit-for-bit (fp32) against outputs of the
reference's own `reference`/`ref`/`error` functions, generated in the build container by
tests/golden/make_golden.py and committed under tests/golden/.
"""
import numpy as np

FP8_MAX = 448.0


# ----------------------------------------------------------------- e4m3fn codec
def _build_decode_table():
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        sign = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        mant = b & 0x7
        if e == 0xF and mant == 0x7:
            v = np.nan                      # the only NaN pattern; e4m3fn has no infinity
        elif e == 0:
            v = sign * (mant / 8.0) * 2.0 ** -6
        else:
            v = sign * (1.0 + mant / 8.0) * 2.0 ** (e - 7)
        t[b] = v
    return t


E4M3_TABLE = _build_decode_table()


def e4m3_decode(u8):
    """uint8 array of float8_e4m3fn bit patterns -> float32."""
    return E4M3_TABLE[np.asarray(u8, dtype=np.uint8)]


def e4m3_encode(x):
    """float32 -> float8_e4m3fn bit patterns (uint8), round-to-nearest-even, the behaviour
    of torch's `.to(torch.float8_e4m3fn)` for |x| <= 448; larger magnitudes and NaN give NaN."""
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    ax = np.abs(x).astype(np.float64)
    out = np.zeros(x.shape, dtype=np.uint8)
    # exponent of the binade, clamped to the subnormal binade (2^-6)
    with np.errstate(divide="ignore", invalid="ignore"):
        e = np.floor(np.log2(np.where(ax > 0, ax, 1.0)))
    e = np.clip(e, -6, 8)
    step = 2.0 ** (e - 3)                   # spacing of representable values in the binade
    q = np.rint(ax / step) * step           # rint = round half to even
    # rounding may carry into the next binade; recompute fields from q
    with np.errstate(divide="ignore", invalid="ignore"):
        e2 = np.floor(np.log2(np.where(q > 0, q, 1.0)))
    e2 = np.clip(e2, -6, 8)
    is_sub = q < 2.0 ** -6
    mant = np.where(is_sub, np.rint(q / 2.0 ** -9), np.rint((q / 2.0 ** e2 - 1.0) * 8.0)).astype(np.int64)
    expf = np.where(is_sub, 0, e2 + 7).astype(np.int64)
    bits = ((expf << 3) | mant).astype(np.uint8)
    out = np.where(q > FP8_MAX, np.uint8(0x7F), bits).astype(np.uint8)
    out = np.where(np.isnan(x), np.uint8(0x7F), out).astype(np.uint8)
    return (out | sign).astype(np.uint8)


def bf16_round(x):
    """float32 -> nearest bfloat16 (ties to even), returned as float32 values."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    out = rounded.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(x), x, out).astype(np.float32)


def bf16_bits(x):
    """float32 -> bfloat16 bit patterns (uint16)."""
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


# ------------------------------------------------------------------- quantiser
def quantize_activations(x, floor=1e-10):
    """x [M,K] f32 -> (A bytes [M,K], As f32 [M,K/128]): amax/448 per 1x128 group
    (scripts/validate.py:26,28; bench.py:17-18), values clamped to +-448."""
    x = np.asarray(x, dtype=np.float32)
    m, k = x.shape
    g = x.reshape(m, k // 128, 128)
    scale = (np.maximum(np.abs(g).max(-1), np.float32(floor)) / np.float32(FP8_MAX)).astype(np.float32)
    q = np.clip(g / scale[..., None], -FP8_MAX, FP8_MAX).astype(np.float32)
    return e4m3_encode(q).reshape(m, k), scale


def quantize_activations_ue8m0(x, floor=1e-10):
    """The same with power-of-two scales: amax/448 rounded UP to 2^e, returned as the UE8M0 byte e + 127
    (the rule of SGLang's quantiser under scale_ue8m0=True, which the reference's adapter meets with
    DEEPGEMM_SCALE_UE8M0, sgl_patch/fp8mm_sglang_patch.py:41).  x [M,K] f32 -> (A bytes, exponents u8)."""
    x = np.asarray(x, dtype=np.float32)
    m, k = x.shape
    g = x.reshape(m, k // 128, 128)
    scale = (np.maximum(np.abs(g).max(-1), np.float32(floor)) / np.float32(FP8_MAX)).astype(np.float32)
    mant, exp = np.frexp(scale)                        # scale = mant * 2^exp, mant in [0.5, 1)
    e = np.where(mant == 0.5, exp - 1, exp).astype(np.int32)     # ceil(log2(scale)), exactly
    pow2 = np.ldexp(np.float32(1.0), e).astype(np.float32)
    q = np.clip(g / pow2[..., None], -FP8_MAX, FP8_MAX).astype(np.float32)
    return e4m3_encode(q).reshape(m, k), np.minimum(e + 127, 254).astype(np.uint8)


def quantize_weights(w, floor=1e-10):
    """w [N,K] f32 -> (B bytes [N,K], Bs f32 [N/128,K/128]): amax/448 per 128x128 block
    (scripts/validate.py:27,29; bench.py:19-21)."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    blk = w.reshape(n // 128, 128, k // 128, 128)
    scale = (np.maximum(np.abs(blk).max((1, 3)), np.float32(floor)) / np.float32(FP8_MAX)).astype(np.float32)
    q = np.clip(blk / scale[:, None, :, None], -FP8_MAX, FP8_MAX).astype(np.float32)
    return e4m3_encode(q).reshape(n, k), scale


# ---------------------------------------------------------------- the GEMM itself
def dequantize(A_u8, As, B_u8, Bs):
    """FP32 dequantised operands: every 1x128 group of A times As[m,kb], every 128x128 block
    of B times Bs[nb,kb] (scripts/validate.py:34)."""
    A_u8 = np.asarray(A_u8, dtype=np.uint8)
    B_u8 = np.asarray(B_u8, dtype=np.uint8)
    m, k = A_u8.shape
    n = B_u8.shape[0]
    a = (e4m3_decode(A_u8).reshape(m, k // 128, 128) * np.asarray(As, np.float32)[..., None]).reshape(m, k)
    b = (e4m3_decode(B_u8).reshape(n // 128, 128, k // 128, 128)
         * np.asarray(Bs, np.float32)[:, None, :, None]).reshape(n, k)
    return a.astype(np.float32), b.astype(np.float32)


def gemm_fp32(A_u8, B_u8, As, Bs):
    """The reference result in float32: dequantise, one FP32 matmul (scripts/validate.py:32-34)."""
    a, b = dequantize(A_u8, As, B_u8, Bs)
    return a @ b.T


def gemm_bf16(A_u8, B_u8, As, Bs):
    """bench.py:25-30: the same, rounded to bfloat16 (returned as float32 values)."""
    return bf16_round(gemm_fp32(A_u8, B_u8, As, Bs))


def gemm_blockwise(A_u8, B_u8, As, Bs, k_order=None):
    """Kernel-order restatement: per 128-wide K block an unscaled partial product, promoted
    into an FP32 accumulator with one scale product (kernel_v2.py:86-91,164-174).  Partial
    products are formed in float64 (the tensor core's block dot is exact or nearly so) and
    rounded once to float32.  Diagnostic: separates summation-order noise from real bugs."""
    A_u8 = np.asarray(A_u8, dtype=np.uint8)
    B_u8 = np.asarray(B_u8, dtype=np.uint8)
    m, k = A_u8.shape
    n = B_u8.shape[0]
    a = e4m3_decode(A_u8).astype(np.float64)
    b = e4m3_decode(B_u8).astype(np.float64)
    As = np.asarray(As, np.float32)
    Bs = np.asarray(Bs, np.float32)
    acc = np.zeros((m, n), dtype=np.float32)
    for kb in (k_order if k_order is not None else range(k // 128)):
        d = (a[:, kb * 128:(kb + 1) * 128] @ b[:, kb * 128:(kb + 1) * 128].T).astype(np.float32)
        sc = As[:, kb][:, None] * np.repeat(Bs[:, kb], 128)[None, :]
        acc = (acc + d * sc).astype(np.float32)
    return acc


# ------------------------------------------------------------------ tolerances
def rel_error(out, ref):
    """max|out-ref| / max(max|ref|, 1e-30)   (scripts/validate.py:36-37)."""
    out = np.asarray(out, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    return float(np.abs(out - ref).max() / max(float(np.abs(ref).max()), 1e-30))


def elementwise_violations(out, ref, rtol=2.0 ** -7, atol=1e-3):
    """How many elements break |out-ref| <= 2^-7 |ref| + 1e-3."""
    out = np.asarray(out, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    return int((np.abs(out - ref) > rtol * np.abs(ref) + atol).sum())


# ------------------------------------------------------------ seeded test inputs
def make_inputs(m, n, k, seed, mode="normal"):
    """numpy twin of fp8_gemm_h20_b200.testing.make_problem for the four validate.py modes
    (independent RNG: numpy PCG64, so values differ from the torch generator)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.05)
    if mode == "outlier":
        x[:, ::127] *= 100.0
    elif mode == "skew":
        w *= np.repeat(np.logspace(-3, 1, n // 128, dtype=np.float32), 128)[:, None]
    elif mode == "zero":
        x[:] = 0
    elif mode != "normal":
        raise ValueError(mode)
    A, As = quantize_activations(x, 1e-6)
    B, Bs = quantize_weights(w, 1e-6)
    return A, B, As, Bs


def expand_ue8m0(e):
    """UE8M0 exponents (uint8 array) -> float32 2^(e-127); 255 is NaN (the format's only special
    value).  The format is the OCP MX scale type that Blackwell's block-scaled MMA and DeepGEMM's
    sm_100 path use; the reference's adapter only tests for it (sgl_patch/fp8mm_sglang_patch.py:41)."""
    e = np.asarray(e, dtype=np.uint8)
    with np.errstate(over="ignore"):
        out = np.ldexp(np.float32(1.0), e.astype(np.int32) - 127).astype(np.float32)
    out[e == 255] = np.float32("nan")
    return out


def unpack_ue8m0_words(words):
    """int32 [rows, w] with four consecutive K-block exponents per word (little endian) ->
    uint8 [rows, 4*w]."""
    w = np.ascontiguousarray(np.asarray(words, dtype=np.int32))
    return w.view(np.uint8).reshape(w.shape[0], w.shape[1] * 4)
