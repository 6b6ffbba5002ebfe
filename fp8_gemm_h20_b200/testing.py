"""Seeded synthetic problems and a plain torch FP32 reference (accuracy gates only).

`matmul` never comes through here.  The quantiser restates the scheme the reference
uses for its synthetic inputs (scripts/validate.py:21-30, bench.py:14-22): per 1x128
activation group and per 128x128 weight block, scale = amax/448 with a floor, values
divided by the scale and cast to float8_e4m3fn.  Everything is generated on the CPU from a
seeded generator so that a CPU checker and the GPU kernel see identical bits.
"""
import math

FP8_MAX = 448.0


def quantize_activations(x, floor=1e-10):
    """x [M,K] float -> (A e4m3 [M,K], As f32 [M,K/128]); 1x128 groups along K."""
    import torch
    m, k = x.shape
    g = x.float().view(m, k // 128, 128)
    scale = g.abs().amax(-1).clamp_min(floor) / FP8_MAX
    q = (g / scale[..., None]).clamp(-FP8_MAX, FP8_MAX).reshape(m, k).to(torch.float8_e4m3fn)
    return q, scale.contiguous()


def quantize_weights(w, floor=1e-10):
    """w [N,K] float -> (B e4m3 [N,K], Bs f32 [N/128,K/128]); 128x128 blocks."""
    import torch
    n, k = w.shape
    blk = w.float().view(n // 128, 128, k // 128, 128)
    scale = blk.abs().amax((1, 3)).clamp_min(floor) / FP8_MAX
    q = (blk / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).reshape(n, k).to(torch.float8_e4m3fn)
    return q, scale.contiguous()


def _raw_problem(m, n, k, seed, mode):
    """Activations x[m,k], weights w[n,k] as float32 and the scale floor of one test problem (see make_problem)."""
    import torch
    gen = torch.Generator().manual_seed(int(seed))
    x = torch.randn(m, k, generator=gen)
    w = torch.randn(n, k, generator=gen)
    if mode == "cfg0":
        n_out = max(1, math.ceil(0.01 * k))
        idx = torch.randperm(k, generator=gen)[:n_out]
        x[:, idx] *= 20.0
        x = x.to(torch.bfloat16).float()
        w = w * 0.02
        floor = 1e-10
    else:
        w = w * 0.05
        floor = 1e-6
        if mode == "outlier":
            x[:, ::127] *= 100.0
        elif mode == "skew":
            w = w * torch.logspace(-3, 1, n // 128).repeat_interleave(128)[:, None]
        elif mode == "zero":
            x.zero_()
        elif mode != "normal":
            raise ValueError(mode)
    return x, w, floor


def make_problem(m, n, k, seed=0, mode="cfg0", device="cpu"):
    """(A, B, As, Bs) on `device`, generated on the CPU from `seed`.

    modes: "cfg0"  X~N(0,1) as bf16 with 1% of the K channels x20, W~N(0,0.02)
           "normal"/"outlier"/"skew"/"zero"  the four distributions of scripts/validate.py:21-25
           (X~N(0,1), W~0.05 N(0,1); every 127th channel x100; weight row blocks x logspace(-3,1);
           all-zero activations), scale floor 1e-6 as there."""
    x, w, floor = _raw_problem(m, n, k, seed, mode)
    A, As = quantize_activations(x, floor)
    B, Bs = quantize_weights(w, floor)
    return tuple(t.to(device) for t in (A, B, As, Bs))


def make_problem_ue8m0(m, n, k, seed=0, device="cpu", mode="cfg0"):
    """(A, B, As_u8, Bs_u8, As, Bs): the problem of `make_problem` (same modes) quantised with power-of-two
    scales (each block's scale rounded UP to 2^e, as UE8M0 checkpoints are made); As_u8/Bs_u8 hold e + 127,
    As/Bs the same scales as float32 for the references."""
    import torch
    x, w, floor = _raw_problem(m, n, k, seed, mode)
    xa = x.view(m, k // 128, 128)
    ea = torch.ceil(torch.log2(xa.abs().amax(-1).clamp_min(floor) / FP8_MAX)).clamp(-127, 127)
    As = torch.exp2(ea)
    A = (xa / As[..., None]).clamp(-FP8_MAX, FP8_MAX).reshape(m, k).to(torch.float8_e4m3fn)
    wb = w.view(n // 128, 128, k // 128, 128)
    eb = torch.ceil(torch.log2(wb.abs().amax((1, 3)).clamp_min(floor) / FP8_MAX)).clamp(-127, 127)
    Bs = torch.exp2(eb)
    B = (wb / Bs[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).reshape(n, k).to(torch.float8_e4m3fn)
    As_u8 = (ea + 127).to(torch.uint8)
    Bs_u8 = (eb + 127).to(torch.uint8)
    return tuple(t.contiguous().to(device) for t in (A, B, As_u8, Bs_u8, As, Bs))


def reference_fp32(A, B, As, Bs):
    """Dequantise, then one FP32 matmul (the reference's accuracy definition,
    scripts/validate.py:32-34).  Returns float32 [M,N] on the inputs' device."""
    m, k = A.shape
    n = B.shape[0]
    a = (A.float().view(m, k // 128, 128) * As[..., None]).reshape(m, k)
    b = (B.float().view(n // 128, 128, k // 128, 128) * Bs[:, None, :, None]).reshape(n, k)
    return a @ b.T


def rel_error(out, ref):
    """max|out-ref| / max|ref|  (scripts/validate.py:36-37)."""
    return ((out.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item()


def elementwise_violations(out, ref, rtol=2.0 ** -7, atol=1e-3):
    """Number of elements with |out-ref| > rtol*|ref| + atol."""
    diff = (out.float() - ref).abs()
    return int((diff > rtol * ref.abs() + atol).sum().item())
