"""GPU parity of the decode kernel (`gemv`: a few tokens, weight rows streamed into registers and
multiplied with FP32 FMAs) against the numpy oracle, through the C ABI.  Same two tolerances as the tile kernels:
max|C-ref|/max|ref| <= 1e-2 (scripts/validate.py:36-37,61 of the reference) and per element
|C-ref| <= 2^-7 |ref| + 1e-3.  Covers every tokens-per-warp variant, token counts that need
several token groups or leave part of one empty, K ranges of one to forty K blocks (chunks that end
inside a four-block group, more chunks than the eight warps of a CTA), strided scales, an output slice of a wider buffer, and bit-repeatability."""
import numpy as np
import pytest
import torch

from fp8_gemm_h20_b200 import engine, testing
from oracle import block_fp8_ref as oracle

pytestmark = pytest.mark.gpu


def oracle_ref(A, B, As, Bs):
    return oracle.gemm_fp32(A.view(torch.uint8).cpu().numpy(), B.view(torch.uint8).cpu().numpy(),
                            As.cpu().numpy(), Bs.cpu().numpy())


def check(out, ref, what):
    o = out.float().cpu().numpy()
    assert np.isfinite(o).all(), what
    err = oracle.rel_error(o, ref)
    assert err <= 1e-2, (what, err)
    assert oracle.elementwise_violations(o, ref) == 0, (what, err)


SHAPES = [(512, 3072), (3072, 256), (1024, 2048), (2048, 4096), (256, 128), (384, 384), (128, 640), (256, 5120)]


@pytest.mark.parametrize("n,k", SHAPES)
def test_gemv_matches_oracle(n, k):
    for m in (1, 2, 3, 4, 5, 8, 11):
        A, B, As, Bs = testing.make_problem(m, n, k, seed=m + n + k + 113, mode="cfg0" if m % 2 else "normal")
        ref = oracle_ref(A, B, As, Bs)
        dev = tuple(t.cuda() for t in (A, B, As, Bs))
        outs = []
        for bt in (1, 2, 4):
            out = engine.launch(*dev, "gemv", dict(BLOCK_T=bt))
            check(out, ref, (m, n, k, bt))
            assert torch.equal(out, engine.launch(*dev, "gemv", dict(BLOCK_T=bt))), ("not bit-repeatable", m, n, k, bt)
            outs.append(out)
        # the tokens-per-warp variants walk K in the same order: same bits
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), (m, n, k)


def test_gemv_strided_scales_and_output_slice():
    m, n, k = 7, 1024, 2048
    A, B, As, Bs = (t.cuda() for t in testing.make_problem(m, n, k, seed=5, mode="outlier"))
    ref = oracle_ref(A, B, As, Bs)
    want = engine.launch(A, B, As, Bs, "gemv", dict(BLOCK_T=4))
    As_t, Bs_t = As.T.contiguous().T, Bs.T.contiguous().T          # column-major scales (validate.py:103-108)
    assert As_t.stride() != As.stride()
    got = engine.launch(A, B, As_t, Bs_t, "gemv", dict(BLOCK_T=4))
    assert torch.equal(got, want)
    check(got, ref, "strided scales")
    wide = torch.full((m, n + 256), float("nan"), dtype=torch.bfloat16, device="cuda")
    engine.launch(A, B, As, Bs, "gemv", dict(BLOCK_T=2), out=wide[:, 128:128 + n])
    assert torch.equal(wide[:, 128:128 + n], want)
    assert torch.isnan(wide[:, :128]).all() and torch.isnan(wide[:, 128 + n:]).all()


def test_gemv_extra_targets_receive_the_same_tiles():
    """The fused all-gather entry point with a second buffer on the same GPU."""
    m, n, k = 4, 512, 3072
    A, B, As, Bs = (t.cuda() for t in testing.make_problem(m, n, k, seed=9))
    want = engine.launch(A, B, As, Bs, "gemv", dict(BLOCK_T=4))
    a = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    b = torch.zeros_like(a)
    engine.launch(A, B, As, Bs, "gemv", dict(BLOCK_T=4), out=a, also_to=[b.data_ptr()])
    torch.cuda.synchronize()
    assert torch.equal(a, want) and torch.equal(b, want)


def test_gemv_rejects_illegal_tiles():
    A, B, As, Bs = (t.cuda() for t in testing.make_problem(2, 256, 256, seed=1))
    for conf in (dict(BLOCK_T=3), dict(BLOCK_T=8), dict(BLOCK_T=4, BLOCK_W=16)):
        with pytest.raises(ValueError):
            engine.launch(A, B, As, Bs, "gemv", conf)
