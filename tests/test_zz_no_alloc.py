"""The allocation-free entry point `fp8mm_b200_gemm_static_scratch`, called through the C ABI.

It serves callers that cannot allocate device memory on the GEMM path: a server whose own pool
owns all of HBM, a plug-in inside another runtime's memory manager, a real-time loop that must
stay off the driver's allocation lock.  They pass inputs and the output; the split-K scratch is
a buffer built into the library.  The checks: the same bits as the regular entry point (which is
given a caller-allocated workspace) on two consecutive calls, for split and unsplit
configurations; a problem whose scratch exceeds the built-in 8 MiB is refused, not truncated.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

from fp8_gemm_h20_b200 import _lib, engine, testing

pytestmark = pytest.mark.gpu


def _args(A, B, As, Bs, out):
    m, k = A.shape
    return _lib.Args(A=A.data_ptr(), B=B.data_ptr(), As=As.data_ptr(), Bs=Bs.data_ptr(), C=out.data_ptr(),
                     M=m, N=B.shape[0], K=k, reserved0=0,
                     as_stride_m=As.stride(0), as_stride_k=As.stride(1),
                     bs_stride_n=Bs.stride(0), bs_stride_k=Bs.stride(1), ldc=out.stride(0))


CASES = [
    (37, 512, 3072, "umma_swap", dict(BLOCK_T=64, SPLIT=3)),      # split-K: counters + partials in the scratch
    (200, 3072, 2048, "umma", dict(BLOCK_W=128, SPLIT=2, SPLIT_VIA_WORKSPACE=True)),   # token-major tiles
    (300, 1024, 2048, "umma", dict(BLOCK_W=256, SPLIT=1)),        # unsplit: status word only
]


@pytest.mark.parametrize("m,n,k,impl,conf", CASES)
def test_static_scratch_matches_regular_entry_point_twice(m, n, k, impl, conf):
    lib = _lib.load()
    A, B, As, Bs = (t.cuda() for t in testing.make_problem(m, n, k, seed=m + n + k, mode="cfg0"))
    want = engine.launch(A, B, As, Bs, impl, conf)                  # regular entry point, torch workspace
    ref = testing.reference_fp32(A, B, As, Bs)
    assert testing.rel_error(want, ref) <= 1e-2 and testing.elementwise_violations(want, ref) == 0
    cfg = engine.make_cfg(impl, conf)
    need = lib.fp8mm_b200_workspace_bytes(m, n, k, ctypes.byref(cfg))
    assert 0 < need <= lib.fp8mm_b200_static_scratch_bytes() == 8 << 20
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):                                           # second call reuses what the first left
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.fp8mm_b200_gemm_static_scratch(ctypes.byref(_args(A, B, As, Bs, out)), ctypes.byref(cfg), stream)
        assert rc == 0, _lib.strerror(rc)
        torch.cuda.synchronize()
        assert torch.equal(out, want), (call, impl, conf)
        assert testing.rel_error(out, ref) <= 1e-2 and testing.elementwise_violations(out, ref) == 0
    # no bounded wait gave up; callers of this entry point read the status without a workspace pointer
    detail = ctypes.c_int32(-1)
    assert lib.fp8mm_b200_static_scratch_status(ctypes.byref(detail)) == 0 and detail.value == 0
    assert lib.fp8mm_b200_last_status(None, ctypes.byref(detail)) == 0 and detail.value == 0


def test_static_scratch_allocates_nothing_and_survives_back_to_back_calls():
    """Free device memory is the same before and after a burst of calls, and two calls with different
    tile counts queued on one stream without a host synchronisation in between (the second finds the
    first one's partial tiles and counters in the shared buffer) both give the regular entry point's bits."""
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    probs = []
    for (m, n, k, impl, conf) in CASES[:2]:
        A, B, As, Bs = (t.cuda() for t in testing.make_problem(m, n, k, seed=11 + m, mode="normal"))
        want = engine.launch(A, B, As, Bs, impl, conf)
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        probs.append((A, B, As, Bs, out, want, engine.make_cfg(impl, conf)))
    A, B, As, Bs, out, _, cfg = probs[0]
    assert lib.fp8mm_b200_gemm_static_scratch(ctypes.byref(_args(A, B, As, Bs, out)), ctypes.byref(cfg), stream) == 0
    torch.cuda.synchronize()                                        # first call per device: address look-up done
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(5):
        for A, B, As, Bs, out, _, cfg in probs:                     # no synchronisation between the calls
            rc = lib.fp8mm_b200_gemm_static_scratch(ctypes.byref(_args(A, B, As, Bs, out)), ctypes.byref(cfg), stream)
            assert rc == 0, _lib.strerror(rc)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    for _, _, _, _, out, want, _ in probs:
        assert torch.equal(out, want)
    assert lib.fp8mm_b200_static_scratch_status(None) == 0


def test_static_scratch_refuses_what_does_not_fit():
    lib = _lib.load()
    m, n, k = 256, 12288, 2048
    conf = dict(BLOCK_T=256, SPLIT=4, SPLIT_VIA_WORKSPACE=True)     # 96 tiles x 4 x 256 x 128 fp32 = 50 MB
    cfg = engine.make_cfg("umma_swap", conf)
    assert lib.fp8mm_b200_workspace_bytes(m, n, k, ctypes.byref(cfg)) > lib.fp8mm_b200_static_scratch_bytes()
    A, B, As, Bs = (t.cuda() for t in testing.make_problem(m, n, k, seed=1))
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    rc = lib.fp8mm_b200_gemm_static_scratch(ctypes.byref(_args(A, B, As, Bs, out)), ctypes.byref(cfg),
                                            torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.E_TOO_LARGE and "8 MiB" in _lib.strerror(rc)
    torch.cuda.synchronize()
    assert (out == 0).all()                                         # nothing was enqueued
    bad = engine.make_cfg("umma_swap", dict(BLOCK_T=48))
    rc = lib.fp8mm_b200_gemm_static_scratch(ctypes.byref(_args(A, B, As, Bs, out)), ctypes.byref(bad),
                                            torch.cuda.current_stream().cuda_stream)
    assert rc == -3
