"""N-sharded layer on two real GPUs: shard GEMMs + NCCL all-gather must reproduce the 1-GPU
result (same kernel config per shard => bit-equal columns).  Skipped on single-GPU boxes."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from fp8_gemm_h20_b200 import engine, sharded, testing
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=120))
    try:
        ok = True
        for m, n, k in [(37, 1024, 512), (300, 2048, 1024)]:
            A, B, As, Bs = (t.cuda() for t in testing.make_problem(m, n, k, seed=9))
            conf = ("umma_swap", dict(BLOCK_T=64, SPLIT=2)) if m <= 64 else ("umma", dict(BLOCK_W=128))
            gemm = lambda a, b, sa, sb, out: engine.launch(a, b, sa, sb, conf[0], conf[1], out=out)
            layer = sharded.ColumnParallelFP8Linear(B, Bs, gemm=gemm)
            out = layer(A, As)
            full = engine.launch(A, B, As, Bs, *conf)
            ref = testing.reference_fp32(A, B, As, Bs)
            ok = ok and torch.equal(out, full) and testing.rel_error(out, ref) <= 1e-2
        # fused path: the GEMM epilogue stores straight into every rank's symmetric output buffer
        for m, n, k in [(37, 5120, 3072), (300, 5120, 3072), (2048, 4608, 3072)]:
            A, B, As, Bs = (t.cuda() for t in testing.make_problem(m, n, k, seed=3))
            plain = sharded.ColumnParallelFP8Linear(B, Bs)
            fused = sharded.ColumnParallelFP8Linear(B, Bs, fused=True, max_tokens=2048)
            want = plain(A, As)
            for _ in range(3):                       # repeated calls reuse the symmetric buffer
                got = fused(A, As).clone()
                ok = ok and torch.equal(got, want)
            ok = ok and testing.rel_error(got, testing.reference_fp32(A, B, As, Bs)) <= 1e-2
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_gather_equals_single_gpu_result():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(300)
    finally:
        # a rank that hangs must not keep holding a GPU of the shared machine after the test
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
            if p.is_alive():
                p.kill()
                p.join(10)
    assert [p.exitcode for p in procs] == [0, 0]
    assert dict(q.get(timeout=5) for _ in range(2)) == {0: True, 1: True}


@pytest.mark.parametrize("impl,conf,m", [
    ("umma", dict(BLOCK_W=256), 300),                              # TMA-store epilogue, two slabs
    ("umma", dict(BLOCK_W=128, SPLIT=2), 200),                     # cluster split-K, plain stores
    ("umma", dict(BLOCK_W=128, SPLIT=2, SPLIT_VIA_WORKSPACE=True), 200),
    ("umma_swap", dict(BLOCK_T=64, SPLIT=1), 37),                  # swap-AB store loop
    ("umma_swap", dict(BLOCK_T=32, SPLIT=4), 17),                  # swap-AB cluster reduction
    ("umma_2cta", dict(), 512),
])
def test_multi_target_epilogue_on_one_gpu(impl, conf, m):
    """fp8mm_b200_gemm_bcast with the extra targets on the SAME GPU: every epilogue variant must put
    the same tiles into all targets (this is the only fused-path coverage a single-GPU run has)."""
    from fp8_gemm_h20_b200 import engine, testing
    n, k = 1024, 1024
    A, B, As, Bs = (t.cuda() for t in testing.make_problem(m, n, k, seed=7))
    want = engine.launch(A, B, As, Bs, impl, conf)
    wide = [torch.full((m, 3 * n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    lo = n          # the shard's column slice inside a wider output
    engine.launch(A, B, As, Bs, impl, conf, out=wide[0][:, lo:lo + n],
                  also_to=[w[:, lo:lo + n].data_ptr() for w in wide[1:]])
    torch.cuda.synchronize()
    for w in wide:
        assert torch.equal(w[:, lo:lo + n], want)
        assert torch.isnan(w[:, :lo]).all() and torch.isnan(w[:, lo + n:]).all()
    assert engine.device_status() == (0, 0)
