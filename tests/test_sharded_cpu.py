"""N-sharded column-parallel layer on CPU ranks (gloo, world_size 2 and 3): partitioning,
all-gather and column assembly, with the numpy oracle standing in for the shard GEMM.
The gathered result must equal the un-sharded oracle result bit for bit (shards are whole
128-row scale blocks, so a shard computes exactly the columns the full GEMM computes)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

from fp8_gemm_h20_b200 import sharded, testing  # noqa: E402


def test_shard_bounds_cover_n_in_whole_blocks():
    for n, g in [(20480, 1), (20480, 2), (20480, 4), (20480, 8), (18432, 8), (1280, 3), (128 * 7, 4)]:
        b = sharded.shard_bounds(n, g)
        assert b[0][0] == 0 and b[-1][1] == n and len(b) == g
        for (lo, hi), (lo2, _) in zip(b, b[1:] + [(n, n)]):
            assert hi == lo2 and lo % 128 == 0 and hi % 128 == 0 and hi > lo
        sizes = [hi - lo for lo, hi in b]
        assert max(sizes) - min(sizes) <= 128
    assert [hi - lo for lo, hi in sharded.shard_bounds(20480, 8)] == [2560] * 8
    assert [hi - lo for lo, hi in sharded.shard_bounds(18432, 4)] == [4608] * 4
    with pytest.raises(ValueError):
        sharded.shard_bounds(1000, 2)
    with pytest.raises(ValueError):
        sharded.shard_bounds(256, 3)


def _oracle_gemm(A, B, As, Bs, out):
    from oracle import block_fp8_ref as oracle
    c = oracle.gemm_bf16(A.view(torch.uint8).numpy(), B.view(torch.uint8).numpy(), As.numpy(), Bs.numpy())
    out.copy_(torch.from_numpy(c).to(torch.bfloat16))
    return out


def _worker(rank, world, port, n, fail_rank, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, k = 37, 384
        A, B, As, Bs = testing.make_problem(m, n, k, seed=5)          # same bits on every rank
        full = torch.empty(m, n, dtype=torch.bfloat16)
        _oracle_gemm(A, B, As, Bs, full)
        layer = sharded.ColumnParallelFP8Linear(B, Bs, gemm=_oracle_gemm)
        lo, hi = layer.bounds[rank]
        assert layer.B.shape[0] == hi - lo and layer.Bs.shape[0] == (hi - lo) // 128
        out = layer(A, As)
        ok = out.shape == (m, n) and torch.equal(out, full)
        # a second call and a shard-only construction give the same answer
        B_sh, Bs_sh = sharded.shard_weights(B, Bs, rank, world)
        layer2 = sharded.ColumnParallelFP8Linear(B_shard=B_sh, Bs_shard=Bs_sh, n_total=n, gemm=_oracle_gemm)
        ok = ok and torch.equal(layer2(A, As), full) and torch.equal(layer.local(A, As), full[:, lo:hi])
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,n", [(2, 512), (3, 896), (2, 384)])
def test_gather_equals_unsharded_result_on_gloo_ranks(world, n):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, None, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=5) for _ in range(world))
    assert results == {r: True for r in range(world)}


def test_wrong_shard_is_rejected():
    A, B, As, Bs = testing.make_problem(4, 256, 128, seed=1)
    with pytest.raises(ValueError):
        sharded.ColumnParallelFP8Linear(B_shard=B[:128], Bs_shard=Bs[:1], n_total=512, gemm=_oracle_gemm)
    with pytest.raises(ValueError):
        sharded.ColumnParallelFP8Linear(gemm=_oracle_gemm)
