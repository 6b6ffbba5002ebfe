"""Long-running randomised check of the kernel family: many (shape, configuration) pairs, each
replayed back to back under a CUDA graph, compared with the FP32 reference on the GPU and for
bit-repeatability.  Rare hand-shake races (ring-slot parity, TMEM buffer reuse) show up only over
many launches; the suite's other tests launch each configuration once or twice."""
import random

import pytest
import torch

from fp8_gemm_h20_b200 import engine, testing

pytestmark = pytest.mark.gpu


def _random_case(rng):
    k = rng.choice([256, 384, 512, 1024, 2048, 3072, 4096])
    n = rng.choice([128, 512, 1024, 2048, 3072, 4608, 9216])
    kb = k // 128
    splits = [d for d in (1, 2, 3, 4, 6, 8) if kb % d == 0]
    kind = rng.random()
    if kind < 0.5:
        m = rng.choice([1, 3, 8, 16, 17, 37, 64, 100, 128, 200, 255])
        bt = rng.choice([16, 32, 64, 128, 256])
        conf = dict(BLOCK_T=bt, SPLIT=rng.choice(splits), NUM_STAGES=rng.choice([2, 3, 4, 5, 8]),
                    K_GROUP=rng.choice([1, 2]), SPLIT_VIA_WORKSPACE=rng.random() < 0.3)
        return m, n, k, "umma_swap", conf
    m = rng.choice([65, 128, 200, 300, 512, 777, 1024, 2049, 4096])
    bw = rng.choice([128, 256]) if n % 256 == 0 else 128
    tiles = -(-m // 128) * (n // bw)
    split = rng.choice([s for s in splits if tiles * s <= 600] or [1])
    conf = dict(BLOCK_W=bw, SPLIT=split, NUM_STAGES=rng.choice([2, 3, 4, 6]), GROUP_SIZE_M=rng.choice([1, 4, 8]),
                MAX_CTAS=rng.choice([0, 0, 37, 148]), SPLIT_VIA_WORKSPACE=rng.random() < 0.3)
    return m, n, k, "umma", conf


def test_many_random_configurations_replayed():
    rng = random.Random(20261125)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for case in range(250):
            m, n, k, impl, conf = _random_case(rng)
            p = tuple(t.cuda() for t in testing.make_problem(m, n, k, seed=case, mode=rng.choice(["normal", "cfg0", "skew"])))
            ref = testing.reference_fp32(*p)
            first = engine.launch(*p, impl, conf).clone()         # also warms the stream's workspace
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(16):
                    out = engine.launch(*p, impl, conf)
            for _ in range(4):
                graph.replay()
            stream.synchronize()
            what = (case, m, n, k, impl, conf)
            assert engine.device_status() == (0, 0), what
            assert torch.equal(out, first), what
            assert testing.rel_error(out, ref) <= 1e-2 and testing.elementwise_violations(out, ref) == 0, what
