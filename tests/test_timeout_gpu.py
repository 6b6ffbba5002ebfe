"""The give-up path of the kernels' bounded waits, exercised once without a fault.

Every mbarrier wait in the tile kernels has a time limit (FP8MM_TIMEOUT_MS).  Here the limit is 5 ms
and the failure is made on the host: a test-only switch encodes the weight operand's tensor map with
half the box rows, so each weight copy delivers fewer bytes than the producer announced and the
ring's `full` barrier never completes.  Nothing faults, traps or waits forever: the MMA-issuing and
promotion threads run into their limit, record a role code in the status word, every role leaves its
loop, tensor memory is freed and the kernel RETURNS.  The host then reads FP8MM_E_DEVICE_TIMEOUT, clears
the status, and the next ordinary launch in the same process is bit-correct.

Runs in a child process: the time limit is read once per process, and a child keeps the doctored
tensor map out of the other tests' cache."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

CHILD = r"""
import ctypes, os, sys
sys.path.insert(0, %r)
import torch
from fp8_gemm_h20_b200 import _lib, engine, testing

m, n, k = 16, 256, 256
conf = dict(BLOCK_T=16, SPLIT=1, NUM_STAGES=2)
A, B, As, Bs = (t.cuda() for t in testing.make_problem(m, n, k, seed=3))
want = engine.launch(A, B, As, Bs, "umma_swap", conf)          # ordinary launch first
torch.cuda.synchronize()
assert engine.device_status() == (0, 0)

# a second copy of the weights: its (doctored) tensor map is cached under its own address
B2 = B.clone()
os.environ["FP8MM_TEST_SHORT_WEIGHT_BOX"] = "1"
out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
engine.launch(A, B2, As, Bs, "umma_swap", conf, out=out)
del os.environ["FP8MM_TEST_SHORT_WEIGHT_BOX"]
torch.cuda.synchronize()                                       # the kernel came back by itself
rc, detail = engine.device_status()
assert rc == _lib.E_DEVICE_TIMEOUT, (rc, detail)
assert detail in (0x21, 0x42), hex(detail)                     # MMA issuer on `full`, or promotion on `tfull`
print("timed out as planned: role code", hex(detail))

# clear the record, then the library must work as before (B's map was encoded without the switch)
lib = _lib.load()
for ws in engine._workspaces.values():
    assert lib.fp8mm_b200_workspace_init(ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream) == 0
torch.cuda.synchronize()
assert engine.device_status() == (0, 0)
again = engine.launch(A, B, As, Bs, "umma_swap", conf)
big = engine.launch(*(t.cuda() for t in testing.make_problem(300, 1024, 1024, seed=4)), "umma", dict(BLOCK_W=256))
torch.cuda.synchronize()
assert torch.equal(again, want)
assert torch.isfinite(big).all() and engine.device_status() == (0, 0)
print("recovered")
"""


def test_bounded_wait_gives_up_and_the_next_launch_is_correct():
    env = dict(__import__("os").environ, FP8MM_TIMEOUT_MS="5")
    res = subprocess.run([sys.executable, "-c", CHILD % str(ROOT)], env=env, capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "timed out as planned" in res.stdout and "recovered" in res.stdout


CHILD_MX = r"""
import os, sys
sys.path.insert(0, %r)
import torch
from fp8_gemm_h20_b200 import _lib, engine, testing

lib = _lib.load()
m, n, k = 40, 256, 1536
A, B, Au, Bu, As, Bs = (t.cuda() for t in testing.make_problem_ue8m0(m, n, k, seed=3))
forms = {"swap-AB": dict(BLOCK_T=16, BLOCK_W=128), "cluster split": dict(BLOCK_T=16, BLOCK_W=128, SPLIT=4),
         "workspace split": dict(BLOCK_T=32, BLOCK_W=128, SPLIT=3), "half-size": dict(BLOCK_T=64, BLOCK_W=128, NUM_STAGES=2, HALF_FORM=True),
         "token-major": dict(BLOCK_T=128, BLOCK_W=256)}
want = {name: engine.launch(A, B, Au, Bu, "umma_mx", conf) for name, conf in forms.items()}
torch.cuda.synchronize()
assert engine.device_status() == (0, 0)
for name, conf in forms.items():
    B2 = B.clone()                      # its (doctored) tensor map is cached under its own address
    os.environ["FP8MM_TEST_SHORT_WEIGHT_BOX"] = "1"
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    engine.launch(A, B2, Au, Bu, "umma_mx", conf, out=out)
    del os.environ["FP8MM_TEST_SHORT_WEIGHT_BOX"]
    torch.cuda.synchronize()            # the kernel came back by itself
    rc, detail = engine.device_status()
    assert rc == _lib.E_DEVICE_TIMEOUT and detail != 0, (name, rc, detail)
    assert not out.any(), name          # no CTA (no rank of a cluster either) stored anything
    print("timed out as planned:", name, hex(detail))
    for ws in engine._workspaces.values():
        assert lib.fp8mm_b200_workspace_init(ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert engine.device_status() == (0, 0)
    assert torch.equal(engine.launch(A, B, Au, Bu, "umma_mx", conf), want[name]), name
print("recovered")
"""


def test_block_scaled_kernels_give_up_and_recover():
    """The same for every form of the block-scaled kernels; with split-K no rank may store a tile to which one
    rank contributed nothing."""
    env = dict(__import__("os").environ, FP8MM_TIMEOUT_MS="5")
    res = subprocess.run([sys.executable, "-c", CHILD_MX % str(ROOT)], env=env, capture_output=True, text=True,
                         timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.count("timed out as planned") == 5 and "recovered" in res.stdout
