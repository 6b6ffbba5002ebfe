"""Build libfp8mm_b200.so in-tree with nvcc for sm_100a.

    python -m fp8_gemm_h20_b200.build [--force] [--verbose]

Cross-compiles without a GPU.  The library is the product's only native code; it has
no torch dependency and is loaded through ctypes (fp8_gemm_h20_b200/_lib.py).
"""
import argparse
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
SOURCES = [PKG / "csrc" / "fp8mm_b200.cu", PKG / "csrc" / "fp8mm_quant.cu"]
HEADERS = [PKG / "csrc" / "fp8mm_kernel.cuh", PKG / "csrc" / "fp8mm_kernel_2cta.cuh", PKG / "csrc" / "fp8mm_gemv.cuh",
           PKG / "csrc" / "ptx_sm100.cuh",
           PKG.parent / "include" / "fp8mm_b200.h"]
OUT = PKG / "libfp8mm_b200.so"
TRACE_OUT = PKG / "libfp8mm_b200_trace.so"      # -DFP8MM_TRACE: clock stamps at the role hand-overs (trace.py)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def up_to_date(out=OUT):
    if not out.is_file():
        return False
    t = out.stat().st_mtime
    return all(p.stat().st_mtime <= t for p in SOURCES + HEADERS + [Path(__file__)])


def build(force=False, verbose=False, trace=False, defines=()):
    """defines: extra -D macros for the trace library, e.g. FP8MM_KNOBS=1 (no tcgen05.ld), =2 (no operand
    copies), =4 (no promotion FMAs), FP8MM_SPIN_MASK=1|2 (no suspend hint on the TMEM-buffer waits)."""
    out = TRACE_OUT if trace else OUT
    if defines and not trace:
        raise ValueError("extra defines are for the trace library only")
    if not force and not defines and up_to_date(out):
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *NVCC_FLAGS, *(["-DFP8MM_TRACE"] if trace else []), *[f"-D{d}" for d in defines],
           *(["-Xptxas", "-v"] if verbose else []), "-o", str(out), *map(str, SOURCES)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode:
        raise RuntimeError(f"nvcc failed ({res.returncode}): {' '.join(cmd)}")
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--trace", action="store_true", help="build the instrumented library (libfp8mm_b200_trace.so)")
    ap.add_argument("-D", dest="defines", action="append", default=[], metavar="MACRO[=VALUE]",
                    help="with --trace: extra macro, e.g. -D FP8MM_KNOBS=1")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.trace, a.defines))
