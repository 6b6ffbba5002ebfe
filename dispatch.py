"""Legacy research API of the 35B experiments, kept so that historical scripts (`import dispatch`)
run against this library unchanged.  New code should import `fp8_gemm_h20`.

Mirrors the reference's root-level dispatch.py (dispatch.py:1-50 there): `pick`, `matmul`,
`_TABLE`, `IMPLS`, the FP8MM_PROFILE switch and the historical DISPATCH_LOOKUP=ceil rule.  The
historical kernel names ("c3" = the generic Triton kernel, "c9"/"c11" = the Gluon kernels) have
no counterpart on sm_100a; here each of them runs the untuned-but-sensible sm_100a
configuration for the problem (fp8_gemm_h20_b200.tune.heuristic), or the configuration that is
passed in.
"""
import os

from fp8_gemm_h20 import matmul as _matmul, select, supports
from fp8_gemm_h20.config import get_profile
from fp8_gemm_h20.engine import KERNELS, kernel

_PROFILE = os.environ.get("FP8MM_PROFILE", "35b_tp1")
_TABLE = {nk: {m: {"impl": e["impl"], "cfg": e["config"]} for m, e in rows.items()}
          for nk, rows in get_profile(_PROFILE)["entries"].items()}
_LOOKUP = os.environ.get("DISPATCH_LOOKUP", "nearest")


def pick(M, N, K):
    """(impl, cfg) for one problem.  A shape outside the 35B table falls back to ("c3", None),
    the generic kernel with its own defaults, as it always did; other profiles raise."""
    if not supports(_PROFILE, M, N, K):
        if _PROFILE not in ("35b_tp1", "b200_35b_tp1"):
            raise ValueError(f"Unsupported shape for {_PROFILE}")
        return "c3", None
    if _LOOKUP == "ceil" and _PROFILE in ("35b_tp1", "b200_35b_tp1"):
        table = _TABLE[f"{N},{K}"]
        ge = [int(m) for m in table if int(m) >= M]
        anchor = str(min(ge)) if ge else max(table, key=int)
        return table[anchor]["impl"], table[anchor]["cfg"]
    entry, _ = select(_PROFILE, M, N, K)
    return entry["impl"], entry["config"]


def _generic(A, B, As, Bs, cfg=None):
    """Historical kernel names: run the configuration given, else the heuristic one."""
    if cfg and "impl" in cfg:
        return kernel(cfg["impl"])(A, B, As, Bs, {k: v for k, v in cfg.items() if k != "impl"})
    from fp8_gemm_h20_b200.tune import heuristic
    entry = heuristic(A.shape[0], B.shape[0], A.shape[1])
    return kernel(entry["impl"])(A, B, As, Bs, entry["config"])


def _named(name):
    def invoke(A, B, As, Bs, cfg=None):
        return kernel(name)(A, B, As, Bs, cfg or {})
    return invoke


IMPLS = {name: _named(name) for name in KERNELS}
IMPLS.update({"c3": _generic, "c9": _generic, "c11": _generic})


def matmul(A, B, As, Bs):
    if supports(_PROFILE, A.shape[0], B.shape[0], A.shape[1]) and _LOOKUP != "ceil":
        return _matmul(A, B, As, Bs, profile=_PROFILE)
    impl, cfg = pick(A.shape[0], B.shape[0], A.shape[1])
    return IMPLS[impl](A, B, As, Bs, cfg)
