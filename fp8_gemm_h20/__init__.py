"""Drop-in import name: `fp8_gemm_h20` is the B200 implementation under the reference's name.

Callers of the reference (`import fp8_gemm_h20`, `from fp8_gemm_h20.config import get_profile`,
`fp8_gemm_h20.engine.kernel(...)`; fp8_gemm_h20/__init__.py:2-5 there) keep working unchanged:
the submodules are the ones of `fp8_gemm_h20_b200`, not copies.
"""
import sys

import fp8_gemm_h20_b200 as _impl
from fp8_gemm_h20_b200 import config, dispatch, engine
from fp8_gemm_h20_b200 import available_profiles, matmul, select, supports

for _name, _mod in (("config", config), ("dispatch", dispatch), ("engine", engine)):
    sys.modules[f"{__name__}.{_name}"] = _mod

__all__ = ["matmul", "available_profiles", "select", "supports"]
