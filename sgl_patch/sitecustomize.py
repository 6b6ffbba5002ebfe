"""Put this directory on PYTHONPATH: runs the interpreter's own sitecustomize first (if any),
then loads the opt-in fp8mm adapter, which does nothing unless FP8MM_ENABLE=1
(reference: sgl_patch/sitecustomize.py:1-16)."""
import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))


def _chain_system_sitecustomize():
    for entry in sys.path:
        if os.path.abspath(entry or ".") == _HERE:
            continue
        candidate = os.path.join(entry, "sitecustomize.py")
        if os.path.isfile(candidate):
            spec = importlib.util.spec_from_file_location("_system_sitecustomize", candidate)
            spec.loader.exec_module(importlib.util.module_from_spec(spec))
            return


_chain_system_sitecustomize()
import fp8mm_sglang_patch  # noqa: E402,F401
