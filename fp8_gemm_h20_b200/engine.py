"""Kernel registry: table `impl` name -> launcher over the native sm_100a library.

Same surface as the reference registry (fp8_gemm_h20/engine.py:5-19): `KERNELS`,
`kernel(name)` returning `fn(A, B, As, Bs, config) -> C`, and `run(entry, args)`.
The callables here do what the reference's per-kernel host wrappers did
(kernels/kernel_v2.py:339-376): merge defaults, keep a zeroed workspace per
(device, stream), allocate the bf16 output, and enqueue one launch on the current
stream.  The kernels themselves are CUDA (csrc/fp8mm_kernel.cuh), not JIT code.
"""
import ctypes
from functools import lru_cache

from . import _lib

# impl name -> (native impl id, defaults merged under the table's config)
KERNELS = {
    "umma": (_lib.IMPL_UMMA, {"BLOCK_T": 128, "BLOCK_W": 256, "NUM_STAGES": 4, "SPLIT": 1,
                              "GROUP_SIZE_M": 8, "MAX_CTAS": 0}),
    "umma_2cta": (_lib.IMPL_UMMA_2CTA, {"BLOCK_T": 256, "BLOCK_W": 256, "NUM_STAGES": 5, "SPLIT": 1,
                                        "GROUP_SIZE_M": 8, "MAX_CTAS": 0}),
    "umma_swap": (_lib.IMPL_UMMA_SWAP, {"BLOCK_T": 16, "BLOCK_W": 128, "NUM_STAGES": 8, "SPLIT": 1,
                                        "GROUP_SIZE_M": 1, "MAX_CTAS": 0}),
    # decode: BLOCK_T tokens per warp (1, 2 or 4), eight weight rows per warp step, FP32 FMAs
    "gemv": (_lib.IMPL_GEMV, {"BLOCK_T": 1, "BLOCK_W": 8, "NUM_STAGES": 1, "SPLIT": 1,
                              "GROUP_SIZE_M": 1, "MAX_CTAS": 0}),
    # power-of-two scales: As, Bs are uint8 UE8M0 exponents, applied by the block-scaled MMA itself
    "umma_mx": (_lib.IMPL_UMMA_MX, {"BLOCK_T": 128, "BLOCK_W": 256, "NUM_STAGES": 4, "SPLIT": 1,
                                    "GROUP_SIZE_M": 8, "MAX_CTAS": 0}),
}

_MIN_WORKSPACE = 1 << 20          # bytes; grown on demand, never shrunk
_workspaces = {}                  # (device index, stream handle) -> uint8 tensor


def _k_group_flag(kg):
    """K blocks per ring slot -> cfg.flags bits (2 keeps its historical bit)."""
    if kg <= 1:
        return 0
    return 2 if kg == 2 else (kg & 15) << 8


def make_cfg(impl, config):
    """Table entry -> native fp8mm_cfg."""
    impl_id, defaults = KERNELS[impl]
    c = dict(defaults)
    c.update(config)
    return _lib.Cfg(impl=impl_id, block_t=int(c["BLOCK_T"]), block_w=int(c["BLOCK_W"]),
                    stages=int(c["NUM_STAGES"]), split=int(c["SPLIT"]),
                    group_m=int(c["GROUP_SIZE_M"]), max_ctas=int(c.get("MAX_CTAS", 0)),
                    flags=(1 if c.get("SPLIT_VIA_WORKSPACE") else 0) | _k_group_flag(int(c.get("K_GROUP", 1)))
                    | (2 if c.get("HALF_FORM") else 0)
                    | (4 if c.get("SCALES_UE8M0") else 0) | (8 if c.get("ACT_SCALES_F32") else 0))


def _workspace(torch, device, stream, nbytes):
    """Zeroed scratch (status word, split-K counters, fp32 partials), one per (device, stream)
    as in the reference (kernel_v2.py:309-324).  The cache is never touched while a CUDA graph
    is being captured: a capture on a stream that has no workspace yet (torch.cuda.graph picks
    its own side stream) gets a private zeroed buffer from the graph's memory pool instead,
    at the price of one memset node per call; warm up on the capture stream to avoid it."""
    key = (device.index, stream)
    ws = _workspaces.get(key)
    if ws is not None and ws.numel() >= nbytes:
        return ws
    if torch.cuda.is_current_stream_capturing():
        return torch.zeros(int(nbytes), dtype=torch.uint8, device=device)
    ws = torch.zeros(max(_MIN_WORKSPACE, int(nbytes)), dtype=torch.uint8, device=device)
    _workspaces[key] = ws
    return ws


@lru_cache(maxsize=8192)
def _plan(impl, conf_items, m, n, k):
    """(native cfg, workspace bytes) for one (table entry, problem): built once, reused by every
    later call with the same entry and shape, so the per-call host path is one struct and one
    foreign call.  The workspace is sized for the workspace reduction even where a cluster launch
    is planned, so that the library can fall back where clusters have no room."""
    lib = _lib.load()
    cfg = make_cfg(impl, dict(conf_items))
    need = lib.fp8mm_b200_workspace_bytes(m, n, k, ctypes.byref(cfg))
    if need == 0:
        rc = lib.fp8mm_b200_validate(m, n, k, ctypes.byref(cfg))
        raise ValueError(f"fp8mm: {_lib.strerror(rc)} (impl={impl}, config={dict(conf_items)}, M,N,K={m},{n},{k})")
    if cfg.split > 1 and not cfg.flags & 1:
        alt = make_cfg(impl, dict(conf_items, SPLIT_VIA_WORKSPACE=True))
        need = max(need, lib.fp8mm_b200_workspace_bytes(m, n, k, ctypes.byref(alt)))
    return cfg, need


def launch(A, B, As, Bs, impl, config, out=None, also_to=()):
    """Enqueue C = blockscaled(A @ B^T) on the current stream of A.device and return C.

    `out`, when given, is a bf16 [M, N] view whose rows may be strided (row stride a
    multiple of 8 elements): the N-sharded layer writes shards into a wider buffer.
    `also_to` lists up to 7 device addresses (ints) of further buffers with the layout of
    `out` — the peers' copies of an N-sharded layer's output — that receive the same tiles
    from the kernel's epilogue (fused all-gather, fp8mm_b200_gemm_bcast)."""
    import torch
    lib = _lib.load()
    m, k = A.shape
    n = B.shape[0]
    cfg, need = _plan(impl, tuple(sorted(config.items())), m, n, k)
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=A.device)
    elif out.dtype != torch.bfloat16 or tuple(out.shape) != (m, n) or out.stride(1) != 1:
        raise ValueError("out must be a bfloat16 [M,N] tensor with unit column stride")
    stream = torch.cuda.current_stream(A.device).cuda_stream
    ws = _workspace(torch, A.device, stream, need)
    args = _lib.Args(A=A.data_ptr(), B=B.data_ptr(), As=As.data_ptr(), Bs=Bs.data_ptr(), C=out.data_ptr(),
                     M=m, N=n, K=k, reserved0=0,
                     as_stride_m=As.stride(0), as_stride_k=As.stride(1),
                     bs_stride_n=Bs.stride(0), bs_stride_k=Bs.stride(1), ldc=out.stride(0))
    if also_to:
        extra = (ctypes.c_void_p * len(also_to))(*[int(x) for x in also_to])
        rc = lib.fp8mm_b200_gemm_bcast(ctypes.byref(args), ctypes.byref(cfg), ws.data_ptr(), ws.numel(), stream,
                                       extra, len(also_to))
    else:
        rc = lib.fp8mm_b200_gemm(ctypes.byref(args), ctypes.byref(cfg), ws.data_ptr(), ws.numel(), stream)
    if rc != 0:
        raise RuntimeError(f"fp8mm_b200_gemm failed: {_lib.strerror(rc)} "
                           f"(impl={impl}, config={dict(config)}, M,N,K={m},{n},{k})")
    return out


def device_status(device=None):
    """Synchronise and return (code, detail) of the workspaces on `device`: code 0 unless a
    bounded device-side wait gave up (then the kernel left early and the output is invalid)."""
    import torch
    lib = _lib.load()
    worst = (0, 0)
    for (dev, _stream), ws in list(_workspaces.items()):
        if device is not None and torch.device(device).index not in (None, dev):
            continue
        torch.cuda.synchronize(dev)
        detail = ctypes.c_int32(0)
        with torch.cuda.device(dev):
            rc = lib.fp8mm_b200_last_status(ws.data_ptr(), ctypes.byref(detail))
        if rc != 0:
            worst = (rc, detail.value)
    return worst


@lru_cache(maxsize=None)
def kernel(name):
    """Callable `fn(A, B, As, Bs, config)` for a table `impl` name (engine.py:13-16)."""
    if name not in KERNELS:
        raise KeyError(name)

    def fn(A, B, As, Bs, config):
        return launch(A, B, As, Bs, name, config)

    fn.__name__ = f"block_fp8_gemm_{name}_b200"
    return fn


def run(entry, args):
    """Run a table entry on (A, B, As, Bs) (engine.py:18-19)."""
    return kernel(entry["impl"])(*args, dict(entry["config"]))
