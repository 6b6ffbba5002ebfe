"""Opt-in SGLang adapter: send SGLang's dense block-FP8 linear to fp8_gemm_h20.matmul.

Same contract as the reference adapter (sgl_patch/fp8mm_sglang_patch.py:11-96): nothing
happens unless FP8MM_ENABLE=1; then an import hook waits for
`sglang.srt.layers.quantization.fp8_utils` and wraps its `dispatch_w8a8_block_fp8_linear`.
Only when SGLang itself would have picked its DeepGEMM linear is the call redirected, and
only for inputs the selected profile covers; everything else goes to SGLang's own function
untouched, before any quantisation work.

Environment:
  FP8MM_ENABLE=1                   turn the adapter on
  FP8MM_PROFILE=35b_tp1|122b_tp4   tuning profile (default 35b_tp1)
  FP8MM_HOME=/path/to/this/repo    prepended to sys.path
  FP8MM_DISABLE_DG_PRECOMPILE=1    also skip DeepGEMM's all-M JIT precompile, unused once patched
  FP8MM_UE8M0_NATIVE=0             with FP8MM_UE8M0=1: expand packed power-of-two weight scales to float32 and use
                                   the profile's table kernels instead of the kernels that take the exponents
  FP8MM_UE8M0=1                    also engage when SGLang runs with DEEPGEMM_SCALE_UE8M0 (its default
                                   on Blackwell): power-of-two scales are taken as float32, or expanded
                                   from the packed int32 form once per weight; the activation quantiser
                                   is asked for power-of-two scales (scale_ue8m0=True).  Without this
                                   switch such calls go to SGLang's own function, as in the reference
                                   adapter (sgl_patch/fp8mm_sglang_patch.py:41).
"""
import os
import sys

if os.environ.get("FP8MM_ENABLE") == "1":
    sys.path.insert(0, os.environ.get("FP8MM_HOME", "/root/fp8mm"))
    if os.environ.get("FP8MM_DISABLE_DG_PRECOMPILE") == "1":
        os.environ["SGLANG_JIT_DEEPGEMM_PRECOMPILE"] = "0"

    import importlib.abc
    import importlib.machinery

    _TARGET = "sglang.srt.layers.quantization.fp8_utils"

    def _install(mod):
        """Wrap mod.dispatch_w8a8_block_fp8_linear (reference :22-71)."""
        import torch
        import fp8_gemm_h20 as fp8mm
        from fp8_gemm_h20.config import get_profile

        profile = os.environ.get("FP8MM_PROFILE", "35b_tp1")
        covered = sorted(get_profile(profile)["entries"])
        sgl_dispatch = mod.dispatch_w8a8_block_fp8_linear
        quantize = mod.sglang_per_token_group_quant_fp8
        stats = {"ours": 0, "fallback": 0}

        ue8m0_mode = os.environ.get("FP8MM_UE8M0") == "1"
        expanded = {}     # packed weight scales -> float32, keyed by storage address (weights are static)

        def weight_scales_f32(weight, weight_scale):
            """float32 [N/128, K/128] scales of a weight whose scales are UE8M0 words (int32, four
            K blocks per word, one row per 128-row block or per weight row)."""
            key = (weight_scale.data_ptr(), tuple(weight_scale.shape), tuple(weight_scale.stride()))
            hit = expanded.get(key)
            if hit is None:
                from fp8_gemm_h20_b200.quant import expand_ue8m0
                n, k = weight.shape
                full = expand_ue8m0(weight_scale)[:, :k // 128]
                hit = (full if full.shape[0] == n // 128 else full[::128]).contiguous()
                expanded[key] = hit
            return hit

        def eligible(input, weight, block_size, weight_scale, input_scale):
            if input_scale is not None or input.dtype != torch.bfloat16:
                return False
            if list(block_size) != [128, 128]:
                return False
            ue8m0 = bool(getattr(mod, "DEEPGEMM_SCALE_UE8M0", False))
            if ue8m0 and not ue8m0_mode:
                return False
            if weight_scale.dtype != torch.float32:
                n, k = weight.shape
                if not (ue8m0 and weight_scale.dtype == torch.int32 and weight_scale.ndim == 2
                        and weight_scale.shape[0] in (n // 128, n)
                        and weight_scale.shape[1] * 4 >= k // 128):
                    return False
            if not (input.is_contiguous() and weight.is_contiguous()):
                return False
            if weight.dtype != torch.float8_e4m3fn:
                return False
            n, k = weight.shape
            return fp8mm.supports(profile, input.numel() // k, n, k)

        def wrap(sgl_linear):
            def fp8mm_w8a8_block_fp8_linear(input, weight, block_size, weight_scale, input_scale=None, bias=None):
                if not eligible(input, weight, block_size, weight_scale, input_scale):
                    stats["fallback"] += 1
                    return sgl_linear(input, weight, block_size, weight_scale, input_scale, bias)
                stats["ours"] += 1
                n, k = weight.shape
                # row-major [M, K/128] float32 activation scales, the layout matmul expects
                if getattr(mod, "DEEPGEMM_SCALE_UE8M0", False):
                    q, s = quantize(input.view(-1, k), block_size[1], column_major_scales=False,
                                    scale_tma_aligned=False, scale_ue8m0=True)
                    if weight_scale.dtype != torch.float32:
                        from fp8_gemm_h20_b200 import quant
                        if os.environ.get("FP8MM_UE8M0_NATIVE", "1") != "0":
                            # the packed exponent words go to the kernels as they are and the float32
                            # power-of-two activation scales too (the kernels take the exponent field): the
                            # tensor cores' own block scaling from five tokens on, the decode kernel below
                            ws = weight_scale if weight_scale.shape[0] == n // 128 else weight_scale[::128]
                            out = quant.matmul_ue8m0(q, weight, s, ws, profile=profile)
                            if bias is not None:
                                out = out + bias
                            return out.view(*input.shape[:-1], n)
                        weight_scale = weight_scales_f32(weight, weight_scale)
                else:
                    q, s = quantize(input.view(-1, k), block_size[1], column_major_scales=False,
                                    scale_tma_aligned=False)
                out = fp8mm.matmul(q, weight, s, weight_scale, profile=profile)
                if bias is not None:
                    out = out + bias
                return out.view(*input.shape[:-1], n)

            fp8mm_w8a8_block_fp8_linear.fp8mm_stats = stats
            return fp8mm_w8a8_block_fp8_linear

        def patched_dispatch():
            chosen = sgl_dispatch()
            if chosen is not mod.deepgemm_w8a8_block_fp8_linear_with_fallback:
                return chosen            # some other backend was selected: leave it alone
            return wrap(chosen)

        mod.dispatch_w8a8_block_fp8_linear = patched_dispatch
        print(f"[fp8mm] patched {_TARGET}.dispatch_w8a8_block_fp8_linear "
              f"(profile={profile}, table NK={covered}, "
              f"dg_precompile={os.environ.get('SGLANG_JIT_DEEPGEMM_PRECOMPILE', '1')})",
              file=sys.stderr, flush=True)

    class _Loader(importlib.abc.Loader):
        """Runs the real loader, then patches the freshly executed module."""

        def __init__(self, inner):
            self.inner = inner

        def create_module(self, spec):
            return self.inner.create_module(spec)

        def exec_module(self, module):
            self.inner.exec_module(module)
            _install(module)

    class _Finder(importlib.abc.MetaPathFinder):
        def find_spec(self, name, path, target=None):
            if name != _TARGET:
                return None
            spec = importlib.machinery.PathFinder.find_spec(name, path)
            if spec is None or spec.loader is None:
                return None
            spec.loader = _Loader(spec.loader)
            return spec

    sys.meta_path.insert(0, _Finder())
