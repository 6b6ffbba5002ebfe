"""Correctness, CUDA-graph replay on two streams, strided scales and optional timing over a whole
profile - the B200 counterpart of the reference's scripts/validate.py (:39-118 there), with the
same options, checks and JSON report:

    python -m fp8_gemm_h20_b200.validate --profile 35b_tp1 --output report.json
                                         [--reference DIR] [--timing] [--quick] [--ue8m0]

* accuracy: every (N,K) of the profile x the reference's M lists x {normal, outlier, skew, zero}:
  finite and max|C-ref|/max|ref| < 1e-2 against dequantise -> FP32 matmul on the GPU;
* --reference DIR: migration check - DIR holds another build of this operator (a checkout whose
  root has a `dispatch.py` with `matmul(A,B,As,Bs)`); every output must be bit-identical to it;
* graphs: one representative problem per kernel path, captured on two streams and replayed 100x;
* strided scales: both scale tensors as transposed-contiguous views;
* --timing: median microseconds under graph replay for M in {1,37,64,128,200,511,512,8192};
* --ue8m0: the same run through `matmul_ue8m0`: the same data quantised with power-of-two scales (exponent
  bytes), the decode / block-scaled kernels chosen by `quant.plan_ue8m0` instead of the profile's table.
Use CUDA_VISIBLE_DEVICES to pick the GPU.
"""
import argparse
import importlib
import json
import statistics
import sys
from pathlib import Path

MS_35 = [1, 8, 16, 37, 64, 100, 128, 200, 256, 333, 512, 777, 1000, 2048, 3000, 4096, 5000, 8192, 12000, 16384]
MS_122 = sorted(set([1, 7, 16, 32, 37, 64, 100, 128, 192, 200, 256, 333, 384, 512, 768, 777, 1024, 2048, 4096,
                     4097, 8192, 16384, 15, 17, 31, 33, 63, 65, 127, 129, 193, 255, 257, 383, 385, 511, 513,
                     1023, 1025, 2049, 23, 39, 95, 130, 191, 258, 510, 1026, 47, 79, 194, 509]))
MS_QUICK = [1, 37, 200, 777, 4097]
MODES = ("normal", "outlier", "skew", "zero")
TIMED_MS = (1, 37, 64, 128, 200, 511, 512, 8192)


def summary_markdown(report, ms, argv):
    """The run in a dozen lines: what the reference keeps as experiments/unification/summary.json."""
    acc = report["accuracy"]
    worst = max(acc, key=lambda r: r["error"])
    by_mode = {mode: max(r["error"] for r in acc if r["mode"] == mode) for mode in MODES}
    shapes = sorted({(r["N"], r["K"]) for r in acc})
    kind = " with power-of-two (UE8M0) scales through `matmul_ue8m0`" if report.get("scales") == "ue8m0" else ""
    lines = [f"# Acceptance run: profile `{report['profile']}`{kind} on {report['device']}", "",
             f"Command: `python -m fp8_gemm_h20_b200.validate {' '.join(argv)}`", "",
             f"* accuracy: **{len(acc)} cases** = {len(shapes)} shapes x {len(ms)} token counts x {len(MODES)} "
             f"distributions, every output finite and max|C-ref|/max|ref| < 1e-2 against dequantise -> FP32 matmul "
             f"(TF32 off) on the GPU; status **{report['status']}**",
             f"* worst error **{report['worst_error']:.3e}** at M={worst['M']}, N={worst['N']}, K={worst['K']}, "
             f"`{worst['mode']}` (the reference's own runs on H20: 3.797e-3 / 3.810e-3, "
             "experiments/unification/summary.json there)",
             "* worst error per distribution: " + ", ".join(f"{m} {e:.3e}" for m, e in by_mode.items()),
             f"* token counts: {ms}",
             f"* two-stream CUDA-graph replay (100 interleaved replays per stream): {len(report['graphs'])} kernel "
             f"paths, worst error {max(max(g['errors']) for g in report['graphs']):.3e}",
             f"* strided (transposed-contiguous) scales: {len(report['strided_scales'])} paths, worst error "
             f"{max(r['error'] for r in report['strided_scales']):.3e}"]
    if report["timing"]:
        lines += ["", "| N | K | M | median us |", "|---|---|---|---|"]
        lines += [f"| {t['N']} | {t['K']} | {t['M']} | {t['median_us']['b200']:.2f} |" for t in report["timing"]]
    return "\n".join(lines) + "\n"


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--profile", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--reference", help="directory of another build whose dispatch.matmul must match bit for bit")
    ap.add_argument("--timing", action="store_true")
    ap.add_argument("--quick", action="store_true", help="five token counts per shape instead of the full list")
    ap.add_argument("--rounds", type=int, default=5)
    ap.add_argument("--summary-md", help="also write a short markdown summary of the run to this path")
    ap.add_argument("--ue8m0", action="store_true",
                    help="power-of-two scales as exponent bytes through matmul_ue8m0 (no table involved)")
    a = ap.parse_args(argv)

    import torch
    from . import matmul, select
    from .config import get_profile
    from .testing import make_problem, make_problem_ue8m0, reference_fp32, rel_error
    from .tune import bench_us
    from . import quant

    torch.backends.cuda.matmul.allow_tf32 = False
    prior = None
    if a.reference:
        sys.path.insert(0, str(Path(a.reference).resolve()))
        prior = importlib.import_module("dispatch").matmul
    config = get_profile(a.profile)
    ms = MS_QUICK if a.quick else (MS_35 if "35b" in a.profile else MS_122)
    report = dict(profile=a.profile, device=torch.cuda.get_device_name(), torch=torch.__version__,
                  scales="ue8m0" if a.ue8m0 else "fp32", accuracy=[], timing=[], graphs=[], strided_scales=[])

    def problem(m, n, k, mode, seed_shift=0):
        seed = m + n + k + 113 + seed_shift
        if not a.ue8m0:
            return tuple(t.cuda() for t in make_problem(m, n, k, seed=seed, mode=mode))
        return tuple(t.cuda() for t in make_problem_ue8m0(m, n, k, seed=seed, mode=mode)[:4])

    if a.ue8m0:
        if a.reference:
            raise SystemExit("--reference compares table kernels; it does not go with --ue8m0")
        plain_reference = reference_fp32

        def reference_fp32(A, B, Au, Bu):        # noqa: F811  (the scales as floats: exact, they are powers of two)
            As, Bs = (torch.exp2(t.float() - 127.0) for t in (Au, Bu))
            return plain_reference(A, B, As, Bs)

        def matmul(A, B, Au, Bu, profile=None):  # noqa: F811
            return quant.matmul_ue8m0(A, B, Au, Bu)

    reps = {}
    for nk in config["entries"]:
        n, k = map(int, nk.split(","))
        for m in ms:
            if a.ue8m0:
                impl, c = quant.plan_ue8m0(m, n, k)
                entry = {"impl": impl, "config": c}
            else:
                entry, _ = select(a.profile, m, n, k)
                c = entry["config"]
            reps.setdefault((entry["impl"], c.get("BLOCK_T"), c.get("BLOCK_W"), c.get("SPLIT", 1) > 1, k), (m, n, k))
            for mode in MODES:
                args = problem(m, n, k, mode)
                ref = reference_fp32(*args)
                out = matmul(*args, profile=a.profile)
                err = rel_error(out, ref)
                if not (bool(torch.isfinite(out).all()) and err < 0.01):
                    raise AssertionError((m, n, k, mode, err))
                parity = None
                if prior is not None:
                    parity = bool(torch.equal(out, prior(*args)))
                    if not parity:
                        raise AssertionError((m, n, k, mode, "migration output mismatch"))
                report["accuracy"].append(dict(M=m, N=n, K=k, mode=mode, error=err, bitwise_equal=parity))
            if a.timing and m in TIMED_MS:
                args = problem(m, n, k, "normal")
                funcs = {"b200": lambda: matmul(*args, profile=a.profile)}
                if prior is not None:
                    funcs["original"] = lambda: prior(*args)
                samples = {name: [] for name in funcs}
                for rnd in range(a.rounds):
                    for name in list(funcs)[::1 if rnd % 2 == 0 else -1]:      # alternate the order
                        samples[name].append(bench_us(funcs[name], torch, rounds=1))
                report["timing"].append(dict(M=m, N=n, K=k, samples_us=samples,
                                             median_us={nm: statistics.median(v) for nm, v in samples.items()}))
            print("checked", a.profile, m, n, k, flush=True)

    for m, n, k in reps.values():
        streams = [torch.cuda.Stream(), torch.cuda.Stream()]
        args_list = [problem(m, n, k, "normal"), problem(m, n, k, "normal", seed_shift=1)]
        refs = [reference_fp32(*args) for args in args_list]
        graphs, outs = [], []
        for stream, args in zip(streams, args_list):
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                for _ in range(3):
                    matmul(*args, profile=a.profile)
        torch.cuda.synchronize()
        for stream, args in zip(streams, args_list):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                out = matmul(*args, profile=a.profile)
            graphs.append(g)
            outs.append(out)
        for _ in range(100):
            for stream, g in zip(streams, graphs):
                with torch.cuda.stream(stream):
                    g.replay()
        torch.cuda.synchronize()
        errs = [rel_error(out, ref) for out, ref in zip(outs, refs)]
        if max(errs) >= 0.01:
            raise AssertionError((m, n, k, errs))
        report["graphs"].append(dict(M=m, N=n, K=k, errors=errs))
        args = list(problem(m, n, k, "normal"))
        for idx in (2, 3):
            args[idx] = args[idx].T.contiguous().T
        out = matmul(*args, profile=a.profile)
        err = rel_error(out, reference_fp32(*args))
        if not (bool(torch.isfinite(out).all()) and err < 0.01):
            raise AssertionError((m, n, k, "strided scales", err))
        report["strided_scales"].append(dict(M=m, N=n, K=k, error=err))

    report["status"] = "passed"
    report["worst_error"] = max(r["error"] for r in report["accuracy"])
    Path(a.output).write_text(json.dumps(report, indent=2) + "\n")
    if a.summary_md:
        Path(a.summary_md).write_text(summary_markdown(report, ms, argv if argv is not None else sys.argv[1:]))
    print("PASS", a.profile, len(report["accuracy"]), report["worst_error"], flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
