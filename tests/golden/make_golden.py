"""Generate the golden fixtures in this directory from the REFERENCE's own code.

Run in the build container only (needs the reference checkout; nothing here is read at
test time except the files it writes):

    cd /tmp && python <repo>/tests/golden/make_golden.py --reference <reference checkout>

1. gemm_golden.npz — for a handful of small seeded problems, the outputs of the reference's
   `reference()` and `error()` (scripts/validate.py:32-37) and `ref()` (bench.py:25-30),
   called on CPU tensors.  Inputs are produced with the reference's quantisation recipe
   (scripts/validate.py:21-30 — its `make` is CUDA-only, so the same statements run here on
   the CPU generator) and stored as raw bytes.
2. routing_golden.json — the answers of the reference's `_select` (fp8_gemm_h20/config.py:76-101)
   for every M in 1..16384 on the synthetic two-policy table routing_table_*.json in this
   directory (kernel names are the B200 ones, so the reference's name set is widened for
   the run; its routing code is untouched).
"""
import argparse
import importlib
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent

CASES = [  # (M, N, K, mode, seed)
    (1, 128, 128, "normal", 1), (5, 128, 256, "outlier", 2), (37, 256, 384, "normal", 3),
    (64, 384, 256, "skew", 4), (200, 256, 512, "normal", 5), (17, 128, 1024, "zero", 6),
    (130, 384, 128, "outlier", 7), (8, 256, 1024, "skew", 8),
]


def make_cpu(torch, m, n, k, mode, seed):
    # scripts/validate.py:21-30 with device='cpu' and an explicit generator
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g)
    b = torch.randn(n, k, generator=g) * .05
    if mode == 'outlier': a[:, ::127] *= 100
    if mode == 'skew': b *= torch.logspace(-3, 1, n // 128).repeat_interleave(128)[:, None]
    if mode == 'zero': a.zero_()
    sa = a.view(m, k // 128, 128).abs().amax(-1).clamp_min(1e-6) / 448
    bb = b.view(n // 128, 128, k // 128, 128)
    sb = bb.abs().amax((1, 3)).clamp_min(1e-6) / 448
    aa = (a.view(m, k // 128, 128) / sa[..., None]).reshape(m, k).to(torch.float8_e4m3fn)
    bq = (bb / sb[:, None, :, None]).reshape(n, k).to(torch.float8_e4m3fn)
    return a, b, aa, bq, sa.contiguous(), sb.contiguous()


def synthetic_tables():
    """Two small profiles exercising both policies, B200 kernel names."""
    def e(impl, bt, bw, split, us=None):
        d = {"impl": impl, "config": {"BLOCK_T": bt, "BLOCK_W": bw, "SPLIT": split, "NUM_STAGES": 4,
                                      "GROUP_SIZE_M": 1}}
        if us is not None:
            d["anchor_us"] = us
        return d
    shapes = [{"name": "a", "N": 3072, "K": 2048, "count": 1}, {"name": "b", "N": 512, "K": 3072, "count": 2}]
    base = {"schema_version": 1, "hardware": "synthetic", "block_size": [128, 128], "m_range": [1, 16384],
            "shapes": shapes}
    log_tab = {"3072,2048": {"16": e("umma_swap", 16, 128, 4), "100": e("umma_swap", 128, 128, 2),
                             "333": e("umma", 128, 128, 1), "4096": e("umma", 128, 128, 1)},
               "512,3072": {"1": e("umma_swap", 16, 128, 8), "64": e("umma_swap", 64, 128, 4),
                            "2048": e("umma", 128, 128, 1)}}
    near = {"3072,2048": {"1": e("umma_swap", 16, 128, 8, 3.1), "7": e("umma_swap", 16, 128, 4, 3.0),
                          "16": e("umma_swap", 16, 128, 4, 3.3), "37": e("umma_swap", 64, 128, 4, 4.0),
                          "40": e("umma_swap", 32, 128, 2, 3.9), "200": e("umma_swap", 256, 128, 2, 6.5),
                          "205": e("umma", 128, 128, 1, 6.4), "512": e("umma", 128, 128, 1, 9.0),
                          "4097": e("umma", 128, 128, 1, 50.0)},
            "512,3072": {"64": e("umma_swap", 64, 128, 8, 4.4), "128": e("umma_swap", 128, 128, 4, 5.0),
                         "130": e("umma", 128, 128, 2, 5.2)}}
    fb = {"3072,2048": {"8": e("umma_swap", 16, 128, 2), "64": e("umma_swap", 64, 128, 2),
                        "1024": e("umma", 128, 128, 1), "16384": e("umma", 128, 128, 1)},
          "512,3072": {"32": e("umma_swap", 32, 128, 2), "1000": e("umma", 128, 128, 1)}}
    t1 = dict(base, profile="routing_table_log", policy={"kind": "log_nearest"}, entries=log_tab)
    t2 = dict(base, profile="routing_table_near",
              policy={"kind": "nearby_equal_tiles", "max_distance": 8, "exact_only": ["umma"]},
              entries=near, fallback_entries=fb)
    return {"routing_table_log": t1, "routing_table_near": t2}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    import numpy as np
    import torch
    torch.manual_seed(0)
    validate = importlib.import_module("scripts.validate")      # reference(), error()
    out = {}
    for i, (m, n, k, mode, seed) in enumerate(CASES):
        x, w, aa, bq, sa, sb = make_cpu(torch, m, n, k, mode, seed)
        ref32 = validate.reference((aa, bq, sa, sb))
        ref16 = ref32.to(torch.bfloat16)                        # bench.py:30
        noisy = ref16.float() * (1 + 1e-3)
        out[f"c{i}_meta"] = np.array([m, n, k, seed], dtype=np.int64)
        out[f"c{i}_mode"] = np.array(mode)
        if m * k + n * k <= 70000:                              # raw inputs pin the quantiser
            out[f"c{i}_x"] = x.numpy()
            out[f"c{i}_w"] = w.numpy()
        out[f"c{i}_A"] = aa.view(torch.uint8).numpy()
        out[f"c{i}_B"] = bq.view(torch.uint8).numpy()
        out[f"c{i}_As"] = sa.numpy()
        out[f"c{i}_Bs"] = sb.numpy()
        out[f"c{i}_ref32"] = ref32.numpy()
        out[f"c{i}_ref16_bits"] = ref16.view(torch.int16).numpy()
        out[f"c{i}_err_bf16"] = np.array(validate.error(ref16, ref32))
        out[f"c{i}_err_noisy"] = np.array(validate.error(noisy, ref32))
    np.savez_compressed(HERE / "gemm_golden.npz", **out)

    cfg = importlib.import_module("fp8_gemm_h20.config")        # the reference's selector
    tables = synthetic_tables()
    for name, data in tables.items():
        (HERE / f"{name}.json").write_text(json.dumps(data, indent=1) + "\n")
    cfg.KERNELS = {"umma": None, "umma_swap": None}
    cfg._PROFILES = tuple(tables)
    cfg._CONFIG_DIR = HERE
    golden = {}
    for name, data in tables.items():
        for nk in data["entries"]:
            n, k = map(int, nk.split(","))
            rows, prev = [], None
            for m in range(1, 16385):
                entry, info = cfg._select(name, m, n, k)
                cur = [info["method"], info["anchor"], entry["impl"], entry["config"]["BLOCK_T"],
                       entry["config"]["SPLIT"]]
                if cur != prev:                                  # run-length: [first M, answer]
                    rows.append([m] + cur)
                    prev = cur
            golden[f"{name}|{nk}"] = rows
    (HERE / "routing_golden.json").write_text(json.dumps(golden) + "\n")
    print("wrote", sorted(p.name for p in HERE.iterdir()))


if __name__ == "__main__":
    main()
