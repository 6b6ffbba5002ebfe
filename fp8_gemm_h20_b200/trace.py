"""Hand-over latencies between the roles of the tile kernel, from clock stamps of one CTA.

    python -m fp8_gemm_h20_b200.build --trace            # libfp8mm_b200_trace.so (-DFP8MM_TRACE)
    python -m fp8_gemm_h20_b200.trace --mnk 8192,12288,2048 [--impl umma --config '{"BLOCK_W":256}']

The instrumented library stamps the SM clock at twelve points of every K block of CTA 0 (128 blocks
after 64 of warm-up; csrc/fp8mm_kernel.cuh lists the slots).  From those this tool prints, as medians
over the window and in SM cycles: the block period, how long each role waits at its barriers, how long
its own work takes, and the two hand-overs that close the loop around a TMEM accumulator buffer
(MMAs committed -> promotion warps awake; buffer released -> issuer's next MMAs).  The stamps cost a
few instructions per block in single threads; the product library is built without them.
"""
import argparse
import json
import os
import statistics
import sys

SLOTS = 16
WINDOW = 128


def analyse(t, nbuf):
    """t: WINDOW x SLOTS list of clock values -> dict of medians (cycles)."""
    def col(s):
        return [row[s] for row in t]

    def med(xs):
        xs = [x for x in xs if x is not None]
        return round(statistics.median(xs), 1) if xs else None

    n = len(t)
    ok = [i for i in range(n) if all(t[i][s] > 0 for s in (0, 1, 2, 3, 4, 5, 6, 8, 9, 10, 11))]
    ok = [i for i in ok if i + nbuf < n and (i + nbuf) in set(ok) and i - 1 in set(ok)]
    out = {"blocks_used": len(ok)}
    if not ok:
        return out
    c = {s: col(s) for s in range(12)}
    out["block_period"] = med([c[5][i + 1] - c[5][i] for i in ok if i + 1 < n and c[5][i + 1] > 0])
    # issuer (the thread that owns this block)
    out["issuer: slot full seen -> TMEM buffer empty seen"] = med([c[3][i] - c[2][i] for i in ok])
    out["issuer: four MMAs issued"] = med([c[4][i] - c[3][i] for i in ok])
    out["issuer: two commits issued"] = med([c[5][i] - c[4][i] for i in ok])
    # promotion
    out["promotion: previous block done -> buffer full seen (idle)"] = med([c[6][i] - c[10][i - 1] for i in ok])
    out["promotion: buffer full seen -> first loads landed"] = med([c[7][i] - c[6][i] for i in ok if c[7][i] > 0])
    out["promotion: buffer full seen -> all loads landed"] = med([c[8][i] - c[6][i] for i in ok])
    out["promotion: all loads landed -> buffer released (fence, warp sync, arrive)"] = med([c[9][i] - c[8][i] for i in ok])
    out["promotion: buffer released -> block's FMAs done"] = med([c[10][i] - c[9][i] for i in ok])
    out["promotion: first warp's release -> last warp's release"] = med([c[11][i] - c[9][i] for i in ok])
    # hand-overs
    out["hand-over: MMAs issued (before commit) -> promotion awake"] = med([c[6][i] - c[4][i] for i in ok])
    out["hand-over: last release -> issuer sees the buffer empty (next use of the buffer)"] = med(
        [c[3][i + nbuf] - max(c[9][i], c[11][i]) for i in ok])
    out["buffer cycle: MMAs issued -> MMAs of the next use issued"] = med([c[4][i + nbuf] - c[4][i] for i in ok])
    # producer
    out["producer: slot empty seen -> copies issued"] = med([c[1][i] - c[0][i] for i in ok])
    out["producer: copies issued -> issuer sees the slot full"] = med([c[2][i] - c[1][i] for i in ok])
    return out


def timeline(t):
    """Stamps of a short call (trace window starting at K block 0) as cycles after kernel entry."""
    t0 = t[0][12]
    rel = lambda v: (v - t0) if v > 0 else None
    out = {"prologue done": rel(t[0][13]), "previous grid's results visible": rel(t[0][14]),
           "producer entered its role": rel(t[1][12]), "producer decoded its first unit": rel(t[1][13]),
           "issuer entered its role": rel(t[1][14]), "promotion entered its role": rel(t[1][15]),
           "promotion staged the first unit's scales": rel(t[2][12]),
           "promotion saw the scales complete": rel(t[2][13])}
    blocks = [i for i in range(len(t)) if t[i][1] > 0 or t[i][5] > 0 or t[i][6] > 0]   # rows with K-block stamps
    names = {0: "producer: slot empty seen", 1: "producer: copies issued", 2: "issuer: slot full seen",
             3: "issuer: TMEM buffer empty seen", 4: "issuer: MMAs issued", 5: "issuer: commits issued",
             6: "promotion: buffer full seen", 8: "promotion: loads landed", 9: "promotion: buffer released",
             10: "promotion: block done", 12: "epilogue of the previous unit entered",
             13: "previous unit converted and staged", 14: "previous unit's stores handed to the TMA unit",
             15: "this unit's scale table seen"}
    for i in blocks:
        for s, nm in names.items():
            if s >= 12 and i < 4:
                continue              # rows 0..3 carry the start-up and reduction stamps there
            if t[i][s] > 0:
                out[f"K block {i}: {nm}"] = rel(t[i][s])
    for (r, sl), nm in {(2, 14): "cluster split-K: partial tile parked", (2, 15): "cluster split-K: CTA in step",
                        (3, 12): "cluster split-K: cluster in step (first barrier passed)",
                        (3, 13): "cluster split-K: this rank's slice reduced and stored"}.items():
        if t[r][sl] > 0:
            out[nm] = rel(t[r][sl])
    out["promotion leader done with the last unit (output stored)"] = rel(t[0][15])
    return out


def boundaries(t, kbn, first_block):
    """Medians (cycles) over the unit boundaries inside the window: what the promotion warps do between
    the last K block of one unit and the first of the next, and how long the MMA issuers stand meanwhile.
    Row r of the record is K block first_block + r of the CTA; a unit has kbn blocks."""
    def med(xs):
        xs = [x for x in xs if x is not None]
        return round(statistics.median(xs), 1) if xs else None

    rows = [r for r in range(1, len(t) - 2) if (r + first_block) % kbn == 0 and t[r][12] > 0 and t[r - 1][10] > 0]

    def d(fn):
        out = []
        for r in rows:
            a, b = fn(r)
            out.append(b - a if a > 0 and b > 0 else None)
        return med(out)

    out = {"boundaries_used": len(rows)}
    if not rows:
        return out
    out["last block's FMAs issued -> epilogue entered"] = d(lambda r: (t[r - 1][10], t[r][12]))
    out["tile converted to bf16 and staged in shared memory"] = d(lambda r: (t[r][12], t[r][13]))
    out["proxy fence"] = d(lambda r: (t[r][13], t[r + 1][12]))
    out["warp in step"] = d(lambda r: (t[r + 1][12], t[r + 1][13]))
    out["first TMA store issued"] = d(lambda r: (t[r + 1][13], t[r + 1][14]))
    out["bulk group committed"] = d(lambda r: (t[r + 1][14], t[r][14]))
    out["next unit's loop entered (coordinates decoded)"] = d(lambda r: (t[r][14], t[r + 1][15]))
    out["next unit's scale table seen"] = d(lambda r: (t[r + 1][15], t[r][15]))
    out["first TMEM buffer of the next unit seen full"] = d(lambda r: (t[r][15], t[r][6]))
    out["its loads landed and the buffer released"] = d(lambda r: (t[r][6], t[r][9]))
    out["promotion: release of the last block -> release of the next unit's first block"] = d(
        lambda r: (t[r - 1][9], t[r][9]))
    out["issuer: MMAs of the next unit's 2nd block -> of its 3rd block (stands for the TMEM buffer)"] = d(
        lambda r: (t[r + 1][4], t[r + 2][4]))
    inner = [t[r + 1][4] - t[r][4] for r in range(1, len(t) - 1)
             if (r + first_block) % kbn not in (0, 1, 2, kbn - 1) and t[r][4] > 0 and t[r + 1][4] > 0]
    out["issuer: block period inside a unit"] = med(inner)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--mnk", default="8192,12288,2048")
    ap.add_argument("--impl", default="umma")
    ap.add_argument("--config", type=json.loads, default={"BLOCK_W": 256, "NUM_STAGES": 4})
    ap.add_argument("--json", help="also write the raw stamps and the table to this file")
    ap.add_argument("--timeline", action="store_true",
                    help="a short call from its start (library built with -D FP8MM_TRACE_FROM=0u): cycles after "
                         "kernel entry at which CTA 0 reached each point")
    ap.add_argument("--boundary", action="store_true",
                    help="medians over the unit boundaries in the window instead of the per-block table")
    ap.add_argument("--first-block", type=int, default=64,
                    help="first K block of the record (the library's FP8MM_TRACE_FROM; 64 unless built otherwise)")
    a = ap.parse_args(argv)

    from pathlib import Path
    lib = Path(__file__).with_name("libfp8mm_b200_trace.so")
    if not lib.is_file():
        raise SystemExit(f"{lib} missing: python -m fp8_gemm_h20_b200.build --trace")
    from .build import up_to_date
    if not up_to_date(lib):
        raise SystemExit(f"{lib} is older than the sources: python -m fp8_gemm_h20_b200.build --trace")
    os.environ["FP8MM_LIB"] = str(lib)
    import torch
    from . import engine, testing
    m, n, k = (int(x) for x in a.mnk.split(","))
    buf = torch.zeros(WINDOW * SLOTS, dtype=torch.int64, device="cuda")
    os.environ["FP8MM_TRACE_PTR"] = hex(buf.data_ptr())
    A, B, As, Bs = (x.cuda() for x in testing.make_problem(m, n, k, seed=m + n + k))
    for _ in range(3):
        buf.zero_()
        engine.launch(A, B, As, Bs, a.impl, a.config)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    engine.launch(A, B, As, Bs, a.impl, a.config)
    e1.record()
    torch.cuda.synchronize()
    t = buf.view(WINDOW, SLOTS).cpu().tolist()
    bw = int(a.config.get("BLOCK_W", 256)) if a.impl == "umma" else int(a.config.get("BLOCK_T", 16))
    nbuf = 2 if bw == 256 else (4 if bw >= 64 else 8)
    if a.boundary:
        table = boundaries(t, (k // 128) // int(a.config.get("SPLIT", 1)), a.first_block)
    else:
        table = timeline(t) if a.timeline else analyse(t, nbuf)
    table["kernel_us_with_stamps"] = round(e0.elapsed_time(e1) * 1e3, 1)
    print(json.dumps({"M": m, "N": n, "K": k, "impl": a.impl, "config": a.config, "tmem_buffers": nbuf}))
    for key, v in table.items():
        print(f"  {key:82s} {v}")
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"table": table, "stamps": t}, f)
    assert engine.device_status() == (0, 0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
