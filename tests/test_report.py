"""Host-side arithmetic of the per-point roofline report (no GPU)."""
import json

from fp8_gemm_h20_b200 import report
from fp8_gemm_h20_b200.tune import algorithmic_bytes


def test_roof_picks_the_larger_time():
    # config 0: 2.517 GFLOP and 7.944 MB -> 0.56 us at 4.5 PFLOP/s, 0.99 us at 8 TB/s: HBM roof
    t, which = report.roof(200, 3072, 2048, 4500.0, 8000.0)
    assert which == "hbm" and abs(t - algorithmic_bytes(200, 3072, 2048) / 8e6) < 1e-9
    assert abs(t - 0.993) < 2e-3
    t, which = report.roof(16384, 12288, 2048, 4500.0, 8000.0)
    assert which == "tensor" and abs(t - 2.0 * 16384 * 12288 * 2048 / 4.5e9) < 1e-6


def test_point_row_fractions():
    r = report.point_row(8192, 12288, 2048, 221.0, None, dict(hbm_gbs=6532.2, fp8_tflops=2760.8))
    assert r["bound"] == "tensor" and "cold_us" not in r
    assert abs(r["tflops"] - 2.0 * 8192 * 12288 * 2048 / 221.0 * 1e-6) < 0.01
    assert abs(r["frac_nominal"] - r["tflops"] / 4500.0) < 1e-3
    assert abs(r["frac_measured"] - r["tflops"] / 2760.8) < 1e-3
    c = report.point_row(1, 12288, 2048, 6.3, 12.0, dict(hbm_gbs=6532.2, fp8_tflops=2760.8))
    assert c["bound"] == "hbm" and abs(c["cold_gbs"] - algorithmic_bytes(1, 12288, 2048) / 12.0 * 1e-3) < 0.1


def test_layer_mix_needs_every_shape():
    shapes = [dict(N=256, K=128, count=3), dict(N=128, K=128, count=2)]
    rows = [dict(M=1, N=256, K=128, us=2.0), dict(M=1, N=128, K=128, us=1.0), dict(M=8, N=256, K=128, us=5.0)]
    assert report.layer_mix(rows, shapes) == {1: 8.0}
    # two layers with the same (N, K): counts add up, duplicate rows are ignored
    shapes.append(dict(N=128, K=128, count=5))
    rows.append(dict(M=1, N=128, K=128, us=1.0))
    assert report.layer_mix(rows, shapes) == {1: 13.0}


def test_markdown_and_summary_render():
    measured = dict(hbm_gbs=6532.2, fp8_tflops=2760.8)
    pts = [report.point_row(8192, 12288, 2048, 221.0, 230.0, measured),
           report.point_row(64, 12288, 2048, 8.0, 11.0, measured)]
    rep = dict(profile="35b_tp1", device="x", rounds=5, command="c", measured_peaks=measured, clocks={},
               points=pts, layer_mix_us={64: 10.0}, two_streams=[dict(M=16384, N=12288, K=2048, alone_us=496.0,
               alone_tflops=1662.0, two_streams_us=990.0, per_stream_tflops=833.0, aggregate_tflops=1666.0)],
               summary=report.summarise(pts))
    md = report.to_markdown(rep)
    assert "| 12288 | 2048 | 8192 | 221.00 |" in md and "Two concurrent streams" in md and "cold us" in md
    assert any("M >= 4096" in k for k in rep["summary"]) and any("M <= 64" in k for k in rep["summary"])
    json.dumps(rep)


def test_render_rebuilds_report_from_saved_json(tmp_path):
    measured = dict(hbm_gbs=6532.2, fp8_tflops=2760.8)
    pts = []
    for (n, k) in [(12288, 2048), (2048, 4096), (9216, 2048), (2048, 4096), (1024, 2048), (2048, 512)]:
        pts.append(report.point_row(8192, n, k, 100.0, None, measured))      # (2048, 4096) twice, as two layers
    saved = dict(profile="35b_tp1", device="x", rounds=5, command="c", measured_peaks=measured, clocks={},
                 points=pts, layer_mix_us={}, two_streams=[], summary={})
    src = tmp_path / "saved.json"
    src.write_text(json.dumps(saved))
    assert report.main(["--profile", "35b_tp1", "--render", str(src), "--out", str(tmp_path / "out")]) == 0
    rep = json.loads((tmp_path / "out.json").read_text())
    assert len(rep["points"]) == 5
    # counts of the 35B profile: 30 + (30 + 10) + 10 + 40 + 40 layers, 100 us each
    assert rep["layer_mix_us"] == {"8192": 16000.0} or rep["layer_mix_us"] == {8192: 16000.0}
    assert "| 8192 | 16000.0 |" in (tmp_path / "out.md").read_text()
