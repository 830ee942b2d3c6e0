"""The sweep chart: reads the driver's logs the way the reference's plot tool does and writes an SVG."""
import json
import xml.dom.minidom

from cuda_hgemm_b200 import plot


def write_log(path, rows):
    # the result line of the driver, byte for byte the reference's format (reference src/common/tester.h:104-106)
    lines = [f"[HGEMM 2026-01-01 00:00:00 1:2 tester.h:120 evaluate] {name} exit, profiling time: {ms:.3f} ms "
             f"({100.0:.2f}%), throughput: {tflops:.3f} TFLOPS ({100.0:.2f}%)" for name, ms, tflops in rows]
    path.write_text("some other line\n" + "\n".join(lines) + "\n")


def test_logs_and_jsonl_give_the_same_series(tmp_path):
    (tmp_path / "log").mkdir()
    data = {256: [("Cublas-Tensor-Op", 0.007, 4.8), ("Mma-Async-Stage4", 0.012, 2.8), ("Wmma-Async-Stage3", 0.010, 3.3),
                  ("B200-Tcgen05-Auto", 0.005, 6.4)],
            512: [("Cublas-Tensor-Op", 0.008, 33.5), ("Mma-Async-Stage4", 0.016, 16.9), ("Wmma-Async-Stage3", 0.017, 15.8),
                  ("B200-Tcgen05-Auto", 0.006, 44.7)]}
    with open(tmp_path / "sweep.jsonl", "w") as f:
        for n, rows in data.items():
            write_log(tmp_path / "log" / f"hgemm_{n}_{n}_{n}.log", rows)
            for name, ms, tflops in rows:
                f.write(json.dumps({"kernel": name, "M": n, "N": n, "K": n, "ms": ms, "tflops": tflops}) + "\n")
    write_log(tmp_path / "log" / "hgemm_512_2048_1024.log", [("Cublas-Tensor-Op", 0.1, 21.0)])  # not square: ignored
    from_logs = plot.read_logs(tmp_path)
    from_jsonl = plot.read_jsonl(tmp_path / "sweep.jsonl")
    assert from_logs == from_jsonl
    assert from_logs["B200-Tcgen05-Auto"] == {256: 6.4, 512: 44.7}
    best = plot.with_reference_best(from_logs)["Reference-Best"]
    assert best == {256: 3.3, 512: 16.9}  # the fastest of the reference's kernels at each size


def test_svg_is_well_formed_and_has_one_line_per_kernel(tmp_path):
    series = {"Cublas-Tensor-Op": {256: 4.8, 512: 33.5, 768: 70.0}, "B200 <auto>": {256: 6.4, 512: 44.7, 768: 138.0}}
    svg = plot.render_svg(series, "throughput & sizes")
    doc = xml.dom.minidom.parseString(svg)
    assert len(doc.getElementsByTagName("polyline")) == 2
    texts = [t.firstChild.data for t in doc.getElementsByTagName("text") if t.firstChild]
    assert "B200 <auto>" in texts and "throughput & sizes" in texts
    out = tmp_path / "chart.svg"
    (tmp_path / "sweep.jsonl").write_text("".join(
        json.dumps({"kernel": k, "M": n, "N": n, "K": n, "tflops": v}) + "\n" for k, pts in series.items() for n, v in pts.items()))
    assert plot.main([str(tmp_path), "--out", str(out), "--kernels", "all"]) == 0
    assert len(xml.dom.minidom.parse(str(out)).getElementsByTagName("polyline")) == 2
    assert plot.main([str(tmp_path), "--kernels", "No-Such-Kernel"]) == 1
