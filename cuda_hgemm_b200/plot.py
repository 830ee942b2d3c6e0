"""Throughput chart of a square sweep as an SVG file, without any plotting library.

The counterpart of the reference's plot tool (reference tools/performance/performance.py:36-78:
one line per kernel, TFLOPS over the matrix size, read from the ``hgemm_M_N_K.log`` files of a
sweep). It reads the same logs (``<dir>/log/hgemm_*.log``, the line format of reference
src/common/tester.h:104-106) or the ``sweep.jsonl`` that ``cuda_hgemm_b200.sweep`` writes, keeps
the kernels named with ``--kernels`` (default: both cuBLAS modes, the reference's best kernel per
size, the B200 kernel) and writes one SVG.

    python -m cuda_hgemm_b200.plot sweep_out --out sweep_out/throughput.svg
"""
from __future__ import annotations

import argparse
import json
import re
import sys
from pathlib import Path
from xml.sax.saxutils import escape

RESULT_LINE = re.compile(r"\]\s*(\S+) exit, profiling time: ([0-9.]+) ms \([0-9.]+%\), throughput: ([0-9.]+) TFLOPS")
LOG_NAME = re.compile(r"hgemm_(\d+)_(\d+)_(\d+)\.log$")
REF_PREFIXES = ("Wmma-", "Mma-", "Simt-")
COLOURS = ("#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#e377c2", "#17becf")


def read_logs(directory: Path):
    """{kernel: {n: tflops}} from the driver's logs of square sizes."""
    series = {}
    for path in sorted((directory / "log").glob("hgemm_*.log")):
        m = LOG_NAME.search(path.name)
        if not m or not (m.group(1) == m.group(2) == m.group(3)):
            continue
        n = int(m.group(1))
        for line in path.read_text(errors="replace").splitlines():
            r = RESULT_LINE.search(line)
            if r:
                series.setdefault(r.group(1), {})[n] = float(r.group(3))
    return series


def read_jsonl(path: Path):
    series = {}
    for line in path.read_text().splitlines():
        if not line.strip():
            continue
        d = json.loads(line)
        if d["M"] == d["N"] == d["K"]:
            series.setdefault(d["kernel"], {})[int(d["M"])] = float(d["tflops"])
    return series


def with_reference_best(series):
    """Adds 'Reference-Best': the fastest of the reference's kernels at every size."""
    best = {}
    for name, points in series.items():
        if name.startswith(REF_PREFIXES):
            for n, v in points.items():
                best[n] = max(best.get(n, 0.0), v)
    if best:
        series = dict(series)
        series["Reference-Best"] = best
    return series


def nice_step(span, target=8):
    raw = span / max(1, target)
    mag = 10 ** len(str(int(raw))) / 10 if raw >= 1 else 1
    for mult in (1, 2, 2.5, 5, 10):
        if raw <= mult * mag:
            return mult * mag
    return 10 * mag


def render_svg(series, title, width=960, height=540):
    left, right, top, bottom = 70, 200, 40, 50
    xs = sorted({n for pts in series.values() for n in pts})
    if not xs:
        raise ValueError("nothing to plot")
    x0, x1 = xs[0], xs[-1] if xs[-1] > xs[0] else xs[0] + 1
    ymax = max(v for pts in series.values() for v in pts.values())
    ystep = nice_step(ymax)
    ytop = ystep * (int(ymax / ystep) + 1)
    pw, ph = width - left - right, height - top - bottom

    def px(n):
        return left + pw * (n - x0) / (x1 - x0)

    def py(v):
        return top + ph * (1.0 - v / ytop)

    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" viewBox="0 0 {width} {height}" '
           'font-family="sans-serif" font-size="12">',
           f'<rect width="{width}" height="{height}" fill="white"/>',
           f'<text x="{left}" y="24" font-size="15">{escape(title)}</text>']
    y = 0.0
    while y <= ytop + 1e-9:
        out.append(f'<line x1="{left}" y1="{py(y):.1f}" x2="{left + pw}" y2="{py(y):.1f}" stroke="#dddddd"/>')
        out.append(f'<text x="{left - 8}" y="{py(y) + 4:.1f}" text-anchor="end">{y:g}</text>')
        y += ystep
    xstep = nice_step(x1 - x0)
    x = (int(x0 / xstep) + (1 if x0 % xstep else 0)) * xstep
    while x <= x1 + 1e-9:
        out.append(f'<line x1="{px(x):.1f}" y1="{top}" x2="{px(x):.1f}" y2="{top + ph}" stroke="#eeeeee"/>')
        out.append(f'<text x="{px(x):.1f}" y="{top + ph + 18}" text-anchor="middle">{int(x)}</text>')
        x += xstep
    out.append(f'<rect x="{left}" y="{top}" width="{pw}" height="{ph}" fill="none" stroke="black"/>')
    out.append(f'<text x="{left + pw / 2:.0f}" y="{height - 10}" text-anchor="middle">M = N = K</text>')
    out.append(f'<text x="18" y="{top + ph / 2:.0f}" text-anchor="middle" transform="rotate(-90 18 {top + ph / 2:.0f})">TFLOPS</text>')
    for i, (name, pts) in enumerate(series.items()):
        colour = COLOURS[i % len(COLOURS)]
        points = " ".join(f"{px(n):.1f},{py(pts[n]):.1f}" for n in sorted(pts))
        out.append(f'<polyline fill="none" stroke="{colour}" stroke-width="1.8" points="{points}"/>')
        ly = top + 14 + 18 * i
        out.append(f'<line x1="{left + pw + 12}" y1="{ly - 4}" x2="{left + pw + 36}" y2="{ly - 4}" stroke="{colour}" stroke-width="2.5"/>')
        out.append(f'<text x="{left + pw + 42}" y="{ly}">{escape(name)}</text>')
    out.append("</svg>")
    return "\n".join(out) + "\n"


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("sweep_dir", help="directory written by cuda_hgemm_b200.sweep (or one holding log/hgemm_*.log)")
    ap.add_argument("--out", default=None, help="SVG file (default: <sweep_dir>/throughput.svg)")
    ap.add_argument("--kernels", default="Cublas-Tensor-Op,Cublas-Tensor-Op-Fp32,Reference-Best,B200-Tcgen05-Auto",
                    help="comma-separated kernel names as they appear in the logs; 'all' plots every kernel")
    ap.add_argument("--title", default="HGEMM throughput, square sizes")
    args = ap.parse_args(argv)

    directory = Path(args.sweep_dir)
    jsonl = directory / "sweep.jsonl"
    series = read_jsonl(jsonl) if jsonl.exists() else read_logs(directory)
    series = with_reference_best(series)
    if args.kernels != "all":
        wanted = [k for k in args.kernels.split(",") if k in series]
        series = {k: series[k] for k in wanted}
    if not series:
        print("no kernel of that name in the sweep", file=sys.stderr)
        return 1
    out = Path(args.out) if args.out else directory / "throughput.svg"
    out.write_text(render_svg(series, args.title))
    print(f"{len(series)} series, {sum(len(p) for p in series.values())} points -> {out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
