"""Regenerates the Nsight Compute summaries under ``profiles/``: one command per capture, one markdown file each.

    python -m cuda_hgemm_b200.profile --list
    python -m cuda_hgemm_b200.profile [--only NAME[,NAME...]] [--out profiles] [--raw DIR] [--summarise-only]

The counterpart of the reference's profiling wrapper (reference run_sample.sh:23-27, one ``ncu`` line kept in a
comment there). Every capture runs its target once WITHOUT ncu first and goes on only if that exits 0; ncu then
gets ``--clock-control none``, one kernel-name filter, a skip count and at most three launches, and a short list
of metrics, so that a capture ends by itself within a minute or two. The launch list of the benchmark collects
``gpu__time_duration.sum`` alone (one pass per launch). The raw CSV goes to ``--raw`` (scratch); the summary
file names the full command, the per-launch values, the algorithmic work of the shape and how the measured DRAM
traffic compares with it. Text after a line ``## Reading`` in an existing summary is kept.
"""
from __future__ import annotations

import argparse
import os
import csv
import shlex
import statistics
import subprocess
import sys
from collections import OrderedDict, defaultdict
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

METRICS = ("dram__bytes_read.sum,dram__bytes_write.sum,lts__t_sectors_srcunit_tex_op_read.sum,lts__t_sector_hit_rate.pct,"
           "gpu__time_duration.sum,sm__cycles_elapsed.avg.per_second,sm__mem_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed,"
           "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed,lts__throughput.avg.pct_of_peak_sustained_elapsed,"
           "launch__grid_size,launch__registers_per_thread")

TARGET = [sys.executable, "-m", "cuda_hgemm_b200.profile_target"]

# name -> (title, target command, kernel regex, launches skipped, launches captured, shape or None)
CAPTURES = OrderedDict([
    ("hgemm_tcgen05_big_square16384", (
        "pairs on 512 x 256 tiles (256 x 256 outputs per CTA) at M=N=K=16384",
        TARGET + ["--shape", "16384x16384x16384", "--plan", "cta2:512", "--launches", "4"],
        "hgemm_tcgen05_big", 1, 3, (16384, 16384, 16384))),
    ("hgemm_tcgen05_mc512_square16384", (
        "groups of four CTAs on 512 x 512 tiles with A multicast (one GPU per process) at M=N=K=16384",
        TARGET + ["--shape", "16384x16384x16384", "--plan", "mcast:512", "--multicast", "--launches", "4"],
        "hgemm_tcgen05_mc512", 1, 3, (16384, 16384, 16384))),
    ("cublas_fp32_compute_square16384", (
        "cuBLAS cublasGemmEx, FP32 compute, at M=N=K=16384 (the comparison)",
        TARGET + ["--shape", "16384x16384x16384", "--plan", "cta2:512", "--launches", "1", "--cublas", "fp32"],
        "nvjet|cutlass", 0, 1, (16384, 16384, 16384))),
    ("hgemm_tcgen05_big_prefill", (
        "pairs on 512 x 256 tiles at the prefill shape M=8192, N=28672, K=8192 (24 full waves; the 16 left-over tiles run as "
        "32 halves on the 128 x 256-per-CTA pair kernel right behind, not captured here)",
        TARGET + ["--shape", "8192x28672x8192", "--dist", "normal", "--launches", "4"],
        "hgemm_tcgen05_big", 1, 3, (8192, 28672, 8192))),
    ("hgemm_skinny_skinny16", (
        "the short-A kernel at the decode shape M=16, N=14336, K=4096 (B cycled through 7 copies)",
        TARGET + ["--shape", "16x14336x4096", "--dist", "normal", "--b-copies", "7", "--launches", "10"],
        "hgemm_skinny", 6, 3, (16, 14336, 4096))),
    ("hgemm_skinny_pair_skinny128", (
        "the short-A kernel on CTA pairs at the decode shape M=128, N=14336, K=4096 (B cycled through 7 copies)",
        TARGET + ["--shape", "128x14336x4096", "--dist", "normal", "--b-copies", "7", "--launches", "10"],
        "hgemm_skinny", 6, 3, (128, 14336, 4096))),
    ("hgemm_skinny_skinny16t", (
        "the short-A kernel with four k-ranges per column tile, summed inside clusters of four, at M=16, N=4096, K=14336 "
        "(B cycled through 7 copies)",
        TARGET + ["--shape", "16x4096x14336", "--dist", "normal", "--b-copies", "7", "--launches", "10"],
        "hgemm_skinny", 6, 3, (16, 4096, 14336))),
    ("hgemm_skinny_skinny128t", (
        "the short-A kernel with four k-ranges per column tile, summed inside clusters of four, at M=128, N=4096, K=14336 "
        "(B cycled through 7 copies)",
        TARGET + ["--shape", "128x4096x14336", "--dist", "normal", "--b-copies", "7", "--launches", "10"],
        "hgemm_skinny", 6, 3, (128, 4096, 14336))),
    ("hgemm_tcgen05_wide288_square2304", (
        "pairs on 256 x 288 tiles (two MMAs side by side per k-step) at M=N=K=2304: 72 tiles, one wave on 74 pairs "
        "(operands and C together are 32 MB: they stay in L2, so the DRAM figures are small)",
        TARGET + ["--shape", "2304x2304x2304", "--plan", "cta2:288", "--launches", "6"],
        "hgemm_tcgen05_kernel", 3, 3, (2304, 2304, 2304))),
    ("launch_list_bench_square16384", (
        "every launch of `bench.py` at the default workload",
        [sys.executable, "bench.py", "--steps", "2", "--warmup", "3", "--no-sweep", "--no-workloads"],
        None, 0, 800, None)),
])


def parse_ncu_csv(path: Path):
    """ncu --csv log -> list of launches [(kernel name, {metric: (value, unit)})] in launch order."""
    lines = path.read_text(errors="replace").splitlines()
    start = next((i for i, line in enumerate(lines) if line.startswith('"ID"')), None)
    if start is None:
        return []
    launches = OrderedDict()
    for row in csv.DictReader(lines[start:]):
        key = row["ID"]
        name = row["Kernel Name"]
        launches.setdefault(key, (name, {}))
        try:
            value = float(row["Metric Value"].replace(",", ""))
        except ValueError:
            continue
        launches[key][1][row["Metric Name"]] = (value, row["Metric Unit"])
    return list(launches.values())


def to_ns(value, unit):
    return value * {"ns": 1.0, "us": 1e3, "usecond": 1e3, "ms": 1e6, "msecond": 1e6, "s": 1e9, "second": 1e9, "nsecond": 1.0}.get(unit, 1.0)


def to_bytes(value, unit):
    return value * {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}.get(unit, 1.0)


def summarise_capture(name, title, plain_cmd, ncu_cmd, launches, shape):
    out = [f"# ncu: {title}", "", "Commands (the first had exited 0 just before the second ran):", "",
           "    " + shlex.join(plain_cmd), "    " + shlex.join(ncu_cmd), ""]
    if not launches:
        out.append("No launch matched the kernel filter.")
        return "\n".join(out) + "\n"
    kernels = sorted({k for k, _ in launches})
    out.append("Kernel(s): " + ", ".join(f"`{k[:110]}`" for k in kernels) + f"; {len(launches)} launch(es) captured.")
    out += ["", "| metric | value per captured launch |", "|---|---|"]
    metric_names = list(OrderedDict.fromkeys(m for _, ms in launches for m in ms))
    for m in metric_names:
        vals = [ms[m] for _, ms in launches if m in ms]
        unit = vals[0][1]
        out.append(f"| {m} ({unit}) | " + " / ".join(f"{v:,.6g}" for v, _ in vals) + " |")
    if shape:
        M, N, K = shape
        flops, algo = 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N)
        traffic = [to_bytes(*ms["dram__bytes_read.sum"]) + to_bytes(*ms["dram__bytes_write.sum"]) for _, ms in launches
                   if "dram__bytes_read.sum" in ms and "dram__bytes_write.sum" in ms]
        dur = [to_ns(*ms["gpu__time_duration.sum"]) for _, ms in launches if "gpu__time_duration.sum" in ms]
        out += ["", f"Algorithmic work of one launch: {flops / 1e9:,.1f} GFLOP, {algo / 1e6:,.1f} MB (2*(M*K + N*K + M*N))."]
        if traffic:
            t = statistics.median(traffic)
            out.append(f"Measured DRAM traffic (read + write, median): {t / 1e6:,.1f} MB per launch = {t / algo:.2f} x algorithmic.")
        if dur:
            d = statistics.median(dur)
            out.append(f"Duration under ncu (median; isolated and serialised, not a benchmark figure): {d / 1e3:,.1f} us "
                       f"= {flops / d / 1e3:,.1f} TFLOP/s, {algo / d:,.1f} GB/s of algorithmic bytes.")
    return "\n".join(out) + "\n"


def summarise_launch_list(title, plain_cmd, ncu_cmd, launches):
    per = defaultdict(list)
    for kname, ms in launches:
        if "gpu__time_duration.sum" in ms:
            per[kname].append(to_ns(*ms["gpu__time_duration.sum"]))
    total = sum(sum(v) for v in per.values()) or 1.0
    out = [f"# ncu launch list: {title}", "", "Commands (the first had exited 0 just before the second ran; one pass per launch):", "",
           "    " + shlex.join(plain_cmd), "    " + shlex.join(ncu_cmd), "",
           "Per kernel over the whole run (per-launch times are cold-cache and serialised: compare shares):", "",
           "| kernel | launches | total ms | min-max per launch (ms) | share |", "|---|---|---|---|---|"]
    for kname, v in sorted(per.items(), key=lambda kv: -sum(kv[1])):
        out.append(f"| `{kname[:100]}` | {len(v)} | {sum(v) / 1e6:.2f} | {min(v) / 1e6:.3f}-{max(v) / 1e6:.3f} | {100 * sum(v) / total:.1f} % |")
    return "\n".join(out) + "\n"


def run_capture(name, out_dir: Path, raw_dir: Path, summarise_only: bool = False) -> int:
    title, target, regex, skip, count, shape = CAPTURES[name]
    raw_dir.mkdir(parents=True, exist_ok=True)
    csv_path = raw_dir / f"{name}.csv"
    metrics = "gpu__time_duration.sum" if regex is None else METRICS
    ncu_cmd = ["ncu", "--metrics", metrics, "--clock-control", "none"]
    if regex is not None:
        ncu_cmd += ["-k", f"regex:{regex}", "-s", str(skip)]
    ncu_cmd += ["-c", str(count), "--csv", "--log-file", str(csv_path.relative_to(ROOT) if csv_path.is_relative_to(ROOT) else csv_path)]
    ncu_cmd += target
    if summarise_only:
        if not csv_path.exists():
            print(f"{name}: no {csv_path} to summarise", file=sys.stderr)
            return 1
    else:
        plain = subprocess.run(target, cwd=ROOT, capture_output=True, text=True)
        (raw_dir / f"{name}.plain.log").write_text(plain.stdout + plain.stderr)
        if plain.returncode != 0:
            print(f"{name}: the target exits {plain.returncode} without ncu; not profiled", file=sys.stderr)
            return 1
        prof = subprocess.run(ncu_cmd, cwd=ROOT, capture_output=True, text=True)
        (raw_dir / f"{name}.ncu.log").write_text(prof.stdout + prof.stderr)
        if prof.returncode != 0 or not csv_path.exists():
            print(f"{name}: ncu exits {prof.returncode}: {(prof.stdout + prof.stderr)[-300:]}", file=sys.stderr)
            return 1
    launches = parse_ncu_csv(csv_path)
    shown_target = ["python" if t == sys.executable else t for t in target]
    shown_ncu = ["python" if t == sys.executable else t for t in ncu_cmd]
    text = (summarise_launch_list(title, shown_target, shown_ncu, launches) if regex is None else
            summarise_capture(name, title, shown_target, shown_ncu, launches, shape))
    md = out_dir / f"{name}.md"
    if md.exists() and "\n## Reading" in md.read_text():
        text += "\n## Reading" + md.read_text().split("\n## Reading", 1)[1]
    out_dir.mkdir(parents=True, exist_ok=True)
    md.write_text(text)
    print(f"{name}: {len(launches)} launch(es) -> {md}")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--only", default="", help="comma-separated capture names (default: all)")
    ap.add_argument("--out", default=str(ROOT / "profiles"))
    ap.add_argument("--raw", default=os.environ.get("B200_PROFILE_RAW", str(ROOT / "ncu_raw")),
                    help="where the CSV files and logs go (scratch; default: $B200_PROFILE_RAW or ncu_raw/ in the repository)")
    ap.add_argument("--summarise-only", action="store_true",
                    help="rewrite the summaries from the CSV files an earlier run left under --raw (e.g. captured on another machine)")
    args = ap.parse_args(argv)
    if args.list:
        for name, (title, *_rest) in CAPTURES.items():
            print(f"{name}: {title}")
        return 0
    names = [n for n in args.only.split(",") if n] or list(CAPTURES)
    unknown = [n for n in names if n not in CAPTURES]
    if unknown:
        ap.error(f"unknown capture(s): {', '.join(unknown)}")
    failures = sum(run_capture(n, Path(args.out), Path(args.raw), args.summarise_only) for n in names)
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())
