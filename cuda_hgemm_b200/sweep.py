"""Square-size sweep with the ``hgemm`` driver: the reference's ``benchmark_hgemm`` loop.

The reference sweeps 20 square sizes with ``-warmup_iterations=1 -profiling_iterations=10`` and
writes one log per size named ``log/hgemm_M_N_K.log`` for its plot tool (reference
run_sample.sh:15-37, tools/performance/performance.py:36-45). This runner keeps the log naming
and format (so that tool still works on the output directory) and sweeps every multiple of
``--step`` from ``--first`` to ``--last``; it also writes ``sweep.jsonl`` (one line per size and
kernel) and ``sweep.md`` (one row per size: cuBLAS in both compute modes, the best reference
kernel, the new kernels).

    python -m cuda_hgemm_b200.sweep --out sweep_out [--ref-lib oracle/_ref/libcuda_hgemm_ref.so]
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from pathlib import Path

from . import build

REF_PREFIXES = ("Wmma-", "Mma-", "Simt-")


def run_size(binary: Path, n: int, out_dir: Path, ref_lib: str | None, warmup: int, iters: int, check: bool,
             multicast: bool = False, sleep_ms: int = 100):
    """Two driver runs per size: cuBLAS and this library back to back, then (with ``ref_lib``) the reference's
    kernels on their own. In one run the reference's thirteen kernels would sit between cuBLAS and this library
    and hand it a GPU that has been under full load for seconds, while cuBLAS started from idle. Every kernel is
    preceded by the driver's idle pause (``sleep_ms``; 100 ms is the reference's default, src/main.cu:42)."""
    log = out_dir / "log" / f"hgemm_{n}_{n}_{n}.log"
    js = out_dir / "json" / f"hgemm_{n}.jsonl"
    log.parent.mkdir(parents=True, exist_ok=True)
    js.parent.mkdir(parents=True, exist_ok=True)
    if js.exists():
        js.unlink()
    base = [str(binary), f"-M={n}", f"-N={n}", f"-K={n}", f"-warmup_iterations={warmup}",
            f"-profiling_iterations={iters}", f"-sleep_duration={sleep_ms}", f"-enable_check={'true' if check else 'false'}",
            "-enable_variants=false", f"-json={js}"]
    ours = base + ["-enable_wmma=false", "-enable_mma=false"] + (["-enable_multicast=true"] if multicast else [])
    with open(log, "w") as f:
        rc = subprocess.run(ours, stdout=f, stderr=subprocess.STDOUT).returncode
        if ref_lib and rc == 0:
            rc = subprocess.run(base + [f"-ref_lib={ref_lib}", "-enable_b200=false"], stdout=f, stderr=subprocess.STDOUT).returncode
    rows = [json.loads(line) for line in js.read_text().splitlines()] if js.exists() else []
    # the second run repeats the two cuBLAS calls: the first run's are the ones compared with this library
    seen, first = set(), []
    for r in rows:
        if r["kernel"].startswith("Cublas-") and r["kernel"] in seen:
            continue
        seen.add(r["kernel"])
        first.append(r)
    return rc, first


def summarise(n: int, rows):
    by = {r["kernel"]: r for r in rows}
    ref = {k: v for k, v in by.items() if k.startswith(REF_PREFIXES)}
    best_ref = max(ref.values(), key=lambda r: r["tflops"]) if ref else None
    ours = by.get("B200-Tcgen05-Auto")
    c16, c32 = by.get("Cublas-Tensor-Op"), by.get("Cublas-Tensor-Op-Fp32")
    return {
        "n": n,
        "cublas_fp16_compute": c16 and c16["tflops"],
        "cublas_fp32_compute": c32 and c32["tflops"],
        "reference_best": best_ref and best_ref["tflops"],
        "reference_best_kernel": best_ref and best_ref["kernel"],
        "b200": ours and ours["tflops"],
        "b200_max_rel_err": ours and ours["max_rel_err"],
        "reference_best_max_rel_err": best_ref and best_ref["max_rel_err"],
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default="sweep_out")
    ap.add_argument("--first", type=int, default=256)
    ap.add_argument("--last", type=int, default=16384)
    ap.add_argument("--step", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ref-lib", default=None, help="library built from the reference's kernels (optional)")
    ap.add_argument("--check-up-to", type=int, default=2048, help="run -enable_check for sizes up to this")
    ap.add_argument("--multicast", action="store_true", help="pass -enable_multicast=true to the driver (one GPU per process)")
    ap.add_argument("--sleep-ms", type=int, default=100, help="the driver's idle pause before every kernel (reference default: 100)")
    args = ap.parse_args(argv)

    binary = build.DRIVER_BIN
    if not binary.exists():
        build.build_driver()
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    summary = []
    with open(out_dir / "sweep.jsonl", "w") as allf:
        for n in range(args.first, args.last + 1, args.step):
            rc, rows = run_size(binary, n, out_dir, args.ref_lib, args.warmup, args.iters, n <= args.check_up_to, args.multicast, args.sleep_ms)
            for r in rows:
                allf.write(json.dumps(r) + "\n")
            s = summarise(n, rows)
            s["driver_rc"] = rc
            summary.append(s)
            print(json.dumps(s), flush=True)

    def fmt(x, nd=1):
        return "-" if x is None else f"{x:.{nd}f}"

    lines = ["| n | cuBLAS FP16-compute | cuBLAS FP32-compute | reference best (kernel) | B200 tcgen05 | vs best cuBLAS | "
             "vs reference best | max rel err (ours / ref best) |", "|---|---|---|---|---|---|---|---|"]
    for s in summary:
        cub = max([v for v in (s["cublas_fp16_compute"], s["cublas_fp32_compute"]) if v] or [0])
        ratio_c = s["b200"] / cub if s["b200"] and cub else None
        ratio_r = s["b200"] / s["reference_best"] if s["b200"] and s["reference_best"] else None
        err = "-"
        if s["b200_max_rel_err"] is not None and s["b200_max_rel_err"] >= 0:
            err = f"{s['b200_max_rel_err']:.1e} / " + (
                f"{s['reference_best_max_rel_err']:.1e}" if s["reference_best_max_rel_err"] not in (None, -1) else "-")
        lines.append(f"| {s['n']} | {fmt(s['cublas_fp16_compute'])} | {fmt(s['cublas_fp32_compute'])} | "
                     f"{fmt(s['reference_best'])} ({s['reference_best_kernel'] or '-'}) | {fmt(s['b200'])} | "
                     f"{fmt(ratio_c, 2)} | {fmt(ratio_r, 2)} | {err} |")
    (out_dir / "sweep.md").write_text("\n".join(lines) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
