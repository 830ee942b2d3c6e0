"""Run the benchmark configurations through the ``hgemm`` driver, one log per shape.

The reference's ``run_sample.sh`` (reference run_sample.sh:15-60) runs its executable over a list
of square sizes and one sample shape and leaves ``log/hgemm_M_N_K.log`` files behind. This does
the same for the shapes this library is measured on, with the reference driver's flags:

    small     256^3 with the result check against the host GEMM
    squares   M = N = K from 256 to 16384 in steps of 256 (``cuda_hgemm_b200.sweep`` does this one
              with its own summary table; here it is a plain list of driver runs)
    large     16384^3
    decode    M in {16, 32, 64, 128} with (N, K) = (14336, 4096) and (4096, 14336); activations
              N(0, 1), weights N(0, 1/K), B cycled through 8 buffers so that it is read from HBM
    prefill   8192 x 28672 x 8192, same distributions

    python -m cuda_hgemm_b200.run_configs --out run_out --configs small,decode,prefill \\
        [--ref-lib oracle/_ref/libcuda_hgemm_ref.so] [--dry-run]

Every run appends its kernels' results to ``<out>/results.jsonl``; the logs keep the reference's
naming and line format, so its plot tool and ``cuda_hgemm_b200.plot`` read them.
"""
from __future__ import annotations

import argparse
import shlex
import subprocess
import sys
from pathlib import Path

from . import build

CONFIGS = ("small", "squares", "large", "decode", "prefill")


def shapes_of(config: str):
    """[(M, N, K, extra driver flags)] of one configuration."""
    normal = ["-dist=normal"]
    if config == "small":
        return [(256, 256, 256, ["-enable_check=true", "-check_rows=0"])]
    if config == "squares":
        return [(n, n, n, ["-enable_check=true"] if n <= 2048 else []) for n in range(256, 16384 + 1, 256)]
    if config == "large":
        return [(16384, 16384, 16384, [])]
    if config == "decode":
        out = []
        for n, k in ((14336, 4096), (4096, 14336)):
            for m in (16, 32, 64, 128):
                out.append((m, n, k, normal + ["-l2_rotate=8", "-enable_check=true", "-check_rows=0"]))
        return out
    if config == "prefill":
        return [(8192, 28672, 8192, normal + ["-enable_check=true"])]
    raise ValueError(f"unknown configuration {config!r}; one of {', '.join(CONFIGS)}")


def command(binary: Path, out_dir: Path, M: int, N: int, K: int, extra, ref_lib, warmup: int, iters: int):
    cmd = [str(binary), f"-M={M}", f"-N={N}", f"-K={K}", f"-warmup_iterations={warmup}", f"-profiling_iterations={iters}",
           "-sleep_duration=100", f"-json={out_dir / 'results.jsonl'}", *extra]
    # the reference's tuned kernels need M % 256 = N % 128 = K % 32 = 0 (reference src/mma/mma_async_stage4.cu:60-66)
    if ref_lib and M % 256 == 0 and N % 128 == 0 and K % 32 == 0:
        cmd.append(f"-ref_lib={ref_lib}")
    else:
        cmd += ["-enable_wmma=false", "-enable_mma=false"]
    return cmd


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default="run_out")
    ap.add_argument("--configs", default="small,large,decode,prefill", help="comma-separated: " + ", ".join(CONFIGS))
    ap.add_argument("--ref-lib", default=None, help="library built from the reference's kernels (optional)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--dry-run", action="store_true", help="print the driver commands instead of running them")
    args = ap.parse_args(argv)

    out_dir = Path(args.out)
    binary = build.DRIVER_BIN
    runs = []
    for config in args.configs.split(","):
        for M, N, K, extra in shapes_of(config.strip()):
            runs.append((M, N, K, command(binary, out_dir, M, N, K, extra, args.ref_lib, args.warmup, args.iters)))
    if args.dry_run:
        for _, _, _, cmd in runs:
            print(" ".join(shlex.quote(c) for c in cmd))
        return 0
    if not binary.exists():
        build.build_driver()
    (out_dir / "log").mkdir(parents=True, exist_ok=True)
    failed = 0
    for M, N, K, cmd in runs:
        log = out_dir / "log" / f"hgemm_{M}_{N}_{K}.log"
        with open(log, "w") as f:
            rc = subprocess.run(cmd, stdout=f, stderr=subprocess.STDOUT).returncode
        print(f"{M}x{N}x{K}: rc={rc} -> {log}", flush=True)
        failed += rc != 0
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
