"""Offline search for the best plan per shape; writes the table the library's dispatch reads.

For every shape the candidates are timed in alternation, ``--rounds`` times over, in the protocol
the reference driver uses (an idle pause, warm-up, ten back-to-back launches: ``timing.time_burst``)
or, with ``--sustained``, after a pre-heat under the power cap (``timing.time_launches``). The plan
the dispatch rules pick stays unless another candidate's median beats it by ``--margin`` (default
3 %): box-to-box variation is of that order, and a table entry should mean something on the next
box too. Only shapes that end up with a plan different from the rules' get a line.

    python -m cuda_hgemm_b200.autotune --squares 256:8192:256 --out cuda_hgemm_b200/plan_table.txt

The table is plain text, ``M N K variant bn parts group_m tma_store`` per line; the library loads
``plan_table.txt`` from the package directory at first use (see ``b200_hgemm_load_plan_table``).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys

from . import _native, api
from .timing import time_burst, time_launches


def candidate_plans(M: int, N: int, K: int):
    """Plans worth timing for this shape: every kernel family whose tiles make sense for it."""
    V = _native
    out = []

    def add(variant, bn, parts=0, group_m=0):
        p = V.Plan()
        p.variant, p.bn, p.parts, p.group_m, p.tma_store = variant, bn, parts, group_m, 1 if N % 8 == 0 else 0
        out.append(p)

    if K % 8 != 0:
        return out
    if M <= 64:
        add(V.VARIANT_SKINNY, 16 if M <= 16 else 32 if M <= 32 else 64)
        if M <= 32:
            add(V.VARIANT_SKINNY, 64)
    if M <= 256:
        for bn in (64, 128):
            add(V.VARIANT_CTA1, bn)
            add(V.VARIANT_STREAMK, bn)
        return out
    tiles256 = -(-M // 128) * -(-N // 256)
    for bn in (256, 128) + ((64,) if tiles256 <= 64 else ()):
        add(V.VARIANT_CTA1, bn)
    for bn in (256, 192, 128):
        add(V.VARIANT_CTA2, bn)
    if N % 8 == 0 and K >= 1024 and M * N >= 2048 * 2048:
        add(V.VARIANT_CTA2, 512)
        add(V.VARIANT_CTA2_MCAST, 512)
    return out


def plan_key(p):
    return (p.variant, p.bn, p.parts, p.group_m)


def tune_shape(torch, M, N, K, rounds, steps, margin, sustained, device):
    g = torch.Generator(device=device)
    g.manual_seed(2023)
    A = (torch.rand((M, K), generator=g, device=device) * 2 - 1).half()
    B = (torch.rand((N, K), generator=g, device=device) * 2 - 1).half()
    C = torch.empty((M, N), dtype=torch.float16, device=device)
    rules = api.select_plan_untuned(M, N, K)
    plans = {plan_key(rules): rules}
    for p in candidate_plans(M, N, K):
        plans.setdefault(plan_key(p), p)
    times = {key: [] for key in plans}
    unusable = set()
    for _ in range(rounds):
        for key, p in plans.items():
            if key in unusable:
                continue
            fn = (lambda p=p: api.hgemm_ex(A, B, C, p))
            try:
                ms = time_launches(torch, fn, 3, steps) if sustained else time_burst(torch, fn, 3, steps, idle_s=0.1)
            except _native.HgemmError:
                unusable.add(key)  # e.g. the multicast companion is not part of this run
                continue
            times[key].append(ms)
    if api.last_device_error() != 0:
        raise RuntimeError("a kernel gave up on a bounded wait")
    med = {key: statistics.median(v) for key, v in times.items() if v}
    rules_key = plan_key(rules)
    best_key = min(med, key=med.get)
    chosen = best_key if med[best_key] < med[rules_key] * (1.0 - margin) else rules_key
    gflop = 2.0 * M * N * K / 1e9
    return plans[chosen], chosen != rules_key, {
        "shape": [M, N, K], "rules": list(rules_key), "chosen": list(chosen),
        "tflops": {"/".join(map(str, key)): round(gflop / ms, 1) for key, ms in sorted(med.items(), key=lambda kv: kv[1])}}


def _options_without_paths(args):
    """The command line as recorded in the table's header: everything but where the files went."""
    out, skip = [], False
    for a in args:
        if skip:
            skip = False
        elif a in ("--out", "--log"):
            skip = True
        elif not a.startswith(("--out=", "--log=")):
            out.append(a)
    return out


def main(argv=None) -> int:
    import torch

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--squares", default="", help="first:last:step of square sizes, e.g. 256:8192:256")
    ap.add_argument("--shapes", default="", help="comma-separated MxNxK shapes")
    ap.add_argument("--out", required=True, help="table file to write")
    ap.add_argument("--log", default="", help="JSON lines with every candidate's TFLOP/s")
    ap.add_argument("--rounds", type=int, default=3)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--margin", type=float, default=0.03)
    ap.add_argument("--sustained", action="store_true", help="time under the power cap instead of in bursts")
    ap.add_argument("--multicast", action="store_true",
                    help="tune for a process that owns one GPU and has switched the multicast kernels on")
    args = ap.parse_args(argv)
    if args.multicast and not api.enable_multicast(True):
        ap.error("the multicast kernels are not available in this process")

    shapes = []
    if args.squares:
        first, last, step = (int(x) for x in args.squares.split(":"))
        shapes += [(n, n, n) for n in range(first, last + 1, step)]
    if args.shapes:
        shapes += [tuple(int(x) for x in s.lower().split("x")) for s in args.shapes.split(",")]
    if not shapes:
        ap.error("no shapes given")

    api.load_plan_table(None)  # measure against the rules, not against an older table
    device = torch.device("cuda", 0)
    lines, log = [], []
    for M, N, K in shapes:
        plan, differs, record = tune_shape(torch, M, N, K, args.rounds, args.steps, args.margin, args.sustained, device)
        log.append(record)
        print(json.dumps(record), flush=True)
        if differs:
            lines.append(f"{M} {N} {K} {plan.variant} {plan.bn} {plan.parts} {plan.group_m} {plan.tma_store}")
    protocol = "sustained (pre-heated, under the power cap)" if args.sustained else "burst (idle pause, 3 warm-up, %d launches)" % args.steps
    header = ["# Plans measured faster than the dispatch rules' own choice by more than %.0f %% (median of %d rounds, %s)." %
              (100 * args.margin, args.rounds, protocol),
              "# Written by: python -m cuda_hgemm_b200.autotune " + " ".join(_options_without_paths(sys.argv[1:] if argv is None else argv)),
              "# M N K variant bn parts group_m tma_store"]
    with open(args.out, "w") as f:
        f.write("\n".join(header + lines) + "\n")
    if args.log:
        with open(args.log, "w") as f:
            for record in log:
                f.write(json.dumps(record) + "\n")
    print(f"{len(lines)} of {len(shapes)} shapes got a table entry -> {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
