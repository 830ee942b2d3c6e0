"""Offline search for the best plan per shape; writes the table the library's dispatch reads.

For every shape the candidates are timed in alternation, ``--rounds`` times over, in the protocol
the reference driver uses (an idle pause, warm-up, ten back-to-back launches: ``timing.time_burst``)
or, with ``--sustained``, after a pre-heat under the power cap (``timing.time_launches``). The plan
the dispatch rules pick stays unless another candidate's median beats it by ``--margin`` (default
3 %): box-to-box variation is of that order, and a table entry should mean something on the next
box too. Only shapes that end up with a plan different from the rules' get a line.

    python -m cuda_hgemm_b200.autotune --squares 256:8192:256 --out cuda_hgemm_b200/plan_table.txt

Two passes per shape: first every kernel family and tile that suits it, with default knobs; then, around the
two fastest and the rules' own plan, the other knobs one at a time -- raster band height (``group_m``), ring
depth (``stages``), number of k-ranges (``parts``), column-tile width of the short-A kernels. Decode shapes
(M <= 128 against a large B) are timed with B cycling through copies larger than L2 in total, inside a CUDA graph.

The table is plain text, ``M N K variant bn parts group_m tma_store stages`` per line; the library loads
``plan_table.txt`` from the package directory at first use (see ``b200_hgemm_load_plan_table``).
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys

from . import _native, api
from .timing import time_burst, time_launches


def make_plan(variant, bn, N, parts=0, group_m=0, stages=0):
    p = _native.Plan()
    p.variant, p.bn, p.parts, p.group_m, p.stages, p.tma_store = variant, bn, parts, group_m, stages, 1 if N % 8 == 0 else 0
    return p


def candidate_plans(M: int, N: int, K: int):
    """First pass: every kernel family whose tiles make sense for the shape, each with its default knobs."""
    V = _native
    out = []

    def add(variant, bn, **kw):
        out.append(make_plan(variant, bn, N, **kw))

    if K % 8 != 0:
        return out
    if M <= 128:
        mt = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
        for variant in (V.VARIANT_SKINNY, V.VARIANT_SKINNY_PAIR):
            add(variant, mt)
            if mt < 128:
                add(variant, 2 * mt)
    if M <= 256:
        for bn in (64, 128):
            add(V.VARIANT_CTA1, bn)
            add(V.VARIANT_STREAMK, bn)
        return out
    tiles256 = -(-M // 128) * -(-N // 256)
    for bn in (256, 128) + ((64,) if tiles256 <= 64 else ()):
        add(V.VARIANT_CTA1, bn)
    for bn in (320, 288, 256, 224, 192, 160, 128):
        add(V.VARIANT_CTA2, bn)
    if N % 8 == 0 and K >= 1024 and M * N >= 2048 * 2048:
        add(V.VARIANT_CTA2, 512)
        add(V.VARIANT_CTA2_MCAST, 512)
    return out


# ring depths that exist besides the default (see b200_hgemm_plan.stages)
OTHER_STAGES = {(_native.VARIANT_CTA1, 256): (3,), (_native.VARIANT_CTA1, 128): (2,), (_native.VARIANT_CTA1, 64): (3,),
                (_native.VARIANT_CTA2, 256): (4, 5), (_native.VARIANT_CTA2, 128): (3,)}


def refinements(plan, M: int, N: int, K: int, sms: int = 148):
    """Second pass around one plan: its other knobs, one at a time -- raster band height, ring depth, number of
    k-ranges, column-tile width of the short-A kernels."""
    V = _native
    out = []
    v, bn = plan.variant, plan.bn
    if v in (V.VARIANT_CTA1, V.VARIANT_CTA2, V.VARIANT_CTA2_MCAST):
        row_blocks = -(-M // (128 if v == V.VARIANT_CTA1 else 512 if bn == 512 else 256))
        for g in (2, 3, 4, 6, 8, 12, 16, 32):
            if g < row_blocks:
                out.append(make_plan(v, bn, N, group_m=g, stages=plan.stages))
        for st in OTHER_STAGES.get((v, bn), ()):
            out.append(make_plan(v, bn, N, group_m=plan.group_m, stages=st))
    elif v in (V.VARIANT_STREAMK, V.VARIANT_HYBRID):
        for parts in (sms // 2, sms, 2 * sms):
            out.append(make_plan(v, bn, N, parts=parts))
    elif v in (V.VARIANT_SKINNY, V.VARIANT_SKINNY_PAIR):
        for w in (128, 120, 112, 104, 96, 80, 64):
            out.append(make_plan(v, bn, N, group_m=w))
        for parts in (1, 2, 3, 4, 6, 8):
            if parts * 8 * 64 <= K:
                out.append(make_plan(v, bn, N, parts=parts))
    return out


def plan_key(p):
    return (p.variant, p.bn, p.parts, p.group_m, p.stages)


def tune_shape(torch, M, N, K, rounds, steps, margin, sustained, device, dist="uniform"):
    from .timing import time_graph

    g = torch.Generator(device=device)
    g.manual_seed(2023)
    if dist == "uniform":
        A = (torch.rand((M, K), generator=g, device=device) * 2 - 1).half()
        B = (torch.rand((N, K), generator=g, device=device) * 2 - 1).half()
    else:
        A = torch.randn((M, K), generator=g, device=device).half()
        B = (torch.randn((N, K), generator=g, device=device) / K ** 0.5).half()
    C = torch.empty((M, N), dtype=torch.float16, device=device)
    # shapes whose operands would stay in L2 between launches although they are meant to come from HBM (the
    # decode shapes: one large B): B cycles through copies, launches are timed inside a CUDA graph
    rotate = M <= 128 and N * K * 2 >= (32 << 20)
    Bs = [B]
    if rotate:
        while len(Bs) * N * K * 2 < (768 << 20) and len(Bs) < 64:
            Bs.append(B.clone())
    turn = [0]
    rules = api.select_plan_untuned(M, N, K)
    times, plans, unusable = {}, {}, set()

    def measure(p):
        key = plan_key(p)
        if key in unusable:
            return
        plans.setdefault(key, p)

        def fn():
            api.hgemm_ex(A, Bs[turn[0] % len(Bs)], C, plans[key])
            turn[0] += 1
        try:
            if rotate:
                ms = time_graph(torch, fn, launches=3 * len(Bs), replays=3)
            elif sustained:
                ms = time_launches(torch, fn, 3, steps)
            else:
                ms = time_burst(torch, fn, 3, steps, idle_s=0.1)
        except _native.HgemmError:
            unusable.add(key)  # e.g. the multicast kernels are not switched on in this run
            return
        times.setdefault(key, []).append(ms)

    def medians():
        return {key: statistics.median(v) for key, v in times.items() if v}

    first = [rules] + candidate_plans(M, N, K)
    for _ in range(rounds):
        for p in first:
            measure(p)
    med = medians()
    rules_key = plan_key(rules)
    leaders = sorted(med, key=med.get)[:2]
    second = []
    for key in dict.fromkeys(leaders + [rules_key]):
        second += refinements(plans[key], M, N, K)
    for _ in range(rounds):
        for p in second:
            measure(p)
        for key in leaders + [rules_key]:  # the references are re-timed beside their variations
            measure(plans[key])
    if api.last_device_error() != 0:
        raise RuntimeError("a kernel gave up on a bounded wait")
    med = medians()
    best_key = min(med, key=med.get)
    chosen = best_key if med[best_key] < med[rules_key] * (1.0 - margin) else rules_key
    gflop = 2.0 * M * N * K / 1e9
    return plans[chosen], chosen != rules_key, {
        "shape": [M, N, K], "rules": list(rules_key), "chosen": list(chosen), "candidates": len(med),
        "protocol": "graph, B rotated" if rotate else "sustained" if sustained else "burst",
        "tflops": {"/".join(map(str, key)): round(gflop / ms, 1) for key, ms in sorted(med.items(), key=lambda kv: kv[1])}}


def _options_without_paths(args):
    """The command line as recorded in the table's header: everything but where the files went."""
    out, skip = [], False
    for a in args:
        if skip:
            skip = False
        elif a in ("--out", "--log", "--md"):
            skip = True
        elif not a.startswith(("--out=", "--log=", "--md=")):
            out.append(a)
    return out


def main(argv=None) -> int:
    import torch

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--squares", default="", help="first:last:step of square sizes, e.g. 256:8192:256")
    ap.add_argument("--shapes", default="", help="comma-separated MxNxK shapes")
    ap.add_argument("--out", required=True, help="table file to write")
    ap.add_argument("--log", default="", help="JSON lines with every candidate's TFLOP/s")
    ap.add_argument("--md", default="", help="markdown table: per shape the rules' plan, the chosen one and the three fastest")
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
        plan, differs, record = tune_shape(torch, M, N, K, args.rounds, args.steps, args.margin, args.sustained, device,
                                           dist="normal" if M <= 128 else "uniform")
        log.append(record)
        print(json.dumps(record), flush=True)
        if differs:
            lines.append(f"{M} {N} {K} {plan.variant} {plan.bn} {plan.parts} {plan.group_m} {plan.tma_store} {plan.stages}")
    protocol = "sustained (pre-heated, under the power cap)" if args.sustained else "burst (idle pause, 3 warm-up, %d launches)" % args.steps
    header = ["# Plans measured faster than the dispatch rules' own choice by more than %.0f %% (median of %d rounds, %s)." %
              (100 * args.margin, args.rounds, protocol),
              "# Written by: python -m cuda_hgemm_b200.autotune " + " ".join(_options_without_paths(sys.argv[1:] if argv is None else argv)),
              "# M N K variant bn parts group_m tma_store stages"]
    with open(args.out, "w") as f:
        f.write("\n".join(header + lines) + "\n")
    if args.log:
        with open(args.log, "w") as f:
            for record in log:
                f.write(json.dumps(record) + "\n")
    if args.md:
        md = ["| shape | rules' plan | TFLOP/s | chosen | TFLOP/s | candidates timed | three fastest (variant/bn/parts/group_m/stages: TFLOP/s) |",
              "|---|---|---|---|---|---|---|"]
        for r in log:
            t = r["tflops"]
            rk, ck = "/".join(map(str, r["rules"])), "/".join(map(str, r["chosen"]))
            top = ", ".join(f"{k}: {v}" for k, v in list(t.items())[:3])
            md.append(f"| {'x'.join(map(str, r['shape']))} | {rk} | {t.get(rk)} | {ck} | {t.get(ck)} | {r['candidates']} | {top} |")
        with open(args.md, "w") as f:
            f.write(f"Protocol per shape as named in the log; margin {args.margin:.0%}; median of {args.rounds} rounds.\n\n")
            f.write("\n".join(md) + "\n")
    print(f"{len(lines)} of {len(shapes)} shapes got a table entry -> {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
