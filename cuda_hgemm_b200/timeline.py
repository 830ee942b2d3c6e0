"""Where the time of one kernel goes: per-CTA time stamps from a profiling build of the library.

    python -m cuda_hgemm_b200.timeline --cases 256x256x256,1024x1024x1024,16x14336x4096:skinny:16 [--md out.md]

A case is ``MxNxK`` (the dispatch's plan) or ``MxNxK:variant:bn[:gN][:pN]`` (a plan as ``abtest`` spells
it). For every case the profiling build (``-DB200_TIMELINE``, built on demand into
``lib/libb200_hgemm_timeline.so``) runs the plan three times untimed and once with a stamp buffer;
every CTA records ``%globaltimer`` at launch, after set-up (barriers, tensor-memory allocation), at
its first TMA load, when its producer / MMA issuer / epilogue finish, and at exit. The table gives the
minimum, median and maximum over the CTAs of each stamp, in microseconds after the first CTA's launch.
The stamps cost a few global stores per CTA; the kernel is otherwise the product's.
"""
from __future__ import annotations

import argparse
import ctypes
import sys

from . import _native, build
from .abtest import parse_plan

STAMPS = ("launch", "set-up done", "first load issued", "producer done", "first MMA", "last MMA issued",
          "epilogue: first tile ready", "epilogue: last tile ready", "epilogue: stores issued",
          "epilogue: stores read out", "exit", "producer: before the dependency wait", "producer: after the dependency wait",
          "producer: first stage free", "producer: first tile located")
# the order in which one CTA passes the stamps (for the cycle counts between consecutive ones)
ORDER = (0, 1, 11, 12, 14, 13, 2, 4, 3, 5, 6, 8, 9, 10)


def run_case(torch, lib, text, device, B_copies=1):
    shape, _, plan_text = text.partition(":")
    M, N, K = (int(x) for x in shape.lower().split("x"))
    plan = _native.Plan()
    if plan_text:
        plan = parse_plan(plan_text)
    else:
        _native.check(lib.b200_hgemm_select(M, N, K, ctypes.byref(plan)))
    a = torch.randn(M, K, device=device).half()
    bs = [torch.randn(N, K, device=device).half() for _ in range(B_copies)]
    c = torch.empty(M, N, device=device, dtype=torch.float16)
    stamps = torch.zeros(8192 * 32, dtype=torch.int64, device=device)
    s = torch.cuda.current_stream().cuda_stream

    def call(b):
        _native.check(lib.b200_hgemm_ex(a.data_ptr(), b.data_ptr(), c.data_ptr(), M, N, K, ctypes.byref(plan), s))

    lib.b200_debug_set_timeline(None)
    for i in range(3):
        call(bs[i % len(bs)])
    torch.cuda.synchronize()
    lib.b200_debug_set_timeline(stamps.data_ptr())
    call(bs[3 % len(bs)])
    torch.cuda.synchronize()
    lib.b200_debug_set_timeline(None)
    both = stamps.cpu().numpy().reshape(-1, 32)
    both = both[both[:, 0] > 0].astype("float64")
    t, cyc = both[:, :16], both[:, 16:]
    t0 = t[:, 0].min()
    rows = []
    for i, name in enumerate(STAMPS):
        col = t[:, i]
        col = col[col > 0]
        if len(col):
            r = sorted((col - t0) / 1e3)
            rows.append((name, r[0], r[len(r) // 2], r[-1]))
    # SM cycles between consecutive stamps of the same CTA (the global timer ticks every 0.256 us only); stamps
    # taken by different warps of the CTA still share the SM's counter
    steps = []
    seen = [i for i in ORDER if (cyc[:, i] > 0).all()]
    for a, b in zip(seen, seen[1:]):
        d = sorted(cyc[:, b] - cyc[:, a])
        steps.append((STAMPS[a], STAMPS[b], d[len(d) // 2]))
    return {"case": text, "shape": (M, N, K), "plan": plan.as_dict(), "ctas": int(len(t)), "rows": rows, "steps": steps}


def main(argv=None) -> int:
    import torch

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--cases", default="256x256x256,1024x1024x1024")
    ap.add_argument("--b-copies", type=int, default=1, help="distinct B buffers cycled through (decode shapes: 8, so B is not in L2)")
    ap.add_argument("--md", default="", help="also write the tables to this markdown file")
    args = ap.parse_args(argv)

    build.build_timeline()
    _native.LIB_PATH = build.TIMELINE_SO
    _native._lib = None
    lib = _native.load()
    lib.b200_debug_set_timeline.argtypes = [ctypes.c_void_p]
    lib.b200_debug_set_timeline.restype = None
    device = torch.device("cuda", 0)
    out = []
    for text in args.cases.split(","):
        r = run_case(torch, lib, text, device, args.b_copies)
        out.append(f"### {r['case']}  (plan {r['plan']}, {r['ctas']} CTAs)\n")
        out.append("| stamp | first CTA (us) | median | last CTA |")
        out.append("|---|---|---|---|")
        for name, lo, med, hi in r["rows"]:
            out.append(f"| {name} | {lo:.2f} | {med:.2f} | {hi:.2f} |")
        out.append("")
        out.append("SM cycles from one stamp to the next (median over the CTAs): " +
                   "; ".join(f"{a} -> {b}: {int(c)}" for a, b, c in r["steps"]))
        out.append("")
    text = "\n".join(out)
    print(text)
    if args.md:
        with open(args.md, "w") as f:
            f.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
