"""A fixed number of launches of one shape and plan: what ``python -m cuda_hgemm_b200.profile`` puts under ncu.

    python -m cuda_hgemm_b200.profile_target --shape 16x14336x4096 [--plan skinny:16] [--launches 6] [--b-copies 7]
                                             [--cublas fp32|fp16] [--multicast] [--dist normal]

Exactly ``--launches`` launches of ours, then (with ``--cublas``) as many of the cuBLAS call, nothing else on the
GPU but the input generation: a profiler can skip and count launches by number. ``--b-copies`` cycles B through
that many copies so that a shape whose B fits L2 still reads it from HBM every time.
"""
from __future__ import annotations

import argparse
import sys

from . import api
from .abtest import parse_plan
from .timing import cublas_callable, load_compare


def main(argv=None) -> int:
    import torch

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shape", required=True, help="MxNxK")
    ap.add_argument("--plan", default="auto", help="auto, or a plan as abtest spells it (cta2:512, skinny2:128:g104, ...)")
    ap.add_argument("--launches", type=int, default=6)
    ap.add_argument("--b-copies", type=int, default=1)
    ap.add_argument("--cublas", choices=("none", "fp32", "fp16"), default="none")
    ap.add_argument("--multicast", action="store_true", help="this process owns one GPU: switch the multicast kernels on")
    ap.add_argument("--dist", choices=("uniform", "normal"), default="uniform")
    args = ap.parse_args(argv)

    if args.multicast and not api.enable_multicast(True):
        print("the multicast kernels are not available in this process", file=sys.stderr)
        return 1
    M, N, K = (int(x) for x in args.shape.lower().split("x"))
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(2023)
    if args.dist == "uniform":
        A = (torch.rand((M, K), generator=g, device=dev) * 2 - 1).half()
        B = (torch.rand((N, K), generator=g, device=dev) * 2 - 1).half()
    else:
        A = torch.randn((M, K), generator=g, device=dev).half()
        B = (torch.randn((N, K), generator=g, device=dev) / K ** 0.5).half()
    Bs = [B] + [B.clone() for _ in range(max(0, args.b_copies - 1))]
    C = torch.empty((M, N), dtype=torch.float16, device=dev)
    plan = None if args.plan == "auto" else parse_plan(args.plan)
    torch.cuda.synchronize()
    for i in range(args.launches):
        if plan is None:
            api.b200Hgemm(A, Bs[i % len(Bs)], C)
        else:
            api.hgemm_ex(A, Bs[i % len(Bs)], C, plan)
    torch.cuda.synchronize()
    if api.last_device_error() != 0:
        print("device-side wait expired", file=sys.stderr)
        return 1
    if args.cublas != "none":
        cmp_lib = load_compare()
        if cmp_lib is None:
            print("the cuBLAS comparison library is not built", file=sys.stderr)
            return 1
        calls = [cublas_callable(torch, cmp_lib, f"hgemm_compare_cublas_{args.cublas}", A, b, C) for b in Bs]
        for i in range(args.launches):
            calls[i % len(calls)]()
        torch.cuda.synchronize()
    used = api.select_plan(M, N, K).as_dict() if plan is None else plan.as_dict()
    print(f"{args.launches} launches of {M}x{N}x{K}, plan {used}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
