"""What the host links give when every rank copies at once: the bound of the end-to-end figures.

    python -m cuda_hgemm_b200.hostlink                                   # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29541 \
        -m cuda_hgemm_b200.hostlink [--up-mib 256] [--down-mib 128] [--iters 10]

Every rank pins one buffer to upload and one to download, and after a barrier all ranks copy at the same time:
uploads alone, downloads alone, then both directions together on two streams (what `b200_hgemm_host` and
`multi_gpu.slab_hgemm_host` do while they multiply). Times are CUDA events around `--iters` copies per direction;
rank 0 prints one JSON line with every rank's GB/s and the sums. An end-to-end GEMM moves every byte of A, B and C
over these links once, however many GPUs share the work, so bytes / (sum of the ranks' rates) is the time it cannot
beat.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    import torch
    import torch.distributed as dist

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--up-mib", type=int, default=256)
    ap.add_argument("--down-mib", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    up_h = torch.empty(args.up_mib << 20, dtype=torch.uint8).pin_memory()
    down_h = torch.empty(args.down_mib << 20, dtype=torch.uint8).pin_memory()
    up_d = torch.empty_like(up_h, device=dev)
    down_d = torch.empty_like(down_h, device=dev)
    s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def timed(do_up: bool, do_down: bool):
        """GB/s of this rank's upload and download streams while the chosen directions run on every rank."""
        for _ in range(2):  # warm-up
            if do_up:
                with torch.cuda.stream(s_up):
                    up_d.copy_(up_h, non_blocking=True)
            if do_down:
                with torch.cuda.stream(s_down):
                    down_h.copy_(down_d, non_blocking=True)
        barrier()
        ev = {name: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for name in ("up", "down")}
        if do_up:
            with torch.cuda.stream(s_up):
                ev["up"][0].record()
                for _ in range(args.iters):
                    up_d.copy_(up_h, non_blocking=True)
                ev["up"][1].record()
        if do_down:
            with torch.cuda.stream(s_down):
                ev["down"][0].record()
                for _ in range(args.iters):
                    down_h.copy_(down_d, non_blocking=True)
                ev["down"][1].record()
        barrier()
        up = args.iters * up_h.numel() / (ev["up"][0].elapsed_time(ev["up"][1]) * 1e-3) / 1e9 if do_up else 0.0
        down = args.iters * down_h.numel() / (ev["down"][0].elapsed_time(ev["down"][1]) * 1e-3) / 1e9 if do_down else 0.0
        return up, down

    mine = {"up_alone": timed(True, False)[0], "down_alone": timed(False, True)[1]}
    mine["up_both"], mine["down_both"] = timed(True, True)
    rows = [mine]
    if world > 1:
        rows = [None] * world
        dist.all_gather_object(rows, mine)
    if rank == 0:
        out = {"n_gpus": world, "up_mib": args.up_mib, "down_mib": args.down_mib, "iters": args.iters, "unit": "GB/s",
               "per_rank": [{k: round(v, 1) for k, v in r.items()} for r in rows],
               "sum": {k: round(sum(r[k] for r in rows), 1) for k in mine}}
        out["sum"]["both_directions"] = round(out["sum"]["up_both"] + out["sum"]["down_both"], 1)
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
