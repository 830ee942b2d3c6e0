#!/usr/bin/env python
"""HGEMM benchmark: TFLOP/s of C[M x N] = A[M x K] * B on B200, next to cuBLAS.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step is one GEMM of the workload. The default workload is the 16384^3 square HGEMM -- the
largest point of the reference's square sweep (reference run_sample.sh:29-37) -- on one GPU; with
N GPUs (one process per GPU under torchrun) the same problem is split into N row slabs of C
(A sharded along M, B replicated, no data exchange), so the series over N is strong scaling.
Inputs are synthetic: FP16 values uniform in [-1, 1) from a fixed seed, as the reference's own
driver draws them (reference src/common/matrix.h:28-33, there unseeded).

Rank 0 prints ONE JSON line. `value` is whole-job TFLOP/s with operands resident in HBM,
timed with CUDA events on the launching stream (max over ranks); `e2e` is the same metric
through the host-pointer entry point of the C ABI, copies included; `roofline` relates the
kernel to the measured tensor-core peak; `cpu_baseline` is the FP32-accumulate host GEMM of the
checker timed on this box's cores. `--impl reference` times the reference project's own kernels
(compiled unmodified for sm_100a) on the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

SEED = 2023
NOMINAL_FP16_DENSE_TFLOPS = 2250.0

WORKLOADS = {
    # name: (M, N, K, distribution, description)
    "square16384": (16384, 16384, 16384, "uniform", "square HGEMM M=N=K=16384, largest point of the 256..16384 sweep"),
    "square8192": (8192, 8192, 8192, "uniform", "square HGEMM M=N=K=8192"),
    "square4096": (4096, 4096, 4096, "uniform", "square HGEMM M=N=K=4096"),
    "prefill": (8192, 28672, 8192, "normal", "prefill-style HGEMM M=8192 N=28672 K=8192"),
    "skinny16": (16, 14336, 4096, "normal", "decode-style HGEMM M=16 N=14336 K=4096"),
    "skinny128": (128, 14336, 4096, "normal", "decode-style HGEMM M=128 N=14336 K=4096"),
    "skinny128t": (128, 4096, 14336, "normal", "decode-style HGEMM M=128 N=4096 K=14336"),
    "skinny32": (32, 14336, 4096, "normal", "decode-style HGEMM M=32 N=14336 K=4096"),
    "skinny64": (64, 14336, 4096, "normal", "decode-style HGEMM M=64 N=14336 K=4096"),
    "skinny16t": (16, 4096, 14336, "normal", "decode-style HGEMM M=16 N=4096 K=14336"),
}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return {"tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)),
                    "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
        except Exception:
            pass
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._ok = False
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            uuid = None
            try:
                import torch

                uuid = str(torch.cuda.get_device_properties(index).uuid)
            except Exception:
                pass
            self.handle = None
            if uuid:
                for i in range(pynvml.nvmlDeviceGetCount()):
                    h = pynvml.nvmlDeviceGetHandleByIndex(i)
                    u = pynvml.nvmlDeviceGetUUID(h)
                    u = u.decode() if isinstance(u, bytes) else u
                    if uuid in u:
                        self.handle = h
            if self.handle is None:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self._ok = True
        except Exception:
            self._ok = False

    REASONS = (("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40),
               ("hw_power_brake_slowdown", 0x80), ("sw_power_cap", 0x4))

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else int(
                    nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                for name, bit in self.REASONS:
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._ok:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_inputs(torch, M, N, K, dist, device, row_lo, row_hi):
    """Seeded operands on the device. Every rank draws the same B; the A slab is cut from the
    same full-size draw a single GPU would use, so the job's inputs do not depend on N."""
    g = torch.Generator(device=device)
    g.manual_seed(SEED)
    if dist == "uniform":
        A = torch.rand((M, K), generator=g, device=device, dtype=torch.float32).mul_(2).sub_(1).to(torch.float16)
        g.manual_seed(SEED + 1)
        B = torch.rand((N, K), generator=g, device=device, dtype=torch.float32).mul_(2).sub_(1).to(torch.float16)
    else:
        A = torch.randn((M, K), generator=g, device=device, dtype=torch.float32).to(torch.float16)
        g.manual_seed(SEED + 1)
        B = (torch.randn((N, K), generator=g, device=device, dtype=torch.float32) / (K ** 0.5)).to(torch.float16)
    return A[row_lo:row_hi].contiguous(), B


from cuda_hgemm_b200 import _native  # noqa: E402
from cuda_hgemm_b200.timing import (PREHEAT_S, cublas_callable, load_compare, time_burst, time_graph,  # noqa: E402
                                    time_launches, time_native_loop, time_native_rotate)

MIN_TIMED_MS = 120.0  # the timed region is at least this long, so that the 2 ms clock sampler sees it often enough


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the committed ncu
# captures under profiles/, keyed by the shape one launch multiplies (a rank's slab, not the job)
# and by the kernel the dispatch picks for it (variant, bn); scaled captures say so there.
NCU_TRAFFIC_BYTES = {
    ((16384, 16384, 16384), _native.VARIANT_CTA2_MCAST, 512): 7.49e9,  # profiles/hgemm_tcgen05_mc512_square16384.md
    ((16384, 16384, 16384), _native.VARIANT_CTA2, 512): 7.80e9,        # profiles/hgemm_tcgen05_big_square16384.md
    ((16384, 16384, 16384), _native.VARIANT_CTA2, 256): 16.5e9,        # profiles/hgemm_tcgen05_big_vs_cublas_square16384.md
    ((8192, 28672, 8192), _native.VARIANT_CTA2, 512): 4.26e9,          # profiles/hgemm_tcgen05_big_prefill.md
    ((8192, 8192, 8192), _native.VARIANT_CTA2_MCAST, 512): 0.936e9,    # profiles/hgemm_tcgen05_mc512_square8192.md
    ((8192, 8192, 8192), _native.VARIANT_CTA2, 256): 1.118e9,          # profiles/hgemm_tcgen05_cta2_square8192.md
    ((16, 14336, 4096), _native.VARIANT_SKINNY, 16): 121.3e6,          # profiles/hgemm_skinny_skinny16.md
    ((128, 14336, 4096), _native.VARIANT_SKINNY_PAIR, 128): 122.3e6,   # profiles/hgemm_skinny_pair_skinny128.md
    ((16, 4096, 14336), _native.VARIANT_SKINNY, 16): 121.4e6,          # profiles/hgemm_skinny_skinny16t.md
    ((128, 4096, 14336), _native.VARIANT_SKINNY, 128): 125.0e6,        # profiles/hgemm_skinny_skinny128t.md
}


def ncu_traffic(shape, plan):
    """Measured DRAM bytes of one launch on `shape` = (rows, N, K), or None where no capture exists."""
    return NCU_TRAFFIC_BYTES.get((tuple(shape), plan.variant, plan.bn)) if plan is not None else None


def roofline(plan, rows, N, K, ms_per_step, peaks):
    """Roofline entry of the dominant kernel for one launch of this rank's slab."""
    skinny = rows <= 128
    if skinny:
        algo = 2.0 * (rows * K + N * K + rows * N)
        achieved = algo / (ms_per_step * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": f"{peaks['source']} copy bandwidth",
                "traffic": ncu_traffic((rows, N, K), plan)}
    achieved = 2.0 * rows * N * K / (ms_per_step * 1e-3) / 1e12
    # the timed region follows a pre-heat and runs back to back under the power cap: the sustained
    # cuBLAS figure is the matching denominator; the burst figure is printed beside it
    peak = peaks["tflops_sustained"] or peaks["tflops"]
    return {"bound": "tensor", "achieved": round(achieved, 2), "peak": peak, "unit": "TFLOP/s",
            "frac": round(achieved / peak, 4),
            "peak_source": f"{peaks['source']} cuBLAS bf16, sustained (kernel timed in a back-to-back loop after a pre-heat)",
            "frac_of_burst_peak": round(achieved / peaks["tflops"], 4), "burst_peak": peaks["tflops"],
            "traffic": ncu_traffic((rows, N, K), plan)}


EXTRA_WORKLOADS = ("skinny16", "skinny32", "skinny64", "skinny128", "skinny16t", "skinny128t", "prefill")


def measure_workload(torch, api, cmp_lib, name, device, peaks, warmup, steps):
    """One more configuration of the benchmark on this GPU: ms, TFLOP/s, roofline and both cuBLAS modes."""
    M, N, K, dist_name, desc = WORKLOADS[name]
    A, B = make_inputs(torch, M, N, K, dist_name, device, 0, M)
    C = torch.empty((M, N), dtype=torch.float16, device=device)
    Bs = [B]
    if (M * K + N * K + M * N) * 2 < (512 << 20):
        while len(Bs) * N * K * 2 < (768 << 20) and len(Bs) < 64:
            Bs.append(B.clone())
    plan = api.select_plan(M, N, K)
    turn = [0]

    def ours():
        api.b200Hgemm(A, Bs[turn[0] % len(Bs)], C)
        turn[0] += 1
    before = api.launch_count()
    ours()
    per_call = api.launch_count() - before
    rotated = len(Bs) > 1 and cmp_lib is not None
    lib = _native.load()
    Cc = torch.empty_like(C)
    contenders = [("ours", lib.b200_hgemm, ours, C)]
    if cmp_lib is not None:
        contenders += [("cublas_fp16_compute_tflops", cmp_lib.hgemm_compare_cublas_fp16, None, Cc),
                       ("cublas_fp32_compute_tflops", cmp_lib.hgemm_compare_cublas_fp32, None, Cc)]
    # The libraries are timed in alternation, twice over, each time after a short idle pause and its own warm-up,
    # and the better round counts: whoever is measured right behind a power-capped GEMM would otherwise be timed
    # on a GPU that is still settling.
    best = {}
    for _ in range(2):
        for key, entry, py_call, out in contenders:
            torch.cuda.synchronize()
            time.sleep(0.2)
            if rotated:
                # kernels of tens of microseconds: launched back to back from native code, so that the interpreter's
                # cost per call (about as long as the kernel) is not what is timed
                t = time_native_rotate(torch, cmp_lib, entry, A, Bs, out, warmup=200, iters=400)
            elif py_call is not None:
                t = time_launches(torch, py_call, warmup, steps)
            else:
                sym = "hgemm_compare_cublas_fp16" if "fp16" in key else "hgemm_compare_cublas_fp32"
                t = time_launches(torch, cublas_callable(torch, cmp_lib, sym, A, B, out), warmup, steps)
            best[key] = min(best.get(key, t), t)
    ms = best["ours"]
    flops = 2.0 * M * N * K
    entry = {"workload": f"{name}: {desc}", "M": M, "N": N, "K": K, "plan": plan.as_dict(), "ms": round(ms, 5),
             "tflops": round(flops / (ms * 1e-3) / 1e12, 2), "kernels_per_call": int(per_call),
             "l2": f"B cycled through {len(Bs)} copies" if len(Bs) > 1 else "operands larger than L2",
             "timing": ("400 back-to-back launches from native code after 200 untimed" if rotated else
                        f"{steps} back-to-back launches after a 0.3 s pre-heat") + "; libraries in alternation, better of 2 rounds",
             "roofline": roofline(plan, M, N, K, ms, peaks)}
    for key in ("cublas_fp16_compute_tflops", "cublas_fp32_compute_tflops"):
        if key in best:
            entry[key] = round(flops / (best[key] * 1e-3) / 1e12, 2)
    if cmp_lib is not None:
        entry["vs_cublas_best"] = round(entry["tflops"] / max(entry["cublas_fp16_compute_tflops"],
                                                              entry["cublas_fp32_compute_tflops"]), 4)
    if api.last_device_error() != 0:
        raise RuntimeError(f"{name}: a kernel gave up on a bounded wait")
    return entry


def cpu_baseline(M, N, K, dist):
    """FP32-accumulate host GEMM (the checker's code) on a bounded row sample of the workload."""
    import numpy as np

    from oracle import hgemm_oracle as oracle

    rng = np.random.default_rng(SEED)
    threads = oracle.max_threads()
    probe_rows = min(M, 64)
    rows_cap = min(M, 4096)
    if dist == "uniform":
        A = rng.uniform(-1, 1, size=(rows_cap, K)).astype(np.float16)
        B = rng.uniform(-1, 1, size=(N, K)).astype(np.float16)
    else:
        A = rng.standard_normal(size=(rows_cap, K), dtype=np.float32).astype(np.float16)
        B = (rng.standard_normal(size=(N, K), dtype=np.float32) / np.sqrt(K)).astype(np.float16)
    t_probe = oracle.time_rows(A, B, probe_rows, threads)
    # aim at about 10 s of CPU work
    rows = int(max(probe_rows, min(rows_cap, probe_rows * 10.0 / max(t_probe, 1e-6))))
    rows = max(1, (rows // 8) * 8) if rows >= 8 else rows
    t = oracle.time_rows(A, B, rows, threads)
    tflops = 2.0 * rows * N * K / t / 1e12
    return {"value": round(tflops, 6), "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"first {rows} of {M} rows of C (rows x {N} x {K}), {t:.2f} s wall; whole-matrix time scales linearly in M"}


ALL_CPUS = set(os.sched_getaffinity(0))  # what this process may run on, before any binding


def bind_to_gpu_cpus(torch, index):
    """Run this process on the CPUs NVML names as local to GPU `index`, so that the pinned host buffers it
    allocates afterwards lie in the memory next to that GPU's host link (with eight ranks on a two-socket host,
    half of them would otherwise copy across the sockets). Returns the CPU count it bound to, or None."""
    try:
        import pynvml

        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(index).uuid)
        handle = None
        for i in range(pynvml.nvmlDeviceGetCount()):
            h = pynvml.nvmlDeviceGetHandleByIndex(i)
            u = pynvml.nvmlDeviceGetUUID(h)
            if uuid in (u.decode() if isinstance(u, bytes) else u):
                handle = h
        if handle is None:
            return None
        n_cpus = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (n_cpus + 63) // 64)
        local = {c for c in range(n_cpus) if (int(words[c // 64]) >> (c % 64)) & 1}
        allowed = local & set(os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return len(allowed)
    except Exception:
        return None


def dist_setup(torch, n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(local)
    return rank, world, local


def dist_teardown(world):
    if world > 1:
        import torch.distributed as dist

        if dist.is_initialized():
            dist.destroy_process_group()


def barrier(torch, world):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(torch, value, world, device):
    if world == 1:
        return value
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_ours(args):
    import torch

    from cuda_hgemm_b200 import api
    from cuda_hgemm_b200.partition import row_slabs

    rank, world, local = dist_setup(torch, args.gpus)
    device = torch.device("cuda", local)
    bound_cpus = bind_to_gpu_cpus(torch, local)
    M, N, K, dist_name, desc = WORKLOADS[args.workload]
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    lo, hi = row_slabs(M, world)[rank]
    A, B = make_inputs(torch, M, N, K, dist_name, device, lo, hi)
    C = torch.empty((hi - lo, N), dtype=torch.float16, device=device)
    rows = hi - lo
    # one process, one GPU: the kernels with multicast operand loads may be switched on (the library
    # refuses in a process that is one rank of several, and works the same without them)
    multicast = api.enable_multicast(True) if world == 1 else False
    plan = api.select_plan(rows, N, K) if rows else None
    # Operands that fit in the 126 MB L2 (the decode-style shapes: B is 117 MB) would be served from
    # L2 on every step after the first: cycle through enough copies of B to exceed L2 several times.
    small = (rows * K + N * K + rows * N) * 2 < (512 << 20)
    Bs = [B]
    if small:
        while len(Bs) * N * K * 2 < (768 << 20) and len(Bs) < 64:
            Bs.append(B.clone())
    counter = [0]

    def step():
        if rows:
            api.b200Hgemm(A, Bs[counter[0] % len(Bs)], C)
            counter[0] += 1

    # ---- device-resident timing: the headline kernel number ----
    # Every N is timed in the same regime: ranks meet at the barrier FIRST, then each runs about
    # 0.3 s of back-to-back steps (the GPU settles under its power cap), and the timed blocks follow
    # with no host synchronisation in between. A block is `steps` launches between two events; blocks
    # repeat until the clock sampler has read the GPU often enough inside the timed region.
    step()
    torch.cuda.synchronize()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record()
    for _ in range(warmup):
        step()
    p1.record()
    torch.cuda.synchronize()
    one_ms = max(p0.elapsed_time(p1) / warmup, 1e-3)
    preheat_steps = int(max_over_ranks(torch, min(20000.0, PREHEAT_S * 1e3 / one_ms), world, device)) if rows else 0
    blocks = max(1, min(64, int(-(-MIN_TIMED_MS // (one_ms * steps))))) if rows else 1
    blocks = int(max_over_ranks(torch, float(blocks), world, device))
    barrier(torch, world)
    for _ in range(preheat_steps):
        step()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
    with ClockSampler(local) as sampler:
        launches_timed0 = api.launch_count()
        marks[0].record()
        for b in range(blocks):
            for _ in range(steps):
                step()
            marks[b + 1].record()
        torch.cuda.synchronize()
        launches_timed = (api.launch_count() - launches_timed0) // blocks
    barrier(torch, world)
    block_ms = [marks[b].elapsed_time(marks[b + 1]) for b in range(blocks)]
    ms_total = max_over_ranks(torch, sum(block_ms) / blocks, world, device)
    if api.last_device_error() != 0:
        raise RuntimeError("a kernel gave up on a bounded wait")
    ms_per_step = ms_total / steps
    flops_job = 2.0 * M * N * K
    value = flops_job / (ms_per_step * 1e-3) / 1e12
    clocks = sampler.summary()
    clocks["timed_blocks"] = blocks
    clocks["enough_samples"] = clocks["samples"] >= 5
    if clocks["sm_mhz"]:
        # time x clock: comparable between runs that were granted different clocks under the cap
        clocks["ms_x_mhz_per_step"] = round(ms_per_step * clocks["sm_mhz"], 2)
    # the reference driver's own protocol beside it: idle pause, 3 warm-up, 10 launches, no pre-heat
    barrier(torch, world)
    burst_ms = max_over_ranks(torch, time_burst(torch, step, 3, 10) if rows else 0.0, world, device)
    barrier(torch, world)

    # ---- end to end through the host-pointer entry point ----
    e2e_steps = max(1, min(steps, 5))
    hA = torch.empty((rows, K), dtype=torch.float16).pin_memory()
    hB = torch.empty((N, K), dtype=torch.float16).pin_memory()
    hC = torch.empty((rows, N), dtype=torch.float16).pin_memory()
    hA.copy_(A)
    hB.copy_(B)
    # Several ranks: every rank uploads its rows of A and 1/world of B, the shares of B are exchanged between
    # the GPUs (NCCL all-gather over NVLink), then the slab is multiplied and comes back: the host link of a GPU
    # carries (M*K + N*K) / world halves up and M*N / world down instead of all of B.
    from cuda_hgemm_b200 import multi_gpu

    sharded_b = world > 1 and N % world == 0
    dB_e2e = torch.empty((N, K), dtype=torch.float16, device=device) if sharded_b else None

    def e2e_once():
        if sharded_b:
            multi_gpu.slab_hgemm_host(hA, hB, hC, dB_e2e)
        elif rows:
            api.hgemm_host(hA, hB, hC)

    e2e_once()  # warm-up: staging buffers, streams and the communicator's buffers are created here
    barrier(torch, world)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_once()
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(torch, (time.perf_counter() - t0) / e2e_steps, world, device)
    barrier(torch, world)
    if rows:
        api.b200Hgemm(A, B, C)
        torch.cuda.synchronize()
    e2e_ok = bool(torch.equal(hC.to(device), C)) if rows else True

    # ---- optional: all-gather of the C slabs (never part of the multiply; timed on its own) ----
    gather_ms = None
    if world > 1 and args.gather:
        from cuda_hgemm_b200 import multi_gpu

        for _ in range(2):
            multi_gpu.allgather_c(C, M, N)
        barrier(torch, world)
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(5):
            multi_gpu.allgather_c(C, M, N)
        g1.record()
        torch.cuda.synchronize()
        gather_ms = max_over_ranks(torch, g0.elapsed_time(g1) / 5, world, device)

    if rank != 0:
        dist_teardown(world)
        return
    peaks = measured_peaks()
    flops_launch = 2.0 * rows * N * K
    out = {
        "metric": "HGEMM TFLOP/s vs cuBLAS and % FP16 TC peak",
        "value": round(value, 2),
        "unit": "TFLOP/s",
        "n_gpus": world,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": round(ms_per_step, 5),
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f16 (FP32 accumulate in tensor memory, FP16 out)",
        "data": f"synthetic: FP16 {dist_name} from seed {SEED}",
        "config": {"workload": f"{args.workload}: {desc}", "M": M, "N": N, "K": K,
                   "partition": f"{world} row slab(s) of C, B replicated, no collective",
                   "l2": (f"B cycled through {len(Bs)} distinct copies ({len(Bs) * N * K * 2 >> 20} MiB in total) so that no step "
                          "finds its operands in L2") if len(Bs) > 1 else "operands larger than L2",
                   "plan": plan.as_dict() if plan else None, "multicast_kernels": multicast},
        "timed_region": (f"barrier, {preheat_steps} untimed steps back to back (about {PREHEAT_S} s), then {blocks} block(s) of "
                         f"{steps} steps between CUDA events with no host synchronisation; ms_per_step is the mean over the blocks"),
        "burst": {"value": round(flops_job / (burst_ms * 1e-3) / 1e12, 2) if burst_ms else None, "unit": "TFLOP/s",
                  "protocol": "idle 0.25 s, 3 warm-up, 10 launches (the reference driver's, reference src/common/tester.h:55-64,91-95)"},
        "gpu_launches": int(launches_timed),
        "pct_fp16_dense_peak": round(100.0 * value / (NOMINAL_FP16_DENSE_TFLOPS * world), 2),
        "clocks": clocks,
        "e2e": {"value": round(flops_job / e2e_s / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": int((rows * K + (N // world if sharded_b else N) * K) * 2),
                "d2h_bytes_per_step": int(rows * N * 2),
                "nvlink_bytes_per_step": int((N - N // world) * K * 2) if sharded_b else 0,
                "steps": e2e_steps, "matches_device_result": e2e_ok, "host_cpus_bound_to_gpu": bound_cpus,
                "api": ("multi_gpu.slab_hgemm_host (per rank: pinned host buffers -> H2D of A's rows and 1/N of B -> "
                        "NCCL all-gather of B -> b200_hgemm_host_a -> D2H)") if sharded_b else
                       "b200_hgemm_host (pinned host buffers -> H2D -> kernel -> D2H, per rank)"},
        "roofline": roofline(plan, rows, N, K, ms_per_step, peaks),
    }

    # ---- comparisons on the same operands (outside the timed region) ----
    cmp_lib = load_compare()
    if cmp_lib is not None and rows:
        Cc = torch.empty_like(C)
        for key, sym in (("cublas_fp16_compute_tflops", "hgemm_compare_cublas_fp16"),
                         ("cublas_fp32_compute_tflops", "hgemm_compare_cublas_fp32")):
            calls = [cublas_callable(torch, cmp_lib, sym, A, b, Cc) for b in Bs]  # same rotation of B as ours
            turn = [0]

            def cublas_step():
                calls[turn[0] % len(calls)]()
                turn[0] += 1
            ms = time_launches(torch, cublas_step, warmup, steps)
            out[key] = round(world * flops_launch / (ms * 1e-3) / 1e12, 2)
        best = max(out["cublas_fp16_compute_tflops"], out["cublas_fp32_compute_tflops"])
        out["vs_cublas_best"] = round(value / best, 4)
        out["vs_cublas_fp32_compute"] = round(value / out["cublas_fp32_compute_tflops"], 4)

    if world == 1 and not args.no_sweep and cmp_lib is not None:
        from cuda_hgemm_b200 import _native

        ours_entry = _native.load().b200_hgemm
        sweep = []
        for n in (256, 512, 1024, 2048, 4096, 8192):
            a, b = make_inputs(torch, n, n, n, "uniform", device, 0, n)
            c = torch.empty((n, n), dtype=torch.float16, device=device)
            f = 2.0 * n ** 3 / 1e9
            row = {"n": n}
            # (1) the reference driver's protocol: 3 warm-up + 10 back-to-back stream launches
            for key, entry in (("tflops", ours_entry), ("cublas_fp32_compute", cmp_lib.hgemm_compare_cublas_fp32),
                               ("cublas_fp16_compute", cmp_lib.hgemm_compare_cublas_fp16)):
                best = min(time_native_loop(torch, cmp_lib, entry, a, b, c) for _ in range(3))
                row[key] = round(f / best, 2)
            # (2) 20 launches per CUDA graph: launch cost removed for every library alike
            row["graph_tflops"] = round(f / time_graph(torch, lambda: api.b200Hgemm(a, b, c)), 2)
            row["graph_cublas_fp32_compute"] = round(
                f / time_graph(torch, cublas_callable(torch, cmp_lib, "hgemm_compare_cublas_fp32", a, b, c)), 2)
            sweep.append(row)
        out["sweep_points"] = sweep
        out["sweep_note"] = ("tflops / cublas_*: reference driver protocol (3 warm-up + 10 back-to-back stream launches from native "
                             "code, best of 3); graph_*: 20 launches per CUDA graph, 5 replays; operands of the small sizes stay "
                             "in L2 for every library alike")

    if world == 1 and not args.no_workloads:
        # the other benchmark configurations, each with its own roofline (decode shapes: HBM bound, B cycled
        # through copies totalling > 768 MiB; prefill: tensor bound), timed like the headline and next to cuBLAS
        out["workloads"] = [measure_workload(torch, api, cmp_lib, name, device, peaks, warmup, steps)
                            for name in EXTRA_WORKLOADS if name != args.workload]
    if world == 1:
        os.sched_setaffinity(0, ALL_CPUS)  # the host GEMM uses every core again
        out["cpu_baseline"] = cpu_baseline(M, N, K, dist_name)
    if gather_ms is not None:
        out["allgather_c"] = {"ms": round(gather_ms, 4), "bytes_received_per_rank": int((M - rows) * N * 2),
                              "note": "NCCL all-gather of the row slabs into full C on every rank; outside the timed multiply"}
    print(json.dumps(out), flush=True)
    dist_teardown(world)


REF_ENABLED = ("wmmaPadding", "wmmaAsync", "wmmaAsyncPg2s", "wmmaAsyncPg2sPs2r", "wmmaAsyncStage2", "wmmaAsyncStage3",
               "mmaPermuted", "mmaAsync", "mmaAsyncPg2s", "mmaAsyncPg2sPs2r", "mmaAsyncStage2", "mmaAsyncStage3",
               "mmaAsyncStage4")
REF_NAIVE = ("mmaNaive", "wmmaNaive")


def run_reference(args):
    """The reference project's own kernels (unmodified sources, built for sm_100a) on the same workload.

    The reference has no CPU implementation of this path; its code IS the GPU kernels, so this arm
    times them: every kernel its driver enables (reference src/main.cu:106-123), best one reported.
    Only rank 0 works; the reference is single-GPU (its only device knob is -gpu_rank)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    from oracle import build as oracle_build

    M, N, K, dist_name, desc = WORKLOADS[args.workload]
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    base = {"impl": "reference", "metric": "HGEMM TFLOP/s vs cuBLAS and % FP16 TC peak", "unit": "TFLOP/s",
            "n_gpus": 1, "steps": steps, "warmup": warmup, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16 (FP16 accumulate, as the reference's kernels compute)",
            "data": f"synthetic: FP16 {dist_name} from seed {SEED}",
            "config": {"workload": f"{args.workload}: {desc}", "M": M, "N": N, "K": K}}
    if not oracle_build.REF_SO.exists() or not torch.cuda.is_available():
        # no build of the reference's kernels travelled here: time the CPU restatement instead
        cb = cpu_baseline(M, N, K, dist_name)
        base.update({"value": cb["value"], "ms_per_step": None, "cpu_baseline": cb, "gpu_launches": 0,
                     "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                     "note": "reference kernel library absent; value is the CPU port of the checker"})
        print(json.dumps(base), flush=True)
        return

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    bind_to_gpu_cpus(torch, 0)  # the same placement of the pinned host buffers as the other arm's
    lib = ctypes.CDLL(str(oracle_build.REF_SO))
    A, B = make_inputs(torch, M, N, K, dist_name, device, 0, M)
    C = torch.empty((M, N), dtype=torch.float16, device=device)
    names = REF_ENABLED if (M % 256 == 0 and N % 128 == 0 and K % 32 == 0 and K >= 128) else REF_NAIVE
    flops = 2.0 * M * N * K
    per_kernel = {}
    launches = 0
    for name in names:
        fn = getattr(lib, oracle_build.mangled(name))
        fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_size_t] * 3
        fn.restype = None
        a, b, c = A.data_ptr(), B.data_ptr(), C.data_ptr()
        ms = time_launches(torch, lambda: fn(a, b, c, M, N, K), warmup, steps)  # launches on the default stream
        launches += steps
        per_kernel[oracle_build.REF_KERNELS[name]] = round(flops / (ms * 1e-3) / 1e12, 2)
    best_name = max(per_kernel, key=per_kernel.get)
    best_fn = getattr(lib, oracle_build.mangled([n for n in names if oracle_build.REF_KERNELS[n] == best_name][0]))
    # end to end the way the reference's Matrix does it: blocking uploads, kernel, blocking download
    hA = torch.empty((M, K), dtype=torch.float16).pin_memory().copy_(A)
    hB = torch.empty((N, K), dtype=torch.float16).pin_memory().copy_(B)
    hC = torch.empty((M, N), dtype=torch.float16).pin_memory()
    e2e_steps = max(1, min(steps, 5))

    def e2e_once():
        A.copy_(hA)
        B.copy_(hB)
        best_fn(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K)
        hC.copy_(C)
        torch.cuda.synchronize()
    e2e_once()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_once()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    value = per_kernel[best_name]
    base.update({"value": value, "ms_per_step": round(flops / value / 1e9, 5), "best_kernel": best_name,
                 "kernels": per_kernel, "gpu_launches": launches,
                 "e2e": {"value": round(flops / e2e_s / 1e12, 2), "unit": "TFLOP/s",
                         "h2d_bytes_per_step": int((M * K + N * K) * 2), "d2h_bytes_per_step": int(M * N * 2)},
                 "note": "reference = its own CUDA kernels built unmodified for sm_100a (it has no CPU path); "
                         "cpu_baseline is the checker's host GEMM"})
    os.sched_setaffinity(0, ALL_CPUS)
    base["cpu_baseline"] = cpu_baseline(M, N, K, dist_name)
    print(json.dumps(base), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="square16384")
    ap.add_argument("--gather", action="store_true", help="with N > 1: also time the optional all-gather of C")
    ap.add_argument("--no-sweep", action="store_true", help="skip the extra square sizes measured after the timed region")
    ap.add_argument("--no-workloads", action="store_true", help="skip the other benchmark configurations measured after the timed region")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
