"""Timing helpers shared by the benchmark and the A/B tool.

Every measurement follows a pre-heat: a dense GEMM on a 1 kW part settles under its power cap
within tens of milliseconds, and a short timed region that starts cold measures that transient
rather than the kernel (results swing by +-15 % with the order of measurement otherwise).
``torch`` is passed in by the caller; it is used for events, streams and graphs only.
"""
from __future__ import annotations

import ctypes

PREHEAT_S = 0.3


def preheat(torch, fn, seconds=PREHEAT_S):
    """Untimed calls for about `seconds` of GPU time: clocks ramp up from idle and then settle under
    the power cap within the first tens of milliseconds of a dense GEMM, so a short timed region that
    starts cold measures that transient, not the kernel. Applied to every library measured, alike."""
    fn()  # first call pays one-time set-up (module load, attributes, tensor maps): not representative
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    one = max(e0.elapsed_time(e1) * 1e-3, 1e-6)
    for _ in range(min(20000, int(seconds / one))):
        fn()
    torch.cuda.synchronize()


def time_launches(torch, fn, warmup, steps):
    """Mean milliseconds of `steps` back-to-back calls after `warmup` calls (events on the current stream)."""
    preheat(torch, fn)
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def time_burst(torch, fn, warmup=3, steps=10, idle_s=0.25):
    """Mean milliseconds of `steps` back-to-back calls issued after an idle pause and `warmup` calls:
    the reference driver's protocol (a short run on a GPU that is not yet under its power cap)."""
    import time

    torch.cuda.synchronize()
    time.sleep(idle_s)
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def time_graph(torch, fn, launches=20, replays=5):
    """Mean milliseconds per call when `launches` calls are captured into one CUDA graph: removes the
    interpreter's per-call cost, which dominates kernels of a few microseconds."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            for _ in range(launches):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
    torch.cuda.current_stream().wait_stream(s)
    return e0.elapsed_time(e1) / (launches * replays)


def load_compare():
    from . import build as pkg_build

    if not pkg_build.COMPARE_SO.exists():
        return None
    lib = ctypes.CDLL(str(pkg_build.COMPARE_SO))
    for name in ("hgemm_compare_cublas_fp16", "hgemm_compare_cublas_fp32"):
        fn = getattr(lib, name)
        fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_size_t] * 3 + [ctypes.c_void_p]
        fn.restype = ctypes.c_int
    lib.hgemm_compare_time_loop.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_size_t] * 3 + [ctypes.c_int] * 2 + [ctypes.c_void_p]
    lib.hgemm_compare_time_loop.restype = ctypes.c_double
    lib.hgemm_compare_time_loop_rotate.argtypes = ([ctypes.c_void_p] * 2 + [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                                   ctypes.c_void_p] + [ctypes.c_size_t] * 3 + [ctypes.c_int] * 2 + [ctypes.c_void_p])
    lib.hgemm_compare_time_loop_rotate.restype = ctypes.c_double
    return lib


def time_native_loop(torch, cmp_lib, entry, A, B, C, warmup=3, iters=10):
    """Mean ms per call of a C-ABI GEMM entry point, launched back to back from native code
    (the reference driver's protocol: no graph, no interpreter between launches)."""
    M, K = A.shape
    N = B.shape[0]
    fn_ptr = ctypes.cast(entry, ctypes.c_void_p)
    ms = cmp_lib.hgemm_compare_time_loop(fn_ptr, A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, warmup, iters,
                                         torch.cuda.current_stream().cuda_stream)
    if ms <= 0:
        raise RuntimeError("native timing loop failed")
    return ms


def cublas_callable(torch, lib, which, A, B, C):
    M, K = A.shape
    N = B.shape[0]
    fn = getattr(lib, which)
    a, b, c = A.data_ptr(), B.data_ptr(), C.data_ptr()

    def call():
        rc = fn(a, b, c, M, N, K, torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError(f"{which} failed with cuBLAS status {rc}")
    return call




def time_native_rotate(torch, cmp_lib, entry, A, Bs, C, warmup=50, iters=200):
    """Mean ms per call of a C-ABI GEMM entry point launched back to back from native code, B taken in turn
    from the list ``Bs`` (copies of one matrix, together several times the L2) so that no call finds B cached.
    ``warmup`` untimed calls come first: enough of them to settle the clocks of a kernel of tens of microseconds."""
    M, K = A.shape
    N = Bs[0].shape[0]
    fn_ptr = ctypes.cast(entry, ctypes.c_void_p)
    ptrs = (ctypes.c_void_p * len(Bs))(*[b.data_ptr() for b in Bs])
    ms = cmp_lib.hgemm_compare_time_loop_rotate(fn_ptr, A.data_ptr(), ptrs, len(Bs), C.data_ptr(), M, N, K, warmup, iters,
                                                torch.cuda.current_stream().cuda_stream)
    if ms <= 0:
        raise RuntimeError("native timing loop failed")
    return ms
