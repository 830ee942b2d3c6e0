"""Python-side mirror of the kernel entry points, for tests and the benchmark.

The reference registers one callable per kernel, all of the shape
``void name(half *A, half *B, half *C, size_t M, size_t N, size_t K)`` (reference
src/main.cu:11-33). The functions here keep that argument order and meaning for torch CUDA
tensors: ``A`` is ``[M, K]`` row-major, ``B`` is ``[N, K]`` row-major (the reference's
"col-major K x N", src/common/tester.h:117-119), ``C`` is ``[M, N]`` row-major; all float16
and contiguous. Everything runs on torch's current stream and returns without synchronising.
torch is used for device memory and streams only; the arithmetic is the native library's.
"""
from __future__ import annotations

import ctypes

from . import _native
from ._native import HgemmError, Plan, check

__all__ = [
    "b200Hgemm", "b200HgemmCta1", "b200HgemmCta2", "b200HgemmSplitK", "b200HgemmStreamK", "b200HgemmSimt",
    "hgemm_ex", "hgemm_host", "select_plan", "workspace_bytes", "last_device_error", "launch_count",
    "KERNEL_LOG_NAMES", "Plan", "HgemmError",
]

# log names, in the reference's style (no spaces: its plot tool splits lines on spaces,
# reference tools/performance/performance.py:57-62)
KERNEL_LOG_NAMES = {
    "b200Hgemm": "B200-Tcgen05-Auto",
    "b200HgemmCta1": "B200-Tcgen05-1Cta",
    "b200HgemmCta2": "B200-Tcgen05-2Cta",
    "b200HgemmSplitK": "B200-Tcgen05-SplitK",
    "b200HgemmStreamK": "B200-Tcgen05-StreamK",
    "b200HgemmSimt": "B200-Simt-Fp32Acc",
}


def _shape_of(A, B, C, c_dtypes=None):
    import torch

    for name, t in (("A", A), ("B", B), ("C", C)):
        ok_types = c_dtypes if (name == "C" and c_dtypes) else (torch.float16,)
        if not isinstance(t, torch.Tensor) or t.dtype not in ok_types or not t.is_cuda or not t.is_contiguous():
            raise TypeError(f"{name} must be a contiguous float16 CUDA tensor")
        if t.dim() != 2:
            raise ValueError(f"{name} must be 2-D")
    M, K = A.shape
    N, Kb = B.shape
    if Kb != K or tuple(C.shape) != (M, N):
        raise ValueError(f"shape mismatch: A {tuple(A.shape)}, B {tuple(B.shape)} (N x K), C {tuple(C.shape)}")
    if A.device != B.device or A.device != C.device:
        raise ValueError("A, B and C must live on one device")
    return int(M), int(N), int(K)


def _stream_of(t) -> int:
    import torch

    return int(torch.cuda.current_stream(t.device).cuda_stream)


def _call(symbol: str, A, B, C):
    import torch

    M, N, K = _shape_of(A, B, C)
    fn = getattr(_native.load(), symbol)
    with torch.cuda.device(A.device):
        check(fn(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, _stream_of(A)))
    return C


def b200Hgemm(A, B, C):
    """Auto-dispatching GEMM (C ABI ``b200_hgemm``)."""
    return _call("b200_hgemm", A, B, C)


def b200HgemmCta1(A, B, C):
    """Single-CTA tcgen05 tiles (C ABI ``b200_hgemm_cta1``)."""
    return _call("b200_hgemm_cta1", A, B, C)


def b200HgemmCta2(A, B, C):
    """CTA-pair tcgen05 tiles (C ABI ``b200_hgemm_cta2``)."""
    return _call("b200_hgemm_cta2", A, B, C)


def b200HgemmSplitK(A, B, C):
    """Fixed k-slices per tile with an FP32 workspace reduce (C ABI ``b200_hgemm_splitk``)."""
    return _call("b200_hgemm_splitk", A, B, C)


def b200HgemmStreamK(A, B, C):
    """Equal k-ranges over all SMs (C ABI ``b200_hgemm_streamk``)."""
    return _call("b200_hgemm_streamk", A, B, C)


def b200HgemmSimt(A, B, C):
    """CUDA-core kernel for any shape (C ABI ``b200_hgemm_simt``)."""
    return _call("b200_hgemm_simt", A, B, C)


def hgemm_ex(A, B, C, plan: Plan):
    """Run an explicit plan (C ABI ``b200_hgemm_ex``): ``plan.variant`` one of the ``_native.VARIANT_*``
    kernel families, ``plan.bn`` the tile width (or, for the large-tile and short-A kernels, the
    arrangement: see ``include/b200_hgemm.h``), ``plan.parts`` the number of k-ranges where k is cut."""
    import torch

    M, N, K = _shape_of(A, B, C)
    with torch.cuda.device(A.device):
        check(_native.load().b200_hgemm_ex(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, ctypes.byref(plan),
                                           _stream_of(A)))
    return C


def hgemm_fused(A, B, C, alpha: float = 1.0, beta: float = 0.0, bias=None, c_in=None, plan: Plan = None):
    """``C = alpha * A @ B.T + beta * c_in + bias`` in one kernel (C ABI ``b200_hgemm_fused``, or
    ``b200_hgemm_fused_ex`` when a ``plan`` is given). ``C`` may be float16, bfloat16 or float32; ``bias`` has one
    FP16 value per column of C; ``c_in`` is an ``[M, N]`` tensor of C's dtype (``C`` itself for an in-place update)."""
    import torch

    c_types = {torch.float16: _native.C_F16, torch.bfloat16: _native.C_BF16, torch.float32: _native.C_F32}
    if not isinstance(C, torch.Tensor) or C.dtype not in c_types or not C.is_cuda or not C.is_contiguous() or C.dim() != 2:
        raise TypeError("C must be a contiguous 2-D float16, bfloat16 or float32 CUDA tensor")
    M, N, K = _shape_of(A, B, C, c_dtypes=tuple(c_types))
    if bias is not None and (bias.dtype != torch.float16 or bias.numel() != N or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous float16 tensor with one value per column of C")
    if c_in is not None and (c_in.dtype != C.dtype or tuple(c_in.shape) != (M, N) or not c_in.is_contiguous()):
        raise ValueError("c_in must be a contiguous [M, N] tensor of C's dtype")
    epi = _native.Epilogue(alpha, beta, bias.data_ptr() if bias is not None else None,
                           c_in.data_ptr() if c_in is not None else None, c_types[C.dtype])
    lib = _native.load()
    with torch.cuda.device(A.device):
        if plan is None:
            check(lib.b200_hgemm_fused(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, ctypes.byref(epi), _stream_of(A)))
        else:
            check(lib.b200_hgemm_fused_ex(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, ctypes.byref(epi),
                                          ctypes.byref(plan), _stream_of(A)))
    return C


def hgemm_bkn(A, B_kn, C):
    """``C = A @ B_kn`` with ``B_kn`` stored ``[K, N]`` row-major (C ABI ``b200_hgemm_bkn``): no transpose is made."""
    import torch

    for name, t in (("A", A), ("B_kn", B_kn), ("C", C)):
        if not isinstance(t, torch.Tensor) or t.dtype != torch.float16 or not t.is_cuda or not t.is_contiguous() or t.dim() != 2:
            raise TypeError(f"{name} must be a contiguous 2-D float16 CUDA tensor")
    M, K = A.shape
    Kb, N = B_kn.shape
    if Kb != K or tuple(C.shape) != (M, N):
        raise ValueError("shape mismatch")
    with torch.cuda.device(A.device):
        check(_native.load().b200_hgemm_bkn(A.data_ptr(), B_kn.data_ptr(), C.data_ptr(), int(M), int(N), int(K), _stream_of(A)))
    return C


def hgemm_batched(A, B, C):
    """``C[i] = A[i] @ B[i].T`` for stacks ``A [batch, M, K]``, ``B [batch, N, K]`` (or one ``[N, K]`` matrix for all),
    ``C [batch, M, N]`` (C ABI ``b200_hgemm_batched``). The innermost two dimensions must be contiguous; the
    stack dimension may have any stride that is a multiple of 8 elements."""
    import torch

    for name, t in (("A", A), ("B", B), ("C", C)):
        if not isinstance(t, torch.Tensor) or t.dtype != torch.float16 or not t.is_cuda:
            raise TypeError(f"{name} must be a float16 CUDA tensor")
    if A.dim() != 3 or C.dim() != 3 or B.dim() not in (2, 3):
        raise ValueError("A and C must be [batch, rows, cols]; B [batch, N, K] or [N, K]")
    batch, M, K = A.shape
    N = B.shape[-2]
    if B.shape[-1] != K or tuple(C.shape) != (batch, M, N) or (B.dim() == 3 and B.shape[0] != batch):
        raise ValueError("shape mismatch")
    for name, t in (("A", A), ("B", B), ("C", C)):
        if t.stride(-1) != 1 or t.stride(-2) != t.shape[-1]:
            raise ValueError(f"the matrices of {name} must be contiguous")
    stride_b = B.stride(0) if B.dim() == 3 else 0
    with torch.cuda.device(A.device):
        check(_native.load().b200_hgemm_batched(A.data_ptr(), B.data_ptr(), C.data_ptr(), int(M), int(N), int(K), int(batch),
                                                int(A.stride(0)), int(stride_b), int(C.stride(0)), _stream_of(A)))
    return C


def hgemm_host(A_host, B_host, C_host):
    """HOST tensors in, HOST tensor out (C ABI ``b200_hgemm_host``): uploads, multiplies, downloads, synchronises."""
    import torch

    for name, t in (("A", A_host), ("B", B_host), ("C", C_host)):
        if not isinstance(t, torch.Tensor) or t.dtype != torch.float16 or t.is_cuda or not t.is_contiguous():
            raise TypeError(f"{name} must be a contiguous float16 CPU tensor")
    M, K = A_host.shape
    N, Kb = B_host.shape
    if Kb != K or tuple(C_host.shape) != (M, N):
        raise ValueError("shape mismatch")
    check(_native.load().b200_hgemm_host(A_host.data_ptr(), B_host.data_ptr(), C_host.data_ptr(), int(M), int(N), int(K)))
    return C_host


def hgemm_host_a(A_host, B_dev, C_host, upload_after=None, gemm_after=None):
    """HOST ``A`` in, HOST ``C`` out, ``B`` already on the GPU (C ABI ``b200_hgemm_host_a``); the current stream's
    work on ``B_dev`` must be complete (this call synchronises that stream first). With ``upload_after`` /
    ``gemm_after`` (``torch.cuda.Event`` objects already recorded; C ABI ``b200_hgemm_host_a_after``) nothing is
    synchronised up front: A's uploads start behind the first event and the multiplies behind the second."""
    import torch

    for name, t in (("A", A_host), ("C", C_host)):
        if not isinstance(t, torch.Tensor) or t.dtype != torch.float16 or t.is_cuda or not t.is_contiguous():
            raise TypeError(f"{name} must be a contiguous float16 CPU tensor")
    if not B_dev.is_cuda or B_dev.dtype != torch.float16 or not B_dev.is_contiguous():
        raise TypeError("B must be a contiguous float16 CUDA tensor")
    M, K = A_host.shape
    N, Kb = B_dev.shape
    if Kb != K or tuple(C_host.shape) != (M, N):
        raise ValueError("shape mismatch")
    with torch.cuda.device(B_dev.device):
        if upload_after is None and gemm_after is None:
            torch.cuda.current_stream().synchronize()
            check(_native.load().b200_hgemm_host_a(A_host.data_ptr(), B_dev.data_ptr(), C_host.data_ptr(), int(M), int(N), int(K)))
        else:
            check(_native.load().b200_hgemm_host_a_after(
                A_host.data_ptr(), B_dev.data_ptr(), C_host.data_ptr(), int(M), int(N), int(K),
                upload_after.cuda_event if upload_after is not None else None,
                gemm_after.cuda_event if gemm_after is not None else None))
    return C_host


def select_plan(M: int, N: int, K: int) -> Plan:
    """The plan ``b200Hgemm`` would run for this shape on the current device (C ABI ``b200_hgemm_select``)."""
    plan = Plan()
    check(_native.load().b200_hgemm_select(M, N, K, ctypes.byref(plan)))
    return plan


def select_plan_untuned(M: int, N: int, K: int) -> Plan:
    """The plan the dispatch rules give, ignoring the table of tuned plans."""
    plan = Plan()
    check(_native.load().b200_hgemm_select_untuned(M, N, K, ctypes.byref(plan)))
    return plan


def load_plan_table(path) -> int:
    """Replace the table of tuned plans with the file at ``path`` (``None``: no table); returns the entry count."""
    n = _native.load().b200_hgemm_load_plan_table(None if path is None else str(path).encode())
    if n < 0:
        check(n)
    return n


def workspace_bytes(M: int, N: int, K: int, plan: Plan) -> int:
    return int(_native.load().b200_hgemm_workspace_bytes(M, N, K, ctypes.byref(plan)))


def last_device_error() -> int:
    return int(_native.load().b200_hgemm_last_device_error())


def enable_multicast(on: bool = True) -> bool:
    """Switch the single-GPU kernels with multicast operand loads on or off (C ABI
    ``b200_hgemm_enable_multicast``). Returns whether they are on afterwards: never in a process that is
    one rank of several or that holds a multi-device handle, and never without the companion library."""
    lib = _native.load()
    lib.b200_hgemm_enable_multicast(1 if on else 0)
    return lib.b200_hgemm_multicast_state() == _native.MULTICAST_ON


def synchronize(device=None) -> None:
    """Wait for torch's current stream and raise if a kernel on it gave up on a bounded wait
    (C ABI ``b200_hgemm_synchronize``)."""
    import torch

    with torch.cuda.device(device):
        check(_native.load().b200_hgemm_synchronize(int(torch.cuda.current_stream().cuda_stream)))


def launch_count() -> int:
    return int(_native.load().b200_hgemm_launch_count())
