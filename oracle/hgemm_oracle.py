"""TEST INFRASTRUCTURE -- not part of the product. Only ``tests/``, the smoke check and the
benchmark's CPU-baseline / reference legs may import this module; the GEMM library never does.

Python face of the CPU checker: a ctypes binding of ``hgemm_oracle.c`` plus a pure-numpy
restatement used to cross-check the C code. Both compute

    C[row, col] = sum_k A[row, k] * B[col, k]

with A ``[M, K]``, B ``[N, K]`` (the reference's layouts, reference src/simt_naive.cu:18-24,
src/common/tester.h:117-119), accumulating in FP32 or FP64 and rounding to FP16 once.

PARITY UNPINNED by the reference: it ships no golden vectors or known-answer tests for this
path and has no CPU implementation; see the header of ``hgemm_oracle.c``.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_double, c_float, c_int, c_size_t, c_uint16
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libhgemm_oracle.so"

#: the tolerance the GEMM is held to: max-norm relative error of the FP16 output against the
#: FP32-accumulate product of the same inputs
RTOL = 1e-2

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            from . import build as _build

            _build.build_oracle()
        lib = ctypes.CDLL(str(LIB_PATH))
        u16p, f32p, f64p = POINTER(c_uint16), POINTER(c_float), POINTER(c_double)
        lib.hgemm_oracle_max_threads.restype = c_int
        lib.hgemm_oracle_f32.argtypes = [u16p, u16p, f32p, c_size_t, c_size_t, c_size_t, c_int]
        lib.hgemm_oracle_f32.restype = c_int
        lib.hgemm_oracle_f32_rows.argtypes = [u16p, u16p, f32p, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t, c_int]
        lib.hgemm_oracle_f32_rows.restype = c_int
        lib.hgemm_oracle_f64.argtypes = [u16p, u16p, f64p, c_size_t, c_size_t, c_size_t, c_int]
        lib.hgemm_oracle_f64.restype = c_int
        lib.hgemm_oracle_f16.argtypes = [u16p, u16p, u16p, c_size_t, c_size_t, c_size_t, c_int]
        lib.hgemm_oracle_f16.restype = c_int
        lib.hgemm_oracle_f16_accumulate.argtypes = [u16p, u16p, u16p, c_size_t, c_size_t, c_size_t]
        lib.hgemm_oracle_f16_accumulate.restype = None
        lib.hgemm_oracle_compare.argtypes = [u16p, f32p, c_size_t, c_double, f64p, c_int]
        lib.hgemm_oracle_compare.restype = None
        lib.hgemm_oracle_time_rows.argtypes = [u16p, u16p, f32p, c_size_t, c_size_t, c_size_t, c_size_t, c_int]
        lib.hgemm_oracle_time_rows.restype = c_double
        _lib = lib
    return _lib


def max_threads() -> int:
    return int(load().hgemm_oracle_max_threads())


def _bits(x: np.ndarray) -> np.ndarray:
    """float16 array -> contiguous uint16 view."""
    x = np.ascontiguousarray(x)
    if x.dtype != np.float16:
        raise TypeError("expected float16")
    return x.view(np.uint16)


def _p(a: np.ndarray, ctype):
    return a.ctypes.data_as(POINTER(ctype))


def _dims(A, B):
    M, K = A.shape
    N, Kb = B.shape
    if K != Kb:
        raise ValueError("A is [M, K], B is [N, K]")
    return M, N, K


def gemm_f32(A: np.ndarray, B: np.ndarray, threads: int | None = None) -> np.ndarray:
    """FP32-accumulate product of float16 A [M,K] and B [N,K] -> float32 [M,N]."""
    M, N, K = _dims(A, B)
    out = np.empty((M, N), dtype=np.float32)
    rc = load().hgemm_oracle_f32(_p(_bits(A), c_uint16), _p(_bits(B), c_uint16), _p(out, c_float), M, N, K,
                                 threads or max_threads())
    if rc != 0:
        raise MemoryError(f"hgemm_oracle_f32 failed ({rc})")
    return out


def gemm_f32_rows(A: np.ndarray, B: np.ndarray, row0: int, rows: int, threads: int | None = None) -> np.ndarray:
    """Rows [row0, row0+rows) of the FP32-accumulate product."""
    M, N, K = _dims(A, B)
    out = np.empty((rows, N), dtype=np.float32)
    rc = load().hgemm_oracle_f32_rows(_p(_bits(A), c_uint16), _p(_bits(B), c_uint16), _p(out, c_float), M, N, K,
                                      row0, rows, threads or max_threads())
    if rc != 0:
        raise RuntimeError(f"hgemm_oracle_f32_rows failed ({rc})")
    return out


def gemm_f64(A: np.ndarray, B: np.ndarray, threads: int | None = None) -> np.ndarray:
    M, N, K = _dims(A, B)
    out = np.empty((M, N), dtype=np.float64)
    rc = load().hgemm_oracle_f64(_p(_bits(A), c_uint16), _p(_bits(B), c_uint16), _p(out, c_double), M, N, K,
                                 threads or max_threads())
    if rc != 0:
        raise MemoryError(f"hgemm_oracle_f64 failed ({rc})")
    return out


def gemm_f16(A: np.ndarray, B: np.ndarray, threads: int | None = None) -> np.ndarray:
    M, N, K = _dims(A, B)
    out = np.empty((M, N), dtype=np.uint16)
    rc = load().hgemm_oracle_f16(_p(_bits(A), c_uint16), _p(_bits(B), c_uint16), _p(out, c_uint16), M, N, K,
                                 threads or max_threads())
    if rc != 0:
        raise MemoryError(f"hgemm_oracle_f16 failed ({rc})")
    return out.view(np.float16)


def gemm_f16_accumulate(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """The reference's FP16-accumulate arithmetic (scalar; small shapes only)."""
    M, N, K = _dims(A, B)
    out = np.empty((M, N), dtype=np.uint16)
    load().hgemm_oracle_f16_accumulate(_p(_bits(A), c_uint16), _p(_bits(B), c_uint16), _p(out, c_uint16), M, N, K)
    return out.view(np.float16)


def compare(C: np.ndarray, ref: np.ndarray, rtol: float = RTOL, threads: int | None = None) -> dict:
    """Difference report of float16 ``C`` against float32 ``ref`` (same shape)."""
    if C.shape != ref.shape:
        raise ValueError("shape mismatch")
    ref = np.ascontiguousarray(ref, dtype=np.float32)
    out = np.zeros(7, dtype=np.float64)
    load().hgemm_oracle_compare(_p(_bits(C), c_uint16), _p(ref, c_float), C.size, rtol, _p(out, c_double),
                                threads or max_threads())
    return {
        "max_abs_diff": float(out[0]), "avg_abs_diff": float(out[1]), "max_ref": float(out[2]),
        "rms_ref": float(out[3]), "max_rel_err": float(out[4]), "violations": int(out[5]),
        "non_finite": int(out[6]),
    }


def passes(report: dict, rtol: float = RTOL) -> bool:
    return report["non_finite"] == 0 and report["max_rel_err"] <= rtol and report["violations"] == 0


def time_rows(A: np.ndarray, B: np.ndarray, rows: int, threads: int | None = None) -> float:
    """Seconds the CPU needs for the first ``rows`` rows of the product (FP32 accumulate)."""
    M, N, K = _dims(A, B)
    rows = min(rows, M)
    out = np.empty((rows, N), dtype=np.float32)
    t = load().hgemm_oracle_time_rows(_p(_bits(A), c_uint16), _p(_bits(B), c_uint16), _p(out, c_float), M, N, K, rows,
                                      threads or max_threads())
    if t < 0:
        raise MemoryError("hgemm_oracle_time_rows failed")
    return float(t)


# ---- pure-numpy restatement (cross-check of the C code; small shapes) -------------------------

def gemm_numpy_f64(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """float64 product through numpy: an implementation independent of hgemm_oracle.c."""
    return A.astype(np.float64) @ B.astype(np.float64).T


def gemm_loops(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """Triple loop over the reference's index arithmetic (reference src/simt_naive.cu:18-24), FP64."""
    M, N, K = _dims(A, B)
    a = A.reshape(-1).astype(np.float64)
    b = B.reshape(-1).astype(np.float64)
    out = np.zeros(M * N, dtype=np.float64)
    for row in range(M):
        for col in range(N):
            tmp = 0.0
            for i in range(K):
                tmp += a[row * K + i] * b[i + col * K]
            out[row * N + col] = tmp
    return out.reshape(M, N)
