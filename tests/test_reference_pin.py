"""Pins the CPU oracle to the reference project's own arithmetic.

The reference ships no golden vectors and no CPU implementation; what it does ship is its CUDA kernels,
and ``oracle/build.py`` compiles those, unmodified, into ``oracle/_ref/libcuda_hgemm_ref.so``. They
accumulate in FP16 (reference src/simt_naive.cu:18-24, src/common/ptx.h:20-23 as used by
src/mma/mma_async_stage4.cu:637-644), the oracle in FP32 -- so on inputs whose every partial sum is
exactly representable in FP16 both must produce the same bits, whatever the order of summation. On
ordinary inputs the reference's kernels may only differ from the oracle by what FP16 accumulation costs.
A disagreement about operand layout, transposition or indexing between the oracle and the reference's
real kernels fails the first test at once.

Shapes are multiples of the kernels' tiles: the reference's kernels have no edge handling (its naive
kernels' bounds guards only hold for exact multiples, reference src/simt_naive.cu:14).
"""
import ctypes
from pathlib import Path

import numpy as np
import pytest

from oracle import build as oracle_build
from oracle import hgemm_oracle as oracle

pytestmark = pytest.mark.gpu

REF_SO = Path(oracle_build.REF_SO)

# entry point -> (M % , N % , K % , K >=) the kernel needs (it does not check)
NAIVE = {"simtNaive": (16, 16, 1, 1), "wmmaNaive": (16, 16, 16, 16), "mmaNaive": (16, 8, 16, 16)}
TILED = ("wmmaPadding", "wmmaAsync", "wmmaAsyncPg2s", "wmmaAsyncPg2sPs2r", "wmmaAsyncStage2", "wmmaAsyncStage3",
         "mmaPermuted", "mmaAsync", "mmaAsyncPg2s", "mmaAsyncPg2sPs2r", "mmaAsyncStage2", "mmaAsyncStage3",
         "mmaAsyncStage4")


@pytest.fixture(scope="module")
def ref_lib():
    if not REF_SO.exists():
        pytest.skip("the reference's kernels were not built (no reference checkout at build time)")
    return ctypes.CDLL(str(REF_SO))


def call_reference(lib, name, A, B, device):
    """Runs one of the reference's entry points (``void name(half*, half*, half*, size_t, size_t, size_t)``,
    reference src/main.cu:11) on the default stream, as its own driver does; returns C as numpy."""
    import torch

    M, K = A.shape
    N = B.shape[0]
    fn = getattr(lib, oracle_build.mangled(name))
    fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_size_t] * 3
    fn.restype = None
    dA, dB = torch.from_numpy(A).to(device), torch.from_numpy(B).to(device)
    dC = torch.full((M, N), float("nan"), dtype=torch.float16, device=device)
    torch.cuda.synchronize(device)
    fn(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M, N, K)
    torch.cuda.synchronize(device)
    return dC.cpu().numpy()


def exact_inputs(M, N, K, seed):
    """A in {-2..2}, B in {-2..2}/64: every product is a multiple of 1/64 of magnitude <= 1/16 and, for
    K <= 512, every partial sum a multiple of 1/64 of magnitude <= 32 -- all exact in FP16 (and FP32)."""
    assert K <= 512
    rng = np.random.default_rng(seed)
    A = rng.integers(-2, 3, size=(M, K)).astype(np.float16)
    B = (rng.integers(-2, 3, size=(N, K)) / 64.0).astype(np.float16)
    return A, B


@pytest.mark.parametrize("name", sorted(NAIVE))
@pytest.mark.parametrize("shape", [(48, 32, 96), (256, 256, 512)], ids=lambda s: "x".join(map(str, s)))
def test_reference_naive_kernels_equal_the_oracle_bit_for_bit(cuda_device, ref_lib, name, shape):
    M, N, K = shape
    A, B = exact_inputs(M, N, K, seed=101)
    got = call_reference(ref_lib, name, A, B, cuda_device)
    assert np.array_equal(got.view(np.uint16), oracle.gemm_f16(A, B).view(np.uint16)), name
    # and the oracle's own FP16-accumulate restatement agrees with both
    if M * N * K <= 48 * 32 * 96:
        assert np.array_equal(oracle.gemm_f16_accumulate(A, B).view(np.uint16), got.view(np.uint16))


@pytest.mark.parametrize("name", TILED)
def test_reference_tiled_kernels_equal_the_oracle_bit_for_bit(cuda_device, ref_lib, name):
    M, N, K = 256, 256, 512  # one 256-row block, two 128-column blocks, sixteen 32-wide k-chunks
    A, B = exact_inputs(M, N, K, seed=102)
    got = call_reference(ref_lib, name, A, B, cuda_device)
    assert np.array_equal(got.view(np.uint16), oracle.gemm_f16(A, B).view(np.uint16)), name


def test_this_library_equals_the_reference_on_exact_inputs(cuda_device, ref_lib):
    """The product under test, the reference's best kernel and the oracle: three implementations, one answer."""
    import torch

    from cuda_hgemm_b200 import api

    M, N, K = 512, 384, 512
    A, B = exact_inputs(M, N, K, seed=103)
    ref_bits = call_reference(ref_lib, "mmaAsyncStage4", A, B, cuda_device).view(np.uint16)
    dA, dB = torch.from_numpy(A).to(cuda_device), torch.from_numpy(B).to(cuda_device)
    for fn in (api.b200Hgemm, api.b200HgemmCta1, api.b200HgemmCta2, api.b200HgemmStreamK):
        C = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda_device)
        fn(dA, dB, C)
        torch.cuda.synchronize()
        assert np.array_equal(C.cpu().numpy().view(np.uint16), ref_bits), fn.__name__
    assert np.array_equal(oracle.gemm_f16(A, B).view(np.uint16), ref_bits)


@pytest.mark.parametrize("name", ["simtNaive", "mmaNaive", "wmmaAsyncStage3", "mmaAsyncStage4"])
def test_reference_kernels_stay_within_fp16_accumulation_of_the_oracle(cuda_device, ref_lib, name):
    """Uniform [-1, 1) inputs at the reference driver's default shape (reference src/main.cu:35-37): the
    reference's kernels differ from the FP32 oracle by FP16 accumulation only. A wrong oracle (or a wrong
    layout) would put the difference at the size of the outputs themselves, a hundred times the bound."""
    from tests.helpers import make_inputs

    M, N, K = 512, 2048, 1024
    A, B = make_inputs(M, N, K, seed=104)
    ref = oracle.gemm_f32(A, B)
    got = call_reference(ref_lib, name, A, B, cuda_device).astype(np.float32)
    assert np.isfinite(got).all()
    scale = float(np.abs(ref).max())
    max_rel = float(np.abs(got - ref).max()) / scale
    # every rounding of a running sum of magnitude <= scale costs at most 2^-11 * scale; the errors of the
    # K / 16 (tensor core) or K (scalar loop) roundings add up like a random walk: a few 1e-3 of the largest
    # output for the former, about 1e-2 for the latter
    assert 0.0 < max_rel < (5e-2 if name == "simtNaive" else 2e-2), (name, max_rel)
    # and it is an accumulation error, not a structural one: correlation with the oracle is essentially one
    corr = float(np.corrcoef(got.ravel(), ref.ravel())[0, 1])
    assert corr > 0.9999, (name, corr)
