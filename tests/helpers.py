"""Shared input generation and checking for the tests (seeded numpy inputs)."""
from __future__ import annotations

import numpy as np

from oracle import hgemm_oracle as oracle


def make_inputs(M, N, K, seed=2023, dist="uniform"):
    """float16 A [M,K] and B [N,K]. 'uniform': U[-1,1) like the reference's Matrix fill
    (reference src/common/matrix.h:28-33); 'normal': A ~ N(0,1), B ~ N(0, 1/K)."""
    rng = np.random.default_rng(seed)
    if dist == "uniform":
        A = rng.uniform(-1.0, 1.0, size=(M, K)).astype(np.float32)
        B = rng.uniform(-1.0, 1.0, size=(N, K)).astype(np.float32)
    elif dist == "normal":
        A = rng.standard_normal(size=(M, K), dtype=np.float32)
        B = rng.standard_normal(size=(N, K), dtype=np.float32) / np.float32(np.sqrt(K))
    else:
        raise ValueError(dist)
    return A.astype(np.float16), B.astype(np.float16)


def assert_close_to_oracle(C: np.ndarray, ref: np.ndarray, what: str = ""):
    """The stated bar: max-norm relative error <= 1e-2 on the FP16 output (no NaN/Inf, and no
    element off by more than 1e-2*|ref| + 1e-2*rms(ref)). A kernel with FP32 accumulation and
    one rounding lands near 2^-11 relative, so a much tighter sanity bound is asserted too."""
    rep = oracle.compare(C, ref, rtol=oracle.RTOL)
    assert rep["non_finite"] == 0, f"{what}: {rep['non_finite']} non-finite outputs ({rep})"
    assert rep["max_rel_err"] <= oracle.RTOL, f"{what}: max-norm relative error {rep['max_rel_err']:.3e} > 1e-2 ({rep})"
    assert rep["violations"] == 0, f"{what}: {rep['violations']} elements outside tolerance ({rep})"
    # expected accuracy of FP32 accumulation + one FP16 rounding
    assert rep["max_rel_err"] <= 2e-3, f"{what}: unexpectedly inaccurate for FP32 accumulation ({rep})"
    return rep
