"""Pins the CPU oracle: against the committed golden fixtures (numpy float64 products), against
a triple loop over the reference's index arithmetic, and on hand-computed cases. CPU only."""
from pathlib import Path

import numpy as np
import pytest

from oracle import hgemm_oracle as oracle
from tests.helpers import make_inputs

GOLDEN = sorted((Path(__file__).parent / "golden").glob("*.npz"))


def test_golden_fixtures_exist():
    assert len(GOLDEN) >= 5


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_oracle_matches_golden(path):
    g = np.load(path)
    A, B = g["A"], g["B"]
    ref32 = oracle.gemm_f32(A, B)
    ref64 = oracle.gemm_f64(A, B)
    K = A.shape[1]
    scale = np.abs(g["ref_f32"]).max()
    # FP64 accumulation reproduces numpy's float64 product to rounding of the FP32 fixture
    assert np.abs(ref64 - g["ref_f32"].astype(np.float64)).max() <= 1e-6 * scale
    # FP32 accumulation: error bounded by K * eps * sum|a||b| -- far inside 1e-4 of the scale here
    assert np.abs(ref32 - g["ref_f32"]).max() <= 1e-4 * scale * max(1.0, K / 1024)
    # rounded output: equal to the float64 product's rounding except where FP32 accumulation
    # error moves a value across an FP16 rounding boundary (one FP16 step of that value)
    c16 = oracle.gemm_f16(A, B).astype(np.float64)
    g16 = g["ref_f16"].astype(np.float64)
    step = 2.0 ** -10 * np.abs(g16) + 1e-5 * scale
    assert (np.abs(c16 - g16) <= step).all()
    assert (c16 != g16).mean() < 0.01


def test_oracle_matches_reference_index_arithmetic():
    A, B = make_inputs(5, 7, 24, seed=1)
    loops = oracle.gemm_loops(A, B)
    assert np.abs(oracle.gemm_f64(A, B) - loops).max() < 1e-12
    assert np.abs(oracle.gemm_numpy_f64(A, B) - loops).max() < 1e-12


def test_hand_computed_cases():
    # identity: B = I (as N x K) gives C = A
    A = (np.arange(16 * 8).reshape(16, 8) % 13 - 6).astype(np.float16)
    I = np.eye(8, dtype=np.float16)
    assert np.array_equal(oracle.gemm_f16(A, I), A)
    # B is N x K: row j of B is column j of the mathematical K x N matrix
    A = np.array([[1, 2, 3]], dtype=np.float16)
    B = np.array([[1, 0, 0], [0, 1, 0], [1, 1, 1], [2, 2, 2]], dtype=np.float16)
    assert np.array_equal(oracle.gemm_f32(A, B), np.array([[1, 2, 6, 12]], dtype=np.float32))
    # FP32 accumulation keeps what FP16 accumulation loses: 2048 + 1 + 1 ...
    A = np.array([[2048] + [1] * 16], dtype=np.float16)
    B = np.ones((1, 17), dtype=np.float16)
    assert oracle.gemm_f32(A, B)[0, 0] == 2064.0
    assert float(oracle.gemm_f16_accumulate(A, B)[0, 0]) == 2048.0  # the reference's arithmetic stalls


def test_rows_subset_equals_full():
    A, B = make_inputs(96, 72, 160, seed=4)
    full = oracle.gemm_f32(A, B)
    part = oracle.gemm_f32_rows(A, B, 32, 40)
    assert np.array_equal(part, full[32:72])


def test_empty_and_ragged_inputs():
    A = np.zeros((0, 8), dtype=np.float16)
    B = np.ones((3, 8), dtype=np.float16)
    assert oracle.gemm_f32(A, B).shape == (0, 3)
    A, B = make_inputs(1, 1, 1, seed=9)
    assert oracle.gemm_f32(A, B)[0, 0] == np.float32(A[0, 0]) * np.float32(B[0, 0])
    with pytest.raises(ValueError):
        oracle.gemm_f32(np.zeros((2, 3), np.float16), np.zeros((2, 4), np.float16))


def test_compare_report():
    A, B = make_inputs(64, 64, 256, seed=2)
    ref = oracle.gemm_f32(A, B)
    good = ref.astype(np.float16)
    rep = oracle.compare(good, ref)
    assert oracle.passes(rep) and rep["max_rel_err"] < 1e-3
    # the reference-style numbers agree with a direct numpy evaluation
    d = np.abs(good.astype(np.float64) - ref.astype(np.float64))
    assert abs(rep["max_abs_diff"] - d.max()) < 1e-12 and abs(rep["avg_abs_diff"] - d.mean()) < 1e-9
    bad = good.copy()
    bad[3, 5] = np.float16(float(bad[3, 5]) + 2.0)
    rep = oracle.compare(bad, ref)
    assert rep["violations"] >= 1 and not oracle.passes(rep)
    nan = good.copy()
    nan[0, 0] = np.float16(np.nan)
    rep = oracle.compare(nan, ref)
    assert rep["non_finite"] == 1 and not oracle.passes(rep)


def test_fp16_accumulation_drift_is_reported_not_hidden():
    # the reference's kernels accumulate in FP16: their error against the FP32 oracle is visibly larger
    A, B = make_inputs(8, 8, 2048, seed=6)
    ref = oracle.gemm_f32(A, B)
    e16 = oracle.compare(oracle.gemm_f16_accumulate(A, B), ref)["max_rel_err"]
    e32 = oracle.compare(oracle.gemm_f16(A, B), ref)["max_rel_err"]
    assert e32 < 1e-3 < e16
