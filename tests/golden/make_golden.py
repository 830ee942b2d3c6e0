"""Generates the golden fixtures in this directory.

The reference project ships no golden vectors for its GEMM path, so these are produced from an
implementation independent of the C oracle: numpy float64 products of seeded float16 inputs,
stored together with the inputs' seeds and the product rounded to float16. Run from the
repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from tests.helpers import make_inputs  # noqa: E402

# (name, M, N, K, seed, dist): small enough to commit, covering one tile, tails in every
# dimension, the 256^3 configuration and a skinny decode-like shape
CASES = [
    ("tile_128x256x64", 128, 256, 64, 11, "uniform"),
    ("square_256", 256, 256, 256, 2023, "uniform"),
    ("tails_200x264x136", 200, 264, 136, 7, "uniform"),
    ("skinny_16x256x512", 16, 256, 512, 5, "normal"),
    ("odd_k_48x40x100", 48, 40, 100, 3, "uniform"),
]


def main():
    for name, M, N, K, seed, dist in CASES:
        A, B = make_inputs(M, N, K, seed=seed, dist=dist)
        ref64 = A.astype(np.float64) @ B.astype(np.float64).T
        np.savez_compressed(HERE / f"{name}.npz", A=A, B=B, ref_f32=ref64.astype(np.float32),
                            ref_f16=ref64.astype(np.float16), meta=np.array([M, N, K, seed]), dist=dist)
        print(name, A.shape, B.shape)


if __name__ == "__main__":
    main()
