"""Row-slab partition of C = A * B over several GPUs.

C (and A) are cut into contiguous row slabs, one per rank; B is replicated. Each rank then
runs the single-GPU entry point on ``(rows, N, K)`` with its own pointers -- row-major A and C
make a slab a plain sub-allocation -- and no data crosses GPUs during the multiply. The
reference itself is single-GPU (its only device knob is ``-gpu_rank``, reference
src/main.cu:45,51).
"""
from __future__ import annotations

from typing import List, Tuple


def row_slabs(M: int, world_size: int, align: int = 128) -> List[Tuple[int, int]]:
    """``[(row_begin, row_end), ...]`` for each rank.

    Slab boundaries fall on multiples of ``align`` rows (one tile height) so that every rank
    computes whole tiles with the same instruction sequence a single GPU would use for those
    rows; the last ranks get the shorter slabs when ``M`` does not divide evenly. Ranks beyond
    the available row blocks get an empty slab.
    """
    if M < 0 or world_size < 1 or align < 1:
        raise ValueError("M >= 0, world_size >= 1, align >= 1 required")
    blocks = (M + align - 1) // align
    base, extra = divmod(blocks, world_size)
    out = []
    begin_block = 0
    for r in range(world_size):
        nb = base + (1 if r < extra else 0)
        lo = min(begin_block * align, M)
        hi = min((begin_block + nb) * align, M)
        out.append((lo, hi))
        begin_block += nb
    return out
