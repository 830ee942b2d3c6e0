"""One process per GPU: each rank multiplies its row slab; C is gathered only on request.

The multiply needs no exchange (A and C are sharded by rows, B is replicated), so the only
collective is an optional all-gather of the C slabs over ``torch.distributed`` (NCCL on GPUs,
gloo in the CPU tests), issued after the GEMM on the same stream.
"""
from __future__ import annotations

from typing import Optional, Tuple

from .partition import row_slabs


def rank_slab(M: int, rank: int, world_size: int, align: int = 128) -> Tuple[int, int]:
    """Row range ``[begin, end)`` of C (and A) that ``rank`` owns."""
    return row_slabs(M, world_size, align)[rank]


def allgather_c(C_slab, M: int, N: int, group=None, align: int = 128):
    """All-gather the ranks' row slabs into the full ``[M, N]`` C on every rank.

    Slabs may differ in height (ragged M); each rank pads its slab to the tallest one for the
    collective and the padding is dropped when the result is assembled.
    """
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    slabs = row_slabs(M, world, align)
    lo, hi = slabs[rank]
    if tuple(C_slab.shape) != (hi - lo, N):
        raise ValueError(f"rank {rank} owns rows [{lo}, {hi}) but passed a slab of shape {tuple(C_slab.shape)}")
    tallest = max(h - l for l, h in slabs)
    if hi - lo == tallest and all(h - l == tallest for l, h in slabs):
        full = torch.empty((M, N), dtype=C_slab.dtype, device=C_slab.device)
        dist.all_gather_into_tensor(full, C_slab.contiguous(), group=group)
        return full
    padded = torch.zeros((tallest, N), dtype=C_slab.dtype, device=C_slab.device)
    padded[: hi - lo] = C_slab
    gathered = torch.empty((world * tallest, N), dtype=C_slab.dtype, device=C_slab.device)
    dist.all_gather_into_tensor(gathered, padded, group=group)
    full = torch.empty((M, N), dtype=C_slab.dtype, device=C_slab.device)
    for r, (l, h) in enumerate(slabs):
        full[l:h] = gathered[r * tallest: r * tallest + (h - l)]
    return full


def slab_hgemm(A_slab, B, C_slab: Optional[object] = None, kernel=None):
    """Multiply this rank's slab: ``C_slab = A_slab * B`` with the single-GPU entry point."""
    import torch

    from . import api

    if C_slab is None:
        C_slab = torch.empty((A_slab.shape[0], B.shape[0]), dtype=torch.float16, device=A_slab.device)
    if A_slab.shape[0] == 0:
        return C_slab
    (kernel or api.b200Hgemm)(A_slab, B, C_slab)
    return C_slab
