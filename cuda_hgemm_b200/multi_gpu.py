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


class SingleProcessGroup:
    """Several GPUs driven from ONE process through the C ABI's ``b200_mg_*`` entry points.

    The same row-slab partition as the one-process-per-GPU path above, for callers that hold all
    devices in one process: ``hgemm`` launches every device's slab on a stream the handle owns and
    returns; ``synchronize`` waits; ``elapsed_ms_max`` is the device time of the last multiply,
    the maximum over the devices; ``gather_c`` copies the slabs into full C buffers by peer copies.
    """

    def __init__(self, devices):
        import ctypes

        from . import _native

        self._native = _native
        self._ct = ctypes
        self.devices = [int(d) for d in devices]
        arr = (ctypes.c_int * len(self.devices))(*self.devices)
        handle = ctypes.c_void_p()
        _native.check(_native.load().b200_mg_create(arr, len(self.devices), ctypes.byref(handle)))
        self._handle = handle

    def close(self):
        if self._handle is not None:
            self._native.load().b200_mg_destroy(self._handle)
            self._handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def slab(self, M: int, index: int) -> Tuple[int, int]:
        ct = self._ct
        row0, rows = ct.c_size_t(), ct.c_size_t()
        self._native.check(self._native.load().b200_mg_slab(self._handle, M, index, ct.byref(row0), ct.byref(rows)))
        return row0.value, row0.value + rows.value

    def _pointers(self, tensors):
        ct = self._ct
        return (ct.c_void_p * len(self.devices))(*[(t.data_ptr() if t is not None and t.numel() else None) for t in tensors])

    def hgemm(self, A_slabs, B_replicas, C_slabs, M: int):
        """``C_slabs[i] = A_slabs[i] * B_replicas[i]`` on ``devices[i]``; returns without waiting."""
        N, K = B_replicas[0].shape
        self._native.check(self._native.load().b200_mg_hgemm(
            self._handle, self._pointers(A_slabs), self._pointers(B_replicas), self._pointers(C_slabs), M, N, K))

    def gather_c(self, C_slabs, C_full, M: int, N: int):
        """``C_full[i]`` (or ``None``) receives all slabs; ordered after the multiply on each owner's stream."""
        self._native.check(self._native.load().b200_mg_gather_c(
            self._handle, self._pointers(C_slabs), self._pointers(C_full), M, N))

    def synchronize(self):
        self._native.check(self._native.load().b200_mg_synchronize(self._handle))

    def elapsed_ms_max(self) -> float:
        ms = self._ct.c_float()
        self._native.check(self._native.load().b200_mg_elapsed_ms_max(self._handle, self._ct.byref(ms)))
        return float(ms.value)


def share_of_b(N: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Rows ``[begin, end)`` of B (columns of C) that ``rank`` brings to the exchange: equal shares."""
    if N % world_size != 0:
        raise ValueError("B is exchanged in equal shares: N must be a multiple of the number of ranks")
    share = N // world_size
    return rank * share, (rank + 1) * share


def exchange_b(B_full, rank: int, world_size: int, group=None):
    """All-gather B in place: on entry rank r's rows ``share_of_b(N, r, world)`` of ``B_full`` are valid,
    on return all of it is, on every rank. The one exchange step of the partitioned multiply when B
    starts on the hosts: every GPU pulls 1/world of B over its own host link and the rest over
    NVLink/NVSwitch (NCCL), instead of all of B over the host link."""
    import torch.distributed as dist

    lo, hi = share_of_b(B_full.shape[0], rank, world_size)
    dist.all_gather_into_tensor(B_full, B_full[lo:hi], group=group)
    return B_full


def slab_hgemm_host(A_host_slab, B_host, C_host_slab, B_dev, group=None):
    """This rank's slab from HOST memory: ``C_host_slab = A_host_slab * B_host^T``.

    ``B_host`` is the whole of B in this rank's (pinned) host memory, ``B_dev`` a device buffer of
    the same shape that the call fills: the rank's own share from the host, the other shares from
    the other ranks. With one rank this is ``api.hgemm_host``.
    """
    import torch
    import torch.distributed as dist

    from . import api

    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    if world == 1 or B_host.shape[0] % world != 0:
        return api.hgemm_host(A_host_slab, B_host, C_host_slab)
    rank = dist.get_rank(group)
    lo, hi = share_of_b(B_host.shape[0], rank, world)
    B_dev[lo:hi].copy_(B_host[lo:hi], non_blocking=True)
    share_up = torch.cuda.Event()
    share_up.record()                      # this rank's share of B is on its way over the host link
    exchange_b(B_dev, rank, world, group)
    b_complete = torch.cuda.Event()
    b_complete.record()                    # ... and behind this, all of B is on the device
    if A_host_slab.shape[0] == 0:
        torch.cuda.current_stream().synchronize()
        return C_host_slab
    # the rows of A follow the share of B over the host link while the other shares arrive over NVLink;
    # the multiplies wait for the exchange
    return api.hgemm_host_a(A_host_slab, B_dev, C_host_slab, upload_after=share_up, gemm_after=b_complete)
